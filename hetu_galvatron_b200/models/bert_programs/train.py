"""Single-device training of the bert family (reference: galvatron/models/bert_hf/train.py)."""
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))  # run from a source checkout

from hetu_galvatron_b200.models.runner import train

if __name__ == "__main__":
    train("bert", random_data=True, single_device=True)
