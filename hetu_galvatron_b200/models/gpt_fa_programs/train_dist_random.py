"""Hybrid-parallel training of the gpt_fa family on synthetic data (reference: galvatron/models/*/train_dist_random.py)."""
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))  # run from a source checkout

from hetu_galvatron_b200.models.runner import train

if __name__ == "__main__":
    train("gpt_fa", random_data=True)
