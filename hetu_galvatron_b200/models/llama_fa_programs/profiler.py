"""Model profiler entry for the llama_fa family (reference: galvatron/models/*/profiler.py)."""
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))  # run from a source checkout

from hetu_galvatron_b200.models.runner import profile

if __name__ == "__main__":
    profile("llama_fa")
