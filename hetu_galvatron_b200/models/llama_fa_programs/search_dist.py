"""Strategy search entry for the llama_fa family (reference: galvatron/models/*/search_dist.py)."""
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))  # run from a source checkout

from hetu_galvatron_b200.models.runner import search

if __name__ == "__main__":
    search("llama_fa")
