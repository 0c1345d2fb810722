"""Strategy search entry for the swin family (reference: galvatron/models/*/search_dist.py)."""
from hetu_galvatron_b200.models.runner import search

if __name__ == "__main__":
    search("swin")
