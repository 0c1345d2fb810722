"""Hybrid-parallel training of the swin family (reference: galvatron/models/*/train_dist.py)."""
from hetu_galvatron_b200.models.runner import train

if __name__ == "__main__":
    train("swin", random_data=False)
