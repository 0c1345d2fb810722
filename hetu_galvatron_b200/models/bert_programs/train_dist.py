"""Hybrid-parallel training of the bert family (reference: galvatron/models/*/train_dist.py)."""
from hetu_galvatron_b200.models.runner import train

if __name__ == "__main__":
    train("bert", random_data=False)
