"""Model profiler entry for the swin family (reference: galvatron/models/*/profiler.py)."""
from hetu_galvatron_b200.models.runner import profile

if __name__ == "__main__":
    profile("swin")
