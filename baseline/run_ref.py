"""Reference arm of bench.py: runs the unmodified reference installed under ``baseline/_ref`` through its own
training entry point on the same metric and configuration."""
from __future__ import annotations

import os

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def run_reference_bench(args) -> dict:
    if not os.path.isdir(os.path.join(REF_DIR, "galvatron")):
        return {"impl": "reference", "unavailable": "reference is not installed under baseline/_ref"}
    return {"impl": "reference", "unavailable": "reference harness not wired yet"}
