"""Zigzag ring attention on 2, 4 and 8 gloo ranks against attention over the whole sequence in one process: forward
output and dq / dk / dv, causal (the diag / first-half-KV / second-half-Q cases) and non-causal, with grouped KV heads
(reference: galvatron/core/runtime/tensor_parallel/transformer.py:2335-2551)."""
import json
import os

import pytest

from dist_utils import ROOT, _spawn_ranks
from hetu_galvatron_b200.parallel.ring_attention import kv_residency_bytes, ring_cases

CASES = [dict(s=64, b=2, hq=4, hk=2, dh=16, causal=True), dict(s=64, b=1, hq=2, hk=2, dh=8, causal=False),
         dict(s=128, b=1, hq=4, hk=1, dh=16, causal=True)]


@pytest.mark.parametrize("cp", [2, 4, 8])
def test_ring_attention_matches_whole_sequence(cp):
    env = dict(os.environ, OMP_NUM_THREADS="1")
    rc, out, err = _spawn_ranks([os.path.join(ROOT, "tests", "ring_worker.py"), json.dumps({"cases": CASES})], cp, env, 300)
    assert rc == 0, out[-2000:] + err[-4000:]
    worst = float([ln for ln in out.splitlines() if ln.startswith("WORST")][-1].split()[1])
    assert worst < 2e-5, worst


def test_ring_cases_cover_the_causal_mask_exactly_once():
    """Every (query chunk, key chunk) pair of the lower triangle is computed by exactly one step of one rank."""
    for cp in (2, 4, 8):
        seen = {}
        for r in range(cp):
            mine = (r, 2 * cp - 1 - r)
            for t, (src, case) in enumerate(ring_cases(cp, r, True)):
                theirs = (src, 2 * cp - 1 - src)
                if case == "diag":
                    pairs = [(mine[0], mine[0]), (mine[1], mine[0]), (mine[1], mine[1])]
                elif case == "kv_first":
                    pairs = [(mine[0], theirs[0]), (mine[1], theirs[0])]
                else:
                    pairs = [(mine[1], theirs[0]), (mine[1], theirs[1])]
                for p in pairs:
                    assert p[1] <= p[0], (cp, r, t, case, p)
                    seen[p] = seen.get(p, 0) + 1
        want = {(i, j) for i in range(2 * cp) for j in range(i + 1)}
        assert set(seen) == want and all(c == 1 for c in seen.values())


def test_ring_keeps_three_blocks_resident():
    m = kv_residency_bytes(seq=32768, batch=1, hk=32, dh=128, cp=8)
    assert m["ring"] * 3 == m["gather_all"]          # 3 blocks against 9
