"""The C++ host modules (search DP core, dataset index builders) built with the address and undefined-behaviour
sanitizers and driven through their Python entry points in a child process. Any report makes the child exit non-zero."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import numpy as np
from hetu_galvatron_b200.search.dynamic_programming import DPAlg
rng = np.random.default_rng(1)
for L, S, M in ((6, 5, 300), (1, 1, 8), (12, 9, 64), (3, 4, 0)):
    v = rng.integers(0, 40, size=(L, S)).astype(np.int32)
    intra, inter = rng.random((L, S)), rng.random((L, S, S)) * 0.1
    inter[0] = 0
    outs = []
    for use_cpp in (True, False):
        dp = DPAlg(M, {1: 5, 2: 9, 4: 10 ** 6}, {1: 0.5, 2: 0.25, 4: 0.1}, L, S, None, True, use_cpp_core=use_cpp)
        dp.set_v_and_cost(v, intra, inter)
        outs.append(dp.fit())
    (c1, r1, m1), (c2, r2, m2) = outs
    for k in c1:
        assert (np.isinf(c1[k]) and np.isinf(c2[k])) or abs(c1[k] - c2[k]) < 1e-12, (L, S, M, k)
        assert m1[k] == m2[k]
from hetu_galvatron_b200 import _build
native = _build.load_pybind("data_index")
sizes = rng.integers(1, 50, size=37).astype(np.int32)
doc_idx = np.concatenate([rng.permutation(37) for _ in range(3)]).astype(np.int32)
tokens = int(sizes.sum())
idx = native.build_sample_idx(sizes, doc_idx, 16, 3, tokens)
assert idx.shape[1] == 2 and idx.shape[0] == (3 * tokens - 1) // 16 + 1
which, index = native.build_blending_indices(np.array([0.2, 0.5, 0.3]), 1000)
assert len(which) == 1000 and abs((np.asarray(which) == 1).mean() - 0.5) < 0.01
print("SANITIZED_OK", _build.load_pybind("dp_core").__file__)
"""


def test_host_modules_under_address_and_ub_sanitizers(tmp_path):
    probe = subprocess.run(["g++", "-print-file-name=libasan.so"], capture_output=True, text=True)
    asan = probe.stdout.strip()
    if probe.returncode != 0 or not os.path.isabs(asan) or not os.path.exists(asan):
        pytest.skip("no address sanitizer runtime")
    env = dict(os.environ, GV_SANITIZE="address,undefined", LD_PRELOAD=asan, PYTHONPATH=ROOT,
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=97", UBSAN_OPTIONS="halt_on_error=1:exitcode=98")
    r = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, env=env, timeout=600, cwd=str(tmp_path))
    assert r.returncode == 0, (r.returncode, r.stdout[-500:], r.stderr[-2000:])
    assert "SANITIZED_OK" in r.stdout and "san_address_undefined" in r.stdout
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error:" not in r.stderr
