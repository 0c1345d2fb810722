"""The flag / epoch protocol of the fused communication kernels, run by a host-side simulator (threads as ranks, plain
memory as payload) under randomised interleavings, also as a thread-sanitizer build. Failures are made on the host: a rank
that stops announcing makes the others' bounded waits give up and report, and every thread still finishes."""
import json
import os
import subprocess

import pytest

SRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "hetu_galvatron_b200", "csrc", "sim",
                   "flag_protocol_sim.cpp")


def _build(tmp, tsan):
    exe = os.path.join(tmp, "sim_tsan" if tsan else "sim")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-pthread"] + (["-fsanitize=thread"] if tsan else []) + [SRC, "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        if tsan:
            pytest.skip("no thread sanitizer runtime: " + r.stderr[-200:])
        raise AssertionError(r.stderr)
    return exe


def _run(exe, *flags, timeout=120):
    r = subprocess.run([exe] + [str(f) for f in flags], capture_output=True, text=True, timeout=timeout)
    line = [l for l in r.stdout.splitlines() if l.startswith("{")]
    return r.returncode, (json.loads(line[-1]) if line else None), r.stderr


@pytest.fixture(scope="module")
def sim(tmp_path_factory):
    return _build(str(tmp_path_factory.mktemp("sim")), tsan=False)


@pytest.mark.parametrize("mode", ["pull", "push"])
@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_double_buffered_protocol_never_shows_stale_data(sim, mode, ranks):
    for seed in (1, 2, 3):
        rc, out, _ = _run(sim, "--ranks", ranks, "--epochs", 200, "--mode", mode, "--seed", seed)
        assert rc == 0 and out["mismatches"] == 0 and out["timeouts"] == 0, out


@pytest.mark.parametrize("mode", ["pull", "push"])
def test_checker_sees_the_hazard_without_double_buffering(sim, mode):
    seen = 0
    for seed in (1, 2, 3, 4):
        rc, out, _ = _run(sim, "--ranks", 4, "--epochs", 300, "--mode", mode, "--seed", seed, "--single-buffer")
        seen += out["mismatches"]
        assert (rc != 0) == (out["mismatches"] > 0)
    assert seen > 0


@pytest.mark.parametrize("mode,site", [("pull", 0x11), ("push", 0x12)])
def test_a_rank_that_stops_announcing_ends_the_others_waits(sim, mode, site):
    rc, out, _ = _run(sim, "--ranks", 4, "--epochs", 50, "--mode", mode, "--drop-rank", 2, "--drop-epoch", 20,
                      "--budget-us", 50000, timeout=60)
    assert rc == 0 and out["mismatches"] == 0
    assert out["timeouts"] == 3                                   # every survivor gave up once, then stopped
    assert out["error"]["site"] == site and out["error"]["src"] == 2 and out["error"]["epoch"] == 20


def test_thread_sanitizer_build_is_clean(tmp_path):
    exe = _build(str(tmp_path), tsan=True)
    for mode in ("pull", "push"):
        rc, out, err = _run(exe, "--ranks", 4, "--epochs", 100, "--mode", mode, "--seed", 5)
        if out is None and "ThreadSanitizer" in err and "unexpected memory mapping" in err:
            pytest.skip("thread sanitizer cannot map its shadow memory on this kernel")
        assert rc == 0 and "data race" not in err and out["mismatches"] == 0, err[-500:]
    # and it does report the unordered accesses of the single-buffer variant
    rc, out, err = _run(exe, "--ranks", 3, "--epochs", 50, "--mode", "push", "--single-buffer")
    assert rc != 0 and "data race" in err


@pytest.mark.parametrize("ranks,clip", [(2, False), (4, False), (8, False), (4, True), (8, True)])
def test_zero_engine_protocol_orders_gradients_and_parameters(sim, ranks, clip):
    """READY / DONE / PARAM of the ZeRO engine's peer-memory path on single-buffered gradient and parameter buffers: every
    owner reads complete gradient slices of the right step, nobody clears a bucket a peer still reads, nobody reads a
    parameter slice before its owner's push, with or without the job-wide all-reduce of the gradient norm in between."""
    for seed in (1, 2, 3):
        rc, out, _ = _run(sim, "--ranks", ranks, "--epochs", 200, "--mode", "zero", "--seed", seed, *(["--clip"] if clip else []))
        assert rc == 0 and out["mode"] == "zero" and out["mismatches"] == 0 and out["timeouts"] == 0, out


def test_zero_engine_checker_sees_a_bucket_cleared_too_early(sim):
    seen = 0
    for seed in (1, 2, 3):
        rc, out, _ = _run(sim, "--ranks", 4, "--epochs", 200, "--mode", "zero", "--seed", seed, "--skip-done-wait")
        seen += out["mismatches"]
        assert (rc != 0) == (out["mismatches"] > 0)
    assert seen > 0


def test_zero_engine_survivors_give_up_when_a_rank_leaves(sim):
    rc, out, _ = _run(sim, "--ranks", 4, "--epochs", 50, "--mode", "zero", "--drop-rank", 2, "--drop-epoch", 20,
                      "--budget-us", 50000, timeout=60)
    assert rc == 0 and out["mismatches"] == 0 and out["timeouts"] == 3
    assert out["error"]["site"] == 0x15 and out["error"]["src"] == 2 and out["error"]["epoch"] == 20   # waiting for READY(20)


def test_zero_engine_protocol_under_the_thread_sanitizer(tmp_path):
    exe = _build(str(tmp_path), tsan=True)
    rc, out, err = _run(exe, "--ranks", 4, "--epochs", 100, "--mode", "zero", "--seed", 5)
    if out is None and "ThreadSanitizer" in err and "unexpected memory mapping" in err:
        pytest.skip("thread sanitizer cannot map its shadow memory on this kernel")
    assert rc == 0 and "data race" not in err and out["mismatches"] == 0, err[-500:]
    rc, out, err = _run(exe, "--ranks", 4, "--epochs", 100, "--mode", "zero", "--seed", 5, "--skip-done-wait")
    assert "data race" in err


@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_mailbox_protocol_with_targeted_reader_waits(sim, ranks):
    """The ring transport: a writer reuses a buffer after waiting only for the ranks that read its publication two epochs
    back; readers are a changing subset of the peers."""
    for seed in (1, 2, 3):
        rc, out, _ = _run(sim, "--ranks", ranks, "--epochs", 300, "--mode", "mailbox", "--seed", seed)
        assert rc == 0 and out["mode"] == "mailbox" and out["mismatches"] == 0 and out["timeouts"] == 0, out


def test_mailbox_checker_sees_a_buffer_reused_under_its_readers(sim):
    seen = 0
    for seed in (1, 2, 3):
        rc, out, _ = _run(sim, "--ranks", 4, "--epochs", 400, "--mode", "mailbox", "--seed", seed, "--skip-reader-wait")
        seen += out["mismatches"]
    assert seen > 0
    rc, out, _ = _run(sim, "--ranks", 4, "--epochs", 50, "--mode", "mailbox", "--drop-rank", 2, "--drop-epoch", 20,
                      "--budget-us", 50000, timeout=60)
    assert rc == 0 and out["mismatches"] == 0 and out["timeouts"] == 3 and out["error"]["site"] in (0x17, 0x18)
