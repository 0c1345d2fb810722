"""The CPU plumbing configuration end to end: a tiny GPT decoder (4 layers, hidden 256, 4 heads, FFN 1024, vocabulary 1024,
learned positions, sequence 128, micro-batch 4) trained in fp32 on two gloo ranks with pure data parallelism, together
with the C++ dynamic-programming search over the same model on a synthetic profile (1 ms forward per layer, 2 GB/s links).
The plan the search writes is then run by the runtime. Needs no GPU."""
import json
import math
import os

import pytest

from dist_utils import run_worker
from hetu_galvatron_b200.search import GalvatronSearchEngine
from search_utils import search_args, write_tiny_gpt_profiles

MODEL = dict(hidden_size=256, num_heads=4, ffn_hidden_size=1024, num_layers=4, vocab_size=1024, seq_length=128)
SEQ = 128


def test_tiny_gpt_data_parallel_on_gloo_and_search_over_the_same_model(tmp_path):
    # ---- runtime: two gloo ranks, pure DP, fp32, micro-batch 4, token ids drawn from seed 0
    steps = 6
    dp2 = run_worker({"family": "gpt", "model": MODEL, "plan": dict(global_bsz=8, chunks=1), "steps": steps, "seed": 0}, 2)
    one = run_worker({"family": "gpt", "model": MODEL, "plan": dict(global_bsz=8, chunks=1), "steps": steps, "seed": 0}, 1)
    assert len(dp2) == steps and abs(dp2[0] - math.log(1024)) < 0.1          # normal(0, 0.02) weights: near-uniform logits
    for a, b in zip(dp2, one):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (dp2, one)

    # ---- search: the C++ dynamic program over the same model on the synthetic profile
    cfg_dir, hw_dir, name = write_tiny_gpt_profiles(str(tmp_path))
    out_dir = str(tmp_path / "out")
    args = search_args(num_gpus_per_node=2, memory_constraint=8, settle_bsz=8, settle_chunk=1, mixed_precision="fp32",
                       max_tp_deg=2, max_pp_deg=2, time_profiling_path=cfg_dir, memory_profiling_path=cfg_dir,
                       allreduce_bandwidth_config_path=hw_dir, p2p_bandwidth_config_path=hw_dir, overlap_coe_path=hw_dir,
                       sp_time_path=hw_dir, output_config_path=out_dir, log_dir=str(tmp_path / "logs"), hidden_size=256)
    eng = GalvatronSearchEngine(args)
    eng.set_search_engine_info(str(tmp_path), [{"hidden_size": 256, "layer_num": 4, "seq_len": SEQ}], name)
    eng.initialize_search_engine(show=False)
    throughput = eng.parallelism_optimization()
    assert throughput > 0
    plan = json.load(open(eng.output_path))
    # at 2 GB/s the per-layer tensor-parallel traffic and the pipeline bubble both cost more than the gradient all-reduce
    assert plan["pp_deg"] == 1 and plan["tp_sizes_enc"] == "1,1,1,1" and plan["global_bsz"] == 8 and plan["chunks"] == 1
    # 8 samples x (4 layers + embedding/head) x 1 ms forward x 3 (forward + backward) on 2 ranks: a step of 50-80 ms
    step_s = 8 / throughput
    assert 0.04 < step_s < 0.12, step_s

    # ---- the searched plan, executed by the runtime, is the data-parallel run above
    searched = run_worker({"family": "gpt", "model": MODEL, "plan_json": eng.output_path, "steps": steps, "seed": 0}, 2)
    for a, b in zip(searched, dp2):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (searched, dp2)


def test_symmetric_workspace_cache_reports_and_releases(monkeypatch):
    """The per-shape workspace cache of the fused paths: one object per (group, tag), statistics, selective release."""
    from types import SimpleNamespace

    from hetu_galvatron_b200.parallel import symm

    made = []

    class FakeWorkspace:
        def __init__(self, group, payload_bytes):
            self.nbytes = symm.FLAG_BYTES + payload_bytes
            made.append(self)

    monkeypatch.setattr(symm, "SymmWorkspace", FakeWorkspace)
    monkeypatch.setattr(symm, "_WORKSPACES", {})
    g01, g23 = SimpleNamespace(ranks=[0, 1]), SimpleNamespace(ranks=[2, 3])
    a = symm.workspace(g01, 1024, tag="act_8_64")
    assert symm.workspace(g01, 4096, tag="act_8_64") is a and len(made) == 1        # the first request fixes the size
    symm.workspace(g01, 2048, tag="u1_8_64")
    symm.workspace(g23, 512, tag="act_8_64")
    assert symm.workspace_stats() == {"count": 3, "bytes": 3 * symm.FLAG_BYTES + 1024 + 2048 + 512}
    assert symm.release_workspaces(g01, tag_prefix="act_") == symm.FLAG_BYTES + 1024
    assert symm.workspace_stats()["count"] == 2
    assert symm.release_workspaces(SimpleNamespace(ranks=[4, 5])) == 0
    assert symm.release_workspaces() == 2 * symm.FLAG_BYTES + 2048 + 512 and symm.workspace_stats() == {"count": 0, "bytes": 0}


def test_symmetric_workspace_guard_zones_catch_a_stray_store(monkeypatch):
    """Debug mode of the peer-memory workspaces: fixed-pattern zones behind the flag area and at the end of the buffer;
    a byte changed there names the zone and the offset."""
    import pytest
    import torch

    from hetu_galvatron_b200.parallel import symm

    buf = torch.zeros(symm.FLAG_BYTES + 2 * symm.CANARY_BYTES + 1024, dtype=torch.uint8)
    guard = symm.CanaryGuard(buf, symm.FLAG_BYTES, buf.numel() - symm.CANARY_BYTES)
    guard.arm()
    payload = buf[symm.FLAG_BYTES + symm.CANARY_BYTES: buf.numel() - symm.CANARY_BYTES]
    payload.fill_(7)                                   # the payload regions are free to change
    buf[:symm.FLAG_BYTES].fill_(1)                     # and so is the flag area
    guard.check()
    buf[buf.numel() - symm.CANARY_BYTES + 5] = 0       # a store one past the payload's end region
    with pytest.raises(RuntimeError, match="tail guard zone overwritten at byte offset %d" % (buf.numel() - symm.CANARY_BYTES + 5)):
        guard.check("act_8_64")
    guard.arm()
    buf[symm.FLAG_BYTES] = 3
    with pytest.raises(RuntimeError, match="head guard zone"):
        guard.check()
    monkeypatch.delenv("GV_SYMM_CANARY", raising=False)
    assert not symm.canaries_enabled() and symm.check_canaries() == 0


def test_groups_that_leave_the_node_keep_the_library_collectives(monkeypatch):
    """Peer-mapped memory exists inside one node only: with 4 ranks per node, a tensor-parallel pair is local, a
    data-parallel group over all 8 ranks is not, and a layer strategy built for such a group falls back to ``nccl``."""
    from hetu_galvatron_b200.core.hybrid_model import _strategy
    from hetu_galvatron_b200.parallel import symm
    from hetu_galvatron_b200.parallel.mesh import Mesh

    monkeypatch.delenv("LOCAL_WORLD_SIZE", raising=False)
    assert symm.ranks_on_one_node(range(16))                       # no launcher information: a single node
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "4")
    assert symm.ranks_on_one_node([0, 1, 2, 3]) and symm.ranks_on_one_node([4, 6])
    assert not symm.ranks_on_one_node([3, 4]) and not symm.ranks_on_one_node(range(8))
    mesh = Mesh(world_size=8, rank=5, pp_deg=1)
    assert _strategy(mesh, 2, "megatron", 1, "zero2", False, "fused").impl == "fused"      # ranks 4, 5
    assert _strategy(mesh, 8, "megatron", 1, "zero2", False, "fused").impl == "nccl"       # ranks 0..7 span two nodes
    assert _strategy(mesh, 2, "megatron", 4, "zero2", False, "fused").impl == "nccl"       # the context-parallel ring leaves the node
    assert _strategy(mesh, 8, "megatron", 1, "zero2", False, "nccl").impl == "nccl"
