"""Hybrid-parallel correctness on CPU ranks (gloo): every plan must reproduce the single-process losses.

Mirrors the reference's distributed correctness tests (tests/core/test_tp.py, test_pp.py, test_fsdp.py,
test_redistributed.py, test_hybrid.py), which need 8 real GPUs; here the same comparisons run as gloo ranks."""
import pytest

from dist_utils import run_worker

MODEL = dict(hidden_size=64, num_heads=4, num_kv_heads=2, ffn_hidden_size=128, num_layers=4, vocab_size=256, seq_length=32)
_BASE = {}


def baseline(family="llama", bsz=8, model=MODEL):
    key = (family, bsz, tuple(sorted(model.items())))
    if key not in _BASE:
        _BASE[key] = run_worker({"family": family, "model": model, "plan": {"global_bsz": bsz, "chunks": 1}, "steps": 3}, 1)
    return _BASE[key]


def check(losses, ref, tol=2e-5):
    assert len(losses) == len(ref)
    for a, b in zip(losses, ref):
        assert abs(a - b) < tol * max(1.0, abs(b)), (losses, ref)


CASES = {
    "dp2": (2, dict(global_bsz=8, chunks=2), {}),
    "dp2_zero2": (2, dict(global_bsz=8, chunks=2, default_dp_type="zero2"), {}),
    "dp2_zero3_ckpt": (2, dict(global_bsz=8, chunks=2, sdp=1, global_checkpoint=1), {}),
    "dp2_zero3_sync_reduce": (2, dict(global_bsz=8, chunks=2, sdp=1), {"async_grad_reduce": False}),
    "tp2": (2, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2), {}),
    "tp2_sp": (2, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2, sequence_parallel=True), {}),
    "ulysses2": (2, dict(global_bsz=8, global_tp_deg=2, use_ulysses=True, vocab_tp=2), {}),
    "cp2": (2, dict(global_bsz=8, global_cp_deg=2, vocab_cp=2), {}),
    "pp2_1f1b": (2, dict(global_bsz=8, pp_deg=2, chunks=4), {}),
    "pp2_gpipe": (2, dict(global_bsz=8, pp_deg=2, chunks=2, pipeline_type="gpipe"), {}),
    "tp2_dp2_zero3": (4, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2, sdp=1, chunks=2, sequence_parallel=True), {}),
    "pp2_tp2_sp": (4, dict(global_bsz=8, pp_deg=2, global_tp_deg=2, vocab_tp=2, chunks=2, sequence_parallel=True), {}),
}


@pytest.mark.parametrize("name", list(CASES))
def test_plan_matches_single_process(name):
    world, plan, extra = CASES[name]
    spec = {"family": "llama", "model": MODEL, "plan": plan, "steps": 3}
    spec.update(extra)
    check(run_worker(spec, world), baseline())


@pytest.mark.parametrize("ckpt", ["0,1,0,0", "0,0,1,0", "1,0,0,0"])
def test_layerwise_hybrid_plan_with_redistribution(ckpt):
    """Per-layer tp sizes 1,2,4,2 with mixed ZeRO types, Ulysses on one layer and checkpointing: exercises the
    relayout at every boundary (reference: tests/core/test_hybrid.py, test_redistributed.py). The checkpointed layer
    sits at boundaries whose local batch differs from the one the stage ends with, so its recomputation must use the
    batch size it saw in the first forward."""
    plan_json = {"pp_deg": 1, "tp_sizes_enc": "1,2,4,2", "tp_consecutive_flags": "1,1,1,1", "dp_types_enc": "0,1,0,1",
                 "use_sp": "0,0,0,1", "checkpoint": ckpt, "global_bsz": 8, "chunks": 2, "pp_division": "4",
                 "pipeline_type": "pipedream_flush", "default_dp_type": "zero2", "vtp": 2, "vsp": 0, "embed_sdp": 1}
    model = dict(MODEL, num_kv_heads=4)
    spec = {"family": "llama", "model": model, "plan_json": plan_json, "steps": 3, "sequence_parallel": True}
    check(run_worker(spec, 4), baseline(model=model))


FAMILY_MODELS = {
    "gpt": dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=4, vocab_size=250, seq_length=32),
    "bert": dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=4, vocab_size=256, seq_length=32),
    "vit": dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=4, image_size=32, patch_size=8, num_labels=16),
    "t5": dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=2, num_decoder_layers=2, vocab_size=256, seq_length=16),
    "swin": dict(model_size="swin-tiny-test"),
}

FAMILY_CASES = [
    ("gpt", 2, dict(global_bsz=8, chunks=2, default_dp_type="zero2")),
    ("gpt", 2, dict(global_bsz=8, pp_deg=2, chunks=4)),                      # tied embedding on two stages
    ("gpt", 2, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2, sequence_parallel=True)),
    ("bert", 2, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2, sequence_parallel=True)),
    ("vit", 2, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2)),
    ("vit", 2, dict(global_bsz=8, chunks=2, sdp=1)),
    ("t5", 2, dict(global_bsz=8, pp_deg=2, chunks=2)),                       # two activations cross the stage boundary
    ("t5", 2, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2)),
    ("t5", 2, dict(global_bsz=8, chunks=2)),                                 # tied embedding used by three blocks, DDP
    ("t5", 2, dict(global_bsz=8, chunks=2, sdp=1, global_checkpoint=1)),     # ZeRO-3 + recomputation of tuple-input blocks
    ("gpt", 2, dict(global_bsz=8, chunks=2)),                                # tied embedding, gradients all-reduced in place
    ("swin", 2, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2)),               # heads and MLP sharded, windows local
    ("swin", 2, dict(global_bsz=8, pp_deg=2, chunks=2)),                         # stage boundary between two resolutions
    ("swin", 2, dict(global_bsz=8, chunks=2, sdp=1, global_checkpoint=1)),       # window gather / bias attention recomputed under ZeRO-3
]


@pytest.mark.parametrize("family,world,plan", FAMILY_CASES, ids=[f"{f}-{i}" for i, (f, _, _) in enumerate(FAMILY_CASES)])
def test_model_families_match_single_process(family, world, plan):
    model = FAMILY_MODELS[family]
    spec = {"family": family, "model": model, "plan": plan, "steps": 3}
    check(run_worker(spec, world), baseline(family, 8, model))


@pytest.mark.parametrize("world,plan", [(2, dict(global_bsz=8, pp_deg=2, chunks=2)),
                                        (4, dict(global_bsz=8, pp_deg=2, global_tp_deg=2, vocab_tp=2, chunks=2, sequence_parallel=True))],
                         ids=["pp2", "pp2_tp2_sp"])          # TP + SP alone and ZeRO-3 + recomputation: see the relative-bias test below
def test_t5_with_a_decoder_length_of_its_own(world, plan):
    """Encoder 16 tokens, decoder 8 (reference: --encoder_seq_length / --decoder_seq_length, models/T5/arguments.py:26-27):
    the two activations that cross a decoder stage boundary differ in shape, cross-attention has more keys than queries, and
    labels follow the decoder; also with padding masks on both sides."""
    model = dict(FAMILY_MODELS["t5"], decoder_seq_length=8)
    ref = baseline("t5", 8, model)
    assert max(abs(a - b) for a, b in zip(ref, baseline("t5", 8, FAMILY_MODELS["t5"]))) > 1e-4
    check(run_worker({"family": "t5", "model": model, "plan": plan, "steps": 3}, world), ref)
    if plan.get("chunks") == 2 and "sdp" not in plan:
        # the mean over micro-batches of per-micro-batch means: compare runs that cut the batch the same way
        padded = {"family": "t5", "model": model, "plan": dict(global_bsz=8, chunks=2), "steps": 3, "padded": True}
        check(run_worker(dict(padded, plan=plan), world), run_worker(padded, 1))


@pytest.mark.parametrize("world,plan", [(2, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2, sequence_parallel=True)),
                                        (2, dict(global_bsz=8, pp_deg=2, chunks=2)),
                                        (2, dict(global_bsz=8, chunks=2, sdp=1, global_checkpoint=1))], ids=["tp2_sp", "pp2", "zero3_ckpt"])
def test_t5_relative_position_bias_trains_the_same_under_every_plan(world, plan):
    """The opt-in relative position bias (a [buckets, heads] table per self-attention layer, sharded by heads under tensor
    parallelism) and the relu feed-forward: three training steps reproduce the single-process losses, so the table's
    gradient is right under head sharding, stage splits and recomputation; and the bias changes the model."""
    model = dict(FAMILY_MODELS["t5"], decoder_seq_length=8, relative_attention_num_buckets=8, relative_attention_max_distance=12, act="relu")
    ref = baseline("t5", 8, model)
    plain = baseline("t5", 8, dict(FAMILY_MODELS["t5"], decoder_seq_length=8, act="relu"))
    assert max(abs(a - b) for a, b in zip(ref, plain)) > 1e-4
    check(run_worker({"family": "t5", "model": model, "plan": plan, "steps": 3}, world), ref)


@pytest.mark.parametrize("family", ["gpt", "t5"])
def test_tied_embedding_counts_once_in_the_gradient_norm_under_pipeline_parallelism(family):
    """Both pipeline ends hold a copy of a tied embedding with the summed gradient; with clipping active the step only
    matches the single-process run if the global norm counts that gradient once."""
    model = FAMILY_MODELS[family]
    one = run_worker({"family": family, "model": model, "plan": dict(global_bsz=8, chunks=1), "steps": 6, "clip": 1.0}, 1)
    pp2 = run_worker({"family": family, "model": model, "plan": dict(global_bsz=8, pp_deg=2, chunks=2), "steps": 6, "clip": 1.0}, 2)
    check(pp2, one, tol=5e-6)


def test_eight_rank_pipeline_with_per_layer_tensor_and_context_parallel_degrees():
    """pp 2 x (tp, cp) = (1, 2), (2, 1) | (4, 1), (2, 2) with one ZeRO-3 layer, GPipe, Megatron-SP: relayouts inside both
    stages, a stage boundary between different layouts, zigzag context parallelism on the first and last layer."""
    plan_json = {"pp_deg": 2, "tp_sizes_enc": "1,2,4,2", "tp_consecutive_flags": "1,1,1,1", "dp_types_enc": "0,1,0,0",
                 "use_sp": "0,0,0,0", "cp_sizes_enc": "2,1,1,2", "checkpoint": "0,0,0,0", "global_bsz": 8, "chunks": 2,
                 "pp_division": "2,2", "pipeline_type": "gpipe", "default_dp_type": "ddp", "vtp": 2, "vsp": 0, "vcp": 1,
                 "embed_sdp": 0}
    model = dict(MODEL, num_kv_heads=4)
    spec = {"family": "llama", "model": model, "plan_json": plan_json, "steps": 3, "sequence_parallel": True}
    check(run_worker(spec, 8), baseline(model=model))


def test_uneven_pipeline_division_with_mixed_tensor_parallel_degrees():
    plan_json = {"pp_deg": 2, "tp_sizes_enc": "2,1,2,1", "tp_consecutive_flags": "1,1,1,1", "dp_types_enc": "0,0,0,0",
                 "use_sp": "0,0,0,0", "checkpoint": "0,0,0,0", "global_bsz": 8, "chunks": 4, "pp_division": "3,1",
                 "pipeline_type": "pipedream_flush", "default_dp_type": "ddp", "vtp": 2, "vsp": 0, "embed_sdp": 0}
    model = dict(MODEL, num_kv_heads=4)
    spec = {"family": "llama", "model": model, "plan_json": plan_json, "steps": 3, "sequence_parallel": True}
    check(run_worker(spec, 4), baseline(model=model))


@pytest.mark.parametrize("family", ["t5", "bert"])
def test_padding_masks_hide_padded_tokens(family):
    """Encoder and decoder padding masks (and the encoder mask in cross-attention): whatever token ids sit at padded
    positions, the losses do not move (reference: galvatron/models/T5/T5Model_tensor_parallel.py:96-115)."""
    model = FAMILY_MODELS[family]
    base = {"family": family, "model": model, "plan": dict(global_bsz=8, chunks=2), "steps": 2, "padded": True}
    a = run_worker(base, 1)
    b = run_worker(dict(base, scramble_padding=True), 1)
    c = run_worker(dict(base, padded=False), 1)
    check(a, b, tol=1e-6)
    assert max(abs(x - y) for x, y in zip(a, c)) > 1e-4          # padding changes the loss, scrambling it does not
    d = run_worker(dict(base, scramble_padding=True, plan=dict(global_bsz=8, chunks=2, global_tp_deg=2, vocab_tp=2)), 2)
    check(d, a)


@pytest.mark.parametrize("plan", [dict(global_bsz=8, chunks=2, default_dp_type="zero2"), dict(global_bsz=8, pp_deg=2, chunks=2)])
def test_scaled_loss_and_an_overflow_on_one_rank(plan):
    """Loss scaling across ranks: scaling the loss by 2^12 and dividing it out in the optimizer step reproduces the
    unscaled run, and a non-finite gradient on ONE rank makes EVERY rank skip that step (the norm is a job-wide sum), after
    which training continues from unchanged weights."""
    base = {"family": "llama", "model": MODEL, "plan": plan, "steps": 4, "clip": 1.0}
    plain = run_worker(base, 2)
    scaled, flags = run_worker(dict(base, loss_scale=4096.0, report_skipped=True), 2)
    check(scaled, plain)
    assert flags == [[False] * 4, [False] * 4]
    hit, flags = run_worker(dict(base, loss_scale=4096.0, report_skipped=True, poison={"iter": 1, "rank": 0}), 2)
    assert flags == [[False, True, False, False]] * 2
    check(hit[:2], plain[:2])                       # the poisoned step still reports its (finite) loss
    # step 1 changed nothing, so step 2 of this run sees the weights that step 1 of the plain run saw; both draw other batches,
    # so only its finiteness and the continued descent can be compared
    assert all(abs(v) < 1e3 for v in hit)
