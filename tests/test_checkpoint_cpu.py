"""Checkpoint round trips: distributed save -> resume, distributed -> HuggingFace -> per-block split -> load.

Follows the reference's checkpoint tests (tests/models/test_checkpoint_convert.py, test_model_correctness.py): a model
restored from disk must continue with the same losses as the run that wrote it."""
import json
import os

import pytest
import torch

from dist_utils import run_worker
from hetu_galvatron_b200.core.checkpoint import qkv_local_to_megatron, qkv_megatron_to_local
from hetu_galvatron_b200.tools import checkpoint_convert_g2h as g2h
from hetu_galvatron_b200.tools import checkpoint_convert_h2g as h2g

MODEL = dict(hidden_size=64, num_heads=4, num_kv_heads=2, ffn_hidden_size=128, num_layers=2, vocab_size=250, seq_length=32)
META = dict(dim=64, n_heads=4, n_kv_heads=2, ffn_dim=128, n_layers=2, vocab_size=250, n_positions=32)


def close(a, b, tol=2e-4):
    assert len(a) == len(b), (a, b)
    for x, y in zip(a, b):
        assert abs(x - y) < tol * max(1.0, abs(y)), (a, b)


def test_qkv_packing_round_trip():
    hq, hk, dh, h = 8, 2, 4, 16
    w = torch.arange((hq + 2 * hk) * dh * h, dtype=torch.float32).view(-1, h)
    m = qkv_local_to_megatron(w, hq, hk, dh)
    # first group: 4 query heads, then its key head, then its value head
    assert torch.equal(m[: 4 * dh], w[: 4 * dh])
    assert torch.equal(m[4 * dh:5 * dh], w[hq * dh:hq * dh + dh])
    assert torch.equal(m[5 * dh:6 * dh], w[(hq + hk) * dh:(hq + hk) * dh + dh])
    assert torch.equal(qkv_megatron_to_local(m, hq, hk, dh), w)


@pytest.mark.parametrize("world,plan", [(1, dict(global_bsz=8, chunks=1)),
                                        (2, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2, sequence_parallel=True)),
                                        (2, dict(global_bsz=8, chunks=2, sdp=1))], ids=["single", "tp2", "zero3"])
def test_resume_continues_the_run(tmp_path, world, plan):
    base = {"family": "llama", "model": MODEL, "plan": plan}
    full = run_worker({**base, "steps": 4, "save": {"dir": str(tmp_path), "iter": 2}}, world)
    assert os.path.exists(tmp_path / "hybrid_parallel_configs.json")
    assert os.path.exists(tmp_path / "iter_2" / "model_layers_0" / "0.pt")
    assert os.path.exists(tmp_path / "iter_2" / "optimizer" / "0.pt")
    resumed = run_worker({**base, "steps": 4, "load": {"dir": str(tmp_path), "iter": 2}}, world)
    close(resumed, full[2:])


def test_resume_rejects_another_plan(tmp_path):
    base = {"family": "llama", "model": MODEL}
    run_worker({**base, "plan": dict(global_bsz=8, chunks=1), "steps": 1, "save": {"dir": str(tmp_path), "iter": 1}}, 1)
    with pytest.raises(RuntimeError, match="Hybrid parallel configs are not equal"):
        run_worker({**base, "plan": dict(global_bsz=16, chunks=1), "steps": 2, "load": {"dir": str(tmp_path), "iter": 1}}, 1)


def test_tp2_checkpoint_to_hf_and_back(tmp_path):
    """tp2 run -> g2h -> HF state dict -> h2g split -> single-process load: same next-step loss."""
    ck, hf, split = tmp_path / "ck", tmp_path / "hf", tmp_path / "split"
    plan = dict(global_bsz=8, global_tp_deg=2, vocab_tp=2)
    full = run_worker({"family": "llama", "model": MODEL, "plan": plan, "steps": 3, "save": {"dir": str(ck), "iter": 2}}, 2)
    meta = tmp_path / "meta.json"
    meta.write_text(json.dumps(META))
    g2h.convert("llama", str(ck), str(hf), 2, str(meta), dtype=torch.float32)
    state = torch.load(hf / "pytorch_model.bin", weights_only=True)
    assert state["model.layers.1.self_attn.k_proj.weight"].shape == (2 * 16, 64)
    assert state["model.embed_tokens.weight"].shape == (250, 64) and state["lm_head.weight"].shape == (250, 64)
    files = h2g.convert("llama", str(hf), str(split), log=lambda s: None)
    assert sorted(os.path.basename(f) for f in set(files)) == ["lm_head.pt", "model_embed_tokens.pt", "model_layers_0.pt",
                                                              "model_layers_1.pt", "model_norm.pt"]
    again = run_worker({"family": "llama", "model": MODEL, "plan": dict(global_bsz=8, chunks=1), "steps": 3,
                        "load": {"dir": str(split), "iter": None, "start": 2}}, 1)
    close(again, full[2:])


def test_h2g_routes_other_families():
    assert h2g.route_key("gpt", "transformer.h.3.attn.c_attn.weight") == ("transformer.h.3", "attn.c_attn.weight")
    assert h2g.route_key("gpt", "transformer.wte.weight") == ("transformer.embedding", "wte.weight")
    assert h2g.route_key("gpt", "transformer.ln_f.bias") == ("transformer.ln_f", "bias")
    assert h2g.route_key("bert-mlm", "bert.encoder.layer.11.output.dense.bias") == ("bert.encoder.layer.11", "output.dense.bias")
    assert h2g.route_key("bert-mlm", "cls.predictions.transform.dense.weight") == ("cls.predictions", "transform.dense.weight")
    assert h2g.route_key("llama", "model.embed_tokens.weight") == ("model.embed_tokens", "embed_tokens.weight")
    assert h2g.route_key("llama", "lm_head.weight") == ("lm_head", "weight")
    assert h2g.route_key("llama", "model.norm.weight") == ("model.norm", "weight")


def test_t5_splits_but_refuses_huggingface_weights(tmp_path):
    """T5 keys are routed to per-block files, and the runtime says plainly that its T5 (no relative position bias, as in the
    reference) cannot take them, instead of starting from random weights without a word."""
    from types import SimpleNamespace

    from hetu_galvatron_b200.core.checkpoint import load_model

    assert h2g.route_key("t5", "encoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight") == \
        ("encoder.block.0", "layer.0.SelfAttention.relative_attention_bias.weight")
    assert h2g.route_key("t5", "shared.weight") == ("shared", "weight")
    with pytest.raises(NotImplementedError, match="relative position"):
        load_model(SimpleNamespace(), str(tmp_path), "t5")


def test_bert_tp2_checkpoint_to_hf_and_back(tmp_path):
    """BERT tp2 run -> g2h -> (HuggingFace model evaluates it) -> h2g split -> single-process run continues it."""
    model = dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=2, vocab_size=256, seq_length=32)
    meta = dict(hidden_size=64, num_attention_heads=4, intermediate_size=128, num_hidden_layers=2, vocab_size=256,
                max_position_embeddings=32, type_vocab_size=2, hidden_act="gelu_new", layer_norm_eps=1e-5)
    ck, hf, split = tmp_path / "ck", tmp_path / "hf", tmp_path / "split"
    plan = dict(global_bsz=4, global_tp_deg=2, vocab_tp=2)
    full = run_worker({"family": "bert", "model": model, "plan": plan, "steps": 3, "save": {"dir": str(ck), "iter": 2}}, 2)
    (tmp_path / "meta.json").write_text(json.dumps(meta))
    g2h.convert("bert", str(ck), str(hf), 2, str(tmp_path / "meta.json"), dtype=torch.float32)
    state = torch.load(hf / "pytorch_model.bin", weights_only=True)
    assert state["bert.encoder.layer.1.attention.self.key.weight"].shape == (64, 64)
    assert state["bert.encoder.layer.0.intermediate.dense.weight"].shape == (128, 64)
    assert state["cls.predictions.decoder.weight"].shape == (256, 64)
    transformers = pytest.importorskip("transformers")
    from hetu_galvatron_b200.models import build_model_specs, synthetic_batch
    cfg = transformers.BertConfig(**json.load(open(hf / "config.json")))
    cfg.hidden_dropout_prob = cfg.attention_probs_dropout_prob = 0.0
    ref = transformers.BertForMaskedLM(cfg).float().eval()
    missing, unexpected = ref.load_state_dict(state, strict=False)
    assert not [k for k in missing if "position_ids" not in k] and not unexpected
    mcfg, _ = build_model_specs("bert", dtype=torch.float32, **model)
    files = h2g.convert("bert-mlm", str(hf), str(split), log=lambda s: None)
    assert sorted(os.path.basename(f) for f in set(files)) == ["bert_embeddings.pt", "bert_encoder_layer_0.pt",
                                                              "bert_encoder_layer_1.pt", "cls_predictions.pt"]
    again = run_worker({"family": "bert", "model": model, "plan": dict(global_bsz=4, chunks=1), "steps": 3,
                        "load": {"dir": str(split), "iter": None, "start": 2}}, 1)
    close(again, full[2:])


@pytest.mark.parametrize("world,plan", [(1, dict(global_bsz=8, chunks=1)),
                                        (2, dict(global_bsz=8, chunks=2, default_dp_type="zero3", sdp=1)),
                                        (2, dict(global_bsz=8, chunks=2, pp_deg=2))],
                         ids=["single", "dp2_zero3", "pp2"])
def test_resume_under_another_plan_with_portable_optimizer_state(tmp_path, world, plan):
    """A dp2 / ZeRO-2 run saves portable optimizer state; runs with another data-parallel degree, ZeRO type or pipeline
    degree (same tensor-parallel degrees) continue it with the losses of the uninterrupted run."""
    base = {"family": "llama", "model": MODEL}
    first = dict(global_bsz=8, chunks=1, default_dp_type="zero2")
    full = run_worker({**base, "plan": first, "steps": 5, "save": {"dir": str(tmp_path), "iter": 2, "portable": True}}, 2)
    assert os.path.exists(tmp_path / "iter_2" / "model_layers_0" / "0.optim.pt")
    state = torch.load(tmp_path / "iter_2" / "model_layers_1" / "0.optim.pt", weights_only=True)
    some = next(iter(state.values()))
    assert set(some) == {"master", "exp_avg", "exp_avg_sq"} and some["master"].dtype == torch.float32
    resumed = run_worker({**base, "plan": plan, "steps": 5,
                          "load": {"dir": str(tmp_path), "iter": 2, "allow_plan_change": True}}, world)
    close(resumed, full[2:])


def test_gpt_tp2_checkpoint_to_hf_and_back(tmp_path):
    """GPT-2 tp2 run -> g2h -> a HuggingFace GPT2LMHeadModel evaluates the converted weights to the run's loss -> h2g split
    -> a single-process run continues with the losses of the uninterrupted run."""
    model = dict(hidden_size=64, num_heads=4, ffn_hidden_size=256, num_layers=2, vocab_size=256, seq_length=32)
    meta = dict(n_embd=64, n_head=4, n_layer=2, vocab_size=256, n_positions=32)
    ck, hf, split = tmp_path / "ck", tmp_path / "hf", tmp_path / "split"
    plan = dict(global_bsz=4, global_tp_deg=2, vocab_tp=2)
    full = run_worker({"family": "gpt", "model": model, "plan": plan, "steps": 3, "save": {"dir": str(ck), "iter": 2}}, 2)
    (tmp_path / "meta.json").write_text(json.dumps(meta))
    g2h.convert("gpt", str(ck), str(hf), 2, str(tmp_path / "meta.json"), dtype=torch.float32)
    state = torch.load(hf / "pytorch_model.bin", weights_only=True)
    assert state["transformer.h.1.attn.c_attn.weight"].shape == (64, 192)          # Conv1D layout [in, out]
    assert state["transformer.h.0.mlp.c_fc.weight"].shape == (64, 256) and state["transformer.wte.weight"].shape == (256, 64)
    transformers = pytest.importorskip("transformers")
    from hetu_galvatron_b200.models import build_model_specs, synthetic_batch
    cfg = transformers.GPT2Config(**json.load(open(hf / "config.json")))
    cfg.resid_pdrop = cfg.embd_pdrop = cfg.attn_pdrop = 0.0
    ref = transformers.GPT2LMHeadModel(cfg).float().eval()
    missing, unexpected = ref.load_state_dict(state, strict=False)
    assert not [k for k in missing if "attn.bias" not in k and "masked_bias" not in k] and not unexpected
    mcfg, _ = build_model_specs("gpt", dtype=torch.float32, **model)
    batch = synthetic_batch("gpt", mcfg, 4, seed=102, device="cpu")             # the batch of step 2 (seed 100 + step)
    with torch.no_grad():
        logits = ref(input_ids=batch[0]).logits
    hf_loss = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), batch[1].reshape(-1)).item()
    assert abs(hf_loss - full[2]) < 2e-4 * max(1.0, abs(full[2])), (hf_loss, full)
    files = h2g.convert("gpt", str(hf), str(split), log=lambda s: None)
    assert sorted(os.path.basename(f) for f in set(files)) == ["transformer_embedding.pt", "transformer_h_0.pt", "transformer_h_1.pt",
                                                              "transformer_ln_f.pt"]
    again = run_worker({"family": "gpt", "model": model, "plan": dict(global_bsz=4, chunks=1), "steps": 3,
                        "load": {"dir": str(split), "iter": None, "start": 2}}, 1)
    close(again, full[2:])


def test_vit_tp2_checkpoint_to_hf_and_back(tmp_path):
    """ViT tp2 run -> g2h -> transformers.ViTModel (+ pooler + the classifier) evaluates the converted weights to the run's
    loss -> h2g split -> a single-process run continues with the losses of the uninterrupted run."""
    model = dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=2, image_size=32, patch_size=8, num_channels=3,
                 num_labels=16, norm_eps=1e-12)
    meta = dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128, image_size=32, patch_size=8,
                num_channels=3, layer_norm_eps=1e-12, hidden_act="gelu_new")
    ck, hf, split = tmp_path / "ck", tmp_path / "hf", tmp_path / "split"
    plan = dict(global_bsz=4, global_tp_deg=2, vocab_tp=2)
    full = run_worker({"family": "vit", "model": model, "plan": plan, "steps": 3, "save": {"dir": str(ck), "iter": 2}}, 2)
    (tmp_path / "meta.json").write_text(json.dumps(meta))
    g2h.convert("vit", str(ck), str(hf), 2, str(tmp_path / "meta.json"), dtype=torch.float32)
    state = torch.load(hf / "pytorch_model.bin", weights_only=True)
    assert state["vit.embeddings.patch_embeddings.projection.weight"].shape == (64, 3, 8, 8)
    assert state["classifier.weight"].shape == (16, 64) and state["vit.encoder.layer.1.attention.attention.key.weight"].shape == (64, 64)
    transformers = pytest.importorskip("transformers")
    from hetu_galvatron_b200.models import build_model_specs, synthetic_batch
    cfg = transformers.ViTConfig(**{k: v for k, v in json.load(open(hf / "config.json")).items()
                                    if k in meta}, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    ref = transformers.ViTModel(cfg, add_pooling_layer=True).float().eval()
    missing, unexpected = ref.load_state_dict({k[len("vit."):]: v for k, v in state.items() if k.startswith("vit.")}, strict=False)
    assert not missing and not unexpected
    mcfg, _ = build_model_specs("vit", dtype=torch.float32, **model)
    pixels, labels = synthetic_batch("vit", mcfg, 4, seed=102, device="cpu")    # the batch of step 2 (seed 100 + step)
    with torch.no_grad():
        logits = ref(pixel_values=pixels.float()).pooler_output @ state["classifier.weight"].t()
    hf_loss = torch.nn.functional.cross_entropy(logits, labels).item()
    assert abs(hf_loss - full[2]) < 3e-4 * max(1.0, abs(full[2])), (hf_loss, full)
    h2g.convert("vit", str(hf), str(split), log=lambda s: None)
    again = run_worker({"family": "vit", "model": model, "plan": dict(global_bsz=4, chunks=1), "steps": 3,
                        "load": {"dir": str(split), "iter": None, "start": 2}}, 1)
    close(again, full[2:])


def test_t5_huggingface_round_trip_through_a_tp2_run(tmp_path):
    """HuggingFace T5 -> h2g split -> loaded by a tp2 run (relative position bias, relu) that saves a distributed checkpoint
    without changing the weights (learning rate 0) -> g2h: every tensor of the original state dict comes back, with the
    factors the loader folded into the query projections and the final decoder norm taken out again and the per-block bias
    tables merged into the one table per stack; a checkpoint whose tables drifted apart is refused."""
    transformers = pytest.importorskip("transformers")
    cfg = transformers.T5Config(vocab_size=256, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_decoder_layers=2, num_heads=4,
                                relative_attention_num_buckets=8, relative_attention_max_distance=20, dropout_rate=0.0,
                                initializer_factor=4.0, feed_forward_proj="relu", tie_word_embeddings=True,
                                decoder_start_token_id=0, pad_token_id=0)
    torch.manual_seed(3)
    hf_model = transformers.T5ForConditionalGeneration(cfg).float().eval()
    src, split, ck, back = tmp_path / "hf", tmp_path / "split", tmp_path / "ck", tmp_path / "back"
    os.makedirs(src)
    torch.save(hf_model.state_dict(), src / "pytorch_model.bin")
    h2g.convert("t5", str(src), str(split), log=lambda s: None)
    model = dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=2, num_decoder_layers=2, vocab_size=256,
                 seq_length=16, norm_eps=1e-6, act="relu", relative_attention_num_buckets=8, relative_attention_max_distance=20)
    run_worker({"family": "t5", "model": model, "plan": dict(global_bsz=4, global_tp_deg=2, vocab_tp=2), "steps": 1, "lr": 0.0,
                "load": {"dir": str(split), "iter": None, "start": 0}, "save": {"dir": str(ck), "iter": 1}}, 2)
    meta = dict(d_model=64, num_heads=4, d_ff=128, num_layers=2, num_decoder_layers=2, vocab_size=256, relative_attention_max_distance=20)
    (tmp_path / "meta.json").write_text(json.dumps(meta))
    g2h.convert("t5", str(ck), str(back), 1, str(tmp_path / "meta.json"), dtype=torch.float32)
    got = torch.load(back / "pytorch_model.bin", weights_only=True)
    want = hf_model.state_dict()
    assert set(want) <= set(got)
    for k, w in want.items():
        assert got[k].shape == w.shape and torch.allclose(got[k], w, rtol=1e-5, atol=1e-6), k
    assert json.load(open(back / "config.json"))["relative_attention_num_buckets"] == 8
    # tables that no longer agree have no HuggingFace form
    shard = ck / "iter_1" / "encoder_block_1" / "0.pt"
    sd = torch.load(shard)
    sd["layer.attn.rel_bias"] = sd["layer.attn.rel_bias"] + 1.0
    torch.save(sd, shard)
    with pytest.raises(ValueError, match="one\\s+table per stack|one table per stack"):
        g2h.convert("t5", str(ck), str(back), 1, str(tmp_path / "meta.json"), dtype=torch.float32)
