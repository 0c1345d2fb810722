"""Weights of a HuggingFace model, split by the h2g tool and loaded through ``load_model``, must reproduce the
HuggingFace model's loss (the reference's correctness tests compare against an un-parallelised HF baseline the same way:
tests/core/test_tp.py:60-69, tests/models/test_model_correctness.py:109-117)."""
import json
import os

import pytest
import torch

from dist_utils import run_worker
from hetu_galvatron_b200.tools import checkpoint_convert_h2g as h2g

transformers = pytest.importorskip("transformers")


def _hf_loss(model, tokens):
    with torch.no_grad():
        out = model(input_ids=tokens[:, :-1], labels=None).logits.float()
    return torch.nn.functional.cross_entropy(out.reshape(-1, out.shape[-1]), tokens[:, 1:].reshape(-1)).item()


def _tokens(vocab, bsz, seq, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (bsz, seq + 1), generator=g)


@pytest.mark.parametrize("world,plan", [(1, dict(global_bsz=4, chunks=1)), (2, dict(global_bsz=4, global_tp_deg=2, vocab_tp=2))],
                         ids=["single", "tp2"])
def test_llama_matches_huggingface(tmp_path, world, plan):
    cfg = transformers.LlamaConfig(initializer_range=0.15, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=256, max_position_embeddings=64, rms_norm_eps=1e-5,
                                   rope_theta=10000.0, tie_word_embeddings=False, attention_bias=False)
    torch.manual_seed(0)
    hf = transformers.LlamaForCausalLM(cfg).float().eval()
    os.makedirs(tmp_path / "hf")
    torch.save(hf.state_dict(), tmp_path / "hf" / "pytorch_model.bin")
    h2g.convert("llama", str(tmp_path / "hf"), str(tmp_path / "split"), log=lambda s: None)
    model = dict(hidden_size=64, num_heads=4, num_kv_heads=2, ffn_hidden_size=128, num_layers=2, vocab_size=256, seq_length=32)
    spec = {"family": "llama", "model": model, "plan": plan, "steps": 1, "lr": 0.0, "data_seed": 100,
            "load": {"dir": str(tmp_path / "split"), "iter": None, "start": 0}}
    ours = run_worker(spec, world)[0]
    # the worker's batch for step 0 is synthetic_batch(seed=100): same generator recipe here
    from hetu_galvatron_b200.models import build_model_specs, synthetic_batch
    mcfg, _ = build_model_specs("llama", dtype=torch.float32, **model)
    tok_in, tok_lab = synthetic_batch("llama", mcfg, 4, seed=100, device="cpu")
    tokens = torch.cat([tok_in, tok_lab[:, -1:]], 1)
    ref = _hf_loss(hf, tokens)
    assert abs(ours - ref) < 2e-4 * max(1.0, abs(ref)), (ours, ref)
    # the same model built without initial values (what --initialize_on_meta 1 --load does): every weight must come
    # from the checkpoint, none may keep its uninitialised storage
    deferred = run_worker(dict(spec, defer_init=True), world)[0]
    assert deferred == ours, (deferred, ours)


def test_gpt2_matches_huggingface(tmp_path):
    cfg = transformers.GPT2Config(initializer_range=0.15, n_embd=64, n_layer=2, n_head=4, n_positions=32, vocab_size=256, n_inner=128,
                                  activation_function="gelu_new", resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0,
                                  layer_norm_epsilon=1e-5)
    torch.manual_seed(0)
    hf = transformers.GPT2LMHeadModel(cfg).float().eval()
    os.makedirs(tmp_path / "hf")
    torch.save({k: v for k, v in hf.state_dict().items() if not k.endswith(".attn.bias") and not k.endswith("masked_bias")},
               tmp_path / "hf" / "pytorch_model.bin")
    h2g.convert("gpt", str(tmp_path / "hf"), str(tmp_path / "split"), log=lambda s: None)
    model = dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=2, vocab_size=256, seq_length=32)
    from hetu_galvatron_b200.models import build_model_specs, synthetic_batch
    mcfg, _ = build_model_specs("gpt", dtype=torch.float32, **model)
    tok_in, tok_lab = synthetic_batch("gpt", mcfg, 4, seed=100, device="cpu")
    ref = _hf_loss(hf, torch.cat([tok_in, tok_lab[:, -1:]], 1))
    for world, plan in ((1, dict(global_bsz=4, chunks=1)), (2, dict(global_bsz=4, global_tp_deg=2, vocab_tp=2))):
        spec = {"family": "gpt", "model": model, "plan": plan, "steps": 1, "lr": 0.0,
                "load": {"dir": str(tmp_path / "split"), "iter": None, "start": 0}}
        ours = run_worker(spec, world)[0]
        assert abs(ours - ref) < 3e-4 * max(1.0, abs(ref)), (world, ours, ref)


def test_bert_mlm_matches_huggingface(tmp_path):
    cfg = transformers.BertConfig(initializer_range=0.15, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                                  vocab_size=256, max_position_embeddings=32, type_vocab_size=2, hidden_act="gelu_new",
                                  hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, layer_norm_eps=1e-12)
    torch.manual_seed(0)
    hf = transformers.BertForMaskedLM(cfg).float().eval()
    os.makedirs(tmp_path / "hf")
    torch.save(hf.state_dict(), tmp_path / "hf" / "pytorch_model.bin")
    h2g.convert("bert-mlm", str(tmp_path / "hf"), str(tmp_path / "split"), log=lambda s: None)
    model = dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=2, vocab_size=256, seq_length=32)
    from hetu_galvatron_b200.models import build_model_specs, synthetic_batch
    mcfg, _ = build_model_specs("bert", dtype=torch.float32, **model)
    ids, labels = synthetic_batch("bert", mcfg, 4, seed=100, device="cpu")
    with torch.no_grad():
        ref = hf(input_ids=ids, labels=labels).loss.item()
    for world, plan in ((1, dict(global_bsz=4, chunks=1)), (2, dict(global_bsz=4, global_tp_deg=2, vocab_tp=2))):
        spec = {"family": "bert", "model": model, "plan": plan, "steps": 1, "lr": 0.0,
                "load": {"dir": str(tmp_path / "split"), "iter": None, "start": 0}}
        ours = run_worker(spec, world)[0]
        assert abs(ours - ref) < 3e-4 * max(1.0, abs(ref)), (world, ours, ref)


def test_bert_padded_batch_matches_huggingface(tmp_path):
    """Sequences of different lengths, padded on the right: the padding mask must keep padded keys out of every softmax
    (reference: galvatron/models/bert_hf/BertModel_sequential.py:12-15, BertModel_tensor_parallel.py:31-33,67-69)."""
    cfg = transformers.BertConfig(initializer_range=0.15, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                                  vocab_size=256, max_position_embeddings=32, type_vocab_size=2, hidden_act="gelu_new",
                                  hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, layer_norm_eps=1e-12)
    torch.manual_seed(0)
    hf = transformers.BertForMaskedLM(cfg).float().eval()
    os.makedirs(tmp_path / "hf")
    torch.save(hf.state_dict(), tmp_path / "hf" / "pytorch_model.bin")
    h2g.convert("bert-mlm", str(tmp_path / "hf"), str(tmp_path / "split"), log=lambda s: None)
    model = dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=2, vocab_size=256, seq_length=32)
    from hetu_galvatron_b200.models import build_model_specs, synthetic_batch
    mcfg, _ = build_model_specs("bert", dtype=torch.float32, **model)
    ids, labels, extra = synthetic_batch("bert", mcfg, 4, seed=100, device="cpu", padded=True)
    assert extra["attention_mask"].sum(1).min() < 32                     # the batch really is ragged
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=extra["attention_mask"], labels=labels).loss.item()
        unmasked = hf(input_ids=ids, labels=labels).loss.item()
    assert abs(ref - unmasked) > 1e-3                                    # and the mask matters for the loss
    for world, plan in ((1, dict(global_bsz=4, chunks=2)), (2, dict(global_bsz=4, global_tp_deg=2, vocab_tp=2))):
        spec = {"family": "bert", "model": model, "plan": plan, "steps": 1, "lr": 0.0, "padded": True,
                "load": {"dir": str(tmp_path / "split"), "iter": None, "start": 0}}
        ours = run_worker(spec, world)[0]
        assert abs(ours - ref) < 3e-4 * max(1.0, abs(ref)), (world, ours, ref)


def test_vit_matches_huggingface(tmp_path):
    """ViT encoder with pooler (the reference adds HuggingFace's ViTPooler in front of the classifier,
    models/vit_hf/ViTModel_sequential.py:116-140) against transformers.ViTModel + a linear classifier."""
    cfg = transformers.ViTConfig(initializer_range=0.15, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                 intermediate_size=128, image_size=32, patch_size=8, num_channels=3, hidden_act="gelu_new",
                                 hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, layer_norm_eps=1e-12)
    torch.manual_seed(0)
    hf = transformers.ViTModel(cfg, add_pooling_layer=True).float().eval()
    classifier = torch.nn.Linear(64, 16, bias=False)
    torch.nn.init.normal_(classifier.weight, std=0.3)
    torch.nn.init.normal_(hf.pooler.dense.weight, std=0.15)
    state = {"vit." + k: v for k, v in hf.state_dict().items()}
    state["classifier.weight"] = classifier.weight.detach()
    os.makedirs(tmp_path / "hf")
    torch.save(state, tmp_path / "hf" / "pytorch_model.bin")
    h2g.convert("vit", str(tmp_path / "hf"), str(tmp_path / "split"), log=lambda s: None)
    model = dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=2, image_size=32, patch_size=8, num_channels=3,
                 num_labels=16, norm_eps=1e-12)
    from hetu_galvatron_b200.models import build_model_specs, synthetic_batch
    mcfg, _ = build_model_specs("vit", dtype=torch.float32, **model)
    pixels, labels = synthetic_batch("vit", mcfg, 4, seed=100, device="cpu")
    with torch.no_grad():
        pooled = hf(pixel_values=pixels.float()).pooler_output
        ref = torch.nn.functional.cross_entropy(classifier(pooled), labels).item()
    assert abs(ref - 2.7726) > 0.05          # the loss depends on the weights (ln 16 = 2.7726 for uniform logits)
    for world, plan in ((1, dict(global_bsz=4, chunks=1)), (2, dict(global_bsz=4, global_tp_deg=2, vocab_tp=2))):
        spec = {"family": "vit", "model": model, "plan": plan, "steps": 1, "lr": 0.0,
                "load": {"dir": str(tmp_path / "split"), "iter": None, "start": 0}}
        ours = run_worker(spec, world)[0]
        assert abs(ours - ref) < 3e-4 * max(1.0, abs(ref)), (world, ours, ref)


def test_swin_matches_huggingface(tmp_path):
    """Four-stage Swin (windowed and shifted-window attention, relative position bias, patch merging) against
    transformers.SwinForImageClassification, single process and TP = 2."""
    cfg = transformers.SwinConfig(initializer_range=0.15, image_size=128, patch_size=4, num_channels=3, embed_dim=32,
                                  depths=[1, 1, 2, 1], num_heads=[2, 2, 4, 4], window_size=4, mlp_ratio=4, qkv_bias=True,
                                  hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, drop_path_rate=0.0,
                                  hidden_act="gelu_new", layer_norm_eps=1e-5, num_labels=16)
    torch.manual_seed(0)
    hf = transformers.SwinForImageClassification(cfg).float().eval()
    with torch.no_grad():
        for name, p in hf.named_parameters():
            if name.endswith("relative_position_bias_table"):
                p.normal_(std=0.5)                       # zero at initialisation: make the bias matter
            if name == "classifier.bias":
                p.zero_()
    os.makedirs(tmp_path / "hf")
    torch.save(hf.state_dict(), tmp_path / "hf" / "pytorch_model.bin")
    files = h2g.convert("swin", str(tmp_path / "hf"), str(tmp_path / "split"), log=lambda s: None)
    assert "swin_encoder_2_1.pt" in {os.path.basename(f) for f in files} and "swin_encoder_2_downsample.pt" in {os.path.basename(f) for f in files}
    model = dict(model_size="swin-tiny-test", image_size=128)      # resolutions 32, 16, 8, 4: every stage holds whole windows
    from hetu_galvatron_b200.models import build_model_specs, synthetic_batch
    mcfg, _ = build_model_specs("swin", dtype=torch.float32, **model)
    pixels, labels = synthetic_batch("swin", mcfg, 4, seed=100, device="cpu")
    with torch.no_grad():
        ref = hf(pixel_values=pixels.float(), labels=labels).loss.item()
    assert abs(ref - 2.7726) > 0.05
    for world, plan in ((1, dict(global_bsz=4, chunks=1)), (2, dict(global_bsz=4, global_tp_deg=2, vocab_tp=2))):
        spec = {"family": "swin", "model": model, "plan": plan, "steps": 1, "lr": 0.0,
                "load": {"dir": str(tmp_path / "split"), "iter": None, "start": 0}}
        ours = run_worker(spec, world)[0]
        assert abs(ours - ref) < 3e-4 * max(1.0, abs(ref)), (world, ours, ref)


def test_t5_with_relative_position_bias_matches_huggingface(tmp_path):
    """T5 built with the relative position bias and the relu feed-forward (both opt-in; the reference's T5 has neither
    bias nor a checkpoint loader) against transformers.T5ForConditionalGeneration: bidirectional buckets in the encoder,
    one-sided buckets + causal mask in the decoder, unscaled scores and the d_model^-0.5 head factor folded into the loaded
    weights, padding masks on both sides, a decoder shorter than the encoder; single process, TP = 2 and PP = 2."""
    cfg = transformers.T5Config(vocab_size=256, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_decoder_layers=2, num_heads=4,
                                relative_attention_num_buckets=8, relative_attention_max_distance=20, dropout_rate=0.0,
                                layer_norm_epsilon=1e-6, initializer_factor=4.0, feed_forward_proj="relu",
                                tie_word_embeddings=True, decoder_start_token_id=0, pad_token_id=0)
    torch.manual_seed(0)
    hf = transformers.T5ForConditionalGeneration(cfg).float().eval()
    os.makedirs(tmp_path / "hf")
    torch.save(hf.state_dict(), tmp_path / "hf" / "pytorch_model.bin")
    files = {os.path.basename(f) for f in h2g.convert("t5", str(tmp_path / "hf"), str(tmp_path / "split"), log=lambda s: None)}
    assert {"shared.pt", "encoder_block_0.pt", "decoder_block_1.pt", "encoder_final_layer_norm.pt"} <= files
    model = dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=2, num_decoder_layers=2, vocab_size=256,
                 seq_length=24, decoder_seq_length=16, norm_eps=1e-6, act="relu", relative_attention_num_buckets=8,
                 relative_attention_max_distance=20)
    from hetu_galvatron_b200.models import build_model_specs, synthetic_batch
    mcfg, _ = build_model_specs("t5", dtype=torch.float32, **model)
    enc, labels, extra = synthetic_batch("t5", mcfg, 4, seed=100, device="cpu", padded=True)
    with torch.no_grad():
        ref = hf(input_ids=enc, attention_mask=extra["attention_mask"], decoder_input_ids=extra["decoder_input_ids"],
                 decoder_attention_mask=extra["decoder_attention_mask"], labels=labels).loss.item()
        flat = hf(input_ids=enc, decoder_input_ids=extra["decoder_input_ids"], labels=labels).loss.item()
    assert abs(ref - 5.545) > 0.05 and abs(ref - flat) > 1e-3        # depends on the weights (ln 256 = 5.545) and on the masks
    for world, plan in ((1, dict(global_bsz=4, chunks=1)), (2, dict(global_bsz=4, global_tp_deg=2, vocab_tp=2)),
                        (2, dict(global_bsz=4, pp_deg=2, chunks=1))):
        spec = {"family": "t5", "model": model, "plan": plan, "steps": 1, "lr": 0.0, "padded": True,
                "load": {"dir": str(tmp_path / "split"), "iter": None, "start": 0}}
        ours = run_worker(spec, world)[0]
        assert abs(ours - ref) < 3e-4 * max(1.0, abs(ref)), (world, plan, ours, ref)
