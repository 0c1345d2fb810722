"""Checkpoint save / load in the reference's on-disk layouts.

* "h2g" input format: a HuggingFace checkpoint split into one ``.pt`` per block, independent of the plan
  (``model_embed_tokens.pt``, ``model_layers_{i}.pt``, ``model_norm.pt``, ``lm_head.pt`` for Llama; reference
  tools/checkpoint_convert_h2g.py:43-82 and models/llama_hf/LlamaModel_checkpoint.py:47-144 for the slicing rules).
* distributed format (reference LlamaModel_checkpoint.py:155-219)::

      {save}/hybrid_parallel_configs.json
      {save}/iter_{N}/opt_param_scheduler.json
      {save}/iter_{N}/{block_name}/{tp_rank}.pt        # full (un-ZeRO-sharded) weights of that block's TP shard
      {save}/iter_{N}/optimizer/{global_rank}.pt

  For the Llama family the tensor keys and the fused-QKV packing are the reference's (Megatron's group-interleaved
  ``[groups, (q_per_group + 2) * head_dim, hidden]`` order, gate|up concatenation), so its conversion tools read
  files written here and vice versa; the other families store this package's parameter names.
Resume asserts that the stored plan equals the running one (hybrid_parallel_config.py:112-124).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist


# ------------------------------------------------------------------ QKV packing
def qkv_local_to_megatron(w: torch.Tensor, hq: int, hk: int, dh: int) -> torch.Tensor:
    """[q_heads | k_heads | v_heads] rows (this package) -> Megatron's per-group interleaved rows."""
    h = w.shape[1]
    q = w[: hq * dh].reshape(hk, hq // hk * dh, h)
    k = w[hq * dh:(hq + hk) * dh].reshape(hk, dh, h)
    v = w[(hq + hk) * dh:].reshape(hk, dh, h)
    return torch.cat([q, k, v], dim=1).reshape(-1, h)


def qkv_megatron_to_local(w: torch.Tensor, hq: int, hk: int, dh: int) -> torch.Tensor:
    h = w.shape[1]
    g = w.reshape(hk, (hq // hk + 2) * dh, h)
    qn = hq // hk * dh
    return torch.cat([g[:, :qn].reshape(-1, h), g[:, qn:qn + dh].reshape(-1, h), g[:, qn + dh:].reshape(-1, h)], dim=0)


# ------------------------------------------------------------------ per-block state dicts
def _llama_block_state(module, kind: str, cfg, st) -> Dict[str, torch.Tensor]:
    t = st.weight_tp
    if kind == "embed":
        return {"embed_tokens.weight": module.embed.wte.data}
    if kind == "norm":
        return {"norm.weight": module.norm.norm.weight.data}
    if kind == "cls":
        return {"lm_head.weight": module.head.weight.data}
    lay = module.layer
    hq, hk, dh = cfg.num_heads // t, cfg.num_kv_heads // t, cfg.head_dim
    return {
        "attention.LayerNorm.weight": lay.ln1.weight.data,
        "attention.attention.query_key_value.weight": qkv_local_to_megatron(lay.attn.wqkv.data, hq, hk, dh),
        "attention.attention.dense.weight": lay.attn.wo.data,
        "mlp.LayerNorm.weight": lay.ln2.weight.data,
        "mlp.mlp.dense_h_to_4h.weight": lay.mlp.w_up.data,
        "mlp.mlp.dense_4h_to_h.weight": lay.mlp.w_down.data,
    }


def _llama_load_block_state(module, kind: str, cfg, st, sd: Dict[str, torch.Tensor]) -> None:
    t = st.weight_tp

    def put(p, w):
        p.data.copy_(w.to(device=p.device, dtype=p.dtype))

    if kind == "embed":
        put(module.embed.wte, sd["embed_tokens.weight"])
    elif kind == "norm":
        put(module.norm.norm.weight, sd["norm.weight"])
    elif kind == "cls":
        put(module.head.weight, sd["lm_head.weight"])
    else:
        lay = module.layer
        hq, hk, dh = cfg.num_heads // t, cfg.num_kv_heads // t, cfg.head_dim
        put(lay.ln1.weight, sd["attention.LayerNorm.weight"])
        put(lay.attn.wqkv, qkv_megatron_to_local(sd["attention.attention.query_key_value.weight"], hq, hk, dh))
        put(lay.attn.wo, sd["attention.attention.dense.weight"])
        put(lay.ln2.weight, sd["mlp.LayerNorm.weight"])
        put(lay.mlp.w_up, sd["mlp.mlp.dense_h_to_4h.weight"])
        put(lay.mlp.w_down, sd["mlp.mlp.dense_4h_to_h.weight"])


def _llama_load_hf_block(module, kind: str, cfg, st, sd: Dict[str, torch.Tensor]) -> None:
    """One block of the plan-independent HF split: slice this rank's TP shard out of the full tensors."""
    t, r = st.weight_tp, (st.tp_rank if st.weight_tp > 1 else 0)

    def put(p, w):
        p.data.copy_(w.to(device=p.device, dtype=p.dtype))

    def rows(w):
        n = w.shape[0] // t
        return w[r * n:(r + 1) * n]

    def cols(w):
        n = w.shape[1] // t
        return w[:, r * n:(r + 1) * n]

    def vocab(w):
        pad = cfg.padded_vocab_size - w.shape[0]
        if pad:
            w = torch.cat([w, torch.zeros(pad, w.shape[1], dtype=w.dtype)], 0)
        return rows(w)

    if kind == "embed":
        put(module.embed.wte, vocab(sd["embed_tokens.weight"]))
    elif kind == "norm":
        put(module.norm.norm.weight, sd["weight"])
    elif kind == "cls":
        put(module.head.weight, vocab(sd["weight"]))
    else:
        lay = module.layer
        put(lay.ln1.weight, sd["input_layernorm.weight"])
        put(lay.attn.wqkv, torch.cat([rows(sd["self_attn.q_proj.weight"]), rows(sd["self_attn.k_proj.weight"]),
                                      rows(sd["self_attn.v_proj.weight"])], 0))
        put(lay.attn.wo, cols(sd["self_attn.o_proj.weight"]))
        put(lay.ln2.weight, sd["post_attention_layernorm.weight"])
        put(lay.mlp.w_up, torch.cat([rows(sd["mlp.gate_proj.weight"]), rows(sd["mlp.up_proj.weight"])], 0))
        put(lay.mlp.w_down, cols(sd["mlp.down_proj.weight"]))


def _gpt_load_hf_block(module, kind: str, cfg, st, sd: Dict[str, torch.Tensor]) -> None:
    """One block of a split HuggingFace GPT-2 checkpoint (``transformer_embedding.pt``, ``transformer_h_{i}.pt``,
    ``transformer_ln_f.pt``; reference models/gpt_hf/GPTModel_checkpoint.py:11-14). GPT-2 stores its linears as Conv1D,
    i.e. [in, out]: they are transposed to [out, in]; the fused ``c_attn`` is split into q | k | v before each is
    sliced for this tensor-parallel rank."""
    t, r = st.weight_tp, (st.tp_rank if st.weight_tp > 1 else 0)

    def put(p, w):
        p.data.copy_(w.to(device=p.device, dtype=p.dtype))

    def rows(w):
        n = w.shape[0] // t
        return w[r * n:(r + 1) * n]

    def cols(w):
        n = w.shape[1] // t
        return w[:, r * n:(r + 1) * n]

    def vocab(w):
        pad = cfg.padded_vocab_size - w.shape[0]
        if pad:
            w = torch.cat([w, torch.zeros(pad, w.shape[1], dtype=w.dtype)], 0)
        return rows(w)

    if kind == "embed":
        put(module.embed.wte, vocab(sd["wte.weight"]))
        put(module.embed.wpe, sd["wpe.weight"][: module.embed.wpe.shape[0]])
    elif kind == "norm":
        put(module.norm.norm.weight, sd["weight"])
        put(module.norm.norm.bias, sd["bias"])
    elif kind == "cls":
        if "lm_head.weight" in sd and not cfg.tie_embeddings:
            put(module.head.weight, vocab(sd["lm_head.weight"]))
    else:
        lay = module.layer
        h = cfg.hidden_size
        put(lay.ln1.weight, sd["ln_1.weight"]); put(lay.ln1.bias, sd["ln_1.bias"])
        put(lay.ln2.weight, sd["ln_2.weight"]); put(lay.ln2.bias, sd["ln_2.bias"])
        w_attn = sd["attn.c_attn.weight"].t()                       # [3h, h]
        b_attn = sd["attn.c_attn.bias"]
        put(lay.attn.wqkv, torch.cat([rows(w_attn[i * h:(i + 1) * h]) for i in range(3)], 0))
        put(lay.attn.bqkv, torch.cat([rows(b_attn[i * h:(i + 1) * h].unsqueeze(1)).squeeze(1) for i in range(3)], 0))
        put(lay.attn.wo, cols(sd["attn.c_proj.weight"].t()))
        put(lay.attn.bo, sd["attn.c_proj.bias"])
        put(lay.mlp.w_up, rows(sd["mlp.c_fc.weight"].t()))
        put(lay.mlp.b_up, rows(sd["mlp.c_fc.bias"].unsqueeze(1)).squeeze(1))
        put(lay.mlp.w_down, cols(sd["mlp.c_proj.weight"].t()))
        put(lay.mlp.b_down, sd["mlp.c_proj.bias"])


def _bert_load_hf_block(module, kind: str, cfg, st, sd: Dict[str, torch.Tensor]) -> None:
    """One block of a split HuggingFace BertForMaskedLM checkpoint (``bert_embeddings.pt``, ``bert_encoder_layer_{i}.pt``,
    ``cls_predictions.pt``; reference models/bert_hf/BertModel_checkpoint.py:9-12). The decoder is tied to the word
    embedding; HuggingFace's separate decoder bias has no counterpart here and must be zero (it is at initialisation)."""
    t, r = st.weight_tp, (st.tp_rank if st.weight_tp > 1 else 0)

    def put(p, w):
        p.data.copy_(w.to(device=p.device, dtype=p.dtype))

    def rows(w):
        n = w.shape[0] // t
        return w[r * n:(r + 1) * n]

    def cols(w):
        n = w.shape[1] // t
        return w[:, r * n:(r + 1) * n]

    def vocab(w):
        pad = cfg.padded_vocab_size - w.shape[0]
        if pad:
            w = torch.cat([w, torch.zeros(pad, w.shape[1], dtype=w.dtype)], 0)
        return rows(w)

    if kind == "embed":
        e = module.embed
        put(e.wte, vocab(sd["word_embeddings.weight"]))
        put(e.wpe, sd["position_embeddings.weight"][: e.wpe.shape[0]])
        put(e.wtt, sd["token_type_embeddings.weight"])
        put(e.ln.weight, sd["LayerNorm.weight"]); put(e.ln.bias, sd["LayerNorm.bias"])
    elif kind == "cls":
        put(module.dense, sd["transform.dense.weight"]); put(module.dense_bias, sd["transform.dense.bias"])
        put(module.ln.weight, sd["transform.LayerNorm.weight"]); put(module.ln.bias, sd["transform.LayerNorm.bias"])
    else:
        lay = module.layer
        put(lay.attn.wqkv, torch.cat([rows(sd["attention.self.%s.weight" % n]) for n in ("query", "key", "value")], 0))
        put(lay.attn.bqkv, torch.cat([rows(sd["attention.self.%s.bias" % n].unsqueeze(1)).squeeze(1) for n in ("query", "key", "value")], 0))
        put(lay.attn.wo, cols(sd["attention.output.dense.weight"])); put(lay.attn.bo, sd["attention.output.dense.bias"])
        put(lay.ln1.weight, sd["attention.output.LayerNorm.weight"]); put(lay.ln1.bias, sd["attention.output.LayerNorm.bias"])
        put(lay.mlp.w_up, rows(sd["intermediate.dense.weight"]))
        put(lay.mlp.b_up, rows(sd["intermediate.dense.bias"].unsqueeze(1)).squeeze(1))
        put(lay.mlp.w_down, cols(sd["output.dense.weight"])); put(lay.mlp.b_down, sd["output.dense.bias"])
        put(lay.ln2.weight, sd["output.LayerNorm.weight"]); put(lay.ln2.bias, sd["output.LayerNorm.bias"])


def _vit_load_hf_block(module, kind: str, cfg, st, sd: Dict[str, torch.Tensor]) -> None:
    """One block of a split HuggingFace ViT checkpoint (``vit_embeddings.pt``, ``vit_encoder_layer_{i}.pt``,
    ``vit_layernorm.pt``, ``classifier.pt`` holding the classifier and, when the source model has one, the pooler;
    reference models/vit_hf/ViTModel_checkpoint.py). The patch projection is the convolution weight flattened over
    (channel, row, column), which is the order the patch GEMM reads its pixels in."""
    t, r = st.weight_tp, (st.tp_rank if st.weight_tp > 1 else 0)

    def put(p, w):
        p.data.copy_(w.to(device=p.device, dtype=p.dtype))

    def rows(w):
        n = w.shape[0] // t
        return w[r * n:(r + 1) * n]

    def cols(w):
        n = w.shape[1] // t
        return w[:, r * n:(r + 1) * n]

    if kind == "embed":
        w = sd["patch_embeddings.projection.weight"].reshape(cfg.hidden_size, -1)
        module.w_patch.data.zero_()
        module.w_patch.data[:, : w.shape[1]].copy_(w.to(device=module.w_patch.device, dtype=module.w_patch.dtype))
        put(module.b_patch, sd["patch_embeddings.projection.bias"])
        put(module.cls_token, sd["cls_token"].reshape(1, -1))
        put(module.pos, sd["position_embeddings"].reshape(-1, cfg.hidden_size))
    elif kind == "norm":
        put(module.norm.norm.weight, sd["weight"]); put(module.norm.norm.bias, sd["bias"])
    elif kind == "cls":
        put(module.w_cls, rows(sd["weight"]))
        if "bias" in sd:
            assert float(sd["bias"].abs().max()) == 0.0, "the classifier of this package has no bias"
        if "pooler.dense.weight" in sd:
            put(module.w_pool, sd["pooler.dense.weight"]); put(module.b_pool, sd["pooler.dense.bias"])
    else:
        lay = module.layer
        put(lay.attn.wqkv, torch.cat([rows(sd["attention.attention.%s.weight" % n]) for n in ("query", "key", "value")], 0))
        put(lay.attn.bqkv, torch.cat([rows(sd["attention.attention.%s.bias" % n].unsqueeze(1)).squeeze(1) for n in ("query", "key", "value")], 0))
        put(lay.attn.wo, cols(sd["attention.output.dense.weight"])); put(lay.attn.bo, sd["attention.output.dense.bias"])
        put(lay.ln1.weight, sd["layernorm_before.weight"]); put(lay.ln1.bias, sd["layernorm_before.bias"])
        put(lay.mlp.w_up, rows(sd["intermediate.dense.weight"]))
        put(lay.mlp.b_up, rows(sd["intermediate.dense.bias"].unsqueeze(1)).squeeze(1))
        put(lay.mlp.w_down, cols(sd["output.dense.weight"])); put(lay.mlp.b_down, sd["output.dense.bias"])
        put(lay.ln2.weight, sd["layernorm_after.weight"]); put(lay.ln2.bias, sd["layernorm_after.bias"])


def _swin_load_hf_block(module, kind: str, cfg, st, sd: Dict[str, torch.Tensor], downsample: Optional[Dict[str, torch.Tensor]]) -> None:
    """One block of a split HuggingFace Swin checkpoint (``swin_embeddings.pt``, ``swin_encoder_{stage}_{block}.pt``,
    ``swin_encoder_{stage}_downsample.pt`` for the patch merging that ends a stage, ``swin_classifier.pt`` holding the
    final LayerNorm and the classifier). The relative-position table is sharded by heads like the projections; the
    2x2 merging concatenates (even row, even col), (odd row, even col), (even row, odd col), (odd row, odd col), the
    order this package's merging uses as well."""
    t, r = st.weight_tp, (st.tp_rank if st.weight_tp > 1 else 0)

    def put(p, w):
        p.data.copy_(w.to(device=p.device, dtype=p.dtype))

    def rows(w):
        n = w.shape[0] // t
        return w[r * n:(r + 1) * n]

    def cols(w):
        n = w.shape[1] // t
        return w[:, r * n:(r + 1) * n]

    if kind == "embed":
        w = sd["patch_embeddings.projection.weight"].reshape(cfg.embed_dim, -1)
        module.w_patch.data.zero_()
        module.w_patch.data[:, : w.shape[1]].copy_(w.to(device=module.w_patch.device, dtype=module.w_patch.dtype))
        put(module.b_patch, sd["patch_embeddings.projection.bias"])
        put(module.ln.weight, sd["norm.weight"]); put(module.ln.bias, sd["norm.bias"])
    elif kind == "cls":
        put(module.ln.weight, sd["layernorm.weight"]); put(module.ln.bias, sd["layernorm.bias"])
        put(module.w_cls, rows(sd["weight"]))
        if "bias" in sd:
            assert float(sd["bias"].abs().max()) == 0.0, "the classifier of this package has no bias"
    else:
        put(module.ln1.weight, sd["layernorm_before.weight"]); put(module.ln1.bias, sd["layernorm_before.bias"])
        put(module.wqkv, torch.cat([rows(sd["attention.self.%s.weight" % n]) for n in ("query", "key", "value")], 0))
        put(module.bqkv, torch.cat([rows(sd["attention.self.%s.bias" % n].unsqueeze(1)).squeeze(1) for n in ("query", "key", "value")], 0))
        put(module.rel_table, cols(sd["attention.self.relative_position_bias_table"]))
        put(module.wo, cols(sd["attention.output.dense.weight"])); put(module.bo, sd["attention.output.dense.bias"])
        put(module.ln2.weight, sd["layernorm_after.weight"]); put(module.ln2.bias, sd["layernorm_after.bias"])
        put(module.w1, rows(sd["intermediate.dense.weight"]))
        put(module.b1, rows(sd["intermediate.dense.bias"].unsqueeze(1)).squeeze(1))
        put(module.w2, cols(sd["output.dense.weight"])); put(module.b2, sd["output.dense.bias"])
        if module.merge:
            assert downsample is not None, "the last block of a stage needs the stage's downsample file"
            put(module.ln_merge.weight, downsample["norm.weight"]); put(module.ln_merge.bias, downsample["norm.bias"])
            put(module.w_merge, downsample["reduction.weight"])


def _t5_load_hf_block(module, name: str, cfg, st, load: str) -> None:
    """One block of a split HuggingFace T5ForConditionalGeneration checkpoint (``shared.pt``, ``encoder_block_{i}.pt``,
    ``decoder_block_{j}.pt``, ``encoder_final_layer_norm.pt``, ``decoder_final_layer_norm.pt``), for a model built with the
    relative position bias (``relative_attention_num_buckets > 0``), the relu feed-forward and tied embeddings.

    Three conventions of that implementation are folded into the weights, so that the blocks stay the generic ones:
    its attention does not scale the scores (the query projection is multiplied by sqrt(head_dim) here, which the kernels'
    1 / sqrt(head_dim) undoes); with tied embeddings it multiplies the decoder output by d_model^-0.5 before the head (the
    final decoder norm's weight carries that factor here); and one bias table per stack, held by block 0, serves every
    block (each block here owns a table and starts from a copy, so the tables are free to drift apart in training)."""
    t, r = st.weight_tp, (st.tp_rank if st.weight_tp > 1 else 0)
    dh = cfg.head_dim

    def read(stem):
        return torch.load(os.path.join(load, stem + ".pt"), map_location="cpu")

    def put(p, w):
        assert p.shape == w.shape, "%s: checkpoint tensor %s does not fit parameter %s" % (name, tuple(w.shape), tuple(p.shape))
        p.data.copy_(w.to(device=p.device, dtype=p.dtype))

    def rows(w):
        n = w.shape[0] // t
        return w[r * n:(r + 1) * n]

    def cols(w):
        n = w.shape[1] // t
        return w[:, r * n:(r + 1) * n]

    def vocab(w):
        pad = cfg.padded_vocab_size - w.shape[0]
        if pad:
            w = torch.cat([w, torch.zeros(pad, w.shape[1], dtype=w.dtype)], 0)
        return rows(w)

    def attention(att, sd, prefix, scaled_q=True):
        q = sd[prefix + ".q.weight"].float() * (math.sqrt(dh) if scaled_q else 1.0)
        assert q.shape[0] == cfg.num_heads * dh, "d_kv * num_heads must equal d_model for this model definition"
        put(att.wqkv, torch.cat([rows(q), rows(sd[prefix + ".k.weight"].float()), rows(sd[prefix + ".v.weight"].float())], 0))
        put(att.wo, cols(sd[prefix + ".o.weight"]))

    if name in ("shared_embedding", "decoder_embedding", "lm_head"):
        w = vocab(read("shared")["weight"])
        target = {"shared_embedding": lambda: module.embed.wte, "decoder_embedding": lambda: module.inner.embed.wte,
                  "lm_head": lambda: module.head.weight}[name]()
        put(target, w)
    elif name == "encoder_final_layer_norm":
        put(module.norm.norm.weight, read(name)["weight"])
    elif name == "decoder_final_layer_norm":
        put(module.norm.norm.weight, read(name)["weight"].float() * cfg.hidden_size ** -0.5)
    else:
        stack, index = name.split("_block_")
        sd = read(name)
        first = sd if index == "0" else read(stack + "_block_0")
        lay = module.layer
        attention(lay.attn, sd, "layer.0.SelfAttention")
        table = first["layer.0.SelfAttention.relative_attention_bias.weight"]          # [buckets, heads]
        n = table.shape[1] // t
        put(lay.attn.rel_bias, table[:, r * n:(r + 1) * n])
        put(lay.ln1.weight, sd["layer.0.layer_norm.weight"])
        ff = 1
        if lay.xattn is not None:
            attention(lay.xattn, sd, "layer.1.EncDecAttention")
            put(lay.ln_x.weight, sd["layer.1.layer_norm.weight"])
            ff = 2
        put(lay.mlp.w_up, rows(sd["layer.%d.DenseReluDense.wi.weight" % ff]))
        put(lay.mlp.w_down, cols(sd["layer.%d.DenseReluDense.wo.weight" % ff]))
        put(lay.ln2.weight, sd["layer.%d.layer_norm.weight" % ff])


def _is_gpt(family: str) -> bool:
    return family in ("gpt", "gpt_hf", "gpt_fa")


def _generic_block_state(module) -> Dict[str, torch.Tensor]:
    return {k: p.data for k, p in module.named_parameters()}


def _generic_load_block_state(module, sd) -> None:
    own = dict(module.named_parameters())
    for k, w in sd.items():
        if k in own:
            own[k].data.copy_(w.to(device=own[k].device, dtype=own[k].dtype))


def _is_llama(family: str) -> bool:
    return family in ("llama", "llama_hf", "llama_fa", "qwen")


# ------------------------------------------------------------------ public API
PLAN_KEYS_OF_THE_FILE_LAYOUT = ("tp_sizes_enc", "use_sp", "vocab_tp", "vocab_sp")


def _portable_optimizer_state(block) -> Dict[str, Dict[str, torch.Tensor]]:
    """Optimizer state of a block's own bucket, per parameter name and unsharded (collective over the bucket's group)."""
    bucket = block.bucket
    if bucket.numel == 0:
        return {}
    names = {id(p): n for n, p in block.module.named_parameters()}
    full = bucket.full_optimizer_state()
    out = {}
    for p, off in zip(bucket.params, bucket.offsets):
        if id(p) in names:
            out[names[id(p)]] = {k: v[off:off + p._gv_numel].clone().view(p._gv_shape) for k, v in full.items()}
    return out


def _load_portable_optimizer_state(block, state: Dict[str, Dict[str, torch.Tensor]]) -> None:
    bucket = block.bucket
    if bucket.numel == 0 or not state:
        return
    names = {id(p): n for n, p in block.module.named_parameters()}
    full = {k: torch.zeros(bucket.numel, dtype=torch.float32) for k in ("master", "exp_avg", "exp_avg_sq")}
    for p, off in zip(bucket.params, bucket.offsets):
        entry = state.get(names.get(id(p)))
        assert entry is not None, "no optimizer state stored for parameter %s" % names.get(id(p))
        for k in full:
            full[k][off:off + p._gv_numel].copy_(entry[k].reshape(-1))
    bucket.load_full_optimizer_state(full)


def save_model(model, save: str, family: str, iteration: int, optimizer=None, portable_optimizer: bool = False) -> None:
    """Write the distributed checkpoint of ``model`` (a GalvatronModel) for ``iteration``.

    ``portable_optimizer``: besides the per-rank optimizer shards (which only the same plan can read back), store the
    fp32 master weights and Adam moments per block, tensor-parallel rank and parameter name
    (``iter_N/{block}/{tp_rank}.optim.pt``), so that a run with another pipeline / data-parallel / ZeRO layout (same
    tensor-parallel degrees) can resume from it."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    it_dir = os.path.join(save, "iter_%d" % iteration)
    if rank == 0:
        os.makedirs(it_dir, exist_ok=True)
        json.dump(model.plan.as_runtime_dict(), open(os.path.join(save, "hybrid_parallel_configs.json"), "w"))
        if optimizer is not None:
            sched = dict(optimizer.scheduler.state_dict())
            if getattr(optimizer, "scaler", None) is not None:
                sched["loss_scaler"] = optimizer.scaler.state_dict()
            json.dump(sched, open(os.path.join(it_dir, "opt_param_scheduler.json"), "w"))
    if dist.is_initialized():
        dist.barrier()
    for spec, block, st in zip(model.my_specs, model.model.blocks, model.strategies):
        for b in block.all_buckets:
            b.unshard()
        wdp_rank = st.wdp_group.rank_in_group(rank) if (st.wdp_group is not None and st.wdp_group.size > 1) else 0
        if wdp_rank == 0:
            sd = _llama_block_state(block.module, spec.kind, model.cfg, st) if _is_llama(family) else _generic_block_state(block.module)
            d = os.path.join(it_dir, spec.name)
            os.makedirs(d, exist_ok=True)
            tp_rank = st.tp_rank if st.weight_tp > 1 else 0
            torch.save({k: v.detach().float().cpu() for k, v in sd.items()}, os.path.join(d, "%d.pt" % tp_rank))
        if portable_optimizer:
            state = _portable_optimizer_state(block)            # collective: every rank of the bucket's group takes part
            if wdp_rank == 0:
                d = os.path.join(it_dir, spec.name)
                os.makedirs(d, exist_ok=True)
                torch.save(state, os.path.join(d, "%d.optim.pt" % (st.tp_rank if st.weight_tp > 1 else 0)))
        for b in block.all_buckets:
            b.reshard()
    os.makedirs(os.path.join(it_dir, "optimizer"), exist_ok=True)
    torch.save(model.engine.state_dict(), os.path.join(it_dir, "optimizer", "%d.pt" % rank))
    if portable_optimizer and rank == 0:
        json.dump({"step": model.engine.step_count}, open(os.path.join(it_dir, "optimizer_step.json"), "w"))
    if dist.is_initialized():
        dist.barrier()


def load_model(model, load: str, family: str, iteration: Optional[int] = None, allow_plan_change: bool = False) -> None:
    """``iteration`` None: plan-independent HF split ("h2g" files); otherwise the distributed checkpoint of that
    iteration, after checking that the stored plan equals the running one.

    ``allow_plan_change``: only the keys that decide the file layout (tensor-parallel degrees per layer and of the
    vocabulary) must match; pipeline / data-parallel degree, ZeRO type, checkpointing and micro-batching may differ,
    and the optimizer state is read from the portable per-block files (``save_model(..., portable_optimizer=True)``)."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    if iteration is None and family == "t5" and not getattr(getattr(model, "cfg", None), "relative_attention_num_buckets", 0):
        # as in the reference (models/T5/T5Model_checkpoint.py:30-32): without the relative position bias the weights of a
        # HuggingFace T5 do not describe the model; its own distributed checkpoints load like any family's
        raise NotImplementedError("loading HuggingFace weights needs the t5 model built with the relative position bias "
                                  "(--relative_attention_num_buckets 32 --t5_feed_forward relu); without it, resume from a "
                                  "distributed checkpoint with --load_iteration")
    if iteration is not None:
        stored = json.load(open(os.path.join(load, "hybrid_parallel_configs.json")))
        mine = json.loads(json.dumps(model.plan.as_runtime_dict()))
        assert stored.keys() == mine.keys(), "Hybrid parallel configs are not equal, %s vs %s" % (stored.keys(), mine.keys())
        for k in (PLAN_KEYS_OF_THE_FILE_LAYOUT if allow_plan_change else mine):
            assert stored[k] == mine[k], f"Hybrid parallel configs are not equal for key {k}, {mine[k]} vs {stored[k]}"
    for spec, block, st in zip(model.my_specs, model.model.blocks, model.strategies):
        for b in block.all_buckets:
            b.unshard()
        tp_rank = st.tp_rank if st.weight_tp > 1 else 0
        if iteration is not None:
            sd = torch.load(os.path.join(load, "iter_%d" % iteration, spec.name, "%d.pt" % tp_rank), map_location="cpu")
            if _is_llama(family):
                _llama_load_block_state(block.module, spec.kind, model.cfg, st, sd)
            else:
                _generic_load_block_state(block.module, sd)
        else:
            if family == "t5":
                _t5_load_hf_block(block.module, spec.name, model.cfg, st, load)
                for b in block.all_buckets:
                    b.commit_loaded_params()
                for b in block.all_buckets:
                    b.reshard()
                continue
            path = os.path.join(load, spec.name + ".pt")
            if not os.path.exists(path) and spec.kind == "cls":
                path = os.path.join(load, model.my_specs[0].name + ".pt") if _is_gpt(family) else path
            sd = torch.load(path, map_location="cpu") if os.path.exists(path) else {}
            if _is_llama(family):
                _llama_load_hf_block(block.module, spec.kind, model.cfg, st, sd)
            elif _is_gpt(family):
                _gpt_load_hf_block(block.module, spec.kind, model.cfg, st, sd)
            elif family in ("bert", "bert_hf"):
                _bert_load_hf_block(block.module, spec.kind, model.cfg, st, sd)
            elif family in ("vit", "vit_hf"):
                _vit_load_hf_block(block.module, spec.kind, model.cfg, st, sd)
            elif family == "swin":
                extra = None
                if getattr(block.module, "merge", False):
                    stage = spec.name.split("_")[2]
                    extra = torch.load(os.path.join(load, "swin_encoder_%s_downsample.pt" % stage), map_location="cpu")
                _swin_load_hf_block(block.module, spec.kind, model.cfg, st, sd, extra)
            else:
                _generic_load_block_state(block.module, sd)
        for b in block.all_buckets:
            b.commit_loaded_params()
        if iteration is not None and allow_plan_change:
            path = os.path.join(load, "iter_%d" % iteration, spec.name, "%d.optim.pt" % tp_rank)
            assert os.path.exists(path), "resuming under another plan needs a checkpoint saved with portable_optimizer=True"
            _load_portable_optimizer_state(block, torch.load(path, map_location="cpu"))
        for b in block.all_buckets:
            b.reshard()
    if iteration is not None and allow_plan_change:
        step_file = os.path.join(load, "iter_%d" % iteration, "optimizer_step.json")
        model.engine.step_count = json.load(open(step_file))["step"]
    elif iteration is not None:
        opt = os.path.join(load, "iter_%d" % iteration, "optimizer", "%d.pt" % rank)
        if os.path.exists(opt):
            model.engine.load_state_dict(torch.load(opt, map_location=model.device))
