"""Distributed checkpoint (``iter_N/{block}/{tp_rank}.pt``) -> HuggingFace state dict.

Counterpart of the reference's galvatron/tools/checkpoint_convert_g2h.py (:11-109 llama, :111-251 bert; its gpt
branch is a stub, here GPT-2 and ViT are converted too): concatenates
the tensor-parallel shards of every block, undoes the grouped QKV packing and the gate|up concatenation (llama) or
splits the fused QKV rows back into query / key / value (bert), trims the vocab padding, and writes
``pytorch_model.bin`` plus ``config.json`` (through the ``transformers`` config class when importable, else the raw
meta config). No model object is instantiated, so a 70B checkpoint converts within host memory of its own size.

    python -m hetu_galvatron_b200.tools.checkpoint_convert_g2h --model_type llama --load_iteration 100 \
        --input_checkpoint <dir> --output_dir <hf dir> --model_config <meta json>
"""
from __future__ import annotations

import argparse
import json
import math
import os
from typing import Dict, List

import torch

from ..core.checkpoint import qkv_megatron_to_local


def _shards(block_dir: str) -> List[Dict[str, torch.Tensor]]:
    assert os.path.isdir(block_dir), "block directory %s does not exist" % block_dir
    files = sorted((f for f in os.listdir(block_dir) if f.endswith(".pt")), key=lambda f: int(f.split(".")[0]))
    return [torch.load(os.path.join(block_dir, f), map_location="cpu", weights_only=True) for f in files]


def assemble_llama(iter_dir: str, meta: dict) -> Dict[str, torch.Tensor]:
    h, nh = meta["dim"], meta["n_heads"]
    nkv, L, vocab = meta.get("n_kv_heads", nh), meta["n_layers"], meta["vocab_size"]
    dh = h // nh
    out: Dict[str, torch.Tensor] = {}
    emb = torch.cat([s["embed_tokens.weight"] for s in _shards(os.path.join(iter_dir, "model_embed_tokens"))], 0)
    out["model.embed_tokens.weight"] = emb[:vocab].contiguous()
    for i in range(L):
        sh = _shards(os.path.join(iter_dir, "model_layers_%d" % i))
        t = len(sh)
        q, k, v, gate, up = [], [], [], [], []
        for s in sh:
            loc = qkv_megatron_to_local(s["attention.attention.query_key_value.weight"], nh // t, nkv // t, dh)
            q.append(loc[: nh // t * dh])
            k.append(loc[nh // t * dh:(nh + nkv) // t * dh])
            v.append(loc[(nh + nkv) // t * dh:])
            w = s["mlp.mlp.dense_h_to_4h.weight"]
            gate.append(w[: w.shape[0] // 2])
            up.append(w[w.shape[0] // 2:])
        p = "model.layers.%d." % i
        out[p + "self_attn.q_proj.weight"] = torch.cat(q, 0).contiguous()
        out[p + "self_attn.k_proj.weight"] = torch.cat(k, 0).contiguous()
        out[p + "self_attn.v_proj.weight"] = torch.cat(v, 0).contiguous()
        out[p + "self_attn.o_proj.weight"] = torch.cat([s["attention.attention.dense.weight"] for s in sh], 1).contiguous()
        out[p + "mlp.gate_proj.weight"] = torch.cat(gate, 0).contiguous()
        out[p + "mlp.up_proj.weight"] = torch.cat(up, 0).contiguous()
        out[p + "mlp.down_proj.weight"] = torch.cat([s["mlp.mlp.dense_4h_to_h.weight"] for s in sh], 1).contiguous()
        out[p + "input_layernorm.weight"] = sh[0]["attention.LayerNorm.weight"]
        out[p + "post_attention_layernorm.weight"] = sh[0]["mlp.LayerNorm.weight"]
    out["model.norm.weight"] = _shards(os.path.join(iter_dir, "model_norm"))[0]["norm.weight"]
    head = torch.cat([s["lm_head.weight"] for s in _shards(os.path.join(iter_dir, "lm_head"))], 0)
    out["lm_head.weight"] = head[:vocab].contiguous()
    return out


def assemble_bert(iter_dir: str, meta: dict) -> Dict[str, torch.Tensor]:
    """BertForMaskedLM state dict from the per-block shards (blocks ``bert_embeddings``, ``bert_encoder_layer_{i}``,
    ``cls_predictions``). Fused QKV rows are stored per rank as [q | k | v] of that rank's heads."""
    L, vocab = meta["num_hidden_layers"], meta["vocab_size"]
    out: Dict[str, torch.Tensor] = {}
    sh = _shards(os.path.join(iter_dir, "bert_embeddings"))
    p = "bert.embeddings."
    out[p + "word_embeddings.weight"] = torch.cat([s["embed.wte"] for s in sh], 0)[:vocab].contiguous()
    out[p + "position_embeddings.weight"] = sh[0]["embed.wpe"]
    out[p + "token_type_embeddings.weight"] = sh[0]["embed.wtt"]
    out[p + "LayerNorm.weight"], out[p + "LayerNorm.bias"] = sh[0]["embed.ln.weight"], sh[0]["embed.ln.bias"]
    for i in range(L):
        sh = _shards(os.path.join(iter_dir, "bert_encoder_layer_%d" % i))
        p = "bert.encoder.layer.%d." % i
        for j, name in enumerate(("query", "key", "value")):
            out[p + "attention.self.%s.weight" % name] = torch.cat([s["layer.attn.wqkv"].chunk(3, 0)[j] for s in sh], 0).contiguous()
            out[p + "attention.self.%s.bias" % name] = torch.cat([s["layer.attn.bqkv"].chunk(3, 0)[j] for s in sh], 0).contiguous()
        out[p + "attention.output.dense.weight"] = torch.cat([s["layer.attn.wo"] for s in sh], 1).contiguous()
        out[p + "attention.output.dense.bias"] = sh[0]["layer.attn.bo"]
        out[p + "attention.output.LayerNorm.weight"], out[p + "attention.output.LayerNorm.bias"] = sh[0]["layer.ln1.weight"], sh[0]["layer.ln1.bias"]
        out[p + "intermediate.dense.weight"] = torch.cat([s["layer.mlp.w_up"] for s in sh], 0).contiguous()
        out[p + "intermediate.dense.bias"] = torch.cat([s["layer.mlp.b_up"] for s in sh], 0).contiguous()
        out[p + "output.dense.weight"] = torch.cat([s["layer.mlp.w_down"] for s in sh], 1).contiguous()
        out[p + "output.dense.bias"] = sh[0]["layer.mlp.b_down"]
        out[p + "output.LayerNorm.weight"], out[p + "output.LayerNorm.bias"] = sh[0]["layer.ln2.weight"], sh[0]["layer.ln2.bias"]
    sh = _shards(os.path.join(iter_dir, "cls_predictions"))
    p = "cls.predictions."
    out[p + "transform.dense.weight"], out[p + "transform.dense.bias"] = sh[0]["dense"], sh[0]["dense_bias"]
    out[p + "transform.LayerNorm.weight"], out[p + "transform.LayerNorm.bias"] = sh[0]["ln.weight"], sh[0]["ln.bias"]
    out[p + "decoder.weight"] = out["bert.embeddings.word_embeddings.weight"]        # tied
    out[p + "bias"] = torch.zeros(vocab)
    out[p + "decoder.bias"] = out[p + "bias"]
    return out


def assemble_gpt(iter_dir: str, meta: dict) -> Dict[str, torch.Tensor]:
    """GPT2LMHeadModel state dict from the per-block shards (blocks ``transformer_embedding``, ``transformer_h_{i}``,
    ``transformer_ln_f``). Every rank stores its fused QKV rows as [q | k | v] of its own heads; GPT-2 keeps linears as
    Conv1D ([in, out]), so every assembled matrix is transposed; the head is tied to the token embedding."""
    L, vocab = meta["n_layer"], meta["vocab_size"]
    out: Dict[str, torch.Tensor] = {}
    sh = _shards(os.path.join(iter_dir, "transformer_embedding"))
    out["transformer.wte.weight"] = torch.cat([s["embed.wte"] for s in sh], 0)[:vocab].contiguous()
    out["transformer.wpe.weight"] = sh[0]["embed.wpe"]
    for i in range(L):
        sh = _shards(os.path.join(iter_dir, "transformer_h_%d" % i))
        p = "transformer.h.%d." % i
        w = torch.cat([torch.cat([s["layer.attn.wqkv"].chunk(3, 0)[j] for s in sh], 0) for j in range(3)], 0)     # [3h, h]: q | k | v
        b = torch.cat([torch.cat([s["layer.attn.bqkv"].chunk(3, 0)[j] for s in sh], 0) for j in range(3)], 0)
        out[p + "attn.c_attn.weight"], out[p + "attn.c_attn.bias"] = w.t().contiguous(), b.contiguous()
        out[p + "attn.c_proj.weight"] = torch.cat([s["layer.attn.wo"] for s in sh], 1).t().contiguous()
        out[p + "attn.c_proj.bias"] = sh[0]["layer.attn.bo"]
        out[p + "mlp.c_fc.weight"] = torch.cat([s["layer.mlp.w_up"] for s in sh], 0).t().contiguous()
        out[p + "mlp.c_fc.bias"] = torch.cat([s["layer.mlp.b_up"] for s in sh], 0).contiguous()
        out[p + "mlp.c_proj.weight"] = torch.cat([s["layer.mlp.w_down"] for s in sh], 1).t().contiguous()
        out[p + "mlp.c_proj.bias"] = sh[0]["layer.mlp.b_down"]
        out[p + "ln_1.weight"], out[p + "ln_1.bias"] = sh[0]["layer.ln1.weight"], sh[0]["layer.ln1.bias"]
        out[p + "ln_2.weight"], out[p + "ln_2.bias"] = sh[0]["layer.ln2.weight"], sh[0]["layer.ln2.bias"]
    sh = _shards(os.path.join(iter_dir, "transformer_ln_f"))
    out["transformer.ln_f.weight"], out["transformer.ln_f.bias"] = sh[0]["norm.norm.weight"], sh[0]["norm.norm.bias"]
    out["lm_head.weight"] = out["transformer.wte.weight"]            # tied
    return out


def assemble_vit(iter_dir: str, meta: dict) -> Dict[str, torch.Tensor]:
    """ViT state dict in HuggingFace names (``vit.*`` + ``classifier.weight``; the pooler under ``vit.pooler.*``) from the
    per-block shards (blocks ``vit_embeddings``, ``vit_encoder_layer_{i}``, ``vit_layernorm``, ``classifier``). The patch
    projection is stored as the convolution weight flattened over (channel, row, column) and zero-padded to the GEMM's
    alignment; it is cut back and reshaped."""
    L, h = meta["num_hidden_layers"], meta["hidden_size"]
    c, ps = meta.get("num_channels", 3), meta["patch_size"]
    out: Dict[str, torch.Tensor] = {}
    e = _shards(os.path.join(iter_dir, "vit_embeddings"))[0]
    p = "vit.embeddings."
    out[p + "patch_embeddings.projection.weight"] = e["w_patch"][:, : c * ps * ps].reshape(h, c, ps, ps).contiguous()
    out[p + "patch_embeddings.projection.bias"] = e["b_patch"]
    out[p + "cls_token"] = e["cls_token"].reshape(1, 1, h)
    out[p + "position_embeddings"] = e["pos"].reshape(1, -1, h)
    for i in range(L):
        sh = _shards(os.path.join(iter_dir, "vit_encoder_layer_%d" % i))
        p = "vit.encoder.layer.%d." % i
        for j, name in enumerate(("query", "key", "value")):
            out[p + "attention.attention.%s.weight" % name] = torch.cat([s["layer.attn.wqkv"].chunk(3, 0)[j] for s in sh], 0).contiguous()
            out[p + "attention.attention.%s.bias" % name] = torch.cat([s["layer.attn.bqkv"].chunk(3, 0)[j] for s in sh], 0).contiguous()
        out[p + "attention.output.dense.weight"] = torch.cat([s["layer.attn.wo"] for s in sh], 1).contiguous()
        out[p + "attention.output.dense.bias"] = sh[0]["layer.attn.bo"]
        out[p + "layernorm_before.weight"], out[p + "layernorm_before.bias"] = sh[0]["layer.ln1.weight"], sh[0]["layer.ln1.bias"]
        out[p + "intermediate.dense.weight"] = torch.cat([s["layer.mlp.w_up"] for s in sh], 0).contiguous()
        out[p + "intermediate.dense.bias"] = torch.cat([s["layer.mlp.b_up"] for s in sh], 0).contiguous()
        out[p + "output.dense.weight"] = torch.cat([s["layer.mlp.w_down"] for s in sh], 1).contiguous()
        out[p + "output.dense.bias"] = sh[0]["layer.mlp.b_down"]
        out[p + "layernorm_after.weight"], out[p + "layernorm_after.bias"] = sh[0]["layer.ln2.weight"], sh[0]["layer.ln2.bias"]
    n = _shards(os.path.join(iter_dir, "vit_layernorm"))[0]
    out["vit.layernorm.weight"], out["vit.layernorm.bias"] = n["norm.norm.weight"], n["norm.norm.bias"]
    sh = _shards(os.path.join(iter_dir, "classifier"))
    out["classifier.weight"] = torch.cat([s["w_cls"] for s in sh], 0).contiguous()
    if "w_pool" in sh[0]:
        out["vit.pooler.dense.weight"], out["vit.pooler.dense.bias"] = sh[0]["w_pool"], sh[0]["b_pool"]
    return out


def assemble_t5(iter_dir: str, meta: dict) -> Dict[str, torch.Tensor]:
    """T5ForConditionalGeneration state dict from the per-block shards of a model built with the relative position bias
    (blocks ``shared_embedding``, ``encoder_block_{i}``, ``decoder_block_{j}``, ``encoder_final_layer_norm``,
    ``decoder_final_layer_norm``). Undoes what the loader folded in (query projection / sqrt(head_dim), final decoder norm
    x d_model^0.5). HuggingFace keeps ONE bias table per stack in block 0; here every block owns one, so the conversion
    is only defined while the tables of a stack still agree (as loaded, or trained with them frozen) and refuses
    otherwise."""
    d, heads = meta["d_model"], meta["num_heads"]
    dh = d // heads
    Le, Ld = meta["num_layers"], meta.get("num_decoder_layers", meta["num_layers"])
    out: Dict[str, torch.Tensor] = {}
    emb = torch.cat([s["embed.wte"] for s in _shards(os.path.join(iter_dir, "shared_embedding"))], 0)[: meta["vocab_size"]].contiguous()
    out["shared.weight"] = out["encoder.embed_tokens.weight"] = out["decoder.embed_tokens.weight"] = out["lm_head.weight"] = emb

    def attention(sh, key, prefix, scaled_q):
        for j, name in enumerate(("q", "k", "v")):
            w = torch.cat([s[key + ".wqkv"].chunk(3, 0)[j] for s in sh], 0).float()
            out[prefix + ".%s.weight" % name] = (w / math.sqrt(dh) if (j == 0 and scaled_q) else w).contiguous()
        out[prefix + ".o.weight"] = torch.cat([s[key + ".wo"] for s in sh], 1).contiguous()

    for stack, n in (("encoder", Le), ("decoder", Ld)):
        tables = []
        for i in range(n):
            sh = _shards(os.path.join(iter_dir, "%s_block_%d" % (stack, i)))
            p = "%s.block.%d." % (stack, i)
            attention(sh, "layer.attn", p + "layer.0.SelfAttention", True)
            tables.append(torch.cat([s["layer.attn.rel_bias"] for s in sh], 1).float())
            out[p + "layer.0.layer_norm.weight"] = sh[0]["layer.ln1.weight"]
            ff = 1
            if stack == "decoder":
                attention(sh, "layer.xattn", p + "layer.1.EncDecAttention", True)
                out[p + "layer.1.layer_norm.weight"] = sh[0]["layer.ln_x.weight"]
                ff = 2
            out[p + "layer.%d.DenseReluDense.wi.weight" % ff] = torch.cat([s["layer.mlp.w_up"] for s in sh], 0).contiguous()
            out[p + "layer.%d.DenseReluDense.wo.weight" % ff] = torch.cat([s["layer.mlp.w_down"] for s in sh], 1).contiguous()
            out[p + "layer.%d.layer_norm.weight" % ff] = sh[0]["layer.ln2.weight"]
        worst = max(float((t - tables[0]).abs().max()) for t in tables)
        if worst > 1e-3 * max(1.0, float(tables[0].abs().max())):
            raise ValueError("the relative position bias tables of the %s blocks differ (by up to %.3g): HuggingFace's T5 has one "
                             "table per stack, so this checkpoint has no HuggingFace form" % (stack, worst))
        out["%s.block.0.layer.0.SelfAttention.relative_attention_bias.weight" % stack] = tables[0].contiguous()
        norm = _shards(os.path.join(iter_dir, "%s_final_layer_norm" % stack))[0]["norm.norm.weight"].float()
        out["%s.final_layer_norm.weight" % stack] = norm * (d ** 0.5 if stack == "decoder" else 1.0)
    return out


def hf_t5_config(meta: dict, tensors: Dict[str, torch.Tensor]) -> dict:
    buckets = tensors["encoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight"].shape[0]
    cfg = dict(vocab_size=meta["vocab_size"], d_model=meta["d_model"], d_kv=meta["d_model"] // meta["num_heads"], d_ff=meta["d_ff"],
               num_layers=meta["num_layers"], num_decoder_layers=meta.get("num_decoder_layers", meta["num_layers"]),
               num_heads=meta["num_heads"], relative_attention_num_buckets=buckets,
               relative_attention_max_distance=meta.get("relative_attention_max_distance", 128),
               layer_norm_epsilon=meta.get("layer_norm_epsilon", 1e-6), feed_forward_proj="relu", tie_word_embeddings=True)
    try:
        from transformers import T5Config
        return T5Config(**cfg).to_dict()
    except Exception:
        return dict(cfg, architectures=["T5ForConditionalGeneration"], model_type="t5")


def hf_vit_config(meta: dict) -> dict:
    keys = ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size", "image_size", "patch_size",
            "num_channels", "layer_norm_eps", "hidden_act")
    cfg = {k: meta[k] for k in keys if k in meta}
    try:
        from transformers import ViTConfig
        return ViTConfig(**cfg).to_dict()
    except Exception:
        return dict(cfg, architectures=["ViTForImageClassification"], model_type="vit")


def hf_gpt_config(meta: dict) -> dict:
    cfg = dict(n_embd=meta["n_embd"], n_head=meta["n_head"], n_layer=meta["n_layer"], vocab_size=meta["vocab_size"],
               n_positions=meta.get("n_positions", 1024), n_inner=meta.get("n_inner"),
               layer_norm_epsilon=meta.get("layer_norm_epsilon", 1e-5), activation_function=meta.get("activation_function", "gelu_new"))
    try:
        from transformers import GPT2Config
        return GPT2Config(**cfg).to_dict()
    except Exception:
        return dict(cfg, architectures=["GPT2LMHeadModel"], model_type="gpt2")


def hf_bert_config(meta: dict) -> dict:
    keys = ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size", "vocab_size",
            "max_position_embeddings", "type_vocab_size", "layer_norm_eps", "hidden_act")
    cfg = {k: meta[k] for k in keys if k in meta}
    try:
        from transformers import BertConfig
        return BertConfig(**cfg).to_dict()
    except Exception:
        return dict(cfg, architectures=["BertForMaskedLM"], model_type="bert")


def hf_llama_config(meta: dict) -> dict:
    from ..models.llama import _ffn_from_multiple_of
    ffn = meta.get("ffn_dim") or _ffn_from_multiple_of(meta["dim"], meta.get("multiple_of", 256))
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=meta["dim"], intermediate_size=ffn,
               num_attention_heads=meta["n_heads"], num_key_value_heads=meta.get("n_kv_heads", meta["n_heads"]),
               num_hidden_layers=meta["n_layers"], vocab_size=meta["vocab_size"], rms_norm_eps=meta.get("norm_eps", 1e-5),
               max_position_embeddings=meta.get("n_positions", 2048), rope_theta=meta.get("rope_theta", 10000.0),
               tie_word_embeddings=False, hidden_act="silu")
    try:
        from transformers import LlamaConfig
        return LlamaConfig(**{k: v for k, v in cfg.items() if k not in ("architectures", "model_type")}).to_dict()
    except Exception:
        return cfg


def convert(model_type: str, input_checkpoint: str, output_dir: str, load_iteration: int, model_config: str,
            dtype: torch.dtype = torch.bfloat16) -> str:
    meta = json.load(open(model_config))
    iter_dir = os.path.join(input_checkpoint, "iter_%d" % load_iteration)
    if model_type in ("llama", "llama_hf", "qwen"):
        tensors, config = assemble_llama(iter_dir, meta), hf_llama_config(meta)
    elif model_type in ("bert", "bert-mlm", "bert_mlm", "bert_hf"):
        tensors, config = assemble_bert(iter_dir, meta), hf_bert_config(meta)
    elif model_type in ("gpt", "gpt2", "gpt_hf", "gpt_fa"):
        tensors, config = assemble_gpt(iter_dir, meta), hf_gpt_config(meta)
    elif model_type in ("vit", "vit_hf"):
        tensors, config = assemble_vit(iter_dir, meta), hf_vit_config(meta)
    elif model_type in ("t5", "T5"):
        tensors = assemble_t5(iter_dir, meta)
        config = hf_t5_config(meta, tensors)
    else:
        raise NotImplementedError("g2h covers the llama, bert, gpt, vit and t5 families; other "
                                  "families are stored with this package's own parameter names and load back "
                                  "through load_model")
    state = {k: v.to(dtype) for k, v in tensors.items()}
    os.makedirs(output_dir, exist_ok=True)
    torch.save(state, os.path.join(output_dir, "pytorch_model.bin"))
    json.dump(config, open(os.path.join(output_dir, "config.json"), "w"), indent=2, default=str)
    print("Successfully converted checkpoint to HuggingFace format at %s" % output_dir)
    return output_dir


# the reference's entry points (galvatron/tools/checkpoint_convert_g2h.py:11,111)
def convert_checkpoints_llama(input_checkpoint_path: str, output_dir: str, load_iteration: int, model_config: str):
    return convert("llama", input_checkpoint_path, output_dir, load_iteration, model_config)


def convert_checkpoints_bert_mlm(input_checkpoint_path: str, output_dir: str, load_iteration: int, model_config: str):
    return convert("bert-mlm", input_checkpoint_path, output_dir, load_iteration, model_config)


def main(argv=None):
    ap = argparse.ArgumentParser(description="Convert a distributed checkpoint to HuggingFace format.")
    ap.add_argument("--load_iteration", type=int, required=True)
    ap.add_argument("--input_checkpoint", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--model_config", required=True)
    ap.add_argument("--model_type", required=True)
    a = ap.parse_args(argv)
    convert(a.model_type, a.input_checkpoint, a.output_dir, a.load_iteration, a.model_config)


if __name__ == "__main__":
    main()
