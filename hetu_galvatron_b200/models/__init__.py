"""Model zoo. ``build_model_specs(family, **config)`` returns (ModelConfig, [ModuleSpec]) for a family name;
``synthetic_batch`` makes the random inputs the reference's ``train_dist_random.py`` programs use."""
from __future__ import annotations

import torch

from .transformer import ModelConfig


def build_model_specs(family: str, dtype=torch.bfloat16, **kw):
    family = family.lower()
    if family in ("llama", "llama_hf", "llama_fa", "qwen"):
        from .llama import llama_config, llama_specs
        if "model_size" in kw:
            cfg = llama_config(kw.pop("model_size"), dtype=dtype, **kw)
        else:
            cfg = ModelConfig(norm="rms", act="swiglu", pos="rope", bias=False, causal=True, dtype=dtype, model_type="llama", **kw)
        return cfg, llama_specs(cfg)
    if family in ("gpt", "gpt_hf", "gpt_fa"):
        from .gpt import gpt_config, gpt_specs
        cfg = gpt_config(kw.pop("model_size"), dtype=dtype, **kw) if "model_size" in kw else ModelConfig(
            norm="layer", act="gelu", pos="learned", bias=True, causal=True, tie_embeddings=True, dtype=dtype,
            model_type="gpt", **kw)
        return cfg, gpt_specs(cfg)
    if family in ("bert", "bert_hf"):
        from .bert import bert_config, bert_specs
        cfg = bert_config(kw.pop("model_size"), dtype=dtype, **kw) if "model_size" in kw else ModelConfig(
            norm="layer", act="gelu", pos="learned", bias=True, causal=False, post_ln=True, type_vocab_size=2,
            tie_embeddings=True, dtype=dtype, model_type="bert", **kw)
        return cfg, bert_specs(cfg)
    if family in ("vit", "vit_hf"):
        from .vit import vit_config, vit_specs
        cfg = vit_config(kw.pop("model_size"), dtype=dtype, **kw) if "model_size" in kw else ModelConfig(
            norm="layer", act="gelu", pos="learned", bias=True, causal=False, dtype=dtype, model_type="vit", **kw)
        cfg.seq_length = (cfg.image_size // cfg.patch_size) ** 2 + 1
        cfg.vocab_size = cfg.num_labels
        return cfg, vit_specs(cfg)
    if family in ("t5",):
        from .t5 import t5_config, t5_specs
        cfg = t5_config(kw.pop("model_size"), dtype=dtype, **kw) if "model_size" in kw else ModelConfig(
            norm="rms", act=kw.pop("act", "gelu"), pos="none", bias=False, causal=False, tie_embeddings=True, dtype=dtype,
            model_type="t5", **kw)
        return cfg, t5_specs(cfg)
    if family in ("swin",):
        from .swin import swin_config, swin_specs
        cfg = swin_config(kw.pop("model_size", "swin-tiny-test"), dtype=dtype, **kw)
        return cfg, swin_specs(cfg)
    raise ValueError("unknown model family %r" % family)


def synthetic_batch(family: str, cfg: ModelConfig, global_bsz: int, seed: int, device, padded: bool = False):
    """Random inputs of the family's shape: (input, labels[, extra dict]), batch-major. ``padded`` (BERT, T5): sequences of
    random length, padded on the right, with the padding masks (1 = token) in the extras as HuggingFace names them."""
    g = torch.Generator().manual_seed(seed)
    family = family.lower()
    if family in ("vit", "vit_hf", "swin"):
        px = torch.randn(global_bsz, cfg.num_channels, cfg.image_size, cfg.image_size, generator=g).to(device=device, dtype=cfg.dtype)
        labels = torch.randint(0, cfg.num_labels, (global_bsz,), generator=g).to(device)
        return px, labels
    if family == "t5":
        sd = getattr(cfg, "decoder_seq_length", None) or cfg.seq_length
        enc = torch.randint(0, cfg.vocab_size, (global_bsz, cfg.seq_length), generator=g).to(device)
        dec = torch.randint(0, cfg.vocab_size, (global_bsz, sd + 1), generator=g).to(device)
        extra = {"decoder_input_ids": dec[:, :-1].contiguous()}
        labels = dec[:, 1:].contiguous()
        if padded:
            pos, dpos = torch.arange(cfg.seq_length).view(1, -1), torch.arange(sd).view(1, -1)
            enc_len = torch.randint(max(cfg.seq_length // 2, 1), cfg.seq_length + 1, (global_bsz, 1), generator=g)
            dec_len = torch.randint(max(sd // 2, 1), sd + 1, (global_bsz, 1), generator=g)
            extra["attention_mask"] = (pos < enc_len).long().to(device)
            extra["decoder_attention_mask"] = (dpos < dec_len).long().to(device)
            labels = labels.masked_fill((dpos >= dec_len).to(device), -100)
        return enc, labels, extra
    tok = torch.randint(0, cfg.vocab_size, (global_bsz, cfg.seq_length + 1), generator=g).to(device)
    if family in ("bert", "bert_hf"):
        ids = tok[:, :-1].contiguous()
        labels = ids.clone()
        mask = torch.rand(ids.shape, generator=g) < 0.15
        labels[~mask.to(device)] = -100
        if padded:
            pos = torch.arange(cfg.seq_length).view(1, -1)
            lens = torch.randint(max(cfg.seq_length // 2, 1), cfg.seq_length + 1, (global_bsz, 1), generator=g)
            labels = labels.masked_fill((pos >= lens).to(device), -100)
            return ids, labels, {"attention_mask": (pos < lens).long().to(device)}
        return ids, labels
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def specs_for(family: str, cfg: ModelConfig, fp32_logits: bool = False):
    family = family.lower()
    if family in ("llama", "llama_hf", "llama_fa", "qwen"):
        from .llama import llama_specs
        return llama_specs(cfg, fp32_logits=fp32_logits)
    if family in ("gpt", "gpt_hf", "gpt_fa"):
        from .gpt import gpt_specs
        return gpt_specs(cfg, fp32_logits=fp32_logits)
    if family in ("bert", "bert_hf"):
        from .bert import bert_specs
        return bert_specs(cfg)
    if family in ("vit", "vit_hf"):
        from .vit import vit_specs
        return vit_specs(cfg)
    if family == "t5":
        from .t5 import t5_specs
        return t5_specs(cfg)
    if family == "swin":
        from .swin import swin_specs
        return swin_specs(cfg)
    raise ValueError("unknown model family %r" % family)


def model_name_and_layer_configs(family: str, cfg: ModelConfig, args=None):
    """(profile-file model name, per-layer-type configs) as the reference's meta_configs/config_utils.py:111-125;
    under sequence-mode profiling the name carries no sequence length (one file for all lengths)."""
    import importlib
    import re

    from .arguments import base_family

    mod = importlib.import_module("." + base_family(family), __package__)
    name = mod.model_name(cfg)
    if getattr(args, "profile_mode", "static") == "sequence":
        name = re.sub(r"_seqlen\d+$", "", name)
    return name, mod.model_layer_configs(cfg)
