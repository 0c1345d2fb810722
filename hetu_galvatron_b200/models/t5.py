"""T5 encoder-decoder family: two layer types, decoder stages carry two activations (encoder states and decoder
states, each with its own sequence length: ``seq_length`` and ``decoder_seq_length``, T5/arguments.py:26-27), shared
embedding tied to the head.

Reference: galvatron/models/T5/ (T5Model_sequential.py:291-321 module types ``embed_1, t5_enc x Le, pre_norm_1,
embed_2, t5_dec x Ld, pre_norm_2, cls``; RMS-style T5LayerNorm). The reference leaves the relative position bias out
(T5Model_tensor_parallel.py:13-14) and so does the default configuration here; ``relative_attention_num_buckets > 0``
adds it (a [buckets, heads] table per self-attention layer, ``models/transformer.py::SelfAttention._position_bias``), and
with ``act="relu"`` the model is the published T5, whose HuggingFace checkpoints ``core/checkpoint.py`` loads."""
from __future__ import annotations

import json
import os
from typing import List

import torch
import torch.nn as nn

from ..core.hybrid_model import ModuleSpec
from .blocks import EmbedBlock, HeadBlock, LayerBlock, NormBlock
from .transformer import BatchCtx, LayerStrategy, ModelConfig, TransformerLayer, FinalNorm

META_DIR = os.path.join(os.path.dirname(__file__), "meta_configs")
T5_SIZES = ["t5-small", "t5-base", "t5-large", "t5-3B"]


def t5_config(model_size: str = "t5-base", seq_length=None, dtype=torch.bfloat16, decoder_seq_length=None, **overrides) -> ModelConfig:
    with open(os.path.join(META_DIR, model_size + ".json")) as fp:
        meta = json.load(fp)
    overrides["decoder_seq_length"] = decoder_seq_length        # None: the decoder runs at the encoder's length
    cfg = ModelConfig(hidden_size=meta["d_model"], num_heads=meta["num_heads"], ffn_hidden_size=meta["d_ff"],
                      num_layers=meta["num_layers"], num_decoder_layers=meta.get("num_decoder_layers", meta["num_layers"]),
                      vocab_size=meta["vocab_size"], seq_length=seq_length or meta.get("n_positions", 512), norm="rms",
                      norm_eps=meta.get("layer_norm_epsilon", 1e-6), act="gelu", pos="none", bias=False, causal=False,
                      tie_embeddings=True, dtype=dtype, model_type="t5", make_vocab_size_divisible_by=128)
    for k, v in overrides.items():
        if v is not None:
            setattr(cfg, k, v)
    cfg.__post_init__()
    return cfg


def decoder_length(cfg: ModelConfig) -> int:
    return getattr(cfg, "decoder_seq_length", None) or cfg.seq_length


class T5DecoderEmbedBlock(nn.Module):
    """Receives the encoder output, embeds the decoder input ids with the shared table, returns both."""

    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device, tied=None):
        super().__init__()
        self.inner = EmbedBlock(cfg, st, device)
        if tied is not None:
            self.inner.embed.wte = tied
        self.tie_key = "wte"

    def forward(self, enc, ctx: BatchCtx):
        dec = self.inner(ctx.extra["decoder_input_ids"], ctx)
        return enc, dec


class T5DecoderLayerBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, st: LayerStrategy, idx: int, device):
        super().__init__()
        self.layer = TransformerLayer(cfg, st, idx, device, cross_attention=True, causal=True)

    def forward(self, x, ctx: BatchCtx):
        enc, dec = x
        return enc, self.layer(dec, ctx, enc=enc)


class T5DecoderNormBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device):
        super().__init__()
        self.norm = FinalNorm(cfg, st, device)

    def forward(self, x, ctx: BatchCtx):
        return self.norm(x[1], ctx)


def t5_specs(cfg: ModelConfig) -> List[ModuleSpec]:
    shared = {}
    le, ld = cfg.num_layers, cfg.num_decoder_layers or cfg.num_layers

    def build_embed(st, dev):
        blk = EmbedBlock(cfg, st, dev)
        shared["wte"] = blk.embed.wte
        return blk

    specs = [ModuleSpec("shared_embedding", "embed", build_embed, None, "embed_1")]
    for i in range(le):
        specs.append(ModuleSpec("encoder_block_%d" % i, "layer", (lambda st, dev, i=i: LayerBlock(cfg, st, i, dev, causal=False)), i, "t5_enc"))
    specs.append(ModuleSpec("encoder_final_layer_norm", "norm", lambda st, dev: NormBlock(cfg, st, dev), None, "pre_norm_1"))
    specs.append(ModuleSpec("decoder_embedding", "other", lambda st, dev: T5DecoderEmbedBlock(cfg, st, dev, shared.get("wte")), None, "embed_2"))
    both = ("seq_length", "decoder_seq_length")       # (encoder states, decoder states) travel together through the decoder
    for j in range(ld):
        specs.append(ModuleSpec("decoder_block_%d" % j, "layer", (lambda st, dev, j=j: T5DecoderLayerBlock(cfg, st, 100 + j, dev)),
                                le + j, "t5_dec", num_inputs=2, seq_attrs=both))
    specs.append(ModuleSpec("decoder_final_layer_norm", "norm", lambda st, dev: T5DecoderNormBlock(cfg, st, dev), None, "pre_norm_2",
                            num_inputs=2, seq_attrs=both))
    specs.append(ModuleSpec("lm_head", "cls", lambda st, dev: HeadBlock(cfg, st, dev, tied=shared.get("wte")), None, "cls",
                            seq_attr="decoder_seq_length"))
    return specs


def model_name(cfg: ModelConfig) -> str:
    if decoder_length(cfg) != cfg.seq_length:
        return "hidden%d_head%d_seqlen[%d,%d]" % (cfg.hidden_size, cfg.num_heads, cfg.seq_length, decoder_length(cfg))
    return "hidden%d_head%d_seqlen%d" % (cfg.hidden_size, cfg.num_heads, cfg.seq_length)


def model_layer_configs(cfg: ModelConfig):
    return [{"hidden_size": cfg.hidden_size, "seq_len": cfg.seq_length, "layer_num": cfg.num_layers},
            {"hidden_size": cfg.hidden_size, "seq_len": decoder_length(cfg), "layer_num": cfg.num_decoder_layers or cfg.num_layers}]


# entry points under the reference's names (models/api.py)
from .api import family_api  # noqa: E402

get_t5_config, t5_model_hp, T5ModelInfo = family_api("t5")
