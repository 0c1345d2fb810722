"""Per-family model flags (the reference keeps one ``arguments.py`` per model directory, e.g.
galvatron/models/llama_hf/arguments.py:3-35, galvatron/models/vit_hf/arguments.py:3-64)."""
from __future__ import annotations

SIZES = {
    "llama": ["llama-0.3b", "llama-7b", "llama-13b", "llama-30b", "llama2-70b", "qwen2.5-1.5b", "qwen2.5-3b", "qwen2.5-7b", "qwen2.5-72b"],
    "gpt": ["gpt-0.3b", "gpt-1.5b", "gpt-2.7b", "gpt-6.7b"],
    "bert": ["bert-base", "bert-large", "bert-huge-32", "bert-huge-48"],
    "vit": ["vit-base", "vit-large", "vit-huge", "vit-huge-patch14", "vit-xhuge"],
    "t5": ["t5-small", "t5-base", "t5-large", "t5-3B"],
    "swin": ["swin-tiny-test", "swin-huge-patch4-window7-224", "swin-large-patch4-window12-384"],
}


_BASE = {"llama_hf": "llama", "llama_fa": "llama", "qwen": "llama", "gpt_hf": "gpt", "gpt_fa": "gpt", "bert_hf": "bert",
         "vit_hf": "vit", "T5": "t5"}


def base_family(family: str) -> str:
    """The model definition behind a family name. The reference keeps separate ``*_hf`` (HuggingFace skeleton) and
    ``*_fa`` (flash-attn skeleton, galvatron/models/llama_fa, gpt_fa) directories of the same architectures; here both
    names run one definition on this package's kernels."""
    return _BASE.get(family, family)


def make_model_args(family: str):
    family = base_family(family)

    def model_args(parser):
        g = parser.add_argument_group(title="Model Arguments")
        g.add_argument("--model_size", type=str, default=SIZES[family][1 if len(SIZES[family]) > 1 else 0], choices=SIZES[family])
        g.add_argument("--hidden_size", type=int, default=768)
        g.add_argument("--num_hidden_layers", type=int, default=12)
        g.add_argument("-a", "--num_attention_heads", type=int, default=12)
        g.add_argument("--ffn_hidden_size", type=int, default=None)
        g.add_argument("-s", "--seq_length", type=int, default=None)
        g.add_argument("--vocab_size", type=int, default=None)
        g.add_argument("--max_predictions_per_seq", type=int, default=20)
        if family in ("vit", "swin"):
            g.add_argument("--image_size", type=int, default=None, help="default: the model size's")
            g.add_argument("--patch_size", type=int, default=None)
            g.add_argument("--num_channels", type=int, default=3)
            g.add_argument("--num_labels", type=int, default=1000)
        if family == "swin":
            g.add_argument("--depths", type=int, nargs="+", default=None, help="blocks per stage (four layer types)")
            g.add_argument("--embed_dim", type=int, default=None)
            g.add_argument("--window_size", type=int, default=None)
            g.add_argument("--num_heads", type=int, nargs="+", default=None, help="attention heads per stage")
            g.add_argument("--mlp_ratio", type=int, default=None)
            g.add_argument("--num_classes", type=int, default=None, help="number of labels (same as --num_labels)")
            g.add_argument("--drop_path_rate", type=float, default=None,
                           help="stochastic depth on the attention branch; default: the model size's rate")
        if family == "vit":
            g.add_argument("--intermediate_size", type=int, default=None, help="MLP width (with --set_model_config_manually)")
            g.add_argument("--hidden_dropout_prob", type=float, default=None, help="same as --dropout_prob")
            g.add_argument("--attention_probs_dropout_prob", type=float, default=None,
                           help="dropout of the attention probabilities; default: the hidden dropout")
            g.add_argument("--layer_norm_eps", type=float, default=None)
        if family == "t5":
            g.add_argument("--num_encoder_layers", type=int, default=None)
            g.add_argument("--num_decoder_layers", type=int, default=None)
            g.add_argument("--relative_attention_num_buckets", type=int, default=0,
                           help="> 0 (32 in the published T5 models): every self-attention layer adds a learned bias per "
                                "(query, key) offset bucket and head to its scores; 0 (default): none, as in the reference")
            g.add_argument("--relative_attention_max_distance", type=int, default=128)
            g.add_argument("--t5_feed_forward", type=str, default="gelu", choices=["gelu", "relu"],
                           help="activation of the feed-forward block (the original T5 checkpoints use relu)")
            g.add_argument("--encoder_seq_length", type=int, default=None, help="with --set_seqlen_manually; default: --seq_length")
            g.add_argument("--decoder_seq_length", type=int, default=None, help="with --set_seqlen_manually; default: the encoder's")
        return parser

    return model_args


def layernum_arg_names(family: str):
    family = base_family(family)
    if family == "swin":
        return ["depths"]          # one list-valued flag: one layer type per entry
    return ["num_encoder_layers", "num_decoder_layers"] if family == "t5" else ["num_hidden_layers"]


def config_from_args(family: str, args, dtype):
    """ModelConfig + specs: the size table, overridden by manual flags the way the reference's
    ``set_model_config`` does (meta_configs/config_utils.py:52-107)."""
    from . import build_model_specs

    family = base_family(family)
    kw = {"model_size": args.model_size}
    if getattr(args, "set_seqlen_manually", 0) and getattr(args, "seq_length", None) and family not in ("vit", "swin"):
        kw["seq_length"] = args.seq_length
    if family == "t5" and getattr(args, "set_seqlen_manually", 0):
        # T5/meta_configs/config_utils.py:49-52: both lengths are set together; --seq_length alone sets both to one value
        if getattr(args, "encoder_seq_length", None):
            kw["seq_length"] = args.encoder_seq_length
        if getattr(args, "decoder_seq_length", None):
            kw["decoder_seq_length"] = args.decoder_seq_length
    if family == "swin" and getattr(args, "set_layernum_manually", 0) and getattr(args, "depths", None):
        kw["depths"] = list(args.depths)
    if family in ("vit", "swin"):
        for flag in ("image_size", "patch_size"):
            if getattr(args, flag, None):
                kw[flag] = getattr(args, flag)
    if family == "swin":
        # models/swin/meta_configs/config_utils.py:30-50: every architecture flag counts with --set_model_config_manually,
        # depths and heads per stage also with --set_layernum_manually
        dp = getattr(args, "drop_path_rate", None)
        kw["drop_path_rate"] = "meta" if dp is None else dp
        if getattr(args, "set_model_config_manually", 0):
            for flag, key in (("embed_dim", "embed_dim"), ("window_size", "window_size"), ("mlp_ratio", "mlp_ratio"),
                              ("depths", "depths"), ("num_heads", "stage_heads"), ("num_channels", "num_channels")):
                if getattr(args, flag, None):
                    kw[key] = list(getattr(args, flag)) if isinstance(getattr(args, flag), (list, tuple)) else getattr(args, flag)
            labels = getattr(args, "num_classes", None) or getattr(args, "num_labels", None)
            if labels:
                kw["num_labels"] = labels
        elif getattr(args, "set_layernum_manually", 0) and getattr(args, "num_heads", None):
            kw["stage_heads"] = list(args.num_heads)
    cfg, _ = build_model_specs(family, dtype=dtype, **kw)
    if family == "swin":
        pass
    elif getattr(args, "set_model_config_manually", 0):
        cfg.hidden_size, cfg.num_heads = args.hidden_size, args.num_attention_heads
        cfg.num_kv_heads = cfg.num_heads
        cfg.num_layers = args.num_hidden_layers
        if args.ffn_hidden_size:
            cfg.ffn_hidden_size = args.ffn_hidden_size
        if args.vocab_size:
            cfg.vocab_size = args.vocab_size
    elif getattr(args, "set_layernum_manually", 0):
        if family == "t5":
            cfg.num_layers = args.num_encoder_layers or cfg.num_layers
            cfg.num_decoder_layers = args.num_decoder_layers or cfg.num_decoder_layers
        else:
            cfg.num_layers = args.num_hidden_layers
    if family == "t5":
        cfg.relative_attention_num_buckets = int(getattr(args, "relative_attention_num_buckets", 0) or 0)
        cfg.relative_attention_max_distance = int(getattr(args, "relative_attention_max_distance", 128) or 128)
        cfg.act = getattr(args, "t5_feed_forward", None) or cfg.act
    if family == "vit":
        if getattr(args, "set_model_config_manually", 0) and getattr(args, "intermediate_size", None):
            cfg.ffn_hidden_size = args.intermediate_size
        if getattr(args, "layer_norm_eps", None):
            cfg.norm_eps = args.layer_norm_eps
        if getattr(args, "attention_probs_dropout_prob", None) is not None:
            cfg.attention_dropout = args.attention_probs_dropout_prob
    # hidden / embedding dropout of the families that have it (the Llama family has none; Swin's blocks do not implement it)
    cfg.dropout = float(getattr(args, "dropout_prob", 0.0) or 0.0) if family in ("gpt", "bert", "vit", "t5") else 0.0
    if family == "vit" and getattr(args, "hidden_dropout_prob", None) is not None:
        cfg.dropout = float(args.hidden_dropout_prob)
    if getattr(args, "init_method_std", None):
        cfg.init_std = float(args.init_method_std)
    from . import specs_for

    return cfg, specs_for(family, cfg, fp32_logits=getattr(args, "entropy_in_fp32", False))
