"""HuggingFace checkpoint -> one ``.pt`` per block, independent of any parallel plan.

Same output contract as the reference's galvatron/tools/checkpoint_convert_h2g.py (file name = block name with dots
replaced by underscores, keys = the parameter name inside that block), written as one routing table per family
instead of one function per family. Reads ``*.bin`` and, when the ``safetensors`` package is present,
``*.safetensors`` shards; a block whose tensors are spread over several shards is merged.

    python -m hetu_galvatron_b200.tools.checkpoint_convert_h2g --model_type llama \
        --input_checkpoint <hf dir> --output_dir <dir>
"""
from __future__ import annotations

import argparse
import os
import re
from collections import defaultdict
from typing import Callable, Dict, List, Optional, Tuple

import torch

# (regex on the HF key, block name template, key-inside-block template); first match wins
Route = Tuple[str, str, str]

ROUTES: Dict[str, List[Route]] = {
    "llama": [
        (r"^model\.layers\.(\d+)\.(.+)$", "model.layers.{0}", "{1}"),
        (r"^model\.norm\.(.+)$", "model.norm", "{0}"),
        (r"^model\.(embed_tokens\..+)$", "model.embed_tokens", "{0}"),
        (r"^lm_head\.(.+)$", "lm_head", "{0}"),
    ],
    "gpt": [
        (r"^transformer\.h\.(\d+)\.(.+)$", "transformer.h.{0}", "{1}"),
        (r"^transformer\.ln_f\.(.+)$", "transformer.ln_f", "{0}"),
        (r"^transformer\.(w[tp]e\..+)$", "transformer.embedding", "{0}"),
        (r"^lm_head\.(.+)$", "transformer.embedding", "lm_head.{0}"),
    ],
    "bert-mlm": [
        (r"^bert\.embeddings\.(.+)$", "bert.embeddings", "{0}"),
        (r"^bert\.encoder\.layer\.(\d+)\.(.+)$", "bert.encoder.layer.{0}", "{1}"),
        (r"^cls\.predictions\.(.+)$", "cls.predictions", "{0}"),
        (r"^bert\.pooler\.(.+)$", "bert.pooler", "{0}"),
    ],
    "vit": [
        (r"^vit\.embeddings\.(.+)$", "vit.embeddings", "{0}"),
        (r"^vit\.encoder\.layer\.(\d+)\.(.+)$", "vit.encoder.layer.{0}", "{1}"),
        (r"^vit\.layernorm\.(.+)$", "vit.layernorm", "{0}"),
        (r"^classifier\.(.+)$", "classifier", "{0}"),
        (r"^vit\.pooler\.(.+)$", "classifier", "pooler.{0}"),
    ],
    "swin": [
        (r"^swin\.embeddings\.(.+)$", "swin.embeddings", "{0}"),
        (r"^swin\.encoder\.layers\.(\d+)\.blocks\.(\d+)\.(.+)$", "swin.encoder.{0}.{1}", "{2}"),
        (r"^swin\.encoder\.layers\.(\d+)\.downsample\.(.+)$", "swin.encoder.{0}.downsample", "{1}"),
        (r"^swin\.layernorm\.(.+)$", "swin.classifier", "layernorm.{0}"),
        (r"^classifier\.(.+)$", "swin.classifier", "{0}"),
    ],
    "t5": [
        (r"^shared\.(.+)$", "shared", "{0}"),
        (r"^(encoder|decoder)\.block\.(\d+)\.(.+)$", "{0}.block.{1}", "{2}"),
        (r"^(encoder|decoder)\.final_layer_norm\.(.+)$", "{0}.final_layer_norm", "{1}"),
        (r"^lm_head\.(.+)$", "lm_head", "{0}"),
    ],
}
ROUTES["bert_mlm"] = ROUTES["bert-mlm"]


def route_key(model_type: str, key: str) -> Optional[Tuple[str, str]]:
    for pattern, block, inner in ROUTES[model_type]:
        m = re.match(pattern, key)
        if m:
            return block.format(*m.groups()), inner.format(*m.groups())
    return None


def _load_shard(path: str):
    if path.endswith(".bin") or path.endswith(".pt"):
        return torch.load(path, mmap=True, map_location="cpu", weights_only=True)
    if path.endswith(".safetensors"):
        import safetensors.torch
        return safetensors.torch.load_file(path, device="cpu")
    return None


def split_state_dict(model_type: str, state: Dict[str, torch.Tensor]) -> Dict[str, Dict[str, torch.Tensor]]:
    blocks: Dict[str, Dict[str, torch.Tensor]] = defaultdict(dict)
    for key, value in state.items():
        dest = route_key(model_type, key)
        if dest is not None:
            blocks[dest[0]][dest[1]] = value
    return blocks


def convert(model_type: str, input_checkpoint: str, output_dir: str, log: Callable[[str], None] = print) -> List[str]:
    os.makedirs(output_dir, exist_ok=True)
    written = []
    for fname in sorted(os.listdir(input_checkpoint)):
        state = _load_shard(os.path.join(input_checkpoint, fname))
        if state is None:
            continue
        for block, params in split_state_dict(model_type, state).items():
            out = os.path.join(output_dir, block.replace(".", "_") + ".pt")
            if os.path.exists(out):
                merged = torch.load(out, map_location="cpu", weights_only=True)
                merged.update(params)
                params = merged
            torch.save({k: v.clone() for k, v in params.items()}, out)
            written.append(out)
            log("Saved parameters for %s to %s" % (block, out))
    return written


# the reference's entry points, one per family it converts (galvatron/tools/checkpoint_convert_h2g.py:6,43,84)
def convert_checkpoints_gpt(input_checkpoint_path: str, output_dir: str) -> List[str]:
    return convert("gpt", input_checkpoint_path, output_dir)


def convert_checkpoints_llama(input_checkpoint_path: str, output_dir: str) -> List[str]:
    return convert("llama", input_checkpoint_path, output_dir)


def convert_checkpoints_bert_mlm(input_checkpoint_path: str, output_dir: str) -> List[str]:
    return convert("bert-mlm", input_checkpoint_path, output_dir)


def main(argv=None):
    ap = argparse.ArgumentParser(description="Split a HuggingFace checkpoint into one file per block.")
    ap.add_argument("--model_type", required=True, choices=sorted(ROUTES))
    ap.add_argument("--input_checkpoint", required=True)
    ap.add_argument("--output_dir", required=True)
    a = ap.parse_args(argv)
    convert(a.model_type, a.input_checkpoint, a.output_dir)


if __name__ == "__main__":
    main()
