"""Profile-file writers. Key grammar and file names are the reference's (galvatron/core/profiler/utils.py:22-64):
memory profiles are keyed ``"{pp}_{tp}_{dp}[_c][_vtp][_sp]"`` -> ``layernum[..]_bsz{B}_seq{S}_rank{r}_{ms|act|act_peak}``
(MB), time profiles ``layernum[..]_bsz{B}_seq{S}`` (ms per iteration)."""
from __future__ import annotations

import os

from ..utils.config_utils import num2str, read_json_config, write_json_config


def memory_strategy_key(pp_deg: int, tp_deg: int, world_size: int, cpt, vocab_tp: int = 1, sequence_parallel: bool = False) -> str:
    key = "%d_%d_%d" % (pp_deg, tp_deg, world_size // pp_deg // tp_deg)
    if cpt:
        key += "_c"
    if vocab_tp == tp_deg and tp_deg != 1:
        key += "_vtp"
    if sequence_parallel:
        key += "_sp"
    return key


def save_profiled_memory(path, pp_deg, tp_deg, world_size, layer_num, bsz, rank, model_states, activation, activation_peak,
                         cpt, sequence_parallel=False, vocab_tp=1, seq=None) -> None:
    config = read_json_config(path) if os.path.exists(path) else {}
    entry = config.setdefault(memory_strategy_key(pp_deg, tp_deg, world_size, cpt, vocab_tp, sequence_parallel), {})
    stem = "%s_bsz%d_%s_rank%d" % (num2str(layer_num, "layernum"), bsz, num2str(seq, "seq"), rank)
    entry[stem + "_ms"] = model_states
    entry[stem + "_act"] = activation
    entry[stem + "_act_peak"] = activation_peak
    write_json_config(config, path)
    print("Already written profiled memory into config file %s!\n" % path)


def save_profiled_time(path, time, bsz, layer_num, seq, suffix: str = "") -> None:
    """``suffix`` "_iter": time of a whole iteration (forward + backward + optimizer step) instead of the forward pass."""
    config = read_json_config(path) if os.path.exists(path) else {}
    config["%s_bsz%d_%s%s" % (num2str(layer_num, "layernum"), bsz, num2str(seq, "seq"), suffix)] = time
    write_json_config(config, path)
    print("Already written profiled time into config file %s!\n" % path)
