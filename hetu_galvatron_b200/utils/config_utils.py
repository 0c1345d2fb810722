"""JSON / strategy / bandwidth-config helpers.

Same function names, argument order and file formats as the reference's ``galvatron/utils/config_utils.py``
(:8-137), so plan files, profile files and hardware files written by either system are interchangeable.
One deliberate difference: ``cp_sizes_enc`` is optional in a plan (the reference's loader requires a key its
own search never writes, config_utils.py:37 vs :46-57).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence

import numpy as np


def str2array(s: str) -> List[int]:
    return [int(x) for x in str(s).split(",") if x != ""]


def array2str(a: Sequence[int]) -> str:
    return ",".join(str(int(x)) for x in a)


def read_json_config(path: str) -> dict:
    with open(path, "r", encoding="utf-8") as fp:
        return json.load(fp)


def write_json_config(config: dict, path: str) -> None:
    d = os.path.dirname(path)
    if d:
        os.makedirs(d, exist_ok=True)
    with open(path, "w") as fp:
        json.dump(config, fp, indent=4)


def config2strategy(config: dict):
    """Plan JSON -> (pp_deg, tp_sizes, cp_sizes, tp_consec_flags, dp_types, use_sp, vtp, vsp, vcp)."""
    pp_deg = config["pp_deg"]
    tp_sizes_enc = str2array(config["tp_sizes_enc"])
    n = len(tp_sizes_enc)
    cp_sizes_enc = str2array(config["cp_sizes_enc"]) if "cp_sizes_enc" in config else [1] * n
    tp_consecutive_flags = str2array(config["tp_consecutive_flags"]) if "tp_consecutive_flags" in config else [1] * n
    dp_types_enc = str2array(config["dp_types_enc"]) if "dp_types_enc" in config else [0] * n
    use_sp = str2array(config["use_sp"]) if "use_sp" in config else [0] * n
    return (pp_deg, tp_sizes_enc, cp_sizes_enc, tp_consecutive_flags, dp_types_enc, use_sp,
            config.get("vtp", 1), config.get("vsp", 0), config.get("vcp", 1))


def strategy2config(strategy_list) -> dict:
    """List of ``[pp, tp, dp, {flags}]`` strategies -> the per-layer part of a plan JSON."""
    if len(strategy_list) == 0:
        return {}
    from .strategy_utils import strategy_flags

    flags = [strategy_flags(s) for s in strategy_list]
    return {
        "pp_deg": strategy_list[0][0],
        "tp_sizes_enc": array2str([s[1] for s in strategy_list]),
        "tp_consecutive_flags": array2str([f["tp_consec"] for f in flags]),
        "dp_types_enc": array2str([f["fsdp"] for f in flags]),
        "use_sp": array2str([f["sp"] for f in flags]),
    }


def read_allreduce_bandwidth_config(config_path, gpu_num: int):
    """Returns (bandwidth_dict, comm_coe_dict) keyed '8', '4_0', '4_1', ..., '1' (coe = 1 / bus bandwidth)."""
    env = read_json_config(config_path) if isinstance(config_path, str) else config_path
    bw: Dict[str, float] = {}
    coe: Dict[str, float] = {}
    size = gpu_num
    if size >= 2:
        bw[str(size)] = env["allreduce_size_%d_consec_1" % size]
        coe[str(size)] = 1.0 / bw[str(size)]
    size //= 2
    while size >= 2:
        for consec in (0, 1):
            key = "%d_%d" % (size, consec)
            bw[key] = env["allreduce_size_%d_consec_%d" % (size, consec)]
            coe[key] = 1.0 / bw[key]
        size //= 2
    bw["1"] = np.inf
    coe["1"] = 0
    return bw, coe


def read_p2p_bandwidth_config(config_path):
    env = read_json_config(config_path) if isinstance(config_path, str) else config_path
    p2p, coe = {}, {}
    for key, val in env.items():
        if "pp_size_" in key:
            k = int(key.split("_")[-1])
            p2p[k] = val
            coe[k] = 1.0 / val
    return p2p, coe


def num2str(num, name: str) -> str:
    if name == "seq" and isinstance(num, (list, tuple)) and len(num) == 1:
        num = num[0]
    if isinstance(num, (list, tuple)):
        return "%s[%s]" % (name, array2str(num))
    return "%s%d" % (name, num)


def dict_join_dirname(dic: dict, dirname: str) -> dict:
    for key, val in dic.items():
        dic[key] = os.path.join(dirname, val)
    return dic


def remap_config(config: dict, op: str) -> dict:
    """Latency table ``{op}_size_{k}_{m}MB_time`` -> {k: {bytes: ms, ..., 'popt': (slope, intercept)}}.

    All-reduce times are halved to model one all-gather / reduce-scatter; ``popt`` is the least-squares line
    through (MB, ms)."""
    out: Dict[int, dict] = {}
    for key, val in config.items():
        if not key.startswith(op):
            continue
        if op == "allreduce":
            val = val / 2
        parts = key.split("_")
        world, mb = int(parts[-3]), int(parts[-2][:-2])
        out.setdefault(world, {})[mb * 1024 * 1024] = val
    for world, table in out.items():
        xs = np.array([size // 1024 // 1024 for size in table], dtype=np.float64)
        ys = np.array(list(table.values()), dtype=np.float64)
        assert len(xs) >= 8, f"Different size in communication profile of {op} should not be lower than 8."
        from scipy.optimize import curve_fit

        popt, _ = curve_fit(lambda x, m, c: m * x + c, xs, ys)
        table["popt"] = popt
    return out
