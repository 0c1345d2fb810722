"""Strategy <-> string codec. A strategy is ``[pp, tp, dp, {fsdp, tp, cpt, sp}]``; its printed form is e.g.
``2-2*-2f-c-sp`` (reference: galvatron/utils/strategy_utils.py:3-95)."""
from __future__ import annotations


def strategy_flags(strategy) -> dict:
    info = strategy[-1] if len(strategy) == 4 and isinstance(strategy[-1], dict) else {}
    return {
        "tp_consec": 0 if ("tp" in info and not info["tp"]) else 1,
        "fsdp": 1 if info.get("fsdp") else 0,
        "cpt": 1 if info.get("cpt") else 0,
        "sp": 1 if info.get("sp") else 0,
    }


def form_strategy(strategy) -> str:
    assert len(strategy) == 4
    info = strategy[-1]
    tp = "%d" % strategy[1]
    dp = "%d" % strategy[2]
    if info.get("fsdp"):
        dp += "f"
    if "tp" in info:
        if info["tp"]:
            tp += "*"
        else:
            dp += "*"
    if info.get("cpt"):
        dp += "-c"
    if info.get("sp"):
        dp += "-sp"
    return "%d-%s-%s" % (strategy[0], tp, dp)


def strategy_str2list(s: str):
    parts = s.split("-")
    tp_consec = None
    if parts[1].endswith("*"):
        tp_consec, parts[1] = 1, parts[1][:-1]
    elif parts[2].endswith("*"):
        tp_consec, parts[2] = 0, parts[2][:-1]
    fsdp = 0
    if parts[2].endswith("f"):
        fsdp, parts[2] = 1, parts[2][:-1]
    tail = parts[3:]
    pp, tp, dp = int(parts[0]), int(parts[1]), int(parts[2])
    info = {}
    if tp > 1 and dp > 1 and tp_consec is not None:
        info["tp"] = tp_consec
    if dp > 1:
        info["fsdp"] = fsdp
    if "c" in tail:
        info["cpt"] = 1
    if "sp" in tail:
        info["sp"] = 1
    return [pp, tp, dp, info]


def strategies_to_string(strategy_list) -> str:
    if strategy_list is None or isinstance(strategy_list, str):
        return "None"
    if len(strategy_list) and isinstance(strategy_list[0][0], list):
        return " || ".join(", ".join(form_strategy(s) for s in sub) for sub in strategy_list)
    return ", ".join(form_strategy(s) for s in strategy_list)


def print_strategies(strategy_list, logger=None) -> None:
    text = strategies_to_string(strategy_list)
    if logger is None:
        print(None if text == "None" else text)
    else:
        logger.info(None if text == "None" else text)
