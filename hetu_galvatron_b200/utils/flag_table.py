"""Command-line flags as tables. A row is ``(name, kind, default[, help])``:

* ``kind`` a type (``int``, ``float``, ``str``): a valued flag;
* ``kind`` a list: a string flag restricted to those choices;
* ``kind`` ``"on"``: a switch that stores True; ``"off:<dest>"``: a switch that stores False into ``<dest>``;
* a name written with dashes (``make-vocab-size-divisible-by``) is stored under its underscore spelling.
"""
from __future__ import annotations

import argparse
from typing import Iterable, Sequence


def add_flags(group, rows: Iterable[Sequence]) -> None:
    for row in rows:
        name, kind, default = row[0], row[1], row[2]
        kw = {"help": row[3]} if len(row) > 3 else {}
        if "-" in name:
            kw["dest"] = name.replace("-", "_")
        if kind == "on":
            group.add_argument("--" + name, action="store_true", **kw)
        elif isinstance(kind, str) and kind.startswith("off:"):
            kw["dest"] = kind[4:]
            group.add_argument("--" + name, action="store_false", **kw)
        elif isinstance(kind, (list, tuple)):
            group.add_argument("--" + name, type=type(kind[0]), default=default, choices=list(kind), **kw)
        else:
            group.add_argument("--" + name, type=kind, default=default, **kw)


def flag_group(parser: argparse.ArgumentParser, title: str, rows: Iterable[Sequence]) -> argparse.ArgumentParser:
    add_flags(parser.add_argument_group(title=title), rows)
    return parser
