"""Command lines that mix options with ``key=value`` configuration overrides in any order
(``prog --config-name X a.b=1 --flag run.c=2``): argparse alone stops collecting a ``nargs="*"`` positional at the first
option, so the overrides after it would be "unrecognized arguments"."""
from __future__ import annotations

import argparse
import re

_OVERRIDE = re.compile(r"^(\+\+|\+|~)?[A-Za-z_][\w.]*(=.*)?$")


def parse_with_overrides(ap: argparse.ArgumentParser, argv=None, dest: str = "overrides") -> argparse.Namespace:
    """``ap.parse_args`` where leftover arguments that look like overrides (``a.b=c``, ``+a.b=c``, ``++a.b=c``, ``~a.b``) are
    appended to ``dest`` wherever they stand; anything else left over is an error, as usual."""
    ns, extra = ap.parse_known_args(argv)
    bad = [e for e in extra if e.startswith("-") or not _OVERRIDE.match(e) or ("=" not in e and not e.startswith("~"))]
    if bad:
        ap.error("unrecognized arguments: %s" % " ".join(bad))
    setattr(ns, dest, list(getattr(ns, dest, None) or []) + extra)
    return ns
