"""``python -m open_transformers_b200.config.describe [--config-name NAME] [overrides...]``

Without a name: every key of the schema with its type and default (the reference for writing recipes and overrides).
With a name: the fully resolved recipe as YAML, after defaults lists, ``key=value`` / ``+key`` / ``++key`` / ``~key``
overrides and validation - the same object that is embedded in every checkpoint's ``meta.json``."""
from __future__ import annotations

import argparse
import json
import sys
import typing

from pydantic import BaseModel
from pydantic_core import PydanticUndefined

from .schema import RootConfig


def schema_rows(model: type[BaseModel] = RootConfig, prefix: str = "") -> list[tuple[str, str, str]]:
    """(dotted key, type, default) for every leaf of the schema, in declaration order."""
    rows = []
    for name, field in model.model_fields.items():
        ann = field.annotation
        inner = [a for a in typing.get_args(ann) if isinstance(a, type) and issubclass(a, BaseModel)] if typing.get_args(ann) else []
        sub = ann if isinstance(ann, type) and issubclass(ann, BaseModel) else (inner[0] if inner and typing.get_origin(ann) is not list else None)
        if sub is not None:
            rows += schema_rows(sub, prefix + name + ".")
            continue
        if field.default is not PydanticUndefined:
            default = json.dumps(field.default, default=str)
        elif field.default_factory is not None:
            made = field.default_factory()
            default = json.dumps(made.model_dump() if isinstance(made, BaseModel) else made, default=str)
        else:
            default = "(required)"
        kind = getattr(ann, "__name__", None) or str(ann).replace("typing.", "")
        rows.append((prefix + name, kind, default))
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m open_transformers_b200.config.describe", description=__doc__.split("\n\n")[1])
    ap.add_argument("--config-name")
    ap.add_argument("overrides", nargs="*")
    from ..cli._args import parse_with_overrides

    a = parse_with_overrides(ap, argv)
    if a.config_name:
        import yaml

        from .load import load_config

        print(yaml.safe_dump(json.loads(load_config(a.config_name, a.overrides).model_dump_json()), sort_keys=False), end="")
        return 0
    width = max(len(k) for k, _, _ in schema_rows())
    for key, kind, default in schema_rows():
        print("%-*s  %-28s %s" % (width, key, kind, default))
    return 0


if __name__ == "__main__":
    sys.exit(main())
