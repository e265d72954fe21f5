"""Config composition: the subset of Hydra that the recipe tree uses, implemented here because
neither hydra-core nor omegaconf is a dependency of this framework.

Supported: ``# @package _global_`` train files; a ``defaults:`` list of ``/group: name`` entries
and ``_self_``; nested-dict deep merge in defaults order; command-line overrides ``a.b=c``
(key must exist), ``+a.b=c`` (key must not exist), ``++a.b=c`` (either), values parsed as YAML
scalars (so ``400_000_000_000``, ``1e-4``, ``[0.9,0.95]``, ``true``, ``null`` work).

API parity: ``load_config`` / ``resolve_to_typed`` / ``parse_config_resolved``
(reference src/pretrain/config/load.py:44-118).
"""
from __future__ import annotations

import copy
import json
import os
import re
from pathlib import Path
from typing import Any, Iterable

import yaml

from .schema import RootConfig

GROUPS = ("model", "data", "optim", "schedule", "run", "train")

# Keys that older checkpoints' embedded configs may still carry; dropped on read so that an
# old meta.json keeps parsing after a field is retired (dotted paths).
RETIRED_CONFIG_KEYS: tuple[str, ...] = (
    "train.clip_algo",
    "train.per_tensor_clip",
    "run.replicate_reduce_algo",
    "optim.amsgrad",
)


class _Loader(yaml.SafeLoader):
    pass


# YAML 1.1 (PyYAML) does not read "1e-4" or "3.0e-4" without a sign in the exponent as floats and
# keeps "400_000" an int already; add the missing float form.
_Loader.add_implicit_resolver(
    "tag:yaml.org,2002:float",
    re.compile(r"""^(?:[-+]?(?:[0-9][0-9_]*)\.[0-9_]*(?:[eE][-+]?[0-9]+)?
                   |[-+]?(?:[0-9][0-9_]*)(?:[eE][-+]?[0-9]+)
                   |\.[0-9_]+(?:[eE][-+]?[0-9]+)?
                   |[-+]?\.(?:inf|Inf|INF)|\.(?:nan|NaN|NAN))$""", re.X),
    list("-+0123456789."),
)


def _yaml_load(text: str) -> Any:
    return yaml.load(text, Loader=_Loader)


def default_configs_dir() -> Path:
    """``$PRETRAIN_CONFIGS`` if set, else the tree shipped inside the package."""
    env = os.environ.get("PRETRAIN_CONFIGS")
    if env:
        p = Path(env)
        if not p.is_dir():
            raise FileNotFoundError("PRETRAIN_CONFIGS=%s is not a directory" % env)
        return p
    return Path(__file__).resolve().parent.parent / "configs"


def _deep_merge(dst: dict, src: dict) -> dict:
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _deep_merge(dst[k], v)
        else:
            dst[k] = copy.deepcopy(v)
    return dst


def _read(path: Path) -> dict:
    if not path.is_file():
        raise FileNotFoundError("config file not found: %s" % path)
    data = _yaml_load(path.read_text()) or {}
    if not isinstance(data, dict):
        raise ValueError("%s: top level must be a mapping" % path)
    return data


def _apply_override(cfg: dict, item: str) -> None:
    m = re.match(r"^(\+\+|\+|~)?([A-Za-z0-9_.\-]+)(?:=(.*))?$", item, re.S)
    if not m:
        raise ValueError("cannot parse override %r" % item)
    mode, dotted, raw = m.group(1) or "", m.group(2), m.group(3)
    keys = dotted.split(".")
    node = cfg
    for k in keys[:-1]:
        if k not in node or not isinstance(node[k], dict):
            if mode in ("+", "++"):
                node[k] = {}
            else:
                raise KeyError("override %r: no such config group %r (use ++ to add)" % (item, k))
        node = node[k]
    leaf = keys[-1]
    if mode == "~":
        node.pop(leaf, None)
        return
    if raw is None:
        raise ValueError("override %r needs a value" % item)
    exists = leaf in node
    if mode == "" and not exists:
        raise KeyError("override %r: key does not exist (use + or ++ to add)" % item)
    if mode == "+" and exists:
        raise KeyError("override %r: key already exists (use ++ to force)" % item)
    node[leaf] = _yaml_load(raw) if raw != "" else ""


def compose(name: str, overrides: Iterable[str] = (), configs_dir: str | os.PathLike | None = None) -> dict:
    """Compose ``train/<name>.yaml`` with its defaults list and overrides into a plain dict."""
    root = Path(configs_dir) if configs_dir else default_configs_dir()
    main = _read(root / "train" / ("%s.yaml" % name))
    defaults = main.pop("defaults", ["_self_"])
    overrides = list(overrides)
    # group re-selection from the command line: "model=llama3_100m_smoke_repop"
    group_choice: dict[str, str] = {}
    rest: list[str] = []
    for ov in overrides:
        m = re.match(r"^/?([a-z_]+)=([A-Za-z0-9_\-]+)$", ov)
        if m and m.group(1) in GROUPS and m.group(1) != "train" and (root / m.group(1) / (m.group(2) + ".yaml")).is_file():
            group_choice[m.group(1)] = m.group(2)
        else:
            rest.append(ov)
    out: dict = {}
    saw_self = False
    for entry in defaults:
        if entry == "_self_":
            _deep_merge(out, main)
            saw_self = True
            continue
        if not isinstance(entry, dict) or len(entry) != 1:
            raise ValueError("unsupported defaults entry %r" % (entry,))
        (group, choice), = entry.items()
        group = group.lstrip("/")
        choice = group_choice.get(group, choice)
        if choice is None:
            continue
        _deep_merge(out, {group: _read(root / group / ("%s.yaml" % choice))})
    if not saw_self:
        _deep_merge(out, main)
    for ov in rest:
        _apply_override(out, ov)
    return out


def resolve_to_typed(cfg: dict) -> RootConfig:
    return RootConfig.model_validate(cfg)


def load_config(name: str, overrides: Iterable[str] = (), configs_dir: str | os.PathLike | None = None) -> RootConfig:
    return resolve_to_typed(compose(name, overrides, configs_dir))


def _drop_retired(cfg: dict) -> dict:
    cfg = copy.deepcopy(cfg)
    for dotted in RETIRED_CONFIG_KEYS:
        node = cfg
        keys = dotted.split(".")
        for k in keys[:-1]:
            node = node.get(k) if isinstance(node, dict) else None
            if node is None:
                break
        if isinstance(node, dict):
            node.pop(keys[-1], None)
    return cfg


def parse_config_resolved(blob: str | dict) -> RootConfig:
    """Parse the resolved-config JSON stored in a checkpoint's ``meta.json``."""
    cfg = json.loads(blob) if isinstance(blob, str) else blob
    return resolve_to_typed(_drop_retired(cfg))
