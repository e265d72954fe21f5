"""Minimal stand-in for `hydra-core`: the subset of config composition the reference uses (config/load.py:55-70).

Supported: a config directory of YAML groups; a primary config with `# @package _global_` and a `defaults:`
list of `/group: name` entries and `_self_`; dotted `key=value`, `+key=value` and `++key=value` overrides with
YAML-parsed values; `group=name` overrides that swap a defaults entry. Interpolations are not supported (the
reference's config tree has none).
"""
import contextlib
from pathlib import Path
from typing import Any

import yaml

from hydra.core.global_hydra import GlobalHydra
from omegaconf import DictConfig


@contextlib.contextmanager
def initialize_config_dir(config_dir: str, version_base: Any = None, job_name: str = "app"):
    GlobalHydra.instance().config_dir = Path(config_dir)
    try:
        yield
    finally:
        GlobalHydra.instance().clear()


def _load(path: Path) -> dict:
    if not path.is_file():
        raise FileNotFoundError("config not found: %s" % path)
    return yaml.safe_load(path.read_text(encoding="utf-8")) or {}


def _merge(dst: dict, src: dict) -> dict:
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _merge(dst[k], v)
        else:
            dst[k] = v
    return dst


def _set(cfg: dict, dotted: str, value: Any, must_exist: bool) -> None:
    parts = dotted.split(".")
    node = cfg
    for p in parts[:-1]:
        if not isinstance(node.get(p), dict):
            if must_exist:
                raise KeyError("override of unknown key %r (use +key=value to add)" % dotted)
            node[p] = {}
        node = node[p]
    if must_exist and parts[-1] not in node:
        raise KeyError("override of unknown key %r (use +key=value to add)" % dotted)
    node[parts[-1]] = value


def compose(config_name: str, overrides: list | None = None) -> DictConfig:
    cdir = GlobalHydra.instance().config_dir
    if cdir is None:
        raise RuntimeError("compose() outside initialize_config_dir()")
    primary = _load(cdir / (config_name + ".yaml"))
    defaults = primary.pop("defaults", [])
    value_overrides = []
    group_choice = {}
    for ov in overrides or []:
        key, _, raw = ov.partition("=")
        bare = key.lstrip("+").lstrip("/")
        if "." not in bare and (cdir / bare).is_dir() and (cdir / bare / (raw + ".yaml")).is_file():
            group_choice[bare] = raw
        else:
            value_overrides.append((key, raw))
    cfg: dict = {}
    seen_self = False
    for entry in defaults:
        if entry == "_self_":
            _merge(cfg, primary)
            seen_self = True
            continue
        if isinstance(entry, dict):
            for group, name in entry.items():
                group = str(group).lstrip("/")
                name = group_choice.get(group, name)
                _merge(cfg, {group.split("/")[-1]: _load(cdir / group / (str(name) + ".yaml"))})
        else:
            _merge(cfg, _load(cdir / (str(entry) + ".yaml")))
    if not seen_self:
        _merge(cfg, primary)
    for key, raw in value_overrides:
        add = key.startswith("+")
        _set(cfg, key.lstrip("+"), yaml.safe_load(raw), must_exist=not add)
    return DictConfig(cfg)
