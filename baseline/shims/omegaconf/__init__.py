"""Minimal stand-in for `omegaconf`: the reference only calls `OmegaConf.to_container` on the composed
config (config/load.py:82), and the composer in the `hydra` stand-in already returns plain containers."""
from typing import Any


class DictConfig(dict):
    """A plain dict that the reference recognises as a config node (it probes `to_container`)."""

    def to_container(self) -> dict:
        return _plain(self)


def _plain(node: Any) -> Any:
    if isinstance(node, dict):
        return {k: _plain(v) for k, v in node.items()}
    if isinstance(node, (list, tuple)):
        return [_plain(v) for v in node]
    return node


class OmegaConf:
    @staticmethod
    def to_container(cfg: Any, resolve: bool = True, throw_on_missing: bool = False) -> Any:
        out = _plain(cfg)
        if throw_on_missing:
            _check_missing(out, "")
        return out

    @staticmethod
    def create(obj: Any = None) -> DictConfig:
        return DictConfig(obj or {})


def _check_missing(node: Any, path: str) -> None:
    if isinstance(node, dict):
        for k, v in node.items():
            _check_missing(v, "%s.%s" % (path, k) if path else str(k))
    elif isinstance(node, list):
        for i, v in enumerate(node):
            _check_missing(v, "%s[%d]" % (path, i))
    elif node == "???":
        raise ValueError("missing mandatory value: " + path)
