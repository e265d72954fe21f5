"""String -> class registries; duplicate or unknown names fail loudly
(reference src/pretrain/util/registry.py:15-49)."""
from __future__ import annotations


class Registry:
    def __init__(self, kind: str):
        self.kind = kind
        self._items: dict[str, type] = {}

    def register(self, name: str):
        def deco(cls):
            if name in self._items:
                raise KeyError("%s %r registered twice" % (self.kind, name))
            self._items[name] = cls
            return cls
        return deco

    def get(self, name: str):
        if name not in self._items:
            raise KeyError("unknown %s %r; known: %s" % (self.kind, name, ", ".join(sorted(self._items))))
        return self._items[name]

    def names(self):
        return sorted(self._items)
