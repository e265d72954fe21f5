"""Null-object wrapper around Weights & Biases: does nothing when the package is missing, when
``WANDB_MODE=disabled`` or off rank 0 (reference src/pretrain/obs/wandb_run.py:24-58)."""
from __future__ import annotations

import os


class WandBRun:
    def __init__(self, project: str, run_id: str, config: dict | None = None, enabled: bool = True):
        self._run = None
        if not enabled or os.environ.get("WANDB_MODE", "").lower() in ("disabled", "off"):
            return
        if not os.environ.get("WANDB_API_KEY") and os.environ.get("WANDB_MODE", "").lower() != "offline":
            return  # no credentials: stay silent instead of prompting inside a training job
        try:
            import wandb  # type: ignore

            self._run = wandb.init(project=project, name=run_id or None, id=run_id or None, config=config or {}, resume="allow")
        except Exception:
            self._run = None

    def log(self, row: dict, step: int | None = None) -> None:
        if self._run is not None:
            self._run.log(row, step=step)

    def finish(self) -> None:
        if self._run is not None:
            self._run.finish()
            self._run = None
