"""Precision policy of a run (reference src/pretrain/model/precision.py:15-61): bf16 compute
weights and activations, fp32 master weights / moments / gradient reduction."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class PrecisionPolicy:
    param_dtype: torch.dtype = torch.bfloat16
    reduce_dtype: torch.dtype = torch.float32
    output_dtype: torch.dtype = torch.bfloat16
    master_dtype: torch.dtype = torch.float32

    @classmethod
    def from_run(cls, mixed_precision: bool) -> "PrecisionPolicy":
        if mixed_precision:
            return cls()
        return cls(torch.float32, torch.float32, torch.float32, torch.float32)
