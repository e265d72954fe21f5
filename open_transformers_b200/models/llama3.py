"""Llama-3 style decoder assembled from the registries (attention / ffn / norm / rope / embedding).

Pre-norm blocks ``x + attn(norm1(x))``, ``x + ffn(norm2(x))`` with both residual adds fused into
the epilogue of the producing GEMM; untied embedding; optional norm on the embedding output;
final norm; vocabulary projection. ``forward`` returns ``ModelOutput(logits, z_loss=None)``;
the loss lives outside (models/fused_loss.py) as in the reference (src/pretrain/model/llama3.py:77-137).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from ..config.schema import ModelConfig
from ..ops import autograd as A
from .registry import ATTENTION, EMBEDDING, FFN, NORM, ROPE
from . import modules as _modules  # noqa: F401  (fills the registries)


@dataclass
class ModelOutput:
    logits: torch.Tensor
    z_loss: torch.Tensor | None = None


class TransformerBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int):
        super().__init__()
        norm = NORM.get(cfg.modules.norm)
        self.layer_idx = layer_idx
        self.norm1 = norm(cfg.d_model, eps=cfg.rms_norm_eps)
        self.attn = ATTENTION.get(cfg.modules.attention)(
            cfg.d_model, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, layer_idx=layer_idx, n_layers=cfg.n_layers,
            swa_window=cfg.swa_window, swa_full_every=cfg.swa_full_every, qk_norm=cfg.qk_norm,
            qk_norm_gain=cfg.qk_norm_gain, eps=cfg.rms_norm_eps, attn_int8_pv=cfg.attn_int8_pv, qat=cfg.qat)
        self.norm2 = norm(cfg.d_model, eps=cfg.rms_norm_eps)
        self.ffn = FFN.get(cfg.modules.ffn)(cfg.d_model, cfg.ffn_intermediate, qat=cfg.qat, layer_idx=layer_idx)

    def forward(self, x, cos, sin):
        x = self.attn(self.norm1(x), cos, sin, residual=x)
        return self.ffn(self.norm2(x), residual=x)


class Llama3(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.cfg = cfg
        self.compute_dtype = torch.float32
        self.embedding = EMBEDDING.get(cfg.modules.embedding)(cfg.vocab_size, cfg.d_model)
        self.emb_norm = NORM.get(cfg.modules.norm)(cfg.d_model, eps=cfg.rms_norm_eps) if cfg.emb_norm else None
        self.rope = ROPE.get(cfg.modules.rope)(cfg.head_dim, cfg.max_seq_len_pretrain, cfg.rope_theta)
        self.blocks = nn.ModuleList(TransformerBlock(cfg, i) for i in range(cfg.n_layers))
        self.norm_out = NORM.get(cfg.modules.norm)(cfg.d_model, eps=cfg.rms_norm_eps)
        self.activation_checkpoint = False
        self.ac_every_other_block = False
        # CPU runs with activation checkpointing: keep each block's attention results for the recomputation
        # (PRETRAIN_CPU_ATTENTION_CHECKPOINT_CACHE=1, or the reference's REPOP_CPU_ATTENTION_CHECKPOINT_CACHE=1)
        import os

        self.cpu_attention_cache = "1" in (os.environ.get("PRETRAIN_CPU_ATTENTION_CHECKPOINT_CACHE"), os.environ.get("REPOP_CPU_ATTENTION_CHECKPOINT_CACHE"))
        # set by the training engine for the last micro-batch of a step: called from the backward pass with a block's
        # index once that block (and everything after it) has produced its weight gradients; -1 = the vocabulary head
        self.bucket_notify = None

    @property
    def lm_head(self) -> nn.Module:
        return self.embedding.output

    def forward_hidden(self, input_ids: torch.Tensor) -> torch.Tensor:
        B, T = input_ids.shape
        cos, sin = self.rope(T)
        st = A.tp()
        if st is not None:
            # tensor parallel: from here to the logits the residual stream is this rank's token rows [B*T / P, d]
            st.batch_shape = (B, T)
            input_ids = input_ids.reshape(-1)[st.rows(B * T)]
        x = self.embedding.encode(input_ids, self.compute_dtype)
        if self.emb_norm is not None:
            x = self.emb_norm(x)
        notify = self.bucket_notify if (torch.is_grad_enabled() and st is None) else None
        for i, blk in enumerate(self.blocks):
            if notify is not None:
                x = A.bucket_mark(x, notify, i)
            if self.activation_checkpoint and self.training and (not self.ac_every_other_block or i % 2 == 0):
                from torch.utils.checkpoint import checkpoint

                extra = {}
                if self.cpu_attention_cache and not x.is_cuda:
                    extra["context_fn"] = A.cpu_attention_checkpoint_contexts
                x = checkpoint(blk, x, cos, sin, use_reentrant=False, preserve_rng_state=False, **extra)
            else:
                x = blk(x, cos, sin)
        x = self.norm_out(x)
        if notify is not None:
            x = A.bucket_mark(x, notify, -1)
        return x

    def forward(self, input_ids: torch.Tensor) -> ModelOutput:
        return ModelOutput(self.embedding.project(self.forward_hidden(input_ids)), None)

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def num_trainable_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad)


def build_model(cfg: ModelConfig, device=None) -> Llama3:
    model = Llama3(cfg)
    if device is not None:
        model = model.to(device)
    return model
