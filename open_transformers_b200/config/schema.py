"""Typed configuration tree (pydantic, unknown keys rejected).

Field set and validation rules follow the reference's ``RootConfig``
(src/pretrain/config/schema.py:17-568) so that its YAML recipes parse unchanged; the
additions are the B200-specific knobs:

* ``run.virtual_dp_size`` - the canonical virtual data-parallel world size V recorded in every
  checkpoint. The hashed arithmetic depends on (V, dp_shard, dp_replicate) only, never on the
  number of physical GPUs: a GPU hosts V / G virtual ranks and steps through them in order.
* ``run.tp_size`` - tensor-parallel group size (fused all-gather->GEMM / GEMM->reduce-scatter).
* ``train.state_hash.tensor_digest`` - ``raw`` feeds tensor bytes straight into the blake2b
  stream (reference wire format); ``tree`` feeds a 32-byte blake2b tree digest of the bytes,
  which a GPU computes in parallel.
"""
from __future__ import annotations

from typing import Literal

from pydantic import BaseModel, ConfigDict, Field, model_validator

FLASH_BLOCK = 32


class _Strict(BaseModel):
    model_config = ConfigDict(extra="forbid")


class InitConfig(_Strict):
    std: float = 0.02


class ZLossConfig(_Strict):
    enabled: bool = True
    coeff: float = Field(1.0e-5, ge=0.0)


class ModuleSelection(_Strict):
    attention: str = "gqa_qknorm_repop"
    ffn: str = "swiglu_repop"
    norm: str = "rmsnorm_repop"
    rope: str = "rope_default"
    embedding: str = "untied_repop"


class QATConfig(_Strict):
    enabled: bool = False
    method: Literal["lsq", "absmax"] = "lsq"
    weight_bits: int = Field(8, ge=2, le=8)   # the int8 tensor-core path carries any symmetric grid up to 8 bits
    act_bits: int = Field(8, ge=2, le=8)
    per_channel_w: bool = True
    exempt_first_n_blocks: int = 0
    scale_refresh_every_n_steps: int = 0
    enable_at_step: int = 0
    ste_bwd_hadamard: bool = False  # run both straight-through backward GEMMs as Hadamard-rotated int8 products

    @model_validator(mode="after")
    def _check(self):
        for key in ("enable_at_step", "scale_refresh_every_n_steps", "exempt_first_n_blocks"):
            if getattr(self, key) < 0:
                raise ValueError("qat.%s must be >= 0, got %d" % (key, getattr(self, key)))
        return self


class ModelConfig(_Strict):
    name: str
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn_intermediate: int
    vocab_size: int
    max_seq_len_pretrain: int
    rope_theta: float = 500_000.0
    rms_norm_eps: float = 1.0e-5
    qk_norm: bool = True
    qk_norm_gain: bool = True
    swa_window: int = 512
    swa_full_every: int = 5
    attn_int8_pv: bool = True
    emb_norm: bool = False
    init: InitConfig = Field(default_factory=InitConfig)
    z_loss: ZLossConfig = Field(default_factory=ZLossConfig)
    modules: ModuleSelection = Field(default_factory=ModuleSelection)
    qat: QATConfig = Field(default_factory=QATConfig)

    @model_validator(mode="after")
    def _check(self):
        if self.n_heads * self.head_dim != self.d_model:
            raise ValueError("d_model=%d != n_heads*head_dim=%d*%d" % (self.d_model, self.n_heads, self.head_dim))
        if self.n_kv_heads <= 0 or self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads=%d not divisible by n_kv_heads=%d" % (self.n_heads, self.n_kv_heads))
        if self.vocab_size % 128:
            raise ValueError("vocab_size=%d must be a multiple of 128" % self.vocab_size)
        if self.swa_window < 0 or self.swa_window % FLASH_BLOCK:
            raise ValueError("swa_window=%d must be a non-negative multiple of %d" % (self.swa_window, FLASH_BLOCK))
        if self.swa_full_every < 1:
            raise ValueError("swa_full_every=%d must be >= 1" % self.swa_full_every)
        return self

    def layer_window(self, layer: int) -> int:
        """Sliding-window width in keys for ``layer`` (0 = full causal).

        Every ``swa_full_every``-th layer and the last layer are full causal
        (reference src/pretrain/model/modules/attention_repop.py:88-96)."""
        if self.swa_window == 0:
            return 0
        if layer % self.swa_full_every == self.swa_full_every - 1 or layer == self.n_layers - 1:
            return 0
        return self.swa_window


class DataSourceConfig(_Strict):
    name: str
    path: str
    weight: float


class DataConfig(_Strict):
    sources: list[DataSourceConfig]
    seq_len: int = 4096
    document_separator_id: int = 0
    pack_strategy: Literal["concat_eos", "varlen"] = "concat_eos"
    weights_are_token_shares: bool = False

    @model_validator(mode="after")
    def _check(self):
        if not self.sources:
            raise ValueError("data.sources is empty")
        if any(s.weight < 0 for s in self.sources):
            raise ValueError("data source weights must be >= 0")
        if sum(s.weight for s in self.sources) <= 0:
            raise ValueError("data source weights sum to zero")
        return self

    def normalised_weights(self) -> list[float]:
        total = sum(s.weight for s in self.sources)
        return [s.weight / total for s in self.sources]


class OptimConfig(_Strict):
    name: Literal["adamw", "adamw_repop", "muon_hybrid"] = "adamw"
    betas: tuple[float, float] = (0.9, 0.95)
    eps: float = 1.0e-8
    weight_decay: float = 0.1
    fused: bool = True
    no_decay_param_names: list[str] = Field(default_factory=lambda: [".bias", "norm.weight", ".rope_"])
    peak_lr: float = Field(3.0e-4, gt=0.0)

    @model_validator(mode="after")
    def _check(self):
        if not (0.0 <= self.betas[0] < 1.0 and 0.0 <= self.betas[1] < 1.0):
            raise ValueError("optim.betas must lie in [0, 1), got %s" % (self.betas,))
        if self.eps <= 0.0 or self.weight_decay < 0.0:
            raise ValueError("optim.eps must be > 0 and optim.weight_decay >= 0")
        return self


class ScheduleConfig(_Strict):
    name: Literal["cosine", "wsd", "linear_anneal"] = "cosine"
    warmup_steps: int = Field(2000, ge=0)
    min_lr_frac: float = Field(0.10, ge=0.0, le=1.0)
    wsd_decay_start_frac: float = Field(0.90, ge=0.0, le=1.0)
    wsd_decay_to_frac: float = Field(0.10, ge=0.0, le=1.0)
    anneal_start_tokens: int = Field(0, ge=0)
    rewarm_tokens: int = Field(0, ge=0)
    rewarm_on_resume: bool = False


class SpikeConfig(_Strict):
    grad_norm_threshold: float = 5.0
    skip_steps_on_spike: int = 5
    skips_in_window_to_halt: int = 5
    halt_window_steps: int = 100
    start_step: int = 0

    @model_validator(mode="after")
    def _check(self):
        # Skips are at least skip_steps_on_spike apart, so k of them span (k-1)*skip steps; if that
        # does not fit in the window the halt can never trigger and the run would skip forever.
        need = (self.skips_in_window_to_halt - 1) * self.skip_steps_on_spike
        if need > self.halt_window_steps:
            raise ValueError(
                "spike halt unreachable: (skips_in_window_to_halt-1)*skip_steps_on_spike=%d exceeds "
                "halt_window_steps=%d" % (need, self.halt_window_steps))
        return self


class GlobalBatchTokens(_Strict):
    warmup: int = 1_048_576
    main: int = 2_097_152
    late: int = 4_194_304


class StateHashConfig(_Strict):
    every_n_steps: int = 0
    include_grads: bool = True
    include_batch: bool = True
    at_init: bool = True
    tensor_digest: Literal["raw", "tree"] = "raw"

    @model_validator(mode="after")
    def _check(self):
        if self.every_n_steps < 0:
            raise ValueError("state_hash.every_n_steps must be >= 0")
        return self


class GradNormLogConfig(_Strict):
    every_n_steps: int = 0
    path: str = "logs/grad_norms.jsonl"
    top_k: int = 12
    weight_stats_every_n_steps: int = 0

    @model_validator(mode="after")
    def _check(self):
        if self.every_n_steps < 0 or self.weight_stats_every_n_steps < 0:
            raise ValueError("grad_norm_log cadences must be >= 0")
        return self


class TrainConfig(_Strict):
    total_tokens: int = Field(150_000_000_000, ge=1)
    seq_len: int = Field(4096, ge=1)
    micro_batch_size: int = Field(4, ge=1)
    global_batch_tokens: GlobalBatchTokens = Field(default_factory=GlobalBatchTokens)
    warmup_to_main_at_tokens: int = 4_000_000_000
    main_to_late_at_tokens: int = 140_000_000_000
    ckpt_every_tokens: int = 5_000_000_000
    ckpt_every_steps: int = 0
    resume_reset_optimizer: bool = False
    spike: SpikeConfig = Field(default_factory=SpikeConfig)
    grad_clip: float = Field(1.0, ge=0.0)   # 0 disables clipping
    qk_gain_clamp: float = Field(0.0, ge=0.0)
    qk_freeze_q_gains_until_step: int = Field(0, ge=0)
    state_hash: StateHashConfig = Field(default_factory=StateHashConfig)
    grad_norm_log: GradNormLogConfig = Field(default_factory=GradNormLogConfig)
    dead_tensor_assert_steps: int = 0


class LoggingConfig(_Strict):
    wandb_project: str = "pretrain-8b"
    metrics_jsonl_path: str = "logs/metrics.jsonl"


class RunConfig(_Strict):
    run_id: str = ""
    seed: int = 42
    output_dir: str = "runs"
    nproc_per_node: int = 8
    dp_shard_size: int = -1
    dp_replicate_size: int = 1
    parallel: Literal["fsdp", "ddp"] = "fsdp"
    reduction_mode: Literal["nccl", "deterministic_allgather"] = "deterministic_allgather"
    mixed_precision: bool = True
    activation_checkpoint: bool = True
    ac_every_other_block: bool = False
    tokenizer_path: str = ""
    # B200 additions
    virtual_dp_size: int = 0  # 0 = dp_shard * dp_replicate of the launch (one virtual rank per process)
    tp_size: int = 1
    tp_fused: bool = False  # tensor-parallel traffic through the peer-memory GEMM kernels instead of library all-gathers (GPUs)
    heartbeat_timeout_s: float = 0.0  # > 0: host-side failure detection between the processes (parallel/heartbeat.py)
    # With sharded ownership: allocate the AdamW moments and the reduced gradient for the OWNED segments only (12 of the 16
    # state bytes per parameter shrink with the process count; the fp32 master weights stay whole). OTB_STATE_SHARDING=1 too.
    state_sharding: bool = False
    # "gather": the bf16 rows of the projection weights stay with their owner after the update and the first forward GEMM
    # pulls the others' rows over peer memory itself (parallel/param_gather.py); "replicate": the AdamW kernel pushes them
    param_sharding: Literal["replicate", "gather"] = "replicate"

    @model_validator(mode="after")
    def _check(self):
        if self.tp_size < 1 or self.virtual_dp_size < 0:
            raise ValueError("run.tp_size must be >= 1 and run.virtual_dp_size >= 0")
        return self


class RootConfig(_Strict):
    model: ModelConfig
    data: DataConfig
    optim: OptimConfig
    schedule: ScheduleConfig
    train: TrainConfig
    run: RunConfig
    logging: LoggingConfig = Field(default_factory=LoggingConfig)

    @model_validator(mode="after")
    def _check(self):
        if self.data.seq_len != self.train.seq_len:
            raise ValueError("data.seq_len=%d must equal train.seq_len=%d" % (self.data.seq_len, self.train.seq_len))
        if self.data.seq_len > self.model.max_seq_len_pretrain:
            raise ValueError("data.seq_len=%d exceeds model.max_seq_len_pretrain=%d (RoPE tables)"
                             % (self.data.seq_len, self.model.max_seq_len_pretrain))
        return self
