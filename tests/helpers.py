import os
import socket
import tempfile

import torch


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def tiny_cfg(tmp, extra=()):
    from open_transformers_b200.config import load_config
    from open_transformers_b200.data.synthetic import ensure_synthetic_sources

    cfg = load_config("tiny_cpu", ["run.output_dir=%s/runs" % tmp, "run.run_id=t", "model.n_layers=1", "model.d_model=128", "model.n_heads=2",
                                   "model.n_kv_heads=2", "model.ffn_intermediate=256", "model.vocab_size=256", "train.seq_len=64", "data.seq_len=64",
                                   "model.max_seq_len_pretrain=64", "train.micro_batch_size=2", "train.global_batch_tokens.warmup=256",
                                   "train.global_batch_tokens.main=256", "train.global_batch_tokens.late=256", "train.total_tokens=768", *extra])
    ensure_synthetic_sources(cfg, tmp, 20000)
    return cfg
