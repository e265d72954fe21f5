"""Worker for the tensor-parallel equivalence test on CPU ranks (gloo): runs a tiny decoder for a few optimizer steps with
``run.tp_size`` = TP (all WORLD_SIZE / TP data-parallel groups share the virtual ranks) and writes, from rank 0, the
gradient norms and chained state hashes to OTB_TEST_OUT. With TP = 1 and one process it produces the baseline."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from open_transformers_b200.config import load_config
from open_transformers_b200.train.engine import TrainEngine


def main():
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    tp, bf16 = int(os.environ.get("OTB_TEST_TP", "1")), os.environ.get("OTB_TEST_BF16", "0") == "1"
    device = os.environ.get("OTB_TEST_DEVICE", "cpu")
    if device == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        device = "cuda:%d" % int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl" if device.startswith("cuda") else "gloo")
    V, B, T, vocab = 2, 2, int(os.environ.get("OTB_TEST_T", "64")), 256
    cfg = load_config("tiny_cpu", ["model.n_layers=2", "model.d_model=128", "model.n_heads=2", "model.n_kv_heads=2", "model.ffn_intermediate=256",
                                   "model.vocab_size=%d" % vocab, "train.seq_len=%d" % T, "data.seq_len=%d" % T, "model.max_seq_len_pretrain=%d" % T,
                                   "run.virtual_dp_size=%d" % V, "run.dp_shard_size=%d" % V, "run.dp_replicate_size=1", "run.tp_size=%d" % tp,
                                   "run.mixed_precision=%s" % ("true" if bf16 else "false")] + os.environ.get("OTB_TEST_EXTRA", "").split())
    eng = TrainEngine(cfg, device, rank, world)
    prev, out = None, []
    for step in range(3):
        eng.zero_grads()
        ces = []
        for k in range(2):                                      # two micro-batches per virtual rank: store, then accumulate
            for vi, v in enumerate(eng.hosted):
                g = torch.Generator().manual_seed(1000 * step + 10 * v + k)
                ids = torch.randint(0, vocab, (B, T), generator=g).to(device)
                lab = torch.randint(0, vocab, (B, T), generator=g).to(device)
                ce, z = eng.forward_backward(vi, ids, lab, 2)
                ces.append(float(ce))
        norm = eng.reduce_gradients()
        eng.optimizer_step(3e-4, eng.clip_coefficient(norm, 1.0))
        prev = eng.sharded_state_hash(prev, None, tensor_digest="raw" if not device.startswith("cuda") else "tree")
        out.append([norm, ces, prev])
    if device.startswith("cuda"):
        from open_transformers_b200.ops.functional import kernel_status

        assert kernel_status(device) == 0, "a bounded wait inside a kernel ran out"
    if rank == 0:
        json.dump(out, open(os.environ["OTB_TEST_OUT"], "w"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
