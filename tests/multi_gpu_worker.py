"""Worker for the multi-GPU equivalence test: trains a small bf16 decoder for a few steps on WORLD_SIZE GPUs with a
fixed virtual topology and writes the chained state hashes (rank 0) to the path in OTB_TEST_OUT."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from open_transformers_b200.config import load_config
from open_transformers_b200.ops.functional import kernel_status
from open_transformers_b200.train.engine import TrainEngine


def main():
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    V, T, vocab = 4, 256, 4096
    cfg = load_config("open1b_b200", ["model.n_layers=2", "model.vocab_size=%d" % vocab, "train.seq_len=%d" % T, "data.seq_len=%d" % T,
                                      "run.virtual_dp_size=%d" % V, "run.dp_shard_size=%d" % int(os.environ.get("OTB_TEST_SHARD", "4")),
                                      "run.dp_replicate_size=%d" % (V // int(os.environ.get("OTB_TEST_SHARD", "4")))])
    eng = TrainEngine(cfg, dev, rank, world)
    prev, out = None, []
    for step in range(3):
        eng.zero_grads()
        for vi, v in enumerate(eng.hosted):
            g = torch.Generator().manual_seed(1000 * step + v)     # the batch depends on (step, virtual rank) only
            ids = torch.randint(0, vocab, (2, T), generator=g).to(dev)
            lab = torch.randint(0, vocab, (2, T), generator=g).to(dev)
            eng.forward_backward(vi, ids, lab, 1, last=vi == len(eng.hosted) - 1)  # the reduction runs under this backward pass
        norm = eng.reduce_gradients()
        eng.optimizer_step(3e-4, eng.clip_coefficient(norm, 1.0))
        prev = eng.sharded_state_hash(prev, None, tensor_digest="tree")
        out.append([norm, prev])
    status = kernel_status(dev)
    if rank == 0:
        json.dump({"hashes": out, "status": status, "overlapped_steps": 0 if eng._ov is None else eng._ov["epoch"], "resident": eng.resident_bytes(),
                   "packed_state": bool(eng._packed_state),
                   "gather_calls": 0 if eng._pg is None else sum(g.calls for g in eng._pg["weights"])}, open(os.environ["OTB_TEST_OUT"], "w"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
