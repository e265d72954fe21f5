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


class HostWorkspace:
    """Stand-in for the peer-memory workspace on CPU ranks: the two fused operations with their documented meaning
    (all-gather -> GEMM; K-split GEMM whose result arrives sharded by token rows), built from gathers."""

    any_device = True

    def __init__(self, rank, P, group=None):
        self.rank, self.P, self.group, self.calls = rank, P, group, []

    def _gather(self, t):
        parts = [torch.empty_like(t.view(torch.uint8)) for _ in range(self.P)]
        dist.all_gather(parts, t.contiguous().view(torch.uint8), group=self.group)
        return [p.view(t.dtype) for p in parts]

    def barrier(self):
        dist.barrier(group=self.group)

    def ag_gemm(self, key, x_shard, w, b_mn=False, out_dtype=torch.bfloat16):
        from open_transformers_b200.ops import functional as K

        self.calls.append(("ag",) + tuple(key[:1]))
        x_full = torch.cat(self._gather(x_shard), 0)
        return K.gemm(x_full, w, b_mn=b_mn), x_full

    def chain_gemm(self, key, a, w, b_mn=False, residual_shard=None):
        from open_transformers_b200.ops import functional as K

        self.calls.append(("chain",) + tuple(key[:1]))
        a_full = torch.cat(self._gather(a), 1)
        w_full = torch.cat(self._gather(w), 0 if b_mn else 1)
        per = a.shape[0] // self.P
        mine = a_full[self.rank * per:(self.rank + 1) * per].contiguous()
        if residual_shard is not None:
            return K.gemm(mine, w_full, b_mn=b_mn, epi=K.EPI_RESIDUAL, residual=residual_shard)
        return K.gemm(mine, w_full, b_mn=b_mn)

    def close(self):
        pass


def main():
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    tp, bf16 = int(os.environ.get("OTB_TEST_TP", "1")), os.environ.get("OTB_TEST_BF16", "0") == "1"
    device = os.environ.get("OTB_TEST_DEVICE", "cpu")
    if device == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        device = "cuda:%d" % int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl" if device.startswith("cuda") else "gloo")
    V, B, T, vocab = int(os.environ.get("OTB_TEST_V", "2")), 2, int(os.environ.get("OTB_TEST_T", "64")), 256
    cfg = load_config("tiny_cpu", ["model.n_layers=2", "model.d_model=128", "model.n_heads=2", "model.n_kv_heads=2", "model.ffn_intermediate=256",
                                   "model.vocab_size=%d" % vocab, "train.seq_len=%d" % T, "data.seq_len=%d" % T, "model.max_seq_len_pretrain=%d" % T,
                                   "run.virtual_dp_size=%d" % V, "run.dp_shard_size=%d" % V, "run.dp_replicate_size=1", "run.tp_size=%d" % tp,
                                   "run.mixed_precision=%s" % ("true" if bf16 else "false")] + os.environ.get("OTB_TEST_EXTRA", "").split())
    eng = TrainEngine(cfg, device, rank, world)
    if os.environ.get("OTB_TEST_HOST_WS") == "1" and tp > 1:
        eng._tp_state.ws = HostWorkspace(eng.tp_rank, eng.tp, eng._tp_group)
    if os.environ.get("OTB_GRAD_TRANSPORT") == "collective" and world > 1:
        assert eng.collective and eng.sharded and not eng.peer and 0 < eng.seg_hi - eng.seg_lo < eng.n_segs
    packed = os.environ.get("OTB_STATE_SHARDING") == "1" and world > 1
    if packed:
        assert eng._packed_state and eng.m1.numel() == eng.grad_red.numel() < eng.layout.total
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
        prev = eng.sharded_state_hash(prev, None, tensor_digest=os.environ.get("OTB_TEST_TD") or ("raw" if not device.startswith("cuda") else "tree"))
        out.append([norm, ces, prev])
    if device.startswith("cuda"):
        from open_transformers_b200.ops.functional import kernel_status

        assert kernel_status(device) == 0, "a bounded wait inside a kernel ran out"
    if os.environ.get("OTB_TEST_HOST_WS") == "1" and tp > 1:
        kinds = {c for c in eng._tp_state.ws.calls}
        assert kinds == {("ag", "col"), ("ag", "row_bwd"), ("chain", "row")}, kinds
    if os.environ.get("OTB_TEST_STATE_OUT"):
        # whole-tensor views of the optimizer state and the reduced gradient (gathered from their owners when sharded)
        st, gr = eng.optimizer_state(), eng.named_grads()
        if rank == 0:
            torch.save({"m1": {n: s["exp_avg"].clone() for n, s in st.items()}, "m2": {n: s["exp_avg_sq"].clone() for n, s in st.items()},
                        "grad": {n: g.clone() for n, g in gr.items()}, "resident": eng.resident_bytes()}, os.environ["OTB_TEST_STATE_OUT"])
    if rank == 0:
        json.dump(out, open(os.environ["OTB_TEST_OUT"], "w"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
