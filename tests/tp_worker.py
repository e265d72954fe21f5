"""Worker of the tensor-parallel kernel test (one process per GPU, started by torchrun): the fused all-gather -> GEMM
and the chained GEMM -> ordered reduction must return exactly the bits of the unsplit GEMM on one GPU."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from open_transformers_b200.ops import functional as K
from open_transformers_b200.parallel.tensor_parallel import TpWorkspace


def main():
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ws = TpWorkspace(dev, rank, world, None, copier_ctas=8)
    res = {}
    for case, (M, N, Kd) in enumerate([(256 * world, 512, 1024), (1024 * world, 384, 256 * world), (2048, 2048, 1408 * world)]):
        g = torch.Generator().manual_seed(100 + case)
        x = torch.randn(M, Kd, generator=g).bfloat16().to(dev)
        w = (torch.randn(N, Kd, generator=g) * 0.05).bfloat16().to(dev)
        r = torch.randn(M, N, generator=g).bfloat16().to(dev)
        rows = ws.shard_rows(M)
        for rep in range(2):  # twice: flags are epoch-numbered, buffers reused
            # column-parallel: every rank owns N/world output columns of the gathered activation
            ncols = slice(rank * (N // world), (rank + 1) * (N // world))
            ws.barrier()
            c, xf = ws.ag_gemm(("ag", case), x[rows].contiguous(), w[ncols].contiguous())
            ok_ag = torch.equal(c, K.gemm(x, w[ncols].contiguous())) and torch.equal(xf, x)
            wt = w[ncols].t().contiguous()  # [K, N/world]: the same product with the weight stored transposed
            ws.barrier()
            c2, _ = ws.ag_gemm(("ag", case), x[rows].contiguous(), wt, b_mn=True)
            ok_ag = ok_ag and torch.equal(c2, c)
            # row-parallel: every rank owns K/world of the reduction
            ks = slice(rank * (Kd // world), (rank + 1) * (Kd // world))
            ws.barrier()
            y = ws.chain_gemm(("ch", case), x[:, ks].contiguous(), w[:, ks].contiguous(), residual_shard=r[rows].contiguous())
            want = K.gemm(x, w, epi=K.EPI_RESIDUAL, residual=r)[rows]
            ok_ch = torch.equal(y, want)
            ws.barrier()
            y2 = ws.chain_gemm(("ch", case), x[:, ks].contiguous(), w[:, ks].t().contiguous(), b_mn=True)
            ok_ch = ok_ch and torch.equal(y2, K.gemm(x, w)[rows])
            res["case%d_rep%d" % (case, rep)] = [bool(ok_ag), bool(ok_ch)]
    torch.cuda.synchronize()
    res["status"] = K.kernel_status(dev)
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        json.dump(allres, open(os.environ["OTB_TEST_OUT"], "w"))
    dist.barrier()
    ws.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
