"""Tensor-level deterministic math: close to the platform's libm (within a unit or two in the last place), identical for
any thread count and any way the tensor is split, canonical sums equal to the flat routine, integer powers by squaring."""
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from open_transformers_b200.ops import elementwise as E
from open_transformers_b200.ops import functional as K


def _ulps(a: torch.Tensor, b: torch.Tensor) -> int:
    ia, ib = a.contiguous().view(torch.int32).to(torch.int64), b.contiguous().view(torch.int32).to(torch.int64)
    return int((ia - ib).abs().max())


def test_maps_track_libm_and_do_not_depend_on_the_split():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(10_000, generator=g) * 5
    pos = x.abs() + 1e-3
    assert _ulps(E.exp(x), torch.exp(x.double()).float()) <= 1
    assert _ulps(E.log(pos), torch.log(pos.double()).float()) <= 1
    assert np.array_equal(E.sqrt(pos).numpy(), np.sqrt(pos.numpy()))       # IEEE square root: exact agreement with a correctly rounded one
    assert _ulps(E.rsqrt(pos), (1.0 / torch.sqrt(pos.double())).float()) <= 2
    assert _ulps(E.sigmoid(x), torch.sigmoid(x.double()).float()) <= 2
    big = torch.rand(10_000, generator=g) * 4096.0                        # RoPE-sized arguments
    assert _ulps(E.sin(big), torch.sin(big.double()).float()) <= 1 and _ulps(E.cos(big), torch.cos(big.double()).float()) <= 1
    for f in (E.exp, E.log, E.sin):
        arg = pos if f is E.log else x
        whole = f(arg)
        assert torch.equal(whole, torch.cat([f(arg[:137]), f(arg[137:])]))
        assert torch.equal(whole.view(100, 100), f(arg.view(100, 100)))
    assert E.exp(x.bfloat16()).dtype == torch.bfloat16


def test_sums_means_and_powers():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(7, 3000, generator=g)
    rows = E.sum_dim(x, -1)
    assert rows.shape == (7,) and all(float(rows[i]) == float(K.det_sum(x[i].contiguous())) for i in range(7))
    assert torch.equal(E.sum_dim(x.t().contiguous(), 0), rows)            # the reduced axis may sit anywhere
    assert torch.allclose(rows, x.double().sum(-1).float(), rtol=1e-5, atol=1e-4)
    assert torch.equal(E.mean_dim(x, -1), E.sum_dim(x, -1, post_scale=1.0 / 3000))
    assert float(E.mean(x)) == float(K.det_sum(x.reshape(-1), False, 1.0 / x.numel()))
    assert torch.equal(E.sum_dim(x, -1, squares=True), torch.stack([K.det_sum(x[i].contiguous(), True) for i in range(7)]).reshape(7))
    b = torch.tensor([0.9, 0.95, 0.999], dtype=torch.float64)

    def by_squaring(v: float, n: int) -> float:       # the same multiplications, in Python doubles
        result, base = 1.0, v
        while n:
            if n & 1:
                result = result * base
            base = base * base
            n >>= 1
        return result

    assert E.pow_int(b, 13).tolist() == [by_squaring(v, 13) for v in b.tolist()]
    assert E.pow_int(b, 1000).tolist() == [by_squaring(v, 1000) for v in b.tolist()]
    assert torch.equal(E.pow_int(b, 0), torch.ones(3, dtype=torch.float64))
    with pytest.raises(ValueError):
        E.pow_int(b, -1)


def test_results_do_not_depend_on_the_thread_count(tmp_path):
    code = ("import torch, sys\n"
            "sys.path.insert(0, %r)\n"
            "from open_transformers_b200.ops import elementwise as E\n"
            "g = torch.Generator().manual_seed(3); x = torch.randn(50000, generator=g) * 3\n"
            "import hashlib\n"
            "h = hashlib.sha256()\n"
            "for t in (E.exp(x), E.sin(x), E.sum_dim(x.view(50, 1000), -1), E.mean(x)): h.update(t.numpy().tobytes())\n"
            "print(h.hexdigest())\n" % os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    outs = [subprocess.run([sys.executable, "-c", code], env=dict(os.environ, OMP_NUM_THREADS=n), capture_output=True, text=True, timeout=300).stdout.strip()
            for n in ("1", "3", "8")]
    assert len(outs[0]) == 64 and outs[0] == outs[1] == outs[2]
