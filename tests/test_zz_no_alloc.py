"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some users of the native library cannot ask CUDA for memory while they run (a host program that links the
library without PyTorch's allocator; a serving loop that reserved all device memory at start-up), so
``otb_rmsnorm_bwd_noalloc`` keeps its work buffer inside the library. This test checks that it returns the
same bits as the regular entry point, twice in a row (the second call sees the first call's leftovers in the
shared buffer), and that it refuses problems larger than the buffer. The file name makes pytest collect it after
every other test file."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE, BAD_SHAPE = -10, -2
MAX_FLOATS = 4 * 1024 * 1024


def _lib():
    from open_transformers_b200.ops.native import cuda_lib

    lib = cuda_lib()
    fn = lib.otb_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_long, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    return lib, fn


def _reference(lib, dy, x, w, rstd, rows, D):
    """The existing entry point with a caller-allocated work buffer."""
    slabs = (rows + 7) // 8
    part = torch.empty(slabs, D, dtype=torch.float32, device=x.device)
    dx = torch.empty_like(x)
    rc = lib.otb_rmsnorm_bwd(ctypes.c_void_p(dy.data_ptr()), ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                             ctypes.c_void_p(rstd.data_ptr()), ctypes.c_void_p(dx.data_ptr()), ctypes.c_void_p(part.data_ptr()),
                             ctypes.c_long(rows), ctypes.c_int(D), ctypes.c_float(1.0 / D), ctypes.c_int(int(x.dtype == torch.bfloat16)),
                             ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return dx, part[0].clone()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_matches_regular_entry_point_twice(dtype):
    lib, fn = _lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (rows, D) in enumerate([(1003, 2048), (517, 768)]):   # second call: smaller problem over the first one's leftovers
        g = torch.Generator().manual_seed(100 + call)
        x = torch.randn(rows, D, generator=g).to(dtype).to(dev)
        dy = torch.randn(rows, D, generator=g).to(dtype).to(dev)
        w = (1 + 0.1 * torch.randn(D, generator=g)).to(dtype).to(dev)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
        want_dx, want_dg = _reference(lib, dy, x, w, rstd, rows, D)
        dx = torch.empty_like(x)
        dg = torch.full((D,), float("nan"), dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dg.data_ptr(), rows, D, 1.0 / D,
                int(dtype == torch.bfloat16), stream)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(dx, want_dx), "dx differs on call %d" % call
        assert torch.equal(dg, want_dg), "dgamma differs on call %d" % call


def test_noalloc_rejects_oversized_and_bad_shapes():
    lib, fn = _lib()
    null = ctypes.c_void_p(0)
    rows = 8 * (MAX_FLOATS // 2048) + 8          # one slab more than fits at D = 2048
    assert fn(null, null, null, null, null, null, rows, 2048, 1.0 / 2048, 1, null) == TOO_LARGE
    assert fn(null, null, null, null, null, null, 16, 100, 0.01, 1, null) == BAD_SHAPE
    assert fn(null, null, null, null, null, null, 0, 2048, 1.0 / 2048, 1, null) == BAD_SHAPE
