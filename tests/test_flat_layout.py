"""Invariants of the flat parameter layout that the reduction / AdamW / digest kernels rely on, over random parameter
lists: every parameter element belongs to exactly one segment, segments are the FSDP-style ceil split by rows, chunks
never straddle a segment and never exceed 8192 elements, every start is 16-byte aligned, and the ownership ranges of any
process count partition the segments in order."""
import numpy as np
from hypothesis import given, settings, strategies as st

from open_transformers_b200.parallel.flat import ALIGN, CHUNK, FlatLayout, shard_rows

shapes = st.lists(st.one_of(st.tuples(st.integers(1, 40), st.sampled_from([4, 8, 12, 64, 100])),   # matrices: rows x (multiple of 4)
                            st.tuples(st.sampled_from([4, 8, 64, 128, 8200]))),                   # vectors
                  min_size=1, max_size=12)


@settings(max_examples=60, deadline=None)
@given(shapes=shapes, num_shards=st.integers(1, 9), world=st.integers(1, 8))
def test_layout_invariants(shapes, num_shards, world):
    # vectors are split by ELEMENTS (dim 0): keep their shard starts aligned as the engine's parameters do (multiples of 4 per shard)
    named = [("p%d" % i, tuple(s)) for i, s in enumerate(shapes)]
    try:
        lay = FlatLayout.build(named, num_shards, [i % 2 for i in range(len(named))])
    except ValueError as e:                       # a shard boundary inside a vector at an unaligned element is refused, loudly
        assert "unaligned" in str(e)
        return
    covered = np.zeros(lay.total, dtype=np.int32)
    for i, (off, n) in enumerate(zip(lay.offsets, lay.numels)):
        assert off % ALIGN == 0 and (i == 0 or off >= lay.offsets[i - 1] + lay.numels[i - 1])
    for seg in lay.segments:
        shape = lay.shapes[seg.param]
        row = lay.numels[seg.param] // shape[0]
        lo, hi = shard_rows(shape[0], num_shards, seg.shard)
        assert seg.start == lay.offsets[seg.param] + lo * row and seg.length == (hi - lo) * row and seg.length > 0
        assert seg.start % 4 == 0
        covered[seg.start:seg.start + seg.length] += 1
        cs = lay.chunk_start[seg.first_chunk:seg.first_chunk + seg.n_chunks]
        cl = lay.chunk_len[seg.first_chunk:seg.first_chunk + seg.n_chunks]
        assert cs[0] == seg.start and int(cs[-1] + cl[-1]) == seg.start + seg.length
        assert (cl <= CHUNK).all() and (cl[:-1] == CHUNK).all() and (np.diff(cs) == CHUNK).all()
        assert (lay.chunk_group[seg.first_chunk:seg.first_chunk + seg.n_chunks] == lay.groups[seg.param]).all()
    for off, n in zip(lay.offsets, lay.numels):
        assert (covered[off:off + n] == 1).all()          # every element of every parameter: exactly one segment
    assert covered.sum() == sum(lay.numels)               # padding belongs to nobody
    order = [(s.shard, s.param) for s in lay.segments]
    assert order == sorted(order)                          # shard-major
    assert list(lay.seg_first) == [s.first_chunk for s in lay.segments] + [len(lay.chunk_start)]
    ranges = lay.owner_ranges(world)
    nxt = 0
    for lo, hi in ranges:
        if hi > lo:
            assert lo == nxt
            nxt = hi
    assert nxt == len(lay.segments)                        # contiguous runs, in order, nothing left out


def test_shard_rows_is_the_ceil_split_with_empty_tails():
    assert [shard_rows(10, 4, s) for s in range(4)] == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert [shard_rows(3, 8, s) for s in range(8)] == [(0, 1), (1, 2), (2, 3)] + [(3, 3)] * 5
    assert [shard_rows(1, 2, s) for s in range(2)] == [(0, 1), (1, 1)]


def test_rows_per_owner_must_describe_the_distribution():
    from open_transformers_b200.parallel.param_gather import uniform_rows_per_owner

    assert uniform_rows_per_owner([(0, 256), (256, 512), (512, 768), (768, 1024)], 1024) == 256
    assert uniform_rows_per_owner([(0, 26), (26, 52), (52, 78), (78, 100)], 100) == 26          # the last owner takes the rest
    assert uniform_rows_per_owner([(0, 50), (50, 100), (0, 0), (0, 0)], 100) == 50              # fewer rows than owners
    assert uniform_rows_per_owner([(0, 30), (30, 50), (50, 100)], 100) is None
    assert uniform_rows_per_owner([(10, 60), (60, 100)], 100) is None


def test_parallel_dims_vocabulary_over_the_virtual_topology():
    from open_transformers_b200.parallel.parallel_dims import ParallelDims

    d = ParallelDims(2, 4, 8)
    assert d.dp_world_size == 8 and d.dp_replicate_enabled and d.dp_shard_enabled and d.fsdp_enabled and d.dp_enabled
    assert [d.dp_rank(r) for r in range(8)] == list(range(8)) and d.coords(5) == (1, 1) and d.make_dp_gloo_group() is None
    one = ParallelDims(1, 1, 1)
    assert not one.dp_enabled and one.dp_world_size == 1
    tp = ParallelDims(1, -1, 8, tp=4)                       # two tensor-parallel groups of four share two batches
    assert tp.dp_world_size == 2 and tp.dp_shard == 2 and [tp.dp_rank(r) for r in (0, 3, 4, 7)] == [0, 0, 1, 1]
    virt = ParallelDims(2, 4, 2, virtual_dp=8)              # eight virtual ranks on two processes
    assert virt.dp_world_size == 8 and virt.hosted_virtual_ranks(1) == [4, 5, 6, 7]


def test_lazy_zeros_is_zero_writable_and_aligned():
    import torch

    from open_transformers_b200.parallel.flat import lazy_zeros

    big = lazy_zeros(5_000_000, torch.float32, "cpu")          # above the threshold: an anonymous mapping
    assert big.dtype == torch.float32 and big.numel() == 5_000_000 and float(big.abs().sum()) == 0.0 and big.data_ptr() % 4096 == 0
    big[123] = 2.5
    big[-1] = -1.0
    assert float(big.sum()) == 1.5 and big.view(torch.uint8).numel() == 20_000_000
    small = lazy_zeros(10, torch.int32, "cpu")
    assert small.dtype == torch.int32 and int(small.sum()) == 0
    half = lazy_zeros(10_000_000, torch.bfloat16, "cpu")
    assert half.dtype == torch.bfloat16 and float(half.float().abs().sum()) == 0.0
