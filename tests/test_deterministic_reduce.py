"""The deterministic gradient reduction against a plain restatement of its rule, bit for bit: per replica the shard
gradients are added in ascending shard order and scaled by 1/S; the replica values are combined by the binary-blocks
tree (power-of-two blocks, largest first, balanced pair tree inside, block sums left to right) and scaled by 1/R. Replica counts 1..9 (powers of two and not), element counts that end
inside a chunk, and the association itself checked symbolically.
(reference test strategy: tests/distributed/test_deterministic_reduce.py:56-185, tests/test_binary_blocks_tree.py:56-70)"""
import ctypes

import numpy as np
import pytest
import torch

from open_transformers_b200.ops.native import I, P, cpu_lib
from open_transformers_b200.train.engine import _ptr_array

CHUNK = 8192


def pair_tree(values, add):
    v = list(values)
    s = 1
    while s < len(v):
        for i in range(0, len(v) - s, 2 * s):
            v[i] = add(v[i], v[i + s])
        s *= 2
    return v[0]


def blocks_tree(values, add):
    v, total, at = list(values), None, 0
    bit = 1 << (len(v).bit_length() - 1)
    while bit:
        if len(v) & bit:
            level = v[at:at + bit]
            at += bit
            while len(level) > 1:
                level = [add(level[i], level[i + 1]) for i in range(0, len(level), 2)]
            total = level[0] if total is None else add(total, level[0])
        bit >>= 1
    return total


def spec(grads, S, R):
    f = np.float32
    reps = []
    for r in range(R):
        acc = grads[r * S].copy()
        for s in range(1, S):
            acc = (acc + grads[r * S + s]).astype(f)
        reps.append((acc * f(1.0 / S)).astype(f))
    return (blocks_tree(reps, lambda a, b: (a + b).astype(f)) * f(1.0 / R)).astype(f)


def native_reduce(grads, S, R, n):
    starts = np.arange(0, n, CHUNK, dtype=np.int64)
    lens = np.minimum(CHUNK, n - starts).astype(np.int32)
    ts = [torch.from_numpy(g) for g in grads]
    out, sos = torch.empty(n), torch.empty(len(starts))
    cs, cl = torch.from_numpy(starts), torch.from_numpy(lens)
    rc = cpu_lib().otb_cpu_grad_reduce(_ptr_array([t.data_ptr() for t in ts]), I(S), I(R), P(cs), P(cl), I(len(starts)), P(out), P(sos))
    assert rc == 0
    return out.numpy(), sos.numpy()


@pytest.mark.parametrize("n", [1, 7, 257, 4097, 2 * CHUNK + 5])
@pytest.mark.parametrize("S,R", [(1, 1), (2, 1), (4, 1), (1, 2), (3, 2), (2, 3), (1, 5), (2, 6), (1, 7), (4, 8), (1, 9), (1, 11), (2, 13), (1, 15),
                                 (1, 16)])
def test_reduction_equals_the_stated_rule_bit_for_bit(S, R, n):
    rng = np.random.default_rng(1000 * S + 10 * R + n)
    grads = [(rng.standard_normal(n) * 10.0 ** rng.integers(-3, 3)).astype(np.float32) for _ in range(S * R)]
    got, sos = native_reduce(grads, S, R, n)
    want = spec(grads, S, R)
    assert got.tobytes() == want.tobytes()
    # the squared-norm partials describe the reduced gradient
    assert abs(float(sos.astype(np.float64).sum()) - float((want.astype(np.float64) ** 2).sum())) <= 1e-5 * float((want.astype(np.float64) ** 2).sum()) + 1e-30


def test_order_matters_so_the_rule_is_really_pinned():
    """a permutation of the shard gradients changes bits somewhere (otherwise the test above would prove nothing)"""
    rng = np.random.default_rng(5)
    n, S, R = 4097, 4, 3
    grads = [(rng.standard_normal(n) * 10.0 ** rng.integers(-3, 3)).astype(np.float32) for _ in range(S * R)]
    a, _ = native_reduce(grads, S, R, n)
    b, _ = native_reduce(grads[::-1], S, R, n)
    assert a.tobytes() != b.tobytes() and np.allclose(a, b, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("n,want", [
    (1, "0"), (2, "(0+1)"), (3, "((0+1)+2)"), (4, "((0+1)+(2+3))"), (5, "(((0+1)+(2+3))+4)"), (6, "(((0+1)+(2+3))+(4+5))"),
    (7, "(((0+1)+(2+3))+((4+5)+6))"), (8, "(((0+1)+(2+3))+((4+5)+(6+7)))"), (9, "((((0+1)+(2+3))+((4+5)+(6+7)))+8)")])
def test_pair_tree_parenthesisation(n, want):
    assert pair_tree([str(i) for i in range(n)], lambda a, b: "(%s+%s)" % (a, b)) == want


def test_every_aligned_power_of_two_range_is_a_subtree():
    """what lets token and K ranges be split over ranks without changing a bit"""
    whole = pair_tree([str(i) for i in range(16)], lambda a, b: "(%s+%s)" % (a, b))
    for size in (2, 4, 8):
        for lo in range(0, 16, size):
            sub = pair_tree([str(i) for i in range(lo, lo + size)], lambda a, b: "(%s+%s)" % (a, b))
            assert sub in whole


def test_reduction_under_the_backward_pass_gives_the_one_shot_bytes(tmp_path, monkeypatch):
    """The bucketed reduction (head, blocks last to first, embedding; started from marks in the backward pass of the
    step's last micro-batch) writes the same reduced gradient, chunk partials, norm and state hash as the reduction that
    runs once after the backward pass. On the CPU the buckets run synchronously inside the hooks, which exercises the
    bucket plan (every owned chunk in exactly one bucket), the stale-buffer rules and the call order."""
    from helpers import tiny_cfg
    from open_transformers_b200.train.engine import TrainEngine

    cfg = tiny_cfg(str(tmp_path), ["model.n_layers=3"])
    g = torch.Generator().manual_seed(11)
    data = [[(torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g), torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g))
             for _ in range(4)] for _ in range(3)]

    def run(mode: str, accum: int):
        monkeypatch.setenv("OTB_REDUCE_OVERLAP", mode)
        eng = TrainEngine(cfg, "cpu")
        assert (eng._ov is not None) == (mode == "1")
        if eng._ov is not None:
            plan = sorted(int(c) for ids in eng._ov["ids"] for c in ids.tolist())
            assert plan == list(range(eng.chunk_lo, eng.chunk_hi))  # every owned chunk in exactly one bucket
        out, prev = [], None
        for step in range(3):
            eng.zero_grads()
            n = 0
            for v in range(eng.V):
                for k in range(accum):
                    ids, lab = data[step][(v * accum + k) % 4]
                    n += 1
                    eng.forward_backward(v, ids, lab, accum, last=n == eng.V * accum)
            norm = eng.reduce_gradients()
            red, sos = eng.grad_red.clone(), eng.chunk_sos.clone()
            eng.optimizer_step(1e-3, eng.clip_coefficient(norm, 1.0))
            prev = eng.sharded_state_hash(prev, None)
            out.append((norm, red, sos, prev))
        launched = None if eng._ov is None else eng._ov["epoch"]
        eng.close()
        return out, launched

    for accum in (1, 2):
        plain, _ = run("0", accum)
        over, epochs = run("1", accum)
        # which parameters never get a gradient is learnt from the first backward pass into a stale buffer (virtual rank
        # 0's, here), so already the first step's last micro-batch reduces under its backward pass
        assert epochs == 3
        for (n0, r0, s0, h0), (n1, r1, s1, h1) in zip(plain, over):
            assert n0 == n1 and torch.equal(r0, r1) and torch.equal(s0, s1) and h0 == h1


# ---- the whole-tensor statement of the same orders (parallel/deterministic_reduce.py)

def test_whole_tensor_fold_equals_the_kernel_twin_bit_for_bit():
    from open_transformers_b200.parallel import deterministic_reduce as DR

    for S, R in [(1, 1), (3, 2), (2, 3), (1, 5), (2, 6), (1, 7), (4, 8), (1, 9), (1, 11), (2, 13)]:
        rng = np.random.default_rng(77 * S + R)
        n = CHUNK + 37
        grads = [(rng.standard_normal(n) * 10.0 ** rng.integers(-3, 3)).astype(np.float32) for _ in range(S * R)]
        got, _ = native_reduce(grads, S, R, n)
        want = DR.fold_virtual_ranks([torch.from_numpy(g) for g in grads], S, R).numpy()
        assert got.tobytes() == want.tobytes(), (S, R)


def test_pair_tree_and_binary_blocks_agree_up_to_two_blocks_and_not_beyond():
    # the reference pins the same strings for its tree_reduce_sum (tests/test_binary_blocks_tree.py:56-70)
    from open_transformers_b200.parallel import deterministic_reduce as DR

    class Sym:
        def __init__(self, s):
            self.s = s

        def __add__(self, o):
            return Sym("(%s+%s)" % (self.s, o.s))

    assert DR.binary_blocks(6) == [4, 2] and DR.binary_blocks(7) == [4, 2, 1] and DR.binary_blocks(8) == [8] and DR.binary_blocks(1) == [1]
    for n in range(1, 17):
        a = DR.pair_tree_sum([Sym(str(i)) for i in range(n)]).s
        b = DR.tree_reduce_sum([Sym(str(i)) for i in range(n)]).s
        assert a == pair_tree([str(i) for i in range(n)], lambda x, y: "(%s+%s)" % (x, y))
        assert b == blocks_tree([str(i) for i in range(n)], lambda x, y: "(%s+%s)" % (x, y))
        assert (a == b) == (bin(n).count("1") <= 2), (n, a, b)
    assert DR.tree_reduce_sum([Sym(str(i)) for i in range(6)]).s == "(((0+1)+(2+3))+(4+5))"
    assert DR.tree_reduce_sum([Sym(str(i)) for i in range(7)]).s == "((((0+1)+(2+3))+(4+5))+6)"
    with pytest.raises(ValueError):
        DR.tree_reduce_sum([])


def test_shard0_helpers():
    from open_transformers_b200.parallel import deterministic_reduce as DR

    t = torch.arange(10 * 3, dtype=torch.float32).view(10, 3)
    assert DR.shard0_full_chunk_size(10, 4) == 3 and DR.shard0_full_chunk_size(8, 4) == 2 and DR.shard0_full_chunk_size(3, 1) == 3
    parts = [DR.shard0_logical_chunk(t, r, 4) for r in range(4)]
    assert [p.shape[0] for p in parts] == [3, 3, 3, 1] and torch.equal(torch.cat(parts), t)
    padded = [DR.shard0_chunk(t, r, 4) for r in range(4)]
    assert all(p.shape == (3, 3) for p in padded) and torch.equal(padded[3][0], t[9]) and float(padded[3][1:].abs().sum()) == 0.0
    # more shards than rows: the trailing shards are empty / all padding
    assert DR.shard0_logical_chunk(t[:2], 3, 4).shape[0] == 0 and DR.shard0_chunk(t[:2], 3, 4).shape == (1, 3)


# ---- telemetry scalars: one fp64 fold in rank order, the same on every rank (gloo ranks on the CPU)

def _scalar_fold_worker(rank, world, init_file, out_dir):
    import json
    import os

    import torch.distributed as dist

    from open_transformers_b200.train.loop import deterministic_scalar_sum, deterministic_scalar_sums

    dist.init_process_group("gloo", init_method="file://" + init_file, rank=rank, world_size=world)
    try:
        # values whose fp64 sum depends on the order: 1e16 + 1 - 1e16 is 0 or 1 depending on the grouping
        mine = [[1e16, 0.25], [1.0], [-1e16, 3.0, 0.5]][rank]
        total, n = deterministic_scalar_sum(mine, world)
        both = deterministic_scalar_sums({"a": mine, "b": [float(rank)] * (rank + 1)}, world)
        with open(os.path.join(out_dir, "rank%d.json" % rank), "w") as f:
            json.dump({"total": total.hex(), "n": n, "a": both["a"][0].hex(), "b": list(both["b"])}, f)
    finally:
        dist.destroy_process_group()


def test_scalar_fold_is_the_rank_ordered_fp64_sum_on_every_rank(tmp_path):
    import json

    import torch.multiprocessing as mp

    world = 3
    mp.spawn(_scalar_fold_worker, args=(world, str(tmp_path / "init"), str(tmp_path)), nprocs=world, join=True)
    want = 0.0
    for v in [1e16, 0.25, 1.0, -1e16, 3.0, 0.5]:
        want += v
    rows = [json.loads((tmp_path / ("rank%d.json" % r)).read_text()) for r in range(world)]
    assert all(r == rows[0] for r in rows)
    assert rows[0]["total"] == want.hex() == rows[0]["a"] and rows[0]["n"] == 6 and rows[0]["b"] == [0.0 + 1.0 + 1.0 + 2.0 + 2.0 + 2.0, 6]
    assert want != sum(sorted([1e16, 0.25, 1.0, -1e16, 3.0, 0.5]))       # another order gives another value: the order is what is pinned
