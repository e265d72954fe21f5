import hashlib
import json

import pytest
import torch

from open_transformers_b200.train import state_hash as SH


def _params():
    g = torch.Generator().manual_seed(0)
    return [("b.weight", torch.randn(6, 4, generator=g)), ("a.weight", torch.randn(5, generator=g))]


def test_v2_wire_format_is_byte_exact():
    params = _params()
    opt = {n: {"step": 3, "exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.ones_like(p)} for n, p in params}
    groups = [{"lr": 1e-3, "params": [0, 1], "betas": (0.9, 0.95)}]
    bd = bytes(range(32))
    got = SH.compute_state_hash(params, opt, groups, prev=None, include_grads=True, grads={"a.weight": None, "b.weight": params[0][1] * 2}, batch_digest=bd)
    h = hashlib.blake2b(digest_size=32)
    h.update(b"pretrain.state_hash.v2\n" + b"prev\0" + b"\0" * 32 + b"params\0")
    for name, p in sorted(params):
        h.update(name.encode() + b"\0")
        h.update(b"weight\0torch.float32\0" + str(tuple(p.shape)).encode() + b"\0" + p.numpy().tobytes())
        h.update(b"optim_step\0" + (3).to_bytes(8, "little", signed=True))
        h.update(b"optim_exp_avg\0torch.float32\0" + str(tuple(p.shape)).encode() + b"\0" + torch.zeros_like(p).numpy().tobytes())
        h.update(b"optim_exp_avg_sq\0torch.float32\0" + str(tuple(p.shape)).encode() + b"\0" + torch.ones_like(p).numpy().tobytes())
        if name == "a.weight":
            h.update(b"grad_none\0")
        else:
            h.update(b"grad\0torch.float32\0(6, 4)\0" + (p * 2).numpy().tobytes())
    h.update(b"param_groups\0" + json.dumps([{"lr": 1e-3, "betas": (0.9, 0.95)}], sort_keys=True, default=str).encode())
    h.update(b"batch_digest\0" + bd)
    assert got == h.hexdigest()


def test_one_ulp_flips_the_hash_and_none_grad_differs_from_zero_grad():
    params = _params()
    base = SH.compute_state_hash(params)
    p2 = [(n, p.clone()) for n, p in params]
    v = p2[0][1].view(torch.int32)
    v[0, 0] += 1
    assert SH.compute_state_hash(p2) != base
    a = SH.compute_state_hash(params, include_grads=True, grads={n: None for n, _ in params})
    b = SH.compute_state_hash(params, include_grads=True, grads={n: torch.zeros_like(p) for n, p in params})
    assert a != b


def test_chaining_and_prev_validation():
    params = _params()
    h1 = SH.compute_state_hash(params)
    assert SH.compute_state_hash(params, prev=h1) != h1
    assert SH.compute_state_hash(params, prev=h1) == SH.compute_state_hash(params, prev=bytes.fromhex(h1))
    # a previous digest of the wrong length is zero-padded or truncated to 32 bytes, as the reference does
    assert SH.compute_state_hash(params, prev=b"short") == SH.compute_state_hash(params, prev=b"short" + b"\0" * 27)
    assert SH.compute_state_hash(params, prev=bytes.fromhex(h1) + b"tail") == SH.compute_state_hash(params, prev=h1)


def test_final_v3_stream_byte_for_byte():
    """The v3 stream against a hand-built one: `param_groups` only with an optimizer, `batch_digest` only when given."""
    import hashlib
    import json

    shard_state, prev, bd = b"\7" * 32, b"\3" * 32, b"\5" * 32
    groups = [{"lr": 0.5, "betas": (0.9, 0.95), "weight_decay": 0.1, "params": [0, 1]}]

    def stream(with_groups, with_batch, with_prev):
        h = hashlib.blake2b(digest_size=32)
        h.update(b"pretrain.state_hash.v3\n")
        h.update(b"prev\0" + (prev if with_prev else b"\0" * 32))
        h.update(b"shard_state\0" + shard_state)
        if with_groups:
            h.update(b"param_groups\0" + json.dumps([{"lr": 0.5, "betas": [0.9, 0.95], "weight_decay": 0.1}], sort_keys=True, default=str).encode())
        if with_batch:
            h.update(b"batch_digest\0" + bd)
        return h.hexdigest()

    assert SH.finalize_state_hash(shard_state, groups, prev, bd) == stream(True, True, True)
    assert SH.finalize_state_hash(shard_state, groups, None, None) == stream(True, False, False)
    assert SH.finalize_state_hash(shard_state, None, prev.hex(), None) == stream(False, False, True)
    with pytest.raises(ValueError):
        SH.finalize_state_hash(shard_state, groups, None, b"short")


def test_sharded_combine_matches_single_process_reconstruction():
    params = _params()
    opt = {n: {"step": 1, "exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.zeros_like(p)} for n, p in params}
    grads = {n: p + 1 for n, p in params}
    for shards, ranks in ((2, 2), (4, 4), (2, 4)):
        locals_ = [SH.local_shard_state_digest(params, opt, grads, shards, s) for s in range(shards)]
        assert SH.combine_shard_state(locals_, ranks) == SH.audit_shard_state_digest(params, opt, grads, shards, ranks)
    # the shard digest covers the LOGICAL rows: 5 rows over 4 shards -> (2, 2, 1, 0)
    assert [SH.shard_rows(5, 4, s) for s in range(4)] == [(0, 2), (2, 4), (4, 5), (5, 5)]
    f = SH.finalize_state_hash(b"\1" * 32, [{"lr": 1.0}], None, None)
    assert len(f) == 64 and f != SH.finalize_state_hash(b"\1" * 32, [{"lr": 2.0}], None, None)


def test_batch_hasher_resume_and_combine():
    b1 = {"input_ids": torch.arange(8).view(2, 4), "labels": torch.arange(8).view(2, 4) + 1}
    b2 = {"input_ids": torch.arange(8).view(2, 4) * 3, "labels": torch.arange(8).view(2, 4)}
    h = SH.RunningBatchHasher()
    h.update(b1)
    mid = h.local_digest()
    h.update(b2)
    r = SH.RunningBatchHasher(mid)
    r.update(b2)
    assert r.local_digest() == h.local_digest() and mid != h.local_digest()
    assert SH.combine_batch_digests([mid]) == mid
    assert SH.combine_batch_digests([mid, h.local_digest()]) == hashlib.blake2b(mid + h.local_digest(), digest_size=32).digest()
    with pytest.raises(ValueError):
        SH.combine_batch_digests([])


def test_tree_digest_definition():
    data = bytes(range(256)) * 100  # 25600 bytes -> 7 leaves -> 224 bytes -> final
    leaves = b"".join(hashlib.blake2b(data[i:i + 4096], digest_size=32).digest() for i in range(0, len(data), 4096))
    want = hashlib.blake2b(leaves + len(data).to_bytes(8, "little"), digest_size=32).digest()
    assert SH.tree_digest_bytes(data) == want
    assert SH.tree_digest_bytes(b"") == hashlib.blake2b((0).to_bytes(8, "little"), digest_size=32).digest()
    t = torch.arange(6400, dtype=torch.float32)
    assert SH.tree_digest_batch([t, t[:10]]) == [SH.tree_digest_tensor(t), SH.tree_digest_tensor(t[:10])]


def test_native_blake2b_is_hashlib_at_every_block_and_leaf_boundary():
    """the C++ compressor behind the tree digests (and its GPU twin's reference) against hashlib, byte for byte
    (reference test strategy: tests/test_native_hash_wire_format.py)"""
    import ctypes

    import numpy as np

    from open_transformers_b200.ops.native import cpu_lib

    lib = cpu_lib()
    rng = np.random.default_rng(0)
    for n in (0, 1, 63, 64, 127, 128, 129, 255, 256, 257, 4095, 4096, 4097, 8191, 8192, 8193, 100_003):
        data = rng.integers(0, 256, n, dtype=np.uint8)
        for outlen in (32, 64):
            out = (ctypes.c_ubyte * outlen)()
            lib.otb_cpu_blake2b(data.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), out, ctypes.c_int(outlen))
            assert bytes(out) == hashlib.blake2b(data.tobytes(), digest_size=outlen).digest(), (n, outlen)
        level = data.tobytes()
        while len(level) > 4096:  # leaves of 4096 bytes -> 32 bytes each, until at most one leaf's worth remains
            level = b"".join(hashlib.blake2b(level[i:i + 4096], digest_size=32).digest() for i in range(0, len(level), 4096))
        assert SH.tree_digest_bytes(data.tobytes()) == hashlib.blake2b(level + n.to_bytes(8, "little"), digest_size=32).digest(), n
    big = rng.integers(0, 256, 4096 * 129 + 5, dtype=np.uint8).tobytes()  # 130 leaves -> 4160 bytes -> a second level
    level = big
    while len(level) > 4096:
        level = b"".join(hashlib.blake2b(level[i:i + 4096], digest_size=32).digest() for i in range(0, len(level), 4096))
    assert SH.tree_digest_bytes(big) == hashlib.blake2b(level + len(big).to_bytes(8, "little"), digest_size=32).digest()


def test_tree_and_raw_digest_modes_separate_and_each_detects_one_flipped_bit():
    g = torch.Generator().manual_seed(1)
    params = [("a.weight", torch.randn(33, 17, generator=g)), ("b.weight", torch.randn(5000, generator=g))]
    state = {n: {"step": 3, "exp_avg": torch.randn(p.shape, generator=g), "exp_avg_sq": torch.rand(p.shape, generator=g)} for n, p in params}
    groups = [{"lr": 1e-3, "betas": [0.9, 0.95], "eps": 1e-8, "weight_decay": 0.1, "amsgrad": False, "params": [0, 1]}]
    out = {}
    for td in ("raw", "tree"):
        base = SH.compute_state_hash(params, state, groups, tensor_digest=td)
        flipped = [(n, p.clone()) for n, p in params]
        flipped[1][1].view(torch.int32)[4999] ^= 1
        assert SH.compute_state_hash(flipped, state, groups, tensor_digest=td) != base
        out[td] = base
    assert out["raw"] != out["tree"]
