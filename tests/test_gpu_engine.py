"""The engine on a GPU: the fp32 (exact family) run must produce the same chained state hashes as the
CPU run, step by step; the bf16 run must be finite, repeatable and free of kernel time-outs."""
import pytest
import torch

from open_transformers_b200.config import load_config
from open_transformers_b200.ops.functional import kernel_status
from open_transformers_b200.train.engine import TrainEngine

pytestmark = pytest.mark.gpu


def _run(cfg, device, steps=2, V=2, T=128, vocab=1024, td="raw"):
    eng = TrainEngine(cfg, device)
    g = torch.Generator().manual_seed(0)
    prev, out = None, []
    for _ in range(steps):
        eng.zero_grads()
        for v in range(V):
            ids = torch.randint(0, vocab, (2, T), generator=g).to(device)
            lab = torch.randint(0, vocab, (2, T), generator=g).to(device)
            ce, z = eng.forward_backward(v, ids, lab, 1, last=v == V - 1)  # on a GPU the reduction runs under this backward pass
        norm = eng.reduce_gradients()
        eng.optimizer_step(3e-4, eng.clip_coefficient(norm, 1.0))
        prev = eng.sharded_state_hash(prev, None, tensor_digest=td)
        out.append((float(ce), norm, prev))
    return out


def test_fp32_gpu_matches_cpu_hashes():
    cfg = load_config("tiny_cpu")
    cpu = _run(cfg, "cpu")
    gpu = _run(cfg, "cuda")
    assert [h for _, _, h in cpu] == [h for _, _, h in gpu], (cpu, gpu)
    assert _run(cfg, "cuda", td="tree")[-1][2] == _run(cfg, "cpu", td="tree")[-1][2]


def test_bf16_gpu_matches_cpu_hashes():
    """bf16 tensor-core run on the GPU == bf16 replay on the CPU (tensor-core accumulation model), hash for hash."""
    cfg = load_config("open1b_b200", ["model.n_layers=2", "model.d_model=256", "model.n_heads=2", "model.n_kv_heads=1", "model.ffn_intermediate=512",
                                      "model.vocab_size=1024", "train.seq_len=128", "data.seq_len=128", "run.virtual_dp_size=2", "run.dp_shard_size=2"])
    cpu = _run(cfg, "cpu", T=128, vocab=1024, td="tree")
    gpu = _run(cfg, "cuda", T=128, vocab=1024, td="tree")
    assert [h for _, _, h in cpu] == [h for _, _, h in gpu], (cpu, gpu)


def test_bf16_gpu_finite_and_repeatable():
    cfg = load_config("open1b_b200", ["model.n_layers=2", "model.vocab_size=4096", "train.seq_len=256", "data.seq_len=256",
                                      "run.virtual_dp_size=2", "run.dp_shard_size=2"])
    a = _run(cfg, "cuda", T=256, vocab=4096, td="tree")
    b = _run(cfg, "cuda", T=256, vocab=4096, td="tree")
    assert all(torch.isfinite(torch.tensor(x[0])) and x[1] > 0 for x in a), a
    assert a == b
    assert kernel_status("cuda") == 0


def test_overlapped_state_hash_equals_the_synchronous_one():
    """begin_state_hash lets the digests run on a side stream under the next step's forward/backward; the chain it
    yields must be the one the synchronous call gives."""
    cfg = load_config("open1b_b200", ["model.n_layers=2", "model.vocab_size=4096", "train.seq_len=256", "data.seq_len=256",
                                      "run.virtual_dp_size=2", "run.dp_shard_size=2"])
    sync = [h for _, _, h in _run(cfg, "cuda", steps=3, T=256, vocab=4096, td="tree")]
    eng = TrainEngine(cfg, "cuda")
    g = torch.Generator().manual_seed(0)
    prev, pending, got = None, None, []
    for _ in range(3):
        eng.zero_grads()
        for v in range(2):
            ids = torch.randint(0, 4096, (2, 256), generator=g).to("cuda")
            lab = torch.randint(0, 4096, (2, 256), generator=g).to("cuda")
            eng.forward_backward(v, ids, lab, 1)
        norm = eng.reduce_gradients()  # waits, on the device, for the digests still in flight
        eng.optimizer_step(3e-4, eng.clip_coefficient(norm, 1.0))
        if pending is not None:
            prev = eng.finish_state_hash(pending, prev, None)
            got.append(prev)
        pending = eng.begin_state_hash(tensor_digest="tree")
    got.append(eng.finish_state_hash(pending, prev, None))
    assert got == sync


def test_offloaded_moments_leave_the_gpu_between_steps_and_change_no_bit(tmp_path):
    """--offload-optimizer on a GPU: the two moment buffers are written to their files after the step's hash and read back for
    the next optimizer step; they are absent during forward and backward and no digest changes."""
    cfg = load_config("open1b_b200", ["model.n_layers=2", "model.vocab_size=4096", "train.seq_len=256", "data.seq_len=256",
                                      "run.virtual_dp_size=2", "run.dp_shard_size=2"])
    want = [h for _, _, h in _run(cfg, "cuda", steps=3, T=256, vocab=4096, td="tree")]
    eng = TrainEngine(cfg, "cuda", offload_optimizer=True, optimizer_offload_dir=str(tmp_path))
    g = torch.Generator().manual_seed(0)
    prev, got = None, []
    for _ in range(3):
        eng.zero_grads()
        for v in range(2):
            ids = torch.randint(0, 4096, (2, 256), generator=g).to("cuda")
            lab = torch.randint(0, 4096, (2, 256), generator=g).to("cuda")
            eng.forward_backward(v, ids, lab, 1)
        assert got == [] or eng._m1 is None  # absent during forward and backward
        norm = eng.reduce_gradients()
        eng.optimizer_step(3e-4, eng.clip_coefficient(norm, 1.0))
        prev = eng.sharded_state_hash(prev, None, tensor_digest="tree")
        got.append(prev)
        eng.release_state()
    assert got == want
    eng.close()
