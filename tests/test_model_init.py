"""Model shapes and initialisation: parameter counts of the shipped architectures on the meta device, and the rules of
the Philox initialisation (same seed -> same bytes, stream position by parameter order, truncation at two standard
deviations, gains one, other vectors zero, learned quantisation steps derived from the final weights).
(reference test strategy: tests/test_model_shapes.py:31-48, tests/test_init.py:81-108, tests/test_init_audit.py)"""
import math

import torch

from open_transformers_b200.config import load_config
from open_transformers_b200.models import build_model, init_weights
from open_transformers_b200.obs.metrics import count_parameters


def test_parameter_counts_of_the_shipped_architectures():
    with torch.device("meta"):
        open1b = build_model(load_config("open1b_b200").model)
        smoke = build_model(load_config("100m_smoke_repop").model)
    n = open1b.num_parameters()
    assert n == count_parameters(open1b.cfg) == 2 * 128256 * 2048 + 24 * (2048 * 2048 * 2 + 2048 * 512 * 2 + 3 * 2048 * 5632 + 2 * 2048) + 2048
    assert 1.60e9 < n < 1.62e9
    assert 150e6 < smoke.num_parameters() < 300e6          # 6 layers of d=768 plus two 128 256 x 768 vocabulary matrices
    names = [k for k, _ in open1b.named_parameters()]
    assert names[0] == "embedding.tok_embeddings.weight" and names[-1] == "norm_out.weight"
    assert all(p.device.type == "meta" for p in open1b.parameters())


def _tiny(extra=()):
    cfg = load_config("tiny_cpu", ["model.n_layers=2", *extra])
    return build_model(cfg.model), cfg


def test_initialisation_rules():
    a, cfg = _tiny()
    b, _ = _tiny()
    c, _ = _tiny()
    init_weights(a, 11)
    init_weights(b, 11)
    init_weights(c, 12)
    sa, sb, sc = dict(a.named_parameters()), dict(b.named_parameters()), dict(c.named_parameters())
    std = cfg.model.init.std
    seen = 0
    for name, p in sa.items():
        assert torch.equal(p, sb[name]), name
        if p.dim() >= 2:
            assert not torch.equal(p, sc[name]), name
            assert float(p.detach().abs().max()) <= 2 * std + 1e-7 and 0.7 * std < float(p.detach().std()) < 1.0 * std, name
            seen += p.numel()
        elif "norm" in name:
            assert torch.all(p == 1), name
        else:
            assert torch.all(p == 0), name
    assert seen > 0
    # the stream position of a parameter is the number of matrix elements before it: a model with one more block shares
    # every earlier parameter's bytes
    d, _ = _tiny(["model.n_layers=3"])
    init_weights(d, 11)
    sd = dict(d.named_parameters())
    assert torch.equal(sd["embedding.tok_embeddings.weight"], sa["embedding.tok_embeddings.weight"])
    assert torch.equal(sd["blocks.1.ffn.w_down.weight"], sa["blocks.1.ffn.w_down.weight"])
    e, _ = _tiny(["model.vocab_size=%d" % (2 * cfg.model.vocab_size)])                        # a longer first matrix moves all later ones
    init_weights(e, 11)
    se = dict(e.named_parameters())
    assert torch.equal(se["embedding.tok_embeddings.weight"][: cfg.model.vocab_size], sa["embedding.tok_embeddings.weight"])
    assert not torch.equal(se["blocks.0.attn.wq.weight"], sa["blocks.0.attn.wq.weight"])


def test_learned_quantisation_steps_follow_the_initialised_weights():
    m, _ = _tiny(["++model.qat.enabled=true"])
    init_weights(m, 3)
    lin = m.blocks[0].ffn.w_down
    want = (lin.weight.detach().abs().mean(1) * (2.0 / math.sqrt(lin.qmax_w))).clamp_min(1e-6)
    assert torch.allclose(lin.weight_scale.detach(), want, rtol=1e-6) and float(lin.weight_scale.detach().min()) > 0


def test_yarn_rope_keeps_high_frequencies_and_stretches_low_ones():
    """NTK-by-parts tables: the fastest-rotating pairs equal the plain tables, the slowest rotate ``factor`` times slower,
    and a model that selects the variant runs a training step"""
    import numpy as np

    from open_transformers_b200.models.modules.core import RoPE, RoPEYarn
    from open_transformers_b200.train.engine import TrainEngine

    plain = RoPE(64, 256, 10000.0)
    yarn = RoPEYarn(64, 256, 10000.0, factor=4.0, original_max=64)
    pc, ps = plain(256)
    yc, ys = yarn(256)
    assert yc.dtype == torch.float32 and yc.shape == pc.shape == (256, 32)
    assert torch.allclose(yc[:, 0], pc[:, 0], atol=1e-6) and torch.allclose(ys[:, 0], ps[:, 0], atol=1e-6)     # highest frequency kept
    inv_last = 1.0 / 10000.0 ** (31 / 32)
    pos = np.arange(256, dtype=np.float64)
    assert np.allclose(yc[:, 31].numpy(), np.cos(pos * inv_last / 4.0), atol=1e-6)                           # lowest: divided by the factor
    assert not torch.allclose(yc[:, 31], pc[:, 31], atol=1e-4)
    cfg = load_config("tiny_cpu", ["model.modules.rope=rope_yarn"])
    eng = TrainEngine(cfg, "cpu")
    assert type(eng.model.rope).__name__ == "RoPEYarn"
    g = torch.Generator().manual_seed(0)
    eng.zero_grads()
    for v in range(eng.V):
        ids = torch.randint(0, cfg.model.vocab_size, (2, 64), generator=g)
        ce, _ = eng.forward_backward(v, ids, ids, 1)
    assert torch.isfinite(ce) and eng.reduce_gradients() > 0
    eng.close()


def test_unseeded_init_uses_the_global_generator_and_keeps_the_rules_for_vectors():
    import torch

    from open_transformers_b200.models.init import init_weights

    torch.manual_seed(3)
    a = torch.nn.Linear(16, 16)
    init_weights(a, None, std=0.02)
    torch.manual_seed(3)
    b = torch.nn.Linear(16, 16)
    init_weights(b, None, std=0.02)
    assert torch.equal(a.weight, b.weight) and float(a.weight.abs().max()) <= 0.04 + 1e-9 and float(a.bias.detach().abs().sum()) == 0.0
    c = torch.nn.Linear(16, 16)
    init_weights(c, 3, std=0.02)
    assert not torch.equal(a.weight, c.weight)
