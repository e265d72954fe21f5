"""`repop.qat.lsq`: learned-step-size (LSQ) and absmax W8A8 layers (reference: model/modules/_linear.py:44-64,
model/modules/qat_warmstart.py:37, train/loop.py:1082-1084).

Stand-in numerics: per-tensor absmax activation quantisation, per-output-channel weight quantisation, both as
fake quantisation with straight-through rounding; the product itself runs in the activation dtype on cuBLAS.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from repop.qat.functional import _qmax_for_bits


def _ste_round(x):
    return (x.round() - x).detach() + x


def _fake_quant_act(x, qmax: int):
    s = x.detach().abs().amax().clamp_min(1e-8) * (1.0 / qmax)
    return _ste_round((x / s).clamp(-qmax - 1, qmax)) * s


class LSQQuantizedLinear(nn.Linear):
    def __init__(self, in_features, out_features, bias=False, weight_bits=8, act_bits=8):
        super().__init__(in_features, out_features, bias=bias)
        self.weight_bits, self.act_bits = int(weight_bits), int(act_bits)
        qmax = _qmax_for_bits(self.weight_bits)
        with torch.no_grad():
            init = self.weight.abs().mean(dim=1) * (2.0 / math.sqrt(qmax))
        self.weight_scale = nn.Parameter(init.clamp_min(1e-6))

    def forward(self, input):  # noqa: A002
        qmax = _qmax_for_bits(self.weight_bits)
        s = self.weight_scale.unsqueeze(1).to(self.weight.dtype)
        w = _ste_round((self.weight / s).clamp(-qmax - 1, qmax)) * s
        return F.linear(_fake_quant_act(input, _qmax_for_bits(self.act_bits)), w.to(input.dtype), self.bias)


class QuantizedLinear(nn.Linear):
    def __init__(self, in_features, out_features, bias=False, weight_bits=8, act_bits=8, per_channel_w=True):
        super().__init__(in_features, out_features, bias=bias)
        self.weight_bits, self.act_bits, self.per_channel_w = int(weight_bits), int(act_bits), bool(per_channel_w)

    def forward(self, input):  # noqa: A002
        qmax = _qmax_for_bits(self.weight_bits)
        w = self.weight
        amax = w.detach().abs().amax(dim=1, keepdim=True) if self.per_channel_w else w.detach().abs().amax()
        s = amax.clamp_min(1e-8) * (1.0 / qmax)
        wq = _ste_round((w / s).clamp(-qmax - 1, qmax)) * s
        return F.linear(_fake_quant_act(input, _qmax_for_bits(self.act_bits)), wq.to(input.dtype), self.bias)


@torch.no_grad()
def refresh_lsq_weight_scales(model: nn.Module) -> int:
    n = 0
    for m in model.modules():
        if isinstance(m, LSQQuantizedLinear):
            w = m.weight.to_local() if hasattr(m.weight, "to_local") else m.weight
            sc = m.weight_scale.to_local() if hasattr(m.weight_scale, "to_local") else m.weight_scale
            qmax = _qmax_for_bits(m.weight_bits)
            sc.copy_((w.to(torch.bfloat16).abs().float().mean(dim=1) * (2.0 / math.sqrt(qmax))).clamp_min(1e-6))
            n += 1
    return n
