"""`repop.qat`: W8A8 quantisation-aware linear layers as straight-through fake quantisation on stock torch."""
from repop.qat.lsq import LSQQuantizedLinear, QuantizedLinear  # noqa: F401
