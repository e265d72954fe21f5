"""`repop.qat.functional._qmax_for_bits` (reference: model/init.py:168)."""


def _qmax_for_bits(bits: int) -> int:
    return (1 << (int(bits) - 1)) - 1
