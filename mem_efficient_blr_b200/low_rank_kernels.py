"""Low-rank operators with the reference's names and layouts (triton_funcs/low_rank_kernels.py).

a is (I, R), b is (R, O) (layer.py:250-251).  Like the reference, the result is 2-D (N, O): the batch
dimensions of x are flattened and not restored (low_rank_kernels.py:416-417).
"""
from __future__ import annotations

from . import _lib as L
from . import ops


def _dims(x, a, b):
    i, r = a.shape
    r2, o = b.shape
    assert x.shape[-1] == i and r2 == r, "incompatible dimensions"
    assert a.is_contiguous() and b.is_contiguous()
    return i, r, o


def triton_low_rank_fp16(x, a, b, config=None):
    """Replaces triton_low_rank_fp16 (low_rank_kernels.py:410-417)."""
    i, r, o = _dims(x, a, b)
    return ops.low_rank(ops._flat2d(x), a, b, L.MMAJOR, L.MMAJOR, i, r, o)


def triton_low_rank_fp32(x, a, b):
    """Replaces triton_low_rank_fp32 (low_rank_kernels.py:394-408): (y (N,O), z (N,R))."""
    i, r, o = _dims(x, a, b)
    return ops.low_rank_f32(ops.flat2d_f32(x), a, b, L.MMAJOR, L.MMAJOR, i, r, o)


def triton_low_rank_load_store_fp16(x, a, b):
    """Replaces triton_low_rank_load_store_fp16 (low_rank_kernels.py:435-449): a bandwidth probe that reads x, a and b
    and writes y (N, O) with the index of the 64-wide output tile in every element (the reference kernel's default
    BLOCK_SIZE_O, low_rank_kernels.py:229-234), no arithmetic."""
    i, r, o = _dims(x, a, b)
    x2 = ops._flat2d(x).contiguous()
    return ops.load_store_probe((x2, a, b), x2.shape[0], o, x.dtype, 64)


def triton_low_rank_load_store_fp32(x, a, b):
    """Replaces triton_low_rank_load_store_fp32 (low_rank_kernels.py:419-433); float32 tensors."""
    i, r, o = _dims(x, a, b)
    x2 = ops.flat2d_f32(x).contiguous()
    return ops.load_store_probe((x2, a, b), x2.shape[0], o, x.dtype, 64)


def low_rank_torch_layout(x, Vt, Ut):
    """torch layouts Vt (R, I), Ut (O, R) (torch_funcs/low_rank_funcs.py:4-28); batch dims restored."""
    r, i = Vt.shape
    o, _ = Ut.shape
    return ops._like_input(ops.low_rank(ops._flat2d(x), Vt, Ut, L.KMAJOR, L.KMAJOR, i, r, o), x)


def get_triton_low_rank_fp16_config():
    return None
