"""Dense operators with the reference's names and layouts (triton_funcs/dense_kernels.py).

w is (I, O) (layer.py:267); the result is 2-D (N, O) like the reference's (dense_kernels.py:375-381).
"""
from __future__ import annotations

from . import _lib as L
from . import ops


def triton_dense_fp16(x, w, config=None):
    """Replaces triton_dense_fp16 (dense_kernels.py:375-381)."""
    i, o = w.shape
    assert x.shape[-1] == i and w.is_contiguous()
    return ops.dense(ops._flat2d(x), w, L.MMAJOR, i, o)


def triton_dense_fp32(x, w):
    """Replaces triton_dense_fp32 (dense_kernels.py:360-373)."""
    i, o = w.shape
    assert x.shape[-1] == i and w.is_contiguous()
    return ops.dense_f32(ops.flat2d_f32(x), w, L.MMAJOR, i, o)


def triton_dense_load_store_fp16(x, w):
    """Replaces triton_dense_load_store_fp16 (dense_kernels.py:398-411): a bandwidth probe that reads x and w and
    writes a zero y (N, O) (dense_kernels.py:222-227), no arithmetic."""
    i, o = w.shape
    assert x.shape[-1] == i and w.is_contiguous()
    x2 = ops._flat2d(x).contiguous()
    return ops.load_store_probe((x2, w), x2.shape[0], o, x.dtype, 0)


def triton_dense_load_store_fp32(x, w):
    """Replaces triton_dense_load_store_fp32 (dense_kernels.py:383-396); float32 tensors."""
    i, o = w.shape
    assert x.shape[-1] == i and w.is_contiguous()
    x2 = ops.flat2d_f32(x).contiguous()
    return ops.load_store_probe((x2, w), x2.shape[0], o, x.dtype, 0)


def dense_torch_layout(x, Wt):
    """torch layout Wt (O, I) (torch_funcs/dense_funcs.py:4-25); batch dims restored."""
    o, i = Wt.shape
    return ops._like_input(ops.dense(ops._flat2d(x), Wt, L.KMAJOR, i, o), x)


def get_triton_dense_fp16_config():
    return None
