"""Monarch operators with the reference's names and layouts (triton_funcs/monarch_kernels.py).

w1_bfly (b, P, rank) has its columns regrouped so that column l*per + jj feeds second-stage block l
(layer.py:221-224); w2 is (b, Q, rank) for ``right`` / ``right_ideal`` and (b, rank, Q) for ``right_left``
(models/wrappers.py:26-31).  ``right`` and ``right_left`` emit output feature s*b + l; ``right_ideal``
emits l*S + s (monarch_kernels.py:1004).
"""
from __future__ import annotations

from . import _lib as L
from . import ops


def _dims(x, w1, w2, w2_kmajor):
    k, p, q = w1.shape
    if w2_kmajor:
        l, s, r = w2.shape
    else:
        l, r, s = w2.shape
    assert k * p == x.shape[-1]
    assert l * r == k * q
    assert k == l, "both factors must have the same number of blocks"
    assert q % k == 0, "rank must be a multiple of the block count"
    assert w1.is_contiguous() and w2.is_contiguous()
    return k, p, q, s


def _run16(x, w1, w2, w2_layout, order):
    b, p, rank, s = _dims(x, w1, w2, w2_layout == L.KMAJOR)
    out = ops.monarch(ops._flat2d(x), w1, w2, L.MMAJOR, L.COLS_GROUPED, w2_layout, b, p, rank, s, order)
    return ops._like_input(out, x)


def _run32(x, w1, w2, w2_layout, order):
    b, p, rank, s = _dims(x, w1, w2, w2_layout == L.KMAJOR)
    out, out1 = ops.monarch_f32(ops.flat2d_f32(x), w1, w2, L.MMAJOR, L.COLS_GROUPED, w2_layout, b, p, rank, s, order)
    return ops._like_input(out, x), out1


def triton_monarch_right_fp16(x, w1_bfly, w2_bfly_t, config=None):
    """Replaces triton_monarch_right_fp16 (monarch_kernels.py:869-909)."""
    return _run16(x, w1_bfly, w2_bfly_t, L.KMAJOR, L.OUT_INTERLEAVED)


def triton_monarch_right_fp32(x, w1_bfly, w2_bfly_t):
    """Replaces triton_monarch_right_fp32 (monarch_kernels.py:823-867): (out2, out1, None)."""
    out, out1 = _run32(x, w1_bfly, w2_bfly_t, L.KMAJOR, L.OUT_INTERLEAVED)
    return out, out1, None


def triton_monarch_right_ideal_fp16(x, w1_bfly, w2_bfly_t, config=None):
    """Replaces triton_monarch_right_ideal_fp16 (monarch_kernels.py:961-1005)."""
    return _run16(x, w1_bfly, w2_bfly_t, L.KMAJOR, L.OUT_BLOCKED)


def triton_monarch_right_ideal_fp32(x, w1_bfly, w2_bfly_t):
    """Replaces triton_monarch_right_ideal_fp32 (monarch_kernels.py:911-959); the reference's harness
    checks element [1] (out1) of the result (layer.py:235-237)."""
    out, out1 = _run32(x, w1_bfly, w2_bfly_t, L.KMAJOR, L.OUT_BLOCKED)
    return out, out1, None


def triton_monarch_right_left_fp16(x, w1_bfly, w2_bfly, config=(None, None)):
    """Replaces triton_monarch_right_left_fp16 (monarch_kernels.py:1060-1099)."""
    return _run16(x, w1_bfly, w2_bfly, L.MMAJOR, L.OUT_INTERLEAVED)


def triton_monarch_right_left_fp32(x, w1_bfly, w2_bfly):
    """Replaces triton_monarch_right_left_fp32 (monarch_kernels.py:1007-1058): (out2, None, out1, None)."""
    out, out1 = _run32(x, w1_bfly, w2_bfly, L.MMAJOR, L.OUT_INTERLEAVED)
    return out, None, out1, None


def monarch_torch_layout(x, w1_t, w2_t, ideal: bool = False):
    """Same operator on the reference's torch layouts (torch_funcs/monarch_funcs.py:4-45):
    w1_t (b, rank, P), w2_t (b, Q, rank); returns out2 only.  ideal = True leaves the output in the block-major order
    of the reference's right_ideal variant (feature l*S + s, monarch_kernels.py:1004) for a consumer that takes it
    that way (ideal_order_index, fold_ideal_order_into_dense)."""
    b, rank, p = w1_t.shape
    l, s, r = w2_t.shape
    assert b == l and r == rank and b * p == x.shape[-1] and rank % b == 0
    out = ops.monarch(ops._flat2d(x), w1_t, w2_t, L.KMAJOR, L.COLS_TORCH, L.KMAJOR, b, p, rank, s,
                      L.OUT_BLOCKED if ideal else L.OUT_INTERLEAVED)
    return ops._like_input(out, x)


# ------------------------------------------------------------------- chaining on the un-interleaved (right_ideal) order
# The reference's Llama configuration runs gate_proj and up_proj with the right_ideal variant, which skips the final
# interleave and "assumes the next layer absorbs the permutation" (configs/networks/llama7b.yaml:164,180,
# monarch_kernels.py:961-1005).  What absorbing means for the layer that follows:
#   * an element-wise step (silu(gate) * up) is order-blind: both operands arrive in the same order;
#   * a dense layer absorbs it exactly by a permutation of its input columns (fold_ideal_order_into_dense);
#   * a Monarch layer with the same block count takes block l of the ideal order (the S outputs of second-stage block
#     l) as its input block l.  That is a different linear map from the same factors on the interleaved order, and no
#     re-packing of block-diagonal factors can turn one into the other (an input block of the interleaved order mixes
#     all l): a chained Monarch MLP is a model of its own, trained in that order, as in the reference's configuration.
def ideal_order_index(features: int, b: int, device=None):
    """idx with y_ideal[..., idx] == y_interleaved: position of interleaved feature s*b + l in the ideal order, l*S + s."""
    import torch
    assert features % b == 0
    S = features // b
    f = torch.arange(features, device=device)
    return (f % b) * S + f // b


def fold_ideal_order_into_dense(weight, b: int):
    """weight (O, I) of a dense layer fed with an interleaved Monarch output -> the weight that gives the same result
    on the ideal-order output: W'[:, l*S + s] = W[:, s*b + l]."""
    idx = ideal_order_index(weight.shape[-1], b, weight.device)
    out = weight.new_empty(weight.shape)
    out[..., idx] = weight
    return out


def get_triton_monarch_right_fp16_config():
    return None


def get_triton_monarch_right_ideal_fp16_config():
    return None


def get_triton_monarch_right_left_fp16_config():
    return (None, None)
