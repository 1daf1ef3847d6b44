"""Torch-facing operators: tensors in, tensors out, arithmetic in libblr_b200.so.

The hot operators (BLAST, quantised BLAST, Monarch, low-rank, dense on 16-bit tensors) are TORCH_LIBRARY ops of the
thin C++ extension (csrc/torch_ext.cpp, ``torch.ops.blr_b200_ext.*``, CUDA + Meta kernels): an eager call costs a
dispatcher hop, and the reference's callers that wrap a model in ``torch.compile(fullgraph=True,
mode='reduce-overhead')`` (models/llama7b.py:65) trace through them.  Where the extension has not been built the
same operators run through ctypes: ``<name>_op`` is then a ``torch.library.custom_op`` with a fake kernel for
tracing, and in eager mode ``<name>`` calls the implementation directly.
Launches go to the current stream, outputs come from torch's allocator, and nothing synchronises the host.
"""
from __future__ import annotations

import collections
import weakref
from typing import Tuple

import torch

from . import _lib as L


def _flat2d(x: torch.Tensor) -> torch.Tensor:
    """(..., I) -> (N, I); a view whenever the leading dims can be merged (traceable by torch.compile).
    A 2-D input is returned as it is: a reshape costs more host time than some of the kernels run."""
    return x if x.dim() == 2 else x.reshape(-1, x.shape[-1])


def _like_input(out: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """(N, W) -> (..., W) with the leading dims of x."""
    return out if x.dim() == 2 else out.reshape(*x.shape[:-1], out.shape[-1])


def _rows(x2: torch.Tensor) -> torch.Tensor:
    """Inside an operator: make the (N, I) input fit the TMA rules (unit inner stride, row stride a multiple
    of 8 elements, 16-byte aligned base); copies only if the input forces it."""
    if x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) % 8 != 0) or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
        if x2.data_ptr() % 16 != 0:
            x2 = x2.clone()
    return x2


def _need_cuda(x: torch.Tensor, *factors: torch.Tensor) -> None:
    """x may be any strided (N, I) view (it is repaired by _rows); factors go to the library as packed arrays, so a
    transposed or sliced view would be read with the wrong strides: refuse it, as the reference's kernels do
    (blast_kernels.py:1951-1952, low_rank_kernels.py:283-285)."""
    for t in (x, *factors):
        if not t.is_cuda:
            raise RuntimeError("blr_b200 operators need CUDA tensors: there is no CPU implementation in this package")
    for t in factors:
        assert t.is_contiguous(), "factor tensors must be contiguous"
        assert t.device == x.device, "x and the factors must live on one device"
    # the library launches on the current device (its descriptor cache and device attributes are per device)
    assert x.device.index is None or x.device.index == torch.cuda.current_device(), \
        f"tensors are on {x.device} but the current CUDA device is {torch.cuda.current_device()}: wrap the call in torch.cuda.device"


def _eager() -> bool:
    return not torch.compiler.is_compiling()


_ws_bytes_cache: dict = {}


def _ws(x: torch.Tensor, n: int, groups: int, width: int, also=None):
    """The stream's workspace, at least blr_workspace_bytes(n, groups, width) bytes (and that of `also` = (groups, width))."""
    st = L.stream_ptr(x.device)
    key = (n, groups, width, also)
    nbytes = _ws_bytes_cache.get(key)
    if nbytes is None:
        nbytes = L.load().blr_workspace_bytes(n, groups, width)
        if also is not None:
            nbytes = max(nbytes, L.load().blr_workspace_bytes(n, also[0], also[1]))
        _ws_bytes_cache[key] = nbytes
    ws = L.workspace(x.device, st, nbytes)
    return ws, st


# ----------------------------------------------------------------------------- BLAST
def _blast_impl(x, U, V, S, u_layout, v_layout, s_i, s_j, s_r, b, P, Q, R, flags, b_out=-1, E=None):
    _need_cuda(x, U, V, S)
    if x.shape[0] == 0:  # an empty batch (e.g. a rank without tokens) is valid and needs no launch
        return x.new_empty((0, (b if b_out < 0 else b_out) * Q))
    x = _rows(x)
    assert U.dtype == x.dtype and V.dtype == x.dtype and S.dtype == x.dtype, "x, U, V, S must share one 16-bit dtype"
    bo = b if b_out < 0 else b_out
    n = x.shape[0]
    out = torch.empty((n, bo * Q), dtype=x.dtype, device=x.device)
    ws, st = _ws(x, n, b, R)
    L.check(L.load().blr_blast_rows_prepared(x.data_ptr(), x.stride(0), n, L.dtype_code(x.dtype), U.data_ptr(), u_layout,
                                             V.data_ptr(), v_layout, S.data_ptr(), s_i, s_j, s_r, b, bo, P, Q, R, flags,
                                             out.data_ptr(), out.stride(0), ws.data_ptr(), ws.numel(), st,
                                             None if E is None else E.data_ptr()))
    return out


@torch.library.custom_op("blr_b200::blast", mutates_args=())
def blast_op(x: torch.Tensor, U: torch.Tensor, V: torch.Tensor, S: torch.Tensor, u_layout: int, v_layout: int,
             s_i: int, s_j: int, s_r: int, b: int, P: int, Q: int, R: int, flags: int, b_out: int = -1) -> torch.Tensor:
    """b_out < b: U and S hold only a slice of the output blocks (sharding by output block)."""
    return _blast_impl(x, U, V, S, u_layout, v_layout, s_i, s_j, s_r, b, P, Q, R, flags, b_out)


# Above this many tokens the library couples on the tensor cores with expanded coupling factors E, a function of S
# alone that blr_blast rebuilds at every call (about 8 us at the headline shape).  The cache below keeps E per S.
_COUPLING_MIN_TOKENS = 256
coupling_cache_bytes = 4 << 30  # upper bound on the cached factors per process (least recently used go first); 0: off
_coupling: "collections.OrderedDict" = collections.OrderedDict()
_coupling_held = 0


def clear_coupling_cache() -> None:
    """Drops every cached set of expanded coupling factors.  The cache notices in-place changes of S that torch
    counts (optimizer steps, copy_, load_state_dict); call this after writing through S.data or from outside torch."""
    global _coupling_held
    _coupling.clear()
    _coupling_held = 0


def _coupling_factors(x, S, s_i, s_j, s_r, b, bo, R):
    """Expanded coupling factors of S for the current stream, built on first use; None where they do not apply
    (few tokens, a shape that couples another way, tracing, stream capture: a captured graph must rebuild them at
    every replay because S may change between replays)."""
    global _coupling_held
    if not (S.is_cuda and S.is_contiguous() and S.dtype == x.dtype) or torch.cuda.is_current_stream_capturing():
        return None
    root = S if S._base is None else S._base  # views made per call (a shard of S) share their base's version counter
    st = L.stream_ptr(S.device)
    key = (S.data_ptr(), s_i, s_j, s_r, b, bo, R, S.dtype, S.device.index, st)
    hit = _coupling.get(key)
    if hit is not None and hit[0]() is root and hit[1] == S._version:
        _coupling.move_to_end(key)
        return hit[2]
    lib = L.load()
    nbytes = lib.blr_blast_coupling_bytes(b, bo, R)
    if nbytes == 0 or nbytes > coupling_cache_bytes:
        return None
    if hit is not None:
        _coupling_held -= hit[2].numel()
        del _coupling[key]
    while _coupling and _coupling_held + nbytes > coupling_cache_bytes:
        _coupling_held -= _coupling.popitem(last=False)[1][2].numel()
    E = torch.empty(nbytes, dtype=torch.uint8, device=S.device)
    L.check(lib.blr_blast_expand_coupling(S.data_ptr(), s_i, s_j, s_r, b, bo, R, L.dtype_code(S.dtype), E.data_ptr(), nbytes, st))
    _coupling[key] = (weakref.ref(root, lambda _r, key=key: _drop_coupling(key)), S._version, E)
    _coupling_held += nbytes
    return E


def _drop_coupling(key) -> None:
    """The tensor an entry was built from is gone: its factors go with it."""
    global _coupling_held
    hit = _coupling.get(key)
    if hit is not None and hit[0]() is None:
        _coupling_held -= hit[2].numel()
        del _coupling[key]


def blast(x, U, V, S, u_layout, v_layout, s_i, s_j, s_r, b, P, Q, R, flags, b_out=-1):
    if not _eager():
        e = L.ext()
        op = blast_op if e is None else e.blast
        return op(x, U, V, S, u_layout, v_layout, s_i, s_j, s_r, b, P, Q, R, flags, b_out)
    E = None
    if x.shape[0] > _COUPLING_MIN_TOKENS and coupling_cache_bytes > 0 and b <= 16:
        E = _coupling_factors(x, S, s_i, s_j, s_r, b, b if b_out < 0 else b_out, R)
    e = L.ext()
    if e is not None:
        return e.blast(x, U, V, S, u_layout, v_layout, s_i, s_j, s_r, b, P, Q, R, flags, b_out, E)
    return _blast_impl(x, U, V, S, u_layout, v_layout, s_i, s_j, s_r, b, P, Q, R, flags, b_out, E)


@blast_op.register_fake
def _(x, U, V, S, u_layout, v_layout, s_i, s_j, s_r, b, P, Q, R, flags, b_out=-1):
    return x.new_empty((x.shape[0], (b if b_out < 0 else b_out) * Q))


def _blast_wq_impl(x, Uq, u_scale, Vq, v_scale, S, s_i, s_j, s_r, bits, group, b, P, Q, R):
    _need_cuda(x, Uq, u_scale, Vq, v_scale, S)
    if x.shape[0] == 0:
        return x.new_empty((0, b * Q))
    x = _rows(x)
    assert u_scale.dtype == torch.float16 and v_scale.dtype == torch.float16, "scales are fp16"
    assert S.dtype == x.dtype
    n = x.shape[0]
    out = torch.empty((n, b * Q), dtype=x.dtype, device=x.device)
    ws, st = _ws(x, n, b, R)
    L.check(L.load().blr_blast_wq(x.data_ptr(), x.stride(0), n, L.dtype_code(x.dtype), Uq.data_ptr(),
                                  u_scale.data_ptr(), Vq.data_ptr(), v_scale.data_ptr(), S.data_ptr(), s_i, s_j, s_r,
                                  bits, group, b, P, Q, R, out.data_ptr(), out.stride(0), ws.data_ptr(), ws.numel(), st))
    return out


@torch.library.custom_op("blr_b200::blast_wq", mutates_args=())
def blast_wq_op(x: torch.Tensor, Uq: torch.Tensor, u_scale: torch.Tensor, Vq: torch.Tensor, v_scale: torch.Tensor,
                S: torch.Tensor, s_i: int, s_j: int, s_r: int, bits: int, group: int, b: int, P: int, Q: int,
                R: int) -> torch.Tensor:
    return _blast_wq_impl(x, Uq, u_scale, Vq, v_scale, S, s_i, s_j, s_r, bits, group, b, P, Q, R)


def blast_wq(x, Uq, u_scale, Vq, v_scale, S, s_i, s_j, s_r, bits, group, b, P, Q, R):
    e = L.ext()
    if e is not None:
        return e.blast_wq(x, Uq, u_scale, Vq, v_scale, S, s_i, s_j, s_r, bits, group, b, P, Q, R)
    if _eager():
        return _blast_wq_impl(x, Uq, u_scale, Vq, v_scale, S, s_i, s_j, s_r, bits, group, b, P, Q, R)
    return blast_wq_op(x, Uq, u_scale, Vq, v_scale, S, s_i, s_j, s_r, bits, group, b, P, Q, R)


@blast_wq_op.register_fake
def _(x, Uq, u_scale, Vq, v_scale, S, s_i, s_j, s_r, bits, group, b, P, Q, R):
    return x.new_empty((x.shape[0], b * Q))


# ----------------------------------------------------------------------------- Monarch
def _monarch_impl(x, w1, w2, w1_layout, w1_cols, w2_layout, b, P, rank, Qs, out_order):
    _need_cuda(x, w1, w2)
    if x.shape[0] == 0:
        return x.new_empty((0, b * Qs))
    x = _rows(x)
    assert w1.dtype == x.dtype and w2.dtype == x.dtype
    n = x.shape[0]
    out = torch.empty((n, b * Qs), dtype=x.dtype, device=x.device)
    ws, st = _ws(x, n, b, rank)
    L.check(L.load().blr_monarch(x.data_ptr(), x.stride(0), n, L.dtype_code(x.dtype), w1.data_ptr(), w1_layout,
                                 w1_cols, w2.data_ptr(), w2_layout, b, P, rank, Qs, out_order, out.data_ptr(),
                                 out.stride(0), ws.data_ptr(), ws.numel(), st))
    return out


@torch.library.custom_op("blr_b200::monarch", mutates_args=())
def monarch_op(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w1_layout: int, w1_cols: int, w2_layout: int,
               b: int, P: int, rank: int, Qs: int, out_order: int) -> torch.Tensor:
    return _monarch_impl(x, w1, w2, w1_layout, w1_cols, w2_layout, b, P, rank, Qs, out_order)


def monarch(x, w1, w2, w1_layout, w1_cols, w2_layout, b, P, rank, Qs, out_order):
    e = L.ext()
    if e is not None:
        return e.monarch(x, w1, w2, w1_layout, w1_cols, w2_layout, b, P, rank, Qs, out_order)
    if _eager():
        return _monarch_impl(x, w1, w2, w1_layout, w1_cols, w2_layout, b, P, rank, Qs, out_order)
    return monarch_op(x, w1, w2, w1_layout, w1_cols, w2_layout, b, P, rank, Qs, out_order)


@monarch_op.register_fake
def _(x, w1, w2, w1_layout, w1_cols, w2_layout, b, P, rank, Qs, out_order):
    return x.new_empty((x.shape[0], b * Qs))


# ----------------------------------------------------------------------------- low rank / dense
def _low_rank_impl(x, V, U, v_layout, u_layout, I, R, O):
    _need_cuda(x, V, U)
    if x.shape[0] == 0:
        return x.new_empty((0, O))
    x = _rows(x)
    assert V.dtype == x.dtype and U.dtype == x.dtype
    n = x.shape[0]
    out = torch.empty((n, O), dtype=x.dtype, device=x.device)
    ws, st = _ws(x, n, 1, R)
    L.check(L.load().blr_low_rank(x.data_ptr(), x.stride(0), n, L.dtype_code(x.dtype), V.data_ptr(), v_layout,
                                  U.data_ptr(), u_layout, I, R, O, out.data_ptr(), out.stride(0), ws.data_ptr(),
                                  ws.numel(), st))
    return out


@torch.library.custom_op("blr_b200::low_rank", mutates_args=())
def low_rank_op(x: torch.Tensor, V: torch.Tensor, U: torch.Tensor, v_layout: int, u_layout: int, I: int, R: int,
                O: int) -> torch.Tensor:
    return _low_rank_impl(x, V, U, v_layout, u_layout, I, R, O)


def low_rank(x, V, U, v_layout, u_layout, I, R, O):
    e = L.ext()
    if e is not None:
        return e.low_rank(x, V, U, v_layout, u_layout, I, R, O)
    if _eager():
        return _low_rank_impl(x, V, U, v_layout, u_layout, I, R, O)
    return low_rank_op(x, V, U, v_layout, u_layout, I, R, O)


@low_rank_op.register_fake
def _(x, V, U, v_layout, u_layout, I, R, O):
    return x.new_empty((x.shape[0], O))


def _dense_impl(x, W, w_layout, I, O):
    _need_cuda(x, W)
    if x.shape[0] == 0:
        return x.new_empty((0, O))
    x = _rows(x)
    assert W.dtype == x.dtype
    n = x.shape[0]
    out = torch.empty((n, O), dtype=x.dtype, device=x.device)
    L.check(L.load().blr_dense(x.data_ptr(), x.stride(0), n, L.dtype_code(x.dtype), W.data_ptr(), w_layout, I, O,
                               out.data_ptr(), out.stride(0), L.stream_ptr(x.device)))
    return out


@torch.library.custom_op("blr_b200::dense", mutates_args=())
def dense_op(x: torch.Tensor, W: torch.Tensor, w_layout: int, I: int, O: int) -> torch.Tensor:
    return _dense_impl(x, W, w_layout, I, O)


def dense(x, W, w_layout, I, O):
    e = L.ext()
    if e is not None:
        return e.dense(x, W, w_layout, I, O)
    if _eager():
        return _dense_impl(x, W, w_layout, I, O)
    return dense_op(x, W, w_layout, I, O)


@dense_op.register_fake
def _(x, W, w_layout, I, O):
    return x.new_empty((x.shape[0], O))


# ----------------------------------------------------------------------------- fp32 verification variants
def _f32(*ts):
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("blr_b200 operators need CUDA tensors: there is no CPU implementation in this package")
        assert t.dtype == torch.float32, "the _fp32 entry points take float32 tensors"


def blast_f32(x2, U, V, S, u_layout, v_layout, s_i, s_j, s_r, b, P, Q, R) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    _f32(x2, U, V, S)
    n = x2.shape[0]
    out = torch.empty((n, b * Q), dtype=torch.float32, device=x2.device)
    z = torch.empty((b, n, R), dtype=torch.float32, device=x2.device)
    y = torch.empty((b, n, R), dtype=torch.float32, device=x2.device)
    L.check(L.load().blr_blast_f32(x2.data_ptr(), x2.stride(0), n, U.data_ptr(), u_layout, V.data_ptr(), v_layout,
                                   S.data_ptr(), s_i, s_j, s_r, b, P, Q, R, out.data_ptr(), out.stride(0),
                                   z.data_ptr(), y.data_ptr(), L.stream_ptr(x2.device)))
    return out, z, y


def monarch_f32(x2, w1, w2, w1_layout, w1_cols, w2_layout, b, P, rank, Qs, out_order):
    _f32(x2, w1, w2)
    n = x2.shape[0]
    out = torch.empty((n, b * Qs), dtype=torch.float32, device=x2.device)
    out1 = torch.empty((b, n, rank), dtype=torch.float32, device=x2.device)
    L.check(L.load().blr_monarch_f32(x2.data_ptr(), x2.stride(0), n, w1.data_ptr(), w1_layout, w1_cols, w2.data_ptr(),
                                     w2_layout, b, P, rank, Qs, out_order, out.data_ptr(), out.stride(0),
                                     out1.data_ptr(), L.stream_ptr(x2.device)))
    return out, out1


def low_rank_f32(x2, V, U, v_layout, u_layout, I, R, O):
    _f32(x2, V, U)
    n = x2.shape[0]
    out = torch.empty((n, O), dtype=torch.float32, device=x2.device)
    z = torch.empty((n, R), dtype=torch.float32, device=x2.device)
    L.check(L.load().blr_low_rank_f32(x2.data_ptr(), x2.stride(0), n, V.data_ptr(), v_layout, U.data_ptr(), u_layout,
                                      I, R, O, out.data_ptr(), out.stride(0), z.data_ptr(), L.stream_ptr(x2.device)))
    return out, z


def dense_f32(x2, W, w_layout, I, O):
    _f32(x2, W)
    n = x2.shape[0]
    out = torch.empty((n, O), dtype=torch.float32, device=x2.device)
    L.check(L.load().blr_dense_f32(x2.data_ptr(), x2.stride(0), n, W.data_ptr(), w_layout, I, O, out.data_ptr(),
                                   out.stride(0), L.stream_ptr(x2.device)))
    return out


def flat2d_f32(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.stride(-1) == 1 else x2.contiguous()


# ----------------------------------------------------------------------------- quantiser
def quantize_sym(w: torch.Tensor, bits: int, group: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric quantisation on the device; w (..., K) contiguous 16-bit.  One fp16 scale per output channel
    (group = 0) or per `group` consecutive contraction indices.
    Returns (q int8 (..., K) | uint8 (..., K/2), scale fp16 (...) | (..., K/group))."""
    _need_cuda(w)
    assert w.is_contiguous() and bits in (8, 4)
    K = w.shape[-1]
    g = K if group == 0 else group
    assert K % g == 0 and g % 2 == 0, f"group {group} must divide the contraction length {K}"
    # a group is quantised exactly like a row of length g, and the layouts coincide
    rows = w.numel() // g
    q = torch.empty((*w.shape[:-1], K if bits == 8 else K // 2), dtype=torch.int8 if bits == 8 else torch.uint8,
                    device=w.device)
    scale = torch.empty(w.shape[:-1] if group == 0 else (*w.shape[:-1], K // g), dtype=torch.float16, device=w.device)
    L.check(L.load().blr_quantize_sym(w.data_ptr(), L.dtype_code(w.dtype), rows, g, bits, q.data_ptr(),
                                      scale.data_ptr(), L.stream_ptr(w.device)))
    return q, scale


def dequantize_sym(q: torch.Tensor, scale: torch.Tensor, bits: int, group: int, dtype: torch.dtype) -> torch.Tensor:
    """16-bit weights q * scale for factors made by quantize_sym (same shapes and group convention)."""
    _need_cuda(q, scale)
    assert q.is_contiguous() and scale.is_contiguous() and bits in (8, 4)
    K = q.shape[-1] * (1 if bits == 8 else 2)
    rows = q.numel() // q.shape[-1]
    w = torch.empty((*q.shape[:-1], K), dtype=dtype, device=q.device)
    L.check(L.load().blr_dequantize_sym(q.data_ptr(), scale.data_ptr(), rows, K, bits, group, L.dtype_code(dtype),
                                        w.data_ptr(), L.stream_ptr(q.device)))
    return w


# ----------------------------------------------------------------------------- load / store probe
def load_store_probe(operands, n: int, out_features: int, dtype: torch.dtype, tile: int) -> torch.Tensor:
    """Streams up to three contiguous operand tensors once and returns out (n, out_features) with out[:, o] = o // tile
    (zeros for tile = 0): the traffic of an operator without its arithmetic."""
    assert 1 <= len(operands) <= 3
    _need_cuda(operands[0], *operands[1:])
    for t in operands:
        assert t.is_contiguous() and (t.numel() * t.element_size()) % 16 == 0 and t.data_ptr() % 16 == 0
    dev = operands[0].device
    out = torch.empty((n, out_features), dtype=dtype, device=dev)
    kind = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[dtype]
    args = []
    for t in list(operands) + [None] * (3 - len(operands)):
        args += [0, 0] if t is None else [t.data_ptr(), t.numel() * t.element_size()]
    L.check(L.load().blr_load_store_probe(*args, kind, out.data_ptr(), n, out_features, out.stride(0) if n else out_features,
                                          tile, L.stream_ptr(dev)))
    return out


# ----------------------------------------------------------------------------- several layers in one pair of launches
def blast_multi(x, layers, bits: int, group: int, b: int, P: int, Q: int, R: int, x_mul=None, biases=None, residuals=None,
                out_act=None):
    """Up to three BLAST layers that share x (N, b*P) and their shapes, through blr_blast_multi.
    layers: tuples (U, Vt, S) of 16-bit factors (bits = 16) or (Uq, u_scale, Vq, v_scale, S) (bits = 8 | 4), torch
    layouts.  x_mul: the input becomes silu(x) * x_mul.  biases / residuals: per layer, None or a tensor added to the
    layer's result ((b*Q,) / (N, b*Q)).  Returns the list of outputs, or None when the fused call does not apply
    (token count or shape outside the two-launch decode path): the caller then runs the layers one by one.
    out_act ("gelu" | "gelu_tanh"): applied to result + bias ahead of the residual; fused above 16 tokens only."""
    n = x.shape[0]
    # decode sizes: the fused pair of launches where it is the faster route; prefill sizes: one call per layer list, worth
    # it when there is a bias or a residual for the last GEMM's epilogue to add (otherwise the plain operators do the same)
    has_res = any(t is not None for t in (residuals or []))
    # (up to 64 tokens the weights are the MMA rows and a thread would fetch its residuals one 2-byte load per token:
    # measured 23.4 us fused against 21.1 us with torch's add at 64 tokens; at 2048 tokens fused and unfused are within
    # 3 % of each other either way - residuals are fused from 65 to 512 tokens, where it gains 1 - 2 us per call)
    if out_act is not None and n <= 16:
        return None
    prefill = (n > 16 and x_mul is None and (any(t is not None for t in (biases or [])) or has_res or out_act is not None)
               and not (has_res and (n <= 64 or n > 512)))
    if n == 0 or torch.compiler.is_compiling() or (n > (8 if bits == 16 else 4) and not prefill):
        return None
    if prefill and bits != 16 and ((P * bits // 8) % 16 != 0 or (R * bits // 8) % 16 != 0 or n > 384):
        return None   # (quantised rows the copy engine cannot stage, or token counts where a widening pass is faster)
    x = _rows(x)
    if x_mul is not None:
        x_mul = _rows(x_mul)
        assert x_mul.shape == x.shape and x_mul.dtype == x.dtype
        if x_mul.stride(0) != x.stride(0):
            x, x_mul = x.contiguous(), x_mul.contiguous()
    k = len(layers)
    arr = (L.BlastProblem * k)()
    outs, keep = [], []
    for i, lay in enumerate(layers):
        if bits == 16:
            U, Vt, S = lay
            us = vs = None
        else:
            U, us, Vt, vs, S = lay
        _need_cuda(x, U, Vt, S)
        out = torch.empty((n, b * Q), dtype=x.dtype, device=x.device)
        bias = None if biases is None else biases[i]
        res = None if residuals is None else residuals[i]
        if res is not None:
            res = _rows(res)
            assert res.shape == out.shape and res.dtype == x.dtype
        arr[i].U, arr[i].V, arr[i].S = U.data_ptr(), Vt.data_ptr(), S.data_ptr()
        arr[i].u_scale = 0 if us is None else us.data_ptr()
        arr[i].v_scale = 0 if vs is None else vs.data_ptr()
        arr[i].bias = 0 if bias is None else bias.data_ptr()
        arr[i].residual = 0 if res is None else res.data_ptr()
        arr[i].ldr = 0 if res is None else res.stride(0)
        arr[i].out, arr[i].ldo = out.data_ptr(), out.stride(0)
        outs.append(out)
        keep.append((bias, res))
    ws, st = _ws(x, n, k * b, R)
    if prefill:
        ws, st = _ws(x, n, k * b, R, also=(b, R))
    rc = L.load().blr_blast_multi(x.data_ptr(), x.stride(0), 0 if x_mul is None else x_mul.data_ptr(),
                                  (L.ACT_NONE if x_mul is None else L.ACT_SILU_MUL) | L.ACT_OUT[out_act], n, L.dtype_code(x.dtype), k, arr,
                                  b * R, R, 1, bits, group, b, P, Q, R, ws.data_ptr(), ws.numel(), st)
    if rc == -6:   # BLR_ERR_UNSUPPORTED: shape outside the fused path
        return None
    L.check(rc)
    return outs


# ----------------------------------------------------------------------------- decoder kernels around the linears
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x (..., d) 16-bit CUDA tensor -> x * rsqrt(mean(x^2) + eps) * weight, fp32 arithmetic, one rounding (LlamaRMSNorm)."""
    _need_cuda(x, weight)
    d = x.shape[-1]
    x2 = x if x.dim() == 2 else x.reshape(-1, d)
    if x2.stride(1) != 1 or x2.stride(0) % 8 != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0], d), dtype=x.dtype, device=x.device)
    L.check(L.load().blr_rmsnorm(x2.data_ptr(), x2.stride(0), x2.shape[0], d, weight.data_ptr(), float(eps), L.dtype_code(x.dtype),
                                 out.data_ptr(), out.stride(0), L.stream_ptr(x.device)))
    return out if x.dim() == 2 else out.reshape(*x.shape[:-1], d)


def _rows16(t: torch.Tensor, d: int) -> torch.Tensor:
    """(..., d) -> (rows, d) with unit inner stride, a row stride that is a multiple of 8 and a 16-byte aligned base."""
    t2 = t if t.dim() == 2 else t.reshape(-1, d)
    if t2.stride(1) != 1 or t2.stride(0) % 8 != 0 or t2.data_ptr() % 16 != 0:
        t2 = t2.contiguous()
    return t2


def layernorm(x: torch.Tensor, weight, bias, eps: float) -> torch.Tensor:
    """x (..., d) 16-bit CUDA tensor -> LayerNorm over d with optional weight / bias (None: none), fp32 arithmetic, one
    rounding; d a multiple of 8, at most 2048."""
    _need_cuda(x)
    d = x.shape[-1]
    x2 = _rows16(x, d)
    out = torch.empty((x2.shape[0], d), dtype=x.dtype, device=x.device)
    L.check(L.load().blr_layernorm(x2.data_ptr(), x2.stride(0), x2.shape[0], d, None if weight is None else weight.data_ptr(),
                                   None if bias is None else bias.data_ptr(), float(eps), L.dtype_code(x.dtype), out.data_ptr(),
                                   out.stride(0), 0, 0, 0, 0, L.stream_ptr(x.device)))
    return out if x.dim() == 2 else out.reshape(x.shape)


def layernorm_modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, eps: float) -> torch.Tensor:
    """norm(x) * (1 + scale) + shift in the norm's own pass: x (B, T, d), shift and scale (B, d) (rows of a wider matrix
    are fine), no affine parameters (the adaLN modulation of a DiT block, DiT/models.py:19-20)."""
    _need_cuda(x, )
    B, T, d = x.shape
    x2 = _rows16(x, d)
    sh, sc = _rows16(shift, d), _rows16(scale, d)
    assert tuple(sh.shape) == (B, d) and tuple(sc.shape) == (B, d) and sh.dtype == x.dtype and sc.dtype == x.dtype
    out = torch.empty((B * T, d), dtype=x.dtype, device=x.device)
    L.check(L.load().blr_layernorm(x2.data_ptr(), x2.stride(0), B * T, d, sc.data_ptr(), sh.data_ptr(), float(eps),
                                   L.dtype_code(x.dtype), out.data_ptr(), out.stride(0), T, sc.stride(0), sh.stride(0), 1,
                                   L.stream_ptr(x.device)))
    return out.view(B, T, d)


def gated_add(x: torch.Tensor, gate: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """x + gate[:, None, :] * y: x, y (B, T, d), gate (B, d) (the gated residual of a DiT block)."""
    _need_cuda(x, )
    B, T, d = x.shape
    x2, y2, g2 = _rows16(x, d), _rows16(y, d), _rows16(gate, d)
    assert y.shape == x.shape and tuple(g2.shape) == (B, d) and y.dtype == x.dtype and g2.dtype == x.dtype
    out = torch.empty((B * T, d), dtype=x.dtype, device=x.device)
    L.check(L.load().blr_gated_add(x2.data_ptr(), x2.stride(0), y2.data_ptr(), y2.stride(0), g2.data_ptr(), g2.stride(0), B * T, T, d,
                                   L.dtype_code(x.dtype), out.data_ptr(), out.stride(0), L.stream_ptr(x.device)))
    return out.view(B, T, d)


def rope_append(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos_table: torch.Tensor, sin_table: torch.Tensor,
                pos: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, n_tok: int) -> torch.Tensor:
    """q, k, v (n_seq * n_tok, heads * head_dim) rows (sequence-major); caches (n_seq, heads, slots, head_dim); cos / sin
    tables (slots, head_dim / 2) fp32; pos (n_tok,) int64 cache slots.  Rotates q in place (returned), writes the
    rotated k and v into the caches at the tokens' slots."""
    _need_cuda(q, k_cache, v_cache)
    n_seq, heads, slots, hd = k_cache.shape
    assert q.dim() == 2 and q.shape == k.shape == v.shape and q.shape[0] == n_seq * n_tok and q.shape[1] == heads * hd
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and v_cache.shape == k_cache.shape
    assert cos_table.dtype == torch.float32 and sin_table.dtype == torch.float32 and cos_table.is_contiguous() and sin_table.is_contiguous()
    assert tuple(cos_table.shape) == (slots, hd // 2) and pos.dtype == torch.int64 and pos.numel() == n_tok and pos.is_cuda
    L.check(L.load().blr_rope_append(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
                                     cos_table.data_ptr(), sin_table.data_ptr(), pos.data_ptr(), n_seq, n_tok, heads, hd, slots,
                                     L.dtype_code(q.dtype), k_cache.data_ptr(), v_cache.data_ptr(), L.stream_ptr(q.device)))
    return q


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, n_keys: int = -1, scale: float = 0.0) -> torch.Tensor:
    """One query token per sequence over the first n_keys slots of the cache (all by default): q (n_seq, heads * head_dim),
    caches (n_seq, heads, slots, head_dim) -> (n_seq, heads * head_dim); scale defaults to head_dim ** -0.5."""
    _need_cuda(q, k_cache, v_cache)
    n_seq, heads, slots, hd = k_cache.shape
    assert q.dim() == 2 and tuple(q.shape) == (n_seq, heads * hd) and q.stride(1) == 1 and v_cache.shape == k_cache.shape
    n_keys = slots if n_keys < 0 else n_keys
    lib = L.load()
    out = torch.empty((n_seq, heads * hd), dtype=q.dtype, device=q.device)
    nbytes = lib.blr_attention_decode_scratch_bytes(n_seq, heads, hd, n_keys)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    L.check(lib.blr_attention_decode(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), n_seq, heads, hd, slots,
                                     n_keys, float(scale) if scale else hd ** -0.5, L.dtype_code(q.dtype), out.data_ptr(),
                                     out.stride(0), scratch.data_ptr(), nbytes, L.stream_ptr(q.device)))
    return out
