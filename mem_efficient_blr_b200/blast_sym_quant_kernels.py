"""Quantised BLAST operators.

``triton_blast_bmm_int8_fp16`` keeps the reference's signature and semantics
(triton_funcs/blast_sym_quant_kernels.py:558-580): 16-bit factors, both intermediates rounded to the
nearest integer in [-128, 127] with no scale.  ``blast_wq`` is the weight-quantised operator
(int8 / packed int4 factors with fp16 per-channel scales), which the reference does not have;
``quantize_blast_factors`` produces its inputs from torch-layout factors.
"""
from __future__ import annotations

import torch

from . import _lib as L
from . import ops
from .blast_kernels import _dims_bmm


def triton_blast_bmm_int8_fp16(x, U, V, S, config=(None, None, None)):
    """U (b,Q,R), V (b,P,R), S (R,b_out,b_in), all 16-bit; activations rounded like the reference's kernels
    (blast_sym_quant_kernels.py:105-108, 227-230)."""
    b, p, q, r = _dims_bmm(x, U, V, S)
    out = ops.blast(ops._flat2d(x), U, V, S, L.KMAJOR, L.MMAJOR, b, 1, b * b, b, p, q, r, L.FLAG_ACT_INT8)
    return ops._like_input(out, x)


def get_triton_blast_bmm_xv_int8_fp16_config():
    return None


def get_triton_blast_bmm_sxv_int8_fp16_config():
    return None


def get_triton_blast_bmm_usxv_int8_fp16_config():
    return None


# Headline layer, int8, cold L2, us per call (in-GEMM widening | widening pass + 16-bit pipeline): 64 tokens 29.7 | 39.9,
# 256: 44.0 | 49.2, 384: 49.1 | 50.2, 512: 59.8 | 56.4, 2048: 147 | 118.
WQ_IN_GEMM_MAX_TOKENS = 384


def quantize_blast_factors(U: torch.Tensor, Vt: torch.Tensor, bits: int, group: int = 0):
    """torch-layout factors U (b,Q,R), Vt (b,R,P) -> (Uq, u_scale, Vq, v_scale).
    One fp16 scale per output channel (group = 0: u_scale (b,Q), v_scale (b,R)) or per `group` contraction
    indices (u_scale (b,Q,R/group), v_scale (b,R,P/group); the kernels take group = 128);
    scale = max|w| / (127 | 7); int4 packed two per byte along the contraction axis, even index in the low nibble."""
    Uq, us = ops.quantize_sym(U.contiguous(), bits, group)
    Vq, vs = ops.quantize_sym(Vt.contiguous(), bits, group)
    return Uq, us, Vq, vs


def blast_wq(x, Uq, u_scale, Vq, v_scale, S, bits: int, group: int = 0):
    """Weight-quantised BLAST. Uq (b,Q,R) int8 or (b,Q,R/2) uint8; Vq (b,R,P) int8 or (b,R,P/2) uint8;
    scales fp16 (b,Q) / (b,R), or (b,Q,R/group) / (b,R,P/group) with per-group scales;
    S (b_out, b_in, R) in x's dtype.  Any token count.  Up to 16 tokens the stored bytes are the MMA operands; up to
    WQ_IN_GEMM_MAX_TOKENS the tensor-core GEMMs stage the stored bytes and widen them in shared memory (the quantised
    arrays are then the only copy of the layer in device memory); above that every weight tile would be widened once
    per 128 tokens, and one widening pass to x's dtype in front of the 16-bit pipeline is cheaper (both routes give
    bit-identical results: the widened weight is q * scale rounded once either way).  Rows of P or R weights that
    are not a multiple of 16 bytes (int4 with P = 48) cannot be staged by the copy engine and take the widening
    pass from 17 tokens on."""
    assert bits in (8, 4)
    per = 1 if bits == 8 else 2
    b, q, r, p = u_scale.size(0), u_scale.size(1), v_scale.size(1), Vq.size(-1) * per
    assert v_scale.size(0) == b and b != 1 and S.size(0) == b and S.size(1) == b and S.size(2) == r
    assert Uq.size(-1) * per == r and x.size(-1) == b * p
    if group == 0:
        assert u_scale.dim() == 2 and v_scale.dim() == 2, "one scale per output channel expected (group = 0)"
    else:
        assert tuple(u_scale.shape) == (b, q, r // group) and tuple(v_scale.shape) == (b, r, p // group)
    x2 = ops._flat2d(x)
    n = x2.shape[0]
    if n > WQ_IN_GEMM_MAX_TOKENS or (n > 16 and ((p * bits // 8) % 16 != 0 or (r * bits // 8) % 16 != 0)):
        U = ops.dequantize_sym(Uq, u_scale, bits, group, x.dtype)
        Vt = ops.dequantize_sym(Vq, v_scale, bits, group, x.dtype)
        out = ops.blast(x2, U, Vt, S, L.KMAJOR, L.KMAJOR, b * r, r, 1, b, p, q, r, L.FLAG_NONE)
    else:
        out = ops.blast_wq(x2, Uq, u_scale, Vq, v_scale, S, b * r, r, 1, bits, group, b, p, q, r)
    return ops._like_input(out, x)


def blast_wq_multi(x, layers, bits: int, group: int = 0, x_mul=None, biases=None, residuals=None, out_act=None):
    """blast_wq for several layers on one input: layers = [(Uq, u_scale, Vq, v_scale, S), ...] with equal shapes; the
    options of blast_kernels.blast_multi_torch_layout.  One pair of launches up to 16 tokens (preceded above 2 tokens, or
    with x_mul, by one launch that converts x to fixed point once), else layer by layer."""
    assert bits in (8, 4)
    per = 1 if bits == 8 else 2
    Uq0, us0, Vq0, vs0, S0 = layers[0]
    b, q, r, p = us0.size(0), us0.size(1), vs0.size(1), Vq0.size(-1) * per
    x2 = ops._flat2d(x)
    xm2 = None if x_mul is None else ops._flat2d(x_mul)
    res2 = None if residuals is None else [None if t is None else ops._flat2d(t) for t in residuals]
    outs = ops.blast_multi(x2, layers, bits, group, b, p, q, r, xm2, biases, res2, out_act) if 1 <= len(layers) <= 3 else None
    if outs is None:
        xe = x2 if xm2 is None else torch.nn.functional.silu(x2) * xm2
        if xm2 is not None and 1 <= len(layers) <= 3:   # the input transform done here, the rest may still fuse
            outs = ops.blast_multi(xe, layers, bits, group, b, p, q, r, None, biases, res2, out_act)
    if outs is None:
        outs = []
        for i, (Uq, us, Vq, vs, S) in enumerate(layers):
            o = ops._flat2d(blast_wq(xe, Uq, us, Vq, vs, S, bits, group))
            if biases is not None and biases[i] is not None:
                o += biases[i]
            if out_act is not None:
                o = torch.nn.functional.gelu(o, approximate="tanh" if out_act == "gelu_tanh" else "none")
            if res2 is not None and res2[i] is not None:
                o += res2[i]
            outs.append(o)
    return [ops._like_input(o, x) for o in outs]


def blast_wq_host(x_host, Uq, u_scale, Vq, v_scale, S, bits: int, group: int = 0, out=None):
    """blast_wq for activations in host memory: x_host (N, b*P) 16-bit CPU tensor (pinned for asynchronous copies),
    factors on the device.  One library call enqueues copy-in, the kernel and copy-out on the device's current
    stream and two copy streams of the library, so that consecutive calls overlap their copies with each other's
    kernels; returns the (pinned) host tensor `out` (N, b*Q), valid after host_flush() and a synchronisation of
    the current stream.  Up to 16 tokens per call; larger batches go through blast_wq on device tensors."""
    assert not x_host.is_cuda and x_host.dim() == 2 and x_host.stride(1) == 1 and bits in (8, 4)
    dev = Uq.device
    per = 1 if bits == 8 else 2
    b, q, r, p = u_scale.size(0), u_scale.size(1), v_scale.size(1), Vq.size(-1) * per
    n = x_host.size(0)
    assert x_host.size(1) == b * p and S.size(0) == b and S.size(1) == b and S.size(2) == r
    if n > 16:
        y = blast_wq(x_host.to(dev, non_blocking=True), Uq, u_scale, Vq, v_scale, S, bits, group)
        if out is None:
            out = torch.empty(y.shape, dtype=y.dtype, pin_memory=True)
        return out.copy_(y, non_blocking=True)
    if out is None:
        out = torch.empty((n, b * q), dtype=x_host.dtype, pin_memory=True)
    assert not out.is_cuda and out.stride(1) == 1 and tuple(out.shape) == (n, b * q) and out.dtype == x_host.dtype
    e = L.ext()
    if e is not None:
        e.blast_wq_host(x_host, out, Uq, u_scale, Vq, v_scale, S, bits, group)
        return out
    lib = L.load()
    st = L.stream_ptr(dev)
    ws = L.workspace(dev, st, lib.blr_workspace_bytes(n, b, r))
    sg = L.staging(dev, st, lib.blr_host_staging_bytes(16, b * p, b * q))  # one size for every token count
    L.check(lib.blr_blast_wq_host(x_host.data_ptr(), x_host.stride(0), n, L.dtype_code(x_host.dtype), Uq.data_ptr(),
                                  u_scale.data_ptr(), Vq.data_ptr(), v_scale.data_ptr(), S.data_ptr(), b * r, r, 1, bits,
                                  group, b, p, q, r, out.data_ptr(), out.stride(0), sg.data_ptr(), sg.numel(),
                                  ws.data_ptr(), ws.numel(), st))
    return out


class BlastWqHostCall:
    """blast_wq_host for a fixed set of factors, prepared once: the factors' pointers, the shapes and the scratch
    buffers are looked up at construction, so that a call costs little more than the library call itself (a decode
    loop issues one such call per layer and token step; the argument checks of blast_wq_host take as long as the
    kernel).  call(x_host, out) has blast_wq_host's meaning: x_host (N <= 16, b*P) and out (N, b*Q) pinned 16-bit
    host tensors; out is valid after host_flush() and a synchronisation of the current stream.  The object keeps
    references to the factors."""

    def __init__(self, Uq, u_scale, Vq, v_scale, S, bits: int, group: int = 0):
        assert bits in (8, 4)
        per = 1 if bits == 8 else 2
        b, q, r, p = u_scale.size(0), u_scale.size(1), v_scale.size(1), Vq.size(-1) * per
        assert v_scale.size(0) == b and b != 1 and tuple(S.shape) == (b, b, r) and Uq.size(-1) * per == r
        for t in (Uq, u_scale, Vq, v_scale, S):
            assert t.is_cuda and t.is_contiguous()
        self._keep = (Uq, u_scale, Vq, v_scale, S)
        self.device = Uq.device
        self.dtype = S.dtype
        self.in_features, self.out_features = b * p, b * q
        self._code = L.dtype_code(S.dtype)
        self._factors = (Uq.data_ptr(), u_scale.data_ptr(), Vq.data_ptr(), v_scale.data_ptr(), S.data_ptr(),
                         b * r, r, 1, bits, group, b, p, q, r)
        lib = L.load()
        self._fn = lib.blr_blast_wq_host
        self._ws_bytes = lib.blr_workspace_bytes(16, b, r)
        self._sg_bytes = lib.blr_host_staging_bytes(16, b * p, b * q)
        self._dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._scratch = {}  # stream -> (workspace, staging)
        self._ext = L.ext()
        self._bits, self._group = bits, group

    def __call__(self, x_host, out):
        if self._ext is not None:  # the C++ operator checks the shapes itself
            self._ext.blast_wq_host(x_host, out, *self._keep, self._bits, self._group)
            return out
        n = x_host.size(0)
        if not (n <= 16 and x_host.size(1) == self.in_features and out.size(0) == n and out.size(1) == self.out_features
                and x_host.dtype == self.dtype and out.dtype == self.dtype and not x_host.is_cuda and not out.is_cuda
                and x_host.stride(1) == 1 and out.stride(1) == 1):
            raise AssertionError("x_host (N <= 16, b*P) and out (N, b*Q) must be 16-bit host tensors of the factors' dtype")
        st = torch._C._cuda_getCurrentRawStream(self._dev_index)
        sc = self._scratch.get(st)
        if sc is None:
            sc = (L.workspace(self.device, st, self._ws_bytes), L.staging(self.device, st, self._sg_bytes))
            self._scratch[st] = sc
        ws, sg = sc
        rc = self._fn(x_host.data_ptr(), x_host.stride(0), n, self._code, *self._factors, out.data_ptr(), out.stride(0),
                      sg.data_ptr(), sg.numel(), ws.data_ptr(), ws.numel(), st)
        if rc != 0:
            L.check(rc)
        return out


def host_flush(device=None) -> None:
    """Makes the current stream of `device` wait for the copy-outs of all blast_wq_host calls issued on it."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    L.check(L.load().blr_host_flush(L.stream_ptr(dev)))
