"""BLAST operators with the reference's names and argument layouts (triton_funcs/blast_kernels.py).

Layouts per family (models/wrappers.py:151-163, layer.py:191-201):
  partial / partial_grouped / partial_grouped_persistent / full:
      U (b, R, Q)   V (b, P, R)   S (b_in, b_out, R)
  bmm:
      U (b, Q, R)   V (b, P, R)   S (R, b_out, b_in)
The ``_fp16`` functions take 16-bit tensors (bfloat16 like the reference, or float16), return the
output only and accept the reference's optional trailing ``config`` (ignored: there is nothing to
autotune at run time).  The ``_fp32`` functions take float32 tensors and return ``(out, z, y)``.
All five families run the same CUDA path; the reference's distinction between them was how far its
Triton kernels managed to fuse (blast_kernels.py:1124-1125).
"""
from __future__ import annotations

import torch

from . import _lib as L
from . import ops


def _dims_partial(x, U, V, S):
    b1, p, r = V.shape
    b2, r2, q = U.shape
    assert b1 == b2, "b1 must equal b2"
    assert b1 != 1 and b2 != 1, "b must not be 1"
    assert r2 == r and tuple(S.shape) == (b1, b2, r), "inconsistent factor shapes"
    assert x.shape[-1] == b1 * p, "x last dim must be b*P"
    assert U.is_contiguous() and V.is_contiguous() and S.is_contiguous()
    return b1, p, q, r


def _dims_bmm(x, U, V, S):
    b1, p, r = V.shape
    b2, q, r2 = U.shape
    assert b1 == b2, "b1 must equal b2"
    assert b1 != 1 and b2 != 1, "b must not be 1"
    assert r2 == r and tuple(S.shape) == (r, b2, b1), "inconsistent factor shapes"
    assert x.shape[-1] == b1 * p, "x last dim must be b*P"
    assert U.is_contiguous() and V.is_contiguous() and S.is_contiguous()
    return b1, p, q, r


def _partial_fp16(x, U, V, S, flags=L.FLAG_NONE):
    b, p, q, r = _dims_partial(x, U, V, S)
    out = ops.blast(ops._flat2d(x), U, V, S, L.MMAJOR, L.MMAJOR, r, b * r, 1, b, p, q, r, flags)
    return ops._like_input(out, x)


def _partial_fp32(x, U, V, S):
    b, p, q, r = _dims_partial(x, U, V, S)
    out, z, y = ops.blast_f32(ops.flat2d_f32(x), U, V, S, L.MMAJOR, L.MMAJOR, r, b * r, 1, b, p, q, r)
    return ops._like_input(out, x), z, y


def triton_blast_partial_fp16(x, U, V, S, config=None):
    """Replaces triton_blast_partial_fp16 (blast_kernels.py:2666-2707)."""
    return _partial_fp16(x, U, V, S)


def triton_blast_partial_fp32(x, U, V, S):
    """Replaces triton_blast_partial_fp32 (blast_kernels.py:2614-2664): (out, z (b,N,R), y (b,N,R))."""
    return _partial_fp32(x, U, V, S)


def triton_blast_partial_grouped_fp16(x, U, V, S, config=None):
    """Replaces triton_blast_partial_grouped_fp16 (blast_kernels.py:2762-2803)."""
    return _partial_fp16(x, U, V, S)


def triton_blast_partial_grouped_fp32(x, U, V, S):
    """Replaces triton_blast_partial_grouped_fp32 (blast_kernels.py:2710-2760)."""
    return _partial_fp32(x, U, V, S)


def triton_blast_partial_grouped_persistent_fp16(x, U, V, S, config=None):
    """Replaces triton_blast_partial_grouped_persistent_fp16 (blast_kernels.py:2858-2899)."""
    return _partial_fp16(x, U, V, S)


def triton_blast_partial_grouped_persistent_fp32(x, U, V, S):
    """Replaces triton_blast_partial_grouped_persistent_fp32 (blast_kernels.py:2806-2856)."""
    return _partial_fp32(x, U, V, S)


def triton_blast_full_fp16(x, U, V, S, config=None):
    """Replaces triton_blast_full_fp16 (blast_kernels.py:2955-2995), which the reference could not make work."""
    return _partial_fp16(x, U, V, S)


def triton_blast_full_fp32(x, U, V, S):
    """Replaces triton_blast_full_fp32 (blast_kernels.py:2902-2953)."""
    return _partial_fp32(x, U, V, S)


def triton_blast_bmm_fp16(x, U, V, S, config=(None, None, None)):
    """Replaces triton_blast_bmm_fp16 (blast_kernels.py:3043-3065)."""
    b, p, q, r = _dims_bmm(x, U, V, S)
    out = ops.blast(ops._flat2d(x), U, V, S, L.KMAJOR, L.MMAJOR, b, 1, b * b, b, p, q, r, L.FLAG_NONE)
    return ops._like_input(out, x)


def triton_blast_bmm_fp32(x, U, V, S):
    """Replaces triton_blast_bmm_fp32 (blast_kernels.py:2998-3041): (out, z (b,R,N), y (R,b,N))."""
    b, p, q, r = _dims_bmm(x, U, V, S)
    out, z, y = ops.blast_f32(ops.flat2d_f32(x), U, V, S, L.KMAJOR, L.MMAJOR, b, 1, b * b, b, p, q, r)
    return ops._like_input(out, x), z.transpose(1, 2), y.permute(2, 0, 1)


def blast_torch_layout(x, U, Vt, S, flags=L.FLAG_NONE):
    """Same operator on the reference's torch layouts (torch_funcs/blast_funcs.py:3-47):
    U (b,Q,R), Vt (b,R,P), S (b_out,b_in,R); returns out only."""
    b, r, p = Vt.shape
    b2, q, r2 = U.shape
    assert b == b2 and b != 1 and r2 == r and tuple(S.shape) == (b2, b, r)
    out = ops.blast(ops._flat2d(x), U, Vt, S, L.KMAJOR, L.KMAJOR, b * r, r, 1, b, p, q, r, flags)
    return ops._like_input(out, x)


def blast_multi_torch_layout(x, layers, x_mul=None, biases=None, residuals=None, out_act=None):
    """Several BLAST layers on one input, torch layouts: layers = [(U (b,Q,R), Vt (b,R,P), S (b,b,R)), ...] with equal
    shapes.  Optional: x_mul - the input becomes silu(x) * x_mul (a down projection fed with the gate and up results);
    biases[i] (O,) and residuals[i] (..., O) are added to layer i's result.  Returns the list of outputs.
    At decode sizes (up to 16 tokens) everything is one pair of launches (blr_blast_multi: no counterpart in the
    reference, which calls one operator per layer and separate torch kernels for the rest, models/wrappers.py:171-177);
    above that the layers run one by one, biases and residuals added by the last GEMM's epilogue.
    out_act ("gelu" | "gelu_tanh"): applied to result + bias ahead of the residual (in that epilogue above 16 tokens)."""
    U0, Vt0, S0 = layers[0]
    b, r, p = Vt0.shape
    q = U0.shape[1]
    for U, Vt, S in layers:
        assert tuple(U.shape) == (b, q, r) and tuple(Vt.shape) == (b, r, p) and tuple(S.shape) == (b, b, r), "layers must share their shapes"
        assert U.is_contiguous() and Vt.is_contiguous() and S.is_contiguous()
    x2 = ops._flat2d(x)
    xm2 = None if x_mul is None else ops._flat2d(x_mul)
    res2 = None if residuals is None else [None if t is None else ops._flat2d(t) for t in residuals]
    outs = ops.blast_multi(x2, layers, 16, 0, b, p, q, r, xm2, biases, res2, out_act) if 1 <= len(layers) <= 3 else None
    if outs is None:
        xe = x2 if xm2 is None else torch.nn.functional.silu(x2) * xm2
        if xm2 is not None and 1 <= len(layers) <= 3:   # the input transform done here, the rest may still fuse
            outs = ops.blast_multi(xe, layers, 16, 0, b, p, q, r, None, biases, res2, out_act)
    if outs is None:
        outs = []
        for i, (U, Vt, S) in enumerate(layers):
            o = ops.blast(xe, U, Vt, S, L.KMAJOR, L.KMAJOR, b * r, r, 1, b, p, q, r, L.FLAG_NONE)
            if biases is not None and biases[i] is not None:
                o += biases[i]
            if out_act is not None:
                o = torch.nn.functional.gelu(o, approximate="tanh" if out_act == "gelu_tanh" else "none")
            if res2 is not None and res2[i] is not None:
                o += res2[i]
            outs.append(o)
    return [ops._like_input(o, x) for o in outs]


def blast_output_blocks(x, U_local, Vt, S_local, flags=L.FLAG_NONE):
    """BLAST restricted to a slice of the output blocks (for sharding a layer over GPUs by output block):
    U_local (b_out,Q,R), Vt (b,R,P), S_local (b_out,b,R) contiguous; returns (..., b_out*Q)."""
    b, r, p = Vt.shape
    bo, q, r2 = U_local.shape
    assert 1 <= bo <= b and r2 == r and tuple(S_local.shape) == (bo, b, r)
    assert U_local.is_contiguous() and S_local.is_contiguous()
    out = ops.blast(ops._flat2d(x), U_local, Vt, S_local, L.KMAJOR, L.KMAJOR, b * r, r, 1, b, p, q, r, flags, bo)
    return ops._like_input(out, x)


def blast_torch_layout_host(x_host, U, Vt, S, out=None, flags=L.FLAG_NONE):
    """blast_torch_layout for activations in host memory: x_host (N, b*P) 16-bit CPU tensor (pinned for asynchronous
    copies), factors on the device.  One library call enqueues copy-in, the kernels and copy-out; the copies run on
    streams of the library so that consecutive calls overlap.  Returns the (pinned) host tensor `out` (N, b*Q),
    valid after host_flush() and a synchronisation of the current stream."""
    assert not x_host.is_cuda and x_host.dim() == 2 and x_host.stride(1) == 1
    dev = U.device
    b, r, p = Vt.shape
    b2, q, r2 = U.shape
    n = x_host.size(0)
    assert b == b2 and b != 1 and r2 == r and tuple(S.shape) == (b2, b, r) and x_host.size(1) == b * p
    assert U.dtype == x_host.dtype and Vt.dtype == x_host.dtype and S.dtype == x_host.dtype
    assert U.is_contiguous() and Vt.is_contiguous() and S.is_contiguous()
    if out is None:
        out = torch.empty((n, b * q), dtype=x_host.dtype, pin_memory=True)
    assert not out.is_cuda and out.stride(1) == 1 and tuple(out.shape) == (n, b * q) and out.dtype == x_host.dtype
    lib = L.load()
    st = L.stream_ptr(dev)
    ws = L.workspace(dev, st, lib.blr_workspace_bytes(n, b, r))
    sg = L.staging(dev, st, lib.blr_host_staging_bytes(max(n, 16), b * p, b * q))
    L.check(lib.blr_blast_host(x_host.data_ptr(), x_host.stride(0), n, L.dtype_code(x_host.dtype), U.data_ptr(), L.KMAJOR,
                               Vt.data_ptr(), L.KMAJOR, S.data_ptr(), b * r, r, 1, b, p, q, r, flags, out.data_ptr(),
                               out.stride(0), sg.data_ptr(), sg.numel(), ws.data_ptr(), ws.numel(), st))
    return out


def host_flush(device=None) -> None:
    """Makes the current stream of `device` wait for the copy-outs of all host-buffer calls issued on it."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    L.check(L.load().blr_host_flush(L.stream_ptr(dev)))


# The reference exposes its autotuner's winning configuration (blast_kernels.py:3068-3086) and pickles
# it (layer.py:310-326).  Tile shapes here are fixed at build time, so there is nothing to report.
def get_triton_blast_partial_fp16_config():
    return None


def get_triton_blast_partial_grouped_fp16_config():
    return None


def get_triton_blast_partial_grouped_persistent_fp16_config():
    return None


def get_triton_blast_full_fp16_config():
    return None


def get_triton_blast_bmm_xv_fp16_config():
    return None


def get_triton_blast_bmm_sxv_fp16_config():
    return None


def get_triton_blast_bmm_usxv_fp16_config():
    return None
