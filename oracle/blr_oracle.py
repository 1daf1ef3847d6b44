"""CPU restatement of the reference's structured matmuls (TEST INFRASTRUCTURE, not product).

Every function here restates, as explicit einsums over fp32 CPU tensors, the arithmetic of
one function of the reference's PyTorch path (``torch_funcs/*.py``).  The restatement is
pinned against outputs of the reference itself: ``tests/golden/make_golden.py`` imports the
reference's functions, runs them on seeded inputs and stores inputs + outputs under
``tests/golden/*.npz``; ``tests/test_oracle.py`` checks these functions against them.

Index conventions (same letters as the reference):
  N tokens, I in_features, O out_features, b blocks, P = I/b, Q = O/b, R rank.
  input feature  = j*P + p   (block j, offset p)
  output feature = i*Q + q   (block i, offset q)   for BLAST / low-rank / dense
  output feature = s*L + l   (block index fastest) for Monarch
"""
from __future__ import annotations

import numpy as np
import torch


# --------------------------------------------------------------------------- helpers
def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(device="cpu", dtype=torch.float32)


def rel_fro(got: torch.Tensor, ref: torch.Tensor) -> float:
    """Relative Frobenius error ||got-ref||_F / ||ref||_F in float64."""
    g = got.detach().cpu().double().reshape(-1)
    r = ref.detach().cpu().double().reshape(-1)
    den = float(torch.linalg.vector_norm(r))
    num = float(torch.linalg.vector_norm(g - r))
    return num / den if den > 0 else num


# --------------------------------------------------------------------------- BLAST
def blast(x, U, Vt, S):
    """BLAST matmul; follows reference torch_funcs/blast_funcs.py:3-47 (torch_blast_baseline).

    x (..., I); U (b, Q, R); Vt (b, R, P); S (b_out, b_in, R).
    Returns (out (..., O), z (b, N, R), y (b, N, R)) in fp32.
      y[j,n,r] = sum_p x[n, j*P+p] * Vt[j,r,p]          (blast_funcs.py:40)
      z[i,n,r] = sum_j S[i,j,r] * y[j,n,r]               (blast_funcs.py:41-42)
      out[n, i*Q+q] = sum_r z[i,n,r] * U[i,q,r]          (blast_funcs.py:44-45)
    """
    x, U, Vt, S = _f32(x), _f32(U), _f32(Vt), _f32(S)
    b1, R, P = Vt.shape
    b2, Q, _ = U.shape
    assert b1 == b2 and b1 != 1, "reference asserts b1 == b2 and b != 1 (blast_funcs.py:33-34)"
    lead = x.shape[:-1]
    xb = x.reshape(-1, b1, P)                               # (N, j, p)
    y = torch.einsum("njp,jrp->jnr", xb, Vt)
    z = torch.einsum("ijr,jnr->inr", S, y)
    o = torch.einsum("inr,iqr->niq", z, U)
    return o.reshape(*lead, b2 * Q), z, y


def blast_bmm(x, U, Vt, S_rij):
    """Three-bmm BLAST; follows torch_funcs/blast_funcs.py:49-91 (torch_blast_bmm).

    Same as :func:`blast` but S is given as (R, b_out, b_in) and z is returned as (R, N, b_out).
    """
    S = _f32(S_rij).permute(1, 2, 0)
    out, z, y = blast(x, U, Vt, S)
    return out, z.permute(2, 1, 0).contiguous(), y


def blast_act_int8(x, U, Vt, S):
    """Activation-rounded BLAST; restates triton_funcs/blast_sym_quant_kernels.py:105-108, 227-230.

    The reference's "int8" BLAST keeps bf16 weights and rounds the two intermediates to the
    nearest integer (ties to even), clamped to [-128, 127], with no scale.
    Returns (out, z_int8 (b,N,R), y_int8 (b,N,R)).
    """
    x, U, Vt, S = _f32(x), _f32(U), _f32(Vt), _f32(S)
    b, R, P = Vt.shape
    Q = U.shape[1]
    lead = x.shape[:-1]
    xb = x.reshape(-1, b, P)
    y = torch.einsum("njp,jrp->jnr", xb, Vt)
    y8 = torch.clamp(torch.round(y), -128, 127)
    z = torch.einsum("ijr,jnr->inr", S, y8)
    z8 = torch.clamp(torch.round(z), -128, 127)
    o = torch.einsum("inr,iqr->niq", z8, U)
    return o.reshape(*lead, b * Q), z8.to(torch.int8), y8.to(torch.int8)


# --------------------------------------------------------------------------- Monarch
def monarch(x, w1_t, w2_t):
    """Monarch matmul; follows torch_funcs/monarch_funcs.py:4-45 (torch_monarch_baseline).

    x (..., I); w1_t (k, q, p) with k*p == I; w2_t (l, s, r) with l*r == k*q.
    Returns (out2 (..., s*l), pre_out2 (l,N,s), out1 (l,N,r), pre_out1 (k,N,q)).
      pre_out1[k,n,q]  = sum_p x[n, k*p_+p] w1_t[k,q,p]           (monarch_funcs.py:40)
      out1[l,n,r]      = pre_out1 flattened over (k,q) at f = r*L + l  (monarch_funcs.py:41)
      pre_out2[l,n,s]  = sum_r out1[l,n,r] w2_t[l,s,r]            (monarch_funcs.py:43)
      out2[n, s*L + l] = pre_out2[l,n,s]                           (monarch_funcs.py:44)
    """
    x, w1_t, w2_t = _f32(x), _f32(w1_t), _f32(w2_t)
    k, q, p = w1_t.shape
    l, s, r = w2_t.shape
    assert k * p == x.shape[-1] and l * r == k * q
    lead = x.shape[:-1]
    xb = x.reshape(-1, k, p)
    n = xb.shape[0]
    pre1 = torch.einsum("nkp,kqp->knq", xb, w1_t)
    flat = pre1.permute(1, 0, 2).reshape(n, k * q)          # f = k*q_ + q
    out1 = flat.reshape(n, r, l).permute(2, 0, 1).contiguous()   # f = r*L + l
    pre2 = torch.einsum("lnr,lsr->lns", out1, w2_t)
    out2 = pre2.permute(1, 2, 0).reshape(*lead, s * l)
    return out2, pre2, out1, pre1


# --------------------------------------------------------------------------- low rank / dense
def low_rank(x, Vt, Ut):
    """x Vt^T Ut^T; follows torch_funcs/low_rank_funcs.py:4-28. Vt (R, I), Ut (O, R). Returns (out, z)."""
    x, Vt, Ut = _f32(x), _f32(Vt), _f32(Ut)
    z = torch.einsum("...i,ri->...r", x, Vt)
    return torch.einsum("...r,or->...o", z, Ut), z


def dense(x, Wt):
    """x Wt^T; follows torch_funcs/dense_funcs.py:4-25. Wt (O, I)."""
    return torch.einsum("...i,oi->...o", _f32(x), _f32(Wt))


# --------------------------------------------------------------------------- layout converters
# The reference's harness builds each kernel-side layout from the torch layout (layer.py:191-201,
# 217-226, 246-251, 264-267).  These restate those conversions so tests can feed both sides.
def blast_to_partial_layout(U, Vt, S):
    """torch (U (b,Q,R), Vt (b,R,P), S (bo,bi,R)) -> partial-family (U (b,R,Q), V (b,P,R), S (bi,bo,R)); layer.py:195-197."""
    return U.transpose(1, 2).contiguous(), Vt.transpose(1, 2).contiguous(), S.transpose(0, 1).contiguous()


def blast_to_bmm_layout(U, Vt, S):
    """torch -> bmm-family (U (b,Q,R), V (b,P,R), S (R,bo,bi)); layer.py:199-201."""
    return U.contiguous(), Vt.transpose(1, 2).contiguous(), S.permute(2, 0, 1).contiguous()


def monarch_w1_to_kernel_layout(w1_t):
    """torch w1_t (b, rank, P) -> kernel w1 (b, P, rank) with columns regrouped so that column
    l*PER + jj holds torch column jj*b + l (PER = rank/b); layer.py:221-224."""
    b, rank, P = w1_t.shape
    per = rank // b
    w = w1_t.transpose(1, 2).contiguous().view(b, P, per, b).permute(0, 1, 3, 2)
    return w.reshape(b, P, rank).contiguous()


def monarch_w2_to_left_layout(w2_t):
    """torch w2_t (b, Q, rank) -> (b, rank, Q); layer.py:226."""
    return w2_t.transpose(1, 2).contiguous()


def monarch_ideal_order(out2, b):
    """Re-order an interleaved Monarch output (feature s*b + l) into the block-major order
    (feature l*S + s) that the reference's right_ideal variant emits (monarch_kernels.py:1004)."""
    lead = out2.shape[:-1]
    S_ = out2.shape[-1] // b
    return out2.reshape(*lead, S_, b).transpose(-1, -2).reshape(*lead, S_ * b)


# --------------------------------------------------------------------------- weight quantiser
# Not in the reference (its "sym_quant" rounds activations).  Spec: symmetric, per output
# channel (group=0) or per group of `group` elements along the contraction (last) axis;
# scale = max|w| / qmax stored as fp16; q = clamp(rint(w / scale), -qmax, qmax); int4 values
# packed two per byte along the contraction axis, even index in the low nibble, as unsigned
# nibbles of the two's complement value.
def quantize_sym(w: torch.Tensor, bits: int, group: int = 0):
    """Returns (q, scale): q int8 (..., K) for bits=8, uint8 (..., K/2) for bits=4;
    scale fp16 (..., ) for group=0 else (..., K/group)."""
    assert bits in (8, 4)
    qmax = 127 if bits == 8 else 7
    wf = _f32(w)
    K = wf.shape[-1]
    g = K if group == 0 else group
    assert K % g == 0
    wg = wf.reshape(*wf.shape[:-1], K // g, g)
    amax = wg.abs().amax(dim=-1)
    scale = (amax / qmax).to(torch.float16)
    sf = scale.float()
    safe = torch.where(sf > 0, sf, torch.ones_like(sf))
    q = torch.clamp(torch.round(wg / safe.unsqueeze(-1)), -qmax, qmax)
    q = torch.where(sf.unsqueeze(-1) > 0, q, torch.zeros_like(q)).reshape(wf.shape).to(torch.int8)
    if group == 0:
        scale = scale.squeeze(-1)
    if bits == 4:
        q = pack_int4(q)
    return q, scale


def pack_int4(q: torch.Tensor) -> torch.Tensor:
    """int8 values in [-8, 7], even count along the last axis -> uint8, low nibble = even index."""
    u = (q.to(torch.int16) & 0xF).to(torch.uint8)
    return (u[..., 0::2] | (u[..., 1::2] << 4)).contiguous()


def unpack_int4(p: torch.Tensor) -> torch.Tensor:
    lo = (p & 0xF).to(torch.int8)
    hi = (p >> 4).to(torch.int8)
    lo = torch.where(lo > 7, lo - 16, lo)
    hi = torch.where(hi > 7, hi - 16, hi)
    return torch.stack([lo, hi], dim=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)


def dequantize_sym(q: torch.Tensor, scale: torch.Tensor, bits: int, group: int = 0) -> torch.Tensor:
    """fp32 weights q * scale ("identically dequantised weights")."""
    qi = unpack_int4(q) if bits == 4 else q
    qf = qi.float()
    K = qf.shape[-1]
    if group == 0:
        return qf * scale.float().unsqueeze(-1)
    return (qf.reshape(*qf.shape[:-1], K // group, group) * scale.float().unsqueeze(-1)).reshape(qf.shape)


def blast_wq(x, Uq, U_scale, Vq, V_scale, S, bits: int, group: int = 0):
    """Weight-quantised BLAST = :func:`blast` on the dequantised factors.
    Uq over (b,Q,R) with scales (b,Q[,R/group]); Vq over (b,R,P) with scales (b,R[,P/group])."""
    U = dequantize_sym(Uq, U_scale, bits, group)
    Vt = dequantize_sym(Vq, V_scale, bits, group)
    return blast(x, U, Vt, S)


# --------------------------------------------------------------------------- seeded inputs
def make_blast_inputs(N, I, O, b, R, dtype=torch.float16, seed=0, lead=None):
    """Seeded factors with the distributions of the headline configuration:
    U, Vt ~ N(0, 1/sqrt(fan_in)), S ~ U(0.5, 1.5), x ~ N(0, 1); generated in fp32 then cast."""
    g = torch.Generator().manual_seed(seed)
    P, Q = I // b, O // b
    U = (torch.randn(b, Q, R, generator=g) / R ** 0.5).to(dtype)
    Vt = (torch.randn(b, R, P, generator=g) / P ** 0.5).to(dtype)
    S = (torch.rand(b, b, R, generator=g) + 0.5).to(dtype)
    shape = (1, N, I) if lead is None else (*lead, I)
    x = torch.randn(*shape, generator=g).to(dtype)
    return x, U, Vt, S


def make_monarch_inputs(N, I, O, b, rank, dtype=torch.float16, seed=0):
    g = torch.Generator().manual_seed(seed)
    w1_t = (torch.randn(b, rank, I // b, generator=g) / (I // b) ** 0.5).to(dtype)
    w2_t = (torch.randn(b, O // b, rank, generator=g) / rank ** 0.5).to(dtype)
    x = torch.randn(1, N, I, generator=g).to(dtype)
    return x, w1_t, w2_t


def make_low_rank_inputs(N, I, O, R, dtype=torch.float16, seed=0):
    g = torch.Generator().manual_seed(seed)
    Vt = (torch.randn(R, I, generator=g) / I ** 0.5).to(dtype)
    Ut = (torch.randn(O, R, generator=g) / R ** 0.5).to(dtype)
    x = torch.randn(1, N, I, generator=g).to(dtype)
    return x, Vt, Ut


def make_dense_inputs(N, I, O, dtype=torch.float16, seed=0):
    g = torch.Generator().manual_seed(seed)
    Wt = (torch.randn(O, I, generator=g) / I ** 0.5).to(dtype)
    x = torch.randn(1, N, I, generator=g).to(dtype)
    return x, Wt
