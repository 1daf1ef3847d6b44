"""GPU parity of the weight-streaming path (1..16 tokens) against the CPU oracle, through the C ABI.

Tolerance: relative Frobenius error <= 1e-2 against the fp32 oracle evaluated on the same 16-bit
inputs (the acceptance bound of the headline configuration); typical errors are ~1e-3.
"""
import os

import numpy as np
import pytest
import torch

from oracle import blr_oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-2
DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import mem_efficient_blr_b200.blast_kernels as bk
    import mem_efficient_blr_b200.blast_sym_quant_kernels as bq
    import mem_efficient_blr_b200.dense_kernels as dk
    import mem_efficient_blr_b200.low_rank_kernels as lk
    import mem_efficient_blr_b200.monarch_kernels as mk
    from mem_efficient_blr_b200 import _lib

    class NS:
        pass

    ns = NS()
    ns.bk, ns.bq, ns.dk, ns.lk, ns.mk, ns.lib = bk, bq, dk, lk, mk, _lib
    return ns


def _cuda(*ts):
    return [t.to(DEV) for t in ts]


def _sync_ok(K):
    torch.cuda.synchronize()
    K.lib.workspace_status(torch.device(DEV))


BLAST_SHAPES = [
    # N, I, O, b, R
    (1, 256, 384, 4, 128),
    (5, 768, 768, 3, 128),        # the reference's ViT setting b=3
    (16, 768, 3072, 16, 192),     # P=48, Q=192
    (8, 4096, 11008, 16, 1024),   # headline layer, Q=688 is not a multiple of 32
    (16, 4096, 11008, 16, 1024),
    (1, 11008, 4096, 16, 1488),   # down_proj with the reference's 50%-parameter rank
    (3, 1152, 2304, 6, 192),      # six blocks: a cluster of 6 CTAs
    (16, 2304, 3456, 9, 384),     # nine blocks, beyond the portable cluster size
    (2, 3456, 1152, 9, 256),
    (13, 768, 1152, 3, 384),      # odd block count with two token tiles and a ragged second tile
    (11, 1152, 2304, 6, 384),
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", BLAST_SHAPES)
def test_blast_all_layout_families(K, shape, dtype):
    N, I, O, b, R = shape
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, dtype, seed=N + R)
    ref, _, _ = orc.blast(x, U, Vt, S)
    xd, Ud, Vtd, Sd = _cuda(x, U, Vt, S)
    got = K.bk.blast_torch_layout(xd, Ud, Vtd, Sd)
    _sync_ok(K)
    assert got.shape == ref.shape and got.dtype == dtype
    assert orc.rel_fro(got.float().cpu(), ref) < TOL
    Up, Vp, Sp = _cuda(*orc.blast_to_partial_layout(U, Vt, S))
    for fn in (K.bk.triton_blast_partial_fp16, K.bk.triton_blast_partial_grouped_fp16,
               K.bk.triton_blast_partial_grouped_persistent_fp16, K.bk.triton_blast_full_fp16):
        got = fn(xd, Up, Vp, Sp)
        _sync_ok(K)
        assert orc.rel_fro(got.float().cpu(), ref) < TOL, fn.__name__
    Ub, Vb, Sb = _cuda(*orc.blast_to_bmm_layout(U, Vt, S))
    got = K.bk.triton_blast_bmm_fp16(xd, Ub, Vb, Sb)
    _sync_ok(K)
    assert orc.rel_fro(got.float().cpu(), ref) < TOL


@pytest.mark.parametrize("tag", ["a", "b"])
def test_blast_reference_golden_vectors(K, golden_dir, tag):
    g = {k: torch.from_numpy(v) for k, v in np.load(os.path.join(golden_dir, f"blast_{tag}.npz")).items()}
    x, U, Vt, S = (g[k].to(torch.bfloat16) for k in ("x", "U", "Vt", "S"))
    ref, _, _ = orc.blast(x, U, Vt, S)
    got = K.bk.blast_torch_layout(*_cuda(x, U, Vt, S))
    _sync_ok(K)
    assert got.shape == g["out"].shape
    assert orc.rel_fro(got.float().cpu(), ref) < TOL
    # and against the reference's own fp32 output: only the bf16 rounding of the inputs separates them
    assert orc.rel_fro(got.float().cpu(), g["out"]) < 3e-2


def test_blast_non_contiguous_x_and_leading_dims(K):
    x, U, Vt, S = orc.make_blast_inputs(6, 512, 256, 4, 64, torch.float16, seed=9, lead=(2, 3))
    big = torch.zeros(2, 3, 1024, dtype=torch.float16)
    big[..., :512] = x
    xv = big.to(DEV)[..., :512]          # row stride 1024, not contiguous
    ref, _, _ = orc.blast(x, U, Vt, S)
    got = K.bk.blast_torch_layout(xv, *_cuda(U, Vt, S))
    _sync_ok(K)
    assert got.shape == (2, 3, 256)
    assert orc.rel_fro(got.float().cpu(), ref) < TOL


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 512, 768, 4, 256), (4, 4096, 11008, 16, 1024), (16, 4096, 11008, 16, 1024),
                                   (1, 4096, 11008, 16, 1024)])
def test_blast_weight_quantised(K, shape, dtype, bits):
    N, I, O, b, R = shape
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, dtype, seed=bits + N)
    Uq, us = orc.quantize_sym(U, bits)
    Vq, vs = orc.quantize_sym(Vt, bits)
    ref, _, _ = orc.blast_wq(x, Uq, us, Vq, vs, S, bits)
    # device quantiser must agree bit for bit with the oracle's
    dUq, dus, dVq, dvs = K.bq.quantize_blast_factors(U.to(DEV), Vt.to(DEV), bits)
    assert torch.equal(dus.cpu(), us) and torch.equal(dvs.cpu(), vs)
    assert torch.equal(dUq.cpu(), Uq) and torch.equal(dVq.cpu(), Vq)
    got = K.bq.blast_wq(x.to(DEV), dUq, dus, dVq, dvs, S.to(DEV), bits)
    _sync_ok(K)
    assert got.shape == ref.shape
    assert orc.rel_fro(got.float().cpu(), ref) < TOL


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("shape", [(1, 4096, 11008, 16, 1024), (7, 4096, 11008, 16, 1024), (16, 4096, 11008, 16, 1024),
                                   (3, 1024, 1536, 4, 384), (2, 2048, 1024, 8, 256)])
def test_blast_weight_quantised_per_group_scales(K, shape, bits):
    """One scale per 128 contraction indices: device quantiser bit-exact against the oracle's, output against the
    oracle on the identically dequantised factors; on the cluster kernel (<= 8 tokens) and the grid-wide one."""
    N, I, O, b, R = shape
    G = 128
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=100 + bits + N)
    # spread the magnitudes of the groups so that a per-channel scale would not do
    U = (U.float() * (1 + 3 * torch.rand(b, O // b, R // G, 1).expand(-1, -1, -1, G).reshape(b, O // b, R))).half()
    Uq, us = orc.quantize_sym(U, bits, G)
    Vq, vs = orc.quantize_sym(Vt, bits, G)
    assert us.shape == (b, O // b, R // G) and vs.shape == (b, R, I // b // G)
    ref, _, _ = orc.blast_wq(x, Uq, us, Vq, vs, S, bits, G)
    dUq, dus, dVq, dvs = K.bq.quantize_blast_factors(U.to(DEV), Vt.to(DEV), bits, G)
    assert torch.equal(dus.cpu(), us) and torch.equal(dvs.cpu(), vs)
    assert torch.equal(dUq.cpu(), Uq) and torch.equal(dVq.cpu(), Vq)
    lib = K.lib.load()
    try:
        for path in (0, 1, 2):   # automatic (two-launch path up to 4 tokens), grid-wide kernel, cluster kernel
            assert lib.blr_debug_decode_path(path) == 0
            got = K.bq.blast_wq(x.to(DEV), dUq, dus, dVq, dvs, S.to(DEV), bits, G)
            _sync_ok(K)
            assert got.shape == ref.shape
            assert orc.rel_fro(got.float().cpu(), ref) < TOL, f"path {path}"
    finally:
        assert lib.blr_debug_decode_path(0) == 0


def test_blast_weight_quantised_rejects_other_group_widths(K):
    x, U, Vt, S = orc.make_blast_inputs(1, 512, 768, 4, 256, torch.float16, seed=5)
    q = K.bq.quantize_blast_factors(U.to(DEV), Vt.to(DEV), 8, 64)
    with pytest.raises(RuntimeError, match="group"):
        K.bq.blast_wq(x.to(DEV), *q, S.to(DEV), 8, 64)


@pytest.mark.parametrize("path", [1, 2])
def test_small_batches_on_the_other_decode_kernels(K, path):
    """BLAST on few tokens normally takes the two-launch path; the cluster kernel (path 2: what runs for the layouts
    and token counts that path does not take) and the grid-wide streaming kernel (path 1: what runs when a shape does
    not fit a cluster) must give the same answers."""
    lib = K.lib.load()
    assert lib.blr_debug_decode_path(path) == 0
    try:
        for N, I, O, b, R, bits in [(1, 4096, 11008, 16, 1024, 16), (5, 768, 768, 3, 128, 16),
                                    (4, 4096, 11008, 16, 1024, 8), (1, 4096, 11008, 16, 1024, 4),
                                    (16, 4096, 11008, 16, 1024, 8), (12, 768, 3072, 4, 192, 16)]:
            x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=N + bits)
            if bits == 16:
                ref, _, _ = orc.blast(x, U, Vt, S)
                got = K.bk.blast_torch_layout(*_cuda(x, U, Vt, S))
            else:
                Uq, us = orc.quantize_sym(U, bits)
                Vq, vs = orc.quantize_sym(Vt, bits)
                ref, _, _ = orc.blast_wq(x, Uq, us, Vq, vs, S, bits)
                got = K.bq.blast_wq(*_cuda(x, Uq, us, Vq, vs, S), bits)
            _sync_ok(K)
            assert orc.rel_fro(got.float().cpu(), ref) < TOL, (N, I, O, b, R, bits)
    finally:
        assert lib.blr_debug_decode_path(0) == 0


def test_blast_act_int8_matches_reference_rounding(K):
    x, U, Vt, S = orc.make_blast_inputs(4, 512, 768, 4, 128, torch.bfloat16, seed=21)
    x = x * 4  # spread the intermediates over the int8 range
    ref, z8, y8 = orc.blast_act_int8(x, U, Vt, S)
    Ub, Vb, Sb = _cuda(*orc.blast_to_bmm_layout(U, Vt, S))
    got = K.bq.triton_blast_bmm_int8_fp16(x.to(DEV), Ub, Vb, Sb)
    _sync_ok(K)
    # rounding ties may flip single intermediates by one unit; the output stays within the bound
    assert orc.rel_fro(got.float().cpu(), ref) < 3e-2


@pytest.mark.parametrize("N", [1, 4, 16])
def test_blast_act_int8_intermediates_on_the_headline_layer(K, N):
    """The reference's activation rounding (blast_sym_quant_kernels.py:105-108, 227-230) on the 4096 -> 11008 layer.
    z is read back from the operator's workspace where the kernel leaves it (two-launch path and tensor-core pipeline
    keep it as (block, token, rank) 16-bit values): it must hold integers in [-128, 127] that equal the oracle's
    except where a product landed within rounding distance of a half-integer.  One unit of y moves z by S_ij <= 1.5, so
    z may differ by up to 2 at such points; they must stay rare.  The output bound follows from the share of moved
    intermediates measured here (a unit error in about 1 % of them is a relative error of about 0.1 / 37 per entry)."""
    I, O, b, R = 4096, 11008, 16, 1024
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.bfloat16, seed=77 + N)
    x = x * 2
    ref, z8, y8 = orc.blast_act_int8(x, U, Vt, S)
    from mem_efficient_blr_b200 import _lib as L
    got = K.bk.blast_torch_layout(*_cuda(x, U, Vt, S), flags=L.FLAG_ACT_INT8)
    _sync_ok(K)
    err = orc.rel_fro(got.float().cpu(), ref)
    assert err < 1e-2, err
    if N <= 16:  # the two-launch path: z sits at the start of the 2-byte region of the workspace
        lib = K.lib.load()
        dev = torch.device(DEV)
        ws = L.workspace(dev, L.stream_ptr(dev), lib.blr_workspace_bytes(N, b, R))
        off = 1024 + (2 << 20) + ((b * N * R * 4 + 255) // 256) * 256
        z = ws[off: off + b * N * R * 2].view(torch.bfloat16).reshape(b, N, R).float().cpu()
        assert torch.equal(z, z.round()) and z.abs().max() <= 128
        d = (z - z8.float().reshape(b, N, R)).abs()
        assert d.max() <= 2 and (d > 0).float().mean() < 0.02, (float(d.max()), float((d > 0).float().mean()))


MONARCH_SHAPES = [(1, 256, 512, 4, 64), (7, 768, 3072, 4, 768), (16, 4096, 4096, 16, 1024), (3, 4096, 11008, 16, 1536),
                  # four blocks on the Llama-7B projections (ranks for about half of the dense parameters)
                  (1, 4096, 4096, 4, 1024), (16, 4096, 11008, 4, 1536), (1, 11008, 4096, 4, 1536)]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", MONARCH_SHAPES)
def test_monarch_all_variants(K, shape, dtype):
    N, I, O, b, rank = shape
    x, w1_t, w2_t = orc.make_monarch_inputs(N, I, O, b, rank, dtype, seed=N)
    ref, _, out1, _ = orc.monarch(x, w1_t, w2_t)
    xd = x.to(DEV)
    got = K.mk.monarch_torch_layout(xd, w1_t.to(DEV), w2_t.to(DEV))
    _sync_ok(K)
    assert orc.rel_fro(got.float().cpu(), ref) < TOL
    w1k = orc.monarch_w1_to_kernel_layout(w1_t).to(DEV)
    got = K.mk.triton_monarch_right_fp16(xd, w1k, w2_t.to(DEV))
    _sync_ok(K)
    assert got.shape == ref.shape and orc.rel_fro(got.float().cpu(), ref) < TOL
    got = K.mk.triton_monarch_right_left_fp16(xd, w1k, orc.monarch_w2_to_left_layout(w2_t).to(DEV))
    _sync_ok(K)
    assert orc.rel_fro(got.float().cpu(), ref) < TOL
    got = K.mk.triton_monarch_right_ideal_fp16(xd, w1k, w2_t.to(DEV))
    _sync_ok(K)
    assert orc.rel_fro(got.float().cpu(), orc.monarch_ideal_order(ref, b)) < TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 256, 384, 64), (16, 4096, 11008, 1024), (5, 11008, 4096, 1024)])
def test_low_rank(K, shape, dtype):
    N, I, O, R = shape
    x, Vt, Ut = orc.make_low_rank_inputs(N, I, O, R, dtype, seed=N)
    ref, _ = orc.low_rank(x, Vt, Ut)
    got = K.lk.low_rank_torch_layout(x.to(DEV), Vt.to(DEV), Ut.to(DEV))
    _sync_ok(K)
    assert orc.rel_fro(got.float().cpu(), ref) < TOL
    got = K.lk.triton_low_rank_fp16(x.to(DEV), Vt.t().contiguous().to(DEV), Ut.t().contiguous().to(DEV))
    _sync_ok(K)
    assert got.shape == (N, O)  # 2-D like the reference
    assert orc.rel_fro(got.float().cpu(), ref.reshape(N, O)) < TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 256, 384), (16, 4096, 11008), (3, 11008, 4096)])
def test_dense(K, shape, dtype):
    N, I, O = shape
    x, Wt = orc.make_dense_inputs(N, I, O, dtype, seed=N)
    ref = orc.dense(x, Wt)
    got = K.dk.dense_torch_layout(x.to(DEV), Wt.to(DEV))
    torch.cuda.synchronize()
    assert orc.rel_fro(got.float().cpu(), ref) < TOL
    got = K.dk.triton_dense_fp16(x.to(DEV), Wt.t().contiguous().to(DEV))
    torch.cuda.synchronize()
    assert got.shape == (N, O) and orc.rel_fro(got.float().cpu(), ref.reshape(N, O)) < TOL


def test_empty_batches_return_empty_outputs(K):
    """Zero tokens (a rank whose token slice is empty) is valid on every operator family and through the C ABI."""
    _, U, Vt, S = orc.make_blast_inputs(1, 512, 768, 4, 128, torch.float16, seed=1)
    x0 = torch.empty(0, 512, dtype=torch.float16, device=DEV)
    assert K.bk.blast_torch_layout(x0, *_cuda(U, Vt, S)).shape == (0, 768)
    q = K.bq.quantize_blast_factors(U.to(DEV), Vt.to(DEV), 8)
    assert K.bq.blast_wq(x0, *q, S.to(DEV), 8).shape == (0, 768)
    Wt = torch.randn(768, 512, dtype=torch.float16, device=DEV)
    assert K.dk.dense_torch_layout(x0, Wt).shape == (0, 768)
    lib = K.lib.load()
    assert lib.blr_dense(None, 512, 0, 0, Wt.data_ptr(), 0, 512, 768, None, 768, None) == 0
    assert lib.blr_blast(None, 512, 0, 0, U.to(DEV).data_ptr(), 0, Vt.to(DEV).data_ptr(), 0, S.to(DEV).data_ptr(), 4 * 128,
                         128, 1, 4, 128, 192, 128, 0, None, 768, None, 0, None) == 0


@pytest.mark.parametrize("bits", [8, 4])
def test_host_buffer_entry_point(K, bits):
    """x and out in pinned host memory, factors on the device: one call copies in, computes and copies out."""
    N, I, O, b, R = 5, 4096, 11008, 16, 1024
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=40 + bits)
    Uq, us = orc.quantize_sym(U, bits)
    Vq, vs = orc.quantize_sym(Vt, bits)
    ref, _, _ = orc.blast_wq(x, Uq, us, Vq, vs, S, bits)
    xh = x.reshape(N, I).pin_memory()
    dq = _cuda(Uq, us, Vq, vs, S)
    out = K.bq.blast_wq_host(xh, *dq, bits)
    K.bq.host_flush()
    _sync_ok(K)
    assert not out.is_cuda and out.shape == (N, O)
    assert orc.rel_fro(out.float(), ref.reshape(N, O)) < TOL
    # a strided host view (rows 2*I apart) and a caller-provided output
    wide = torch.zeros(N, 2 * I, dtype=torch.float16).pin_memory()
    wide[:, :I] = xh
    out2 = torch.empty(N, O, dtype=torch.float16).pin_memory()
    got = K.bq.blast_wq_host(wide[:, :I], *dq, bits, out=out2)
    K.bq.host_flush()
    _sync_ok(K)
    # the slices' partial sums meet in fp32 atomics, whose order varies from run to run: equal up to the last bit
    assert got is out2 and orc.rel_fro(out2.float(), out.float()) < 1e-3
    # a burst of calls with changing token counts through the ring of staging slots
    outs = [torch.empty(n, O, dtype=torch.float16).pin_memory() for n in (1, 5, 3, 5, 1, 2, 5, 4, 5)]
    for o in outs:
        K.bq.blast_wq_host(xh[: o.shape[0]], *dq, bits, out=o)
    K.bq.host_flush()
    _sync_ok(K)
    for o in outs:
        assert orc.rel_fro(o.float(), out[: o.shape[0]].float()) < 1e-3
    # the prepared call: same entry point, arguments converted once
    call = K.bq.BlastWqHostCall(*dq, bits)
    outs = [torch.empty(n, O, dtype=torch.float16).pin_memory() for n in (5, 1, 4)]
    for o in outs:
        assert call(xh[: o.shape[0]], o) is o
    K.bq.host_flush()
    _sync_ok(K)
    for o in outs:
        assert orc.rel_fro(o.float(), out[: o.shape[0]].float()) < 1e-3
    with pytest.raises((AssertionError, RuntimeError)):  # (the C++ operator reports a RuntimeError)
        call(xh[:, : I // 2], outs[0])


def test_host_buffer_entry_point_16_bit(K):
    for N in (3, 40):  # streaming / cluster kernel, and the tensor-core pipeline
        x, U, Vt, S = orc.make_blast_inputs(N, 768, 3072, 4, 192, torch.bfloat16, seed=N)
        ref, _, _ = orc.blast(x, U, Vt, S)
        out = K.bk.blast_torch_layout_host(x.reshape(N, 768).pin_memory(), *_cuda(U, Vt, S))
        K.bk.host_flush()
        _sync_ok(K)
        assert orc.rel_fro(out.float(), ref.reshape(N, 3072)) < TOL


def test_repeated_calls_reuse_the_workspace(K):
    """The grid-barrier words re-arm themselves: 50 back-to-back calls give the same answer."""
    x, U, Vt, S = orc.make_blast_inputs(16, 1024, 1024, 4, 256, torch.float16, seed=2)
    ref, _, _ = orc.blast(x, U, Vt, S)
    args = _cuda(x, U, Vt, S)
    outs = [K.bk.blast_torch_layout(*args) for _ in range(50)]
    _sync_ok(K)
    for o in (outs[0], outs[-1]):
        assert orc.rel_fro(o.float().cpu(), ref) < TOL
    assert orc.rel_fro(outs[-1].float().cpu(), outs[0].float().cpu()) < 1e-3


def test_two_launch_path_is_bitwise_reproducible(K):
    """Up to 4 tokens (8 with 16-bit factors) every sum has a fixed order: repeated calls agree bit for bit."""
    for bits, N in ((16, 1), (16, 8), (8, 1), (8, 4), (4, 3)):
        x, U, Vt, S = orc.make_blast_inputs(N, 4096, 11008, 16, 1024, torch.float16, seed=N)
        if bits == 16:
            args = _cuda(x, U, Vt, S)
            outs = [K.bk.blast_torch_layout(*args) for _ in range(4)]
        else:
            q = K.bq.quantize_blast_factors(U.to(DEV), Vt.to(DEV), bits)
            xd, Sd = _cuda(x, S)
            outs = [K.bq.blast_wq(xd, *q, Sd, bits) for _ in range(4)]
        _sync_ok(K)
        for o in outs[1:]:
            assert torch.equal(o, outs[0]), (bits, N)


def test_timeout_status_is_reported_and_cleared(K):
    """A kernel that gives up on a device-side wait leaves a non-zero status word in the workspace.  No wait is made
    to run out here: the word is written from the host, as a kernel would have left it, and the host side must
    report BLR_ERR_TIMEOUT, and after blr_workspace_init report success and compute correctly again."""
    from mem_efficient_blr_b200 import _lib as L
    x, U, Vt, S = orc.make_blast_inputs(2, 512, 768, 4, 128, torch.float16, seed=8)
    args = _cuda(x, U, Vt, S)
    K.bk.blast_torch_layout(*args)
    _sync_ok(K)
    dev = torch.device(DEV)
    st = L.stream_ptr(dev)
    lib = K.lib.load()
    ws = L.workspace(dev, st, lib.blr_workspace_bytes(2, 4, 128))
    for word in (3, 255):   # grid-wide kernel's status, cluster / two-launch kernels' status
        ws[4 * word: 4 * word + 4].copy_(torch.tensor([1, 0, 0, 0], dtype=torch.uint8))
        torch.cuda.synchronize()
        assert lib.blr_workspace_status(ws.data_ptr(), st) == -7
        assert b"gave up" in lib.blr_last_error()
        with pytest.raises(RuntimeError):
            ws[4 * word: 4 * word + 4].copy_(torch.tensor([1, 0, 0, 0], dtype=torch.uint8))
            torch.cuda.synchronize()
            L.workspace_status(dev)      # raises and re-initialises the workspace
        assert lib.blr_workspace_status(ws.data_ptr(), st) == 0
        got = K.bk.blast_torch_layout(*args)
        _sync_ok(K)
        assert orc.rel_fro(got.float().cpu(), orc.blast(x, U, Vt, S)[0]) < TOL


def test_non_contiguous_factors_are_refused(K):
    """A transposed view has the right shape but the wrong strides for the packed layouts the library reads."""
    x, Wt = orc.make_dense_inputs(3, 256, 256, torch.float16, seed=3)
    xd, Wd = _cuda(x, Wt)
    with pytest.raises((AssertionError, RuntimeError), match="contiguous"):
        K.dk.dense_torch_layout(xd, Wd.t())
    x, Vt, Ut = orc.make_low_rank_inputs(3, 256, 256, 64, torch.float16, seed=3)
    with pytest.raises((AssertionError, RuntimeError), match="contiguous"):
        K.lk.low_rank_torch_layout(x.to(DEV), Vt.to(DEV), Ut.to(DEV).t().contiguous().t())


def test_argument_errors_are_reported(K):
    x, U, Vt, S = orc.make_blast_inputs(2, 256, 256, 4, 64, torch.float16, seed=1)
    with pytest.raises(AssertionError):
        K.bk.blast_torch_layout(*_cuda(x, U, Vt, S[:, :3].contiguous()))
    with pytest.raises(RuntimeError):  # CPU tensors: there is no fallback
        K.bk.blast_torch_layout(x, U, Vt, S)
    # P = 12 is not a multiple of 8: rejected by the C ABI with a message
    x, U, Vt, S = orc.make_blast_inputs(2, 48, 64, 4, 64, torch.float16, seed=1)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        K.bk.blast_torch_layout(*_cuda(x, U, Vt, S))


@pytest.mark.parametrize("bits", [16, 8, 4])
@pytest.mark.parametrize("N", [1, 3, 12, 20])
def test_fused_layers_bias_residual_and_swiglu_input(K, bits, N):
    """blr_blast_multi: q/k/v-style layers on one input with bias and residual in the epilogue, and a down projection
    fed with silu(gate) * up, against the oracle composition (N = 20 takes the layer-by-layer route)."""
    I, O, b, R = 1024, 1536, 8, 256
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=200 + N)
    sets = [(U, Vt, S)]
    for s in (1, 2):
        _, U2, Vt2, S2 = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=300 + s)
        sets.append((U2, Vt2, S2))
    g = torch.Generator().manual_seed(N)
    biases = [torch.randn(O, generator=g).half() for _ in sets]
    res = torch.randn(1, N, O, generator=g).half()
    xm = torch.randn(1, N, I, generator=g).half()
    xe = torch.nn.functional.silu(x.float()) * xm.float()

    def ref_one(inp, f, bias, residual):
        if bits == 16:
            o = orc.blast(inp, *f)[0]
        else:
            Uq, us = orc.quantize_sym(f[0], bits)
            Vq, vs = orc.quantize_sym(f[1], bits)
            o = orc.blast_wq(inp, Uq, us, Vq, vs, f[2], bits)[0]
        return o + bias.float() + residual.float()

    if bits == 16:
        dev_sets = [tuple(_cuda(*f)) for f in sets]
        call = lambda inp, ls, **kw: K.bk.blast_multi_torch_layout(inp, ls, **kw)
    else:
        dev_sets = []
        for f in sets:
            Uq, us, Vq, vs = K.bq.quantize_blast_factors(f[0].to(DEV), f[1].to(DEV), bits)
            dev_sets.append((Uq, us, Vq, vs, f[2].to(DEV)))
        call = lambda inp, ls, **kw: K.bq.blast_wq_multi(inp, ls, bits, **kw)
    # three layers, one input
    got = call(x.to(DEV), dev_sets, biases=[t.to(DEV) for t in biases], residuals=[res.to(DEV)] * 3)
    _sync_ok(K)
    for o, f, bias in zip(got, sets, biases):
        assert o.shape == (1, N, O)
        assert orc.rel_fro(o.float().cpu(), ref_one(x, f, bias, res)) < TOL
    # one layer on silu(x) * x_mul (the activations are rounded to 16 bits once, like the unfused product)
    (got,) = call(x.to(DEV), dev_sets[:1], x_mul=xm.to(DEV), residuals=[res.to(DEV)])
    _sync_ok(K)
    assert orc.rel_fro(got.float().cpu(), ref_one(xe.half(), sets[0], torch.zeros(O), res)) < TOL
