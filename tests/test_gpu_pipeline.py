"""GPU parity of the tensor-core pipeline (more than 16 tokens) against the CPU oracle, through the C ABI.

Tolerance: relative Frobenius error <= 1e-2 against the fp32 oracle on the same 16-bit inputs.
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

    class NS:
        pass

    ns = NS()
    ns.bk, ns.bq, ns.dk, ns.lk, ns.mk = bk, bq, dk, lk, mk
    return ns


def _cuda(*ts):
    return [t.to(DEV) for t in ts]


def _err(got, ref):
    torch.cuda.synchronize()
    return orc.rel_fro(got.float().cpu(), ref)


BLAST_SHAPES = [
    # N, I, O, b, R
    (17, 256, 384, 4, 128),
    (197, 768, 2304, 3, 128),      # the reference's ViT-B setting (b = 3, fused qkv)
    (197, 768, 3072, 16, 192),
    (128, 4096, 11008, 16, 1024),  # headline layer, 128 tokens
    (2048, 4096, 11008, 16, 1024),
    (129, 11008, 4096, 16, 1488),  # down_proj at the reference's 50 %-parameter rank, ragged token count
    (65, 1152, 2304, 6, 192),      # six and nine blocks
    (197, 2304, 3456, 9, 384),
    (100, 512, 288, 4, 64),        # Q = 72: 16-byte but not 32-byte output pieces
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", BLAST_SHAPES)
def test_blast_prefill_all_layout_families(K, shape, dtype):
    N, I, O, b, R = shape
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, dtype, seed=N % 97)
    ref, _, _ = orc.blast(x, U, Vt, S)
    xd, Ud, Vtd, Sd = _cuda(x, U, Vt, S)
    got = K.bk.blast_torch_layout(xd, Ud, Vtd, Sd)
    assert got.shape == ref.shape and got.dtype == dtype
    assert _err(got, ref) < TOL
    Up, Vp, Sp = _cuda(*orc.blast_to_partial_layout(U, Vt, S))
    assert _err(K.bk.triton_blast_partial_grouped_fp16(xd, Up, Vp, Sp), ref) < TOL
    assert _err(K.bk.triton_blast_full_fp16(xd, Up, Vp, Sp), ref) < TOL
    Ub, Vb, Sb = _cuda(*orc.blast_to_bmm_layout(U, Vt, S))
    assert _err(K.bk.triton_blast_bmm_fp16(xd, Ub, Vb, Sb), ref) < TOL


def test_blast_reference_golden_vector_17_tokens(K, golden_dir):
    g = {k: torch.from_numpy(v) for k, v in np.load(os.path.join(golden_dir, "blast_c.npz")).items()}
    x, U, Vt, S = (g[k].to(torch.bfloat16) for k in ("x", "U", "Vt", "S"))
    ref, _, _ = orc.blast(x, U, Vt, S)
    got = K.bk.blast_torch_layout(*_cuda(x, U, Vt, S))
    assert got.shape == g["out"].shape
    assert _err(got, ref) < TOL
    assert _err(got, g["out"]) < 3e-2  # vs the reference's own fp32 output (inputs rounded to bf16 here)


def test_blast_act_int8_prefill(K):
    x, U, Vt, S = orc.make_blast_inputs(64, 512, 768, 4, 128, torch.bfloat16, seed=21)
    x = x * 4
    ref, _, _ = orc.blast_act_int8(x, U, Vt, S)
    Ub, Vb, Sb = _cuda(*orc.blast_to_bmm_layout(U, Vt, S))
    assert _err(K.bq.triton_blast_bmm_int8_fp16(x.to(DEV), Ub, Vb, Sb), ref) < 3e-2


WQ_SHAPES = [
    # N, I, O, b, R
    (17, 512, 768, 4, 128),        # weights as the MMA rows (up to 64 tokens)
    (64, 4096, 11008, 16, 1024),
    (65, 4096, 11008, 16, 1024),   # tokens as the MMA rows
    (300, 768, 1152, 3, 384),      # three blocks, the coupling over expanded factors
    (200, 512, 288, 4, 128),       # Q = 72: a ragged weight tile
    (1024, 4096, 4096, 16, 1024),
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits,group", [(8, 0), (4, 0), (8, 128), (4, 128)])
@pytest.mark.parametrize("shape", WQ_SHAPES)
def test_quantised_factors_widened_inside_the_gemms(K, shape, bits, group, dtype):
    """Above 16 tokens the C entry point stages the stored bytes and widens them in shared memory.  The widened tile
    equals what blr_dequantize_sym writes (q * scale rounded once), so the result is bit-identical to the 16-bit
    pipeline on the widened factors, which needs a second copy of the layer in device memory."""
    from mem_efficient_blr_b200 import ops
    N, I, O, b, R = shape
    P, Q = I // b, O // b
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, dtype, seed=N + bits + group)
    Uq, us = orc.quantize_sym(U, bits, group)
    Vq, vs = orc.quantize_sym(Vt, bits, group)
    xd, Uqd, usd, Vqd, vsd, Sd = _cuda(x.reshape(-1, I), Uq, us, Vq, vs, S)
    got = ops.blast_wq(xd, Uqd, usd, Vqd, vsd, Sd, b * R, R, 1, bits, group, b, P, Q, R)
    Uw = ops.dequantize_sym(Uqd, usd, bits, group, dtype)
    Vw = ops.dequantize_sym(Vqd, vsd, bits, group, dtype)
    keep = ops.coupling_cache_bytes
    ops.coupling_cache_bytes = 0
    try:
        want = ops.blast(xd, Uw, Vw, Sd, 0, 0, b * R, R, 1, b, P, Q, R, 0)
    finally:
        ops.coupling_cache_bytes = keep
    torch.cuda.synchronize()
    assert got.shape == want.shape and torch.equal(got, want)
    ref, _, _ = orc.blast_wq(x, Uq, us, Vq, vs, S, bits, group)
    assert _err(got, ref.reshape(-1, O)) < TOL


def test_quantised_rows_the_copy_engine_cannot_stage(K):
    """int4 rows of P = 48 weights are 24 bytes: the C entry point refuses them above 16 tokens, the Python operator
    widens such a layer for the call."""
    from mem_efficient_blr_b200 import ops
    N, I, O, b, R = 40, 768, 768, 16, 64
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=2)
    Uq, us = orc.quantize_sym(U, 4, 0)
    Vq, vs = orc.quantize_sym(Vt, 4, 0)
    xd, Uqd, usd, Vqd, vsd, Sd = _cuda(x, Uq, us, Vq, vs, S)
    with pytest.raises(RuntimeError, match="multiple of 16 bytes"):
        ops.blast_wq(xd.reshape(-1, I), Uqd, usd, Vqd, vsd, Sd, b * R, R, 1, 4, 0, b, I // b, O // b, R)
    ref, _, _ = orc.blast_wq(x, Uq, us, Vq, vs, S, 4, 0)
    assert _err(K.bq.blast_wq(xd, Uqd, usd, Vqd, vsd, Sd, 4, 0), ref) < TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(33, 256, 512, 4, 64), (197, 768, 3072, 4, 768), (128, 4096, 4096, 16, 1024),
                                   (2048, 4096, 11008, 16, 1536)])
def test_monarch_prefill_all_variants(K, shape, dtype):
    N, I, O, b, rank = shape
    x, w1_t, w2_t = orc.make_monarch_inputs(N, I, O, b, rank, dtype, seed=N % 89)
    ref = orc.monarch(x, w1_t, w2_t)[0]
    xd = x.to(DEV)
    assert _err(K.mk.monarch_torch_layout(xd, w1_t.to(DEV), w2_t.to(DEV)), ref) < TOL
    w1k = orc.monarch_w1_to_kernel_layout(w1_t).to(DEV)
    assert _err(K.mk.triton_monarch_right_fp16(xd, w1k, w2_t.to(DEV)), ref) < TOL
    assert _err(K.mk.triton_monarch_right_left_fp16(xd, w1k, orc.monarch_w2_to_left_layout(w2_t).to(DEV)), ref) < TOL
    assert _err(K.mk.triton_monarch_right_ideal_fp16(xd, w1k, w2_t.to(DEV)), orc.monarch_ideal_order(ref, b)) < TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(17, 256, 384, 64), (128, 4096, 11008, 1024), (2048, 11008, 4096, 1024),
                                   (300, 2000, 1000, 200)])  # (the last: two contraction slices of 1000, not whole 64-wide blocks)
def test_low_rank_prefill(K, shape, dtype):
    N, I, O, R = shape
    x, Vt, Ut = orc.make_low_rank_inputs(N, I, O, R, dtype, seed=N % 83)
    ref, _ = orc.low_rank(x, Vt, Ut)
    assert _err(K.lk.low_rank_torch_layout(*_cuda(x, Vt, Ut)), ref) < TOL
    got = K.lk.triton_low_rank_fp16(x.to(DEV), Vt.t().contiguous().to(DEV), Ut.t().contiguous().to(DEV))
    assert got.shape == (N, O) and _err(got, ref.reshape(N, O)) < TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(17, 256, 384), (200, 512, 1000), (130, 264, 1000), (2048, 4096, 11008)])
def test_dense_prefill(K, shape, dtype):
    N, I, O = shape
    x, Wt = orc.make_dense_inputs(N, I, O, dtype, seed=N % 79)
    ref = orc.dense(x, Wt)
    assert _err(K.dk.dense_torch_layout(*_cuda(x, Wt)), ref) < TOL
    got = K.dk.triton_dense_fp16(x.to(DEV), Wt.t().contiguous().to(DEV))
    assert got.shape == (N, O) and _err(got, ref.reshape(N, O)) < TOL


def test_linearity_at_full_size(K):
    """Size-independent property at the headline size: f(a*x1 + x2) = a*f(x1) + f(x2) within rounding."""
    N, I, O, b, R = 2048, 4096, 11008, 16, 1024
    x1, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=5)
    x2 = torch.randn(1, N, I, generator=torch.Generator().manual_seed(6)).half()
    Ud, Vtd, Sd = _cuda(U, Vt, S)
    f = lambda t: K.bk.blast_torch_layout(t.to(DEV), Ud, Vtd, Sd).float()
    lhs = f((0.5 * x1.float() + x2.float()).half())
    rhs = 0.5 * f(x1) + f(x2)
    torch.cuda.synchronize()
    assert orc.rel_fro(lhs.cpu(), rhs.cpu()) < 5e-3


@pytest.mark.parametrize("bits,group", [(8, 0), (4, 0), (8, 128), (4, 128)])
def test_weight_quantised_blast_above_16_tokens(K, bits, group):
    """Quantised layers on prefill sizes through the reference-facing operator.  The widening (here in shared
    memory, inside the GEMMs) rounds q * scale to the 16-bit type, which the oracle (fp32 dequantisation) does not;
    the bound is the same 1e-2."""
    N, I, O, b, R = 197, 4096, 11008, 16, 1024
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=bits + group)
    Uq, us = orc.quantize_sym(U, bits, group)
    Vq, vs = orc.quantize_sym(Vt, bits, group)
    ref, _, _ = orc.blast_wq(x, Uq, us, Vq, vs, S, bits, group)
    import mem_efficient_blr_b200.blast_sym_quant_kernels as bq
    from mem_efficient_blr_b200 import ops
    # the widening itself is exact up to the rounding to fp16
    Ud = ops.dequantize_sym(Uq.to(DEV), us.to(DEV), bits, group, torch.float16)
    want = orc.dequantize_sym(Uq, us, bits, group).half()
    assert torch.equal(Ud.cpu(), want)
    got = bq.blast_wq(x.to(DEV), Uq.to(DEV), us.to(DEV), Vq.to(DEV), vs.to(DEV), S.to(DEV), bits, group)
    assert got.shape == ref.shape
    assert _err(got, ref) < TOL


# ------------------------------------------------------------------------- expanded coupling factors kept per S
def test_coupling_factors_cached_per_S_and_rebuilt_after_a_change(K):
    """Above 256 tokens the expanded coupling factors are built once per S (ops._coupling_factors): the cached call is
    bit-identical to the uncached one, and an in-place change of S (a version bump) rebuilds them."""
    from mem_efficient_blr_b200 import ops
    N, I, O, b, R = 300, 512, 768, 4, 128
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=5)
    xd, Ud, Vtd, Sd = _cuda(x, U, Vt, S)
    ops.clear_coupling_cache()
    keep = ops.coupling_cache_bytes
    try:
        ops.coupling_cache_bytes = 0
        plain = K.bk.blast_torch_layout(xd, Ud, Vtd, Sd)
        assert len(ops._coupling) == 0
        ops.coupling_cache_bytes = keep
        first = K.bk.blast_torch_layout(xd, Ud, Vtd, Sd)
        assert len(ops._coupling) == 1
        held = next(iter(ops._coupling.values()))[2]
        second = K.bk.blast_torch_layout(xd, Ud, Vtd, Sd)
        assert len(ops._coupling) == 1 and next(iter(ops._coupling.values()))[2] is held
        torch.cuda.synchronize()
        assert torch.equal(plain, first) and torch.equal(plain, second)
        assert _err(first, orc.blast(x, U, Vt, S)[0]) < TOL
        # a shard of S made per call is a fresh view object of one base: still one entry per pointer
        half = K.bk.blast_torch_layout(xd, Ud, Vtd, Sd[:])
        assert torch.equal(half, plain) and len(ops._coupling) == 1
        Sd.mul_(-0.5)
        changed = K.bk.blast_torch_layout(xd, Ud, Vtd, Sd)
        assert _err(changed, orc.blast(x, U, Vt, S * -0.5)[0]) < TOL
        assert len(ops._coupling) == 1
        # the factors of a tensor that is gone are dropped with it
        S2 = Sd.clone()
        K.bk.blast_torch_layout(xd, Ud, Vtd, S2)
        assert len(ops._coupling) == 2
        del S2
        assert len(ops._coupling) == 1 and ops._coupling_held == next(iter(ops._coupling.values()))[2].numel()
        # few tokens never touch the cache
        ops.clear_coupling_cache()
        K.bk.blast_torch_layout(xd.reshape(-1, I)[:200], Ud, Vtd, Sd)
        assert len(ops._coupling) == 0
    finally:
        ops.coupling_cache_bytes = keep
        ops.clear_coupling_cache()


def test_coupling_factors_stay_out_of_captured_graphs(K):
    """A captured graph expands S at every replay (S may change between replays), so capture neither reads nor fills
    the cache."""
    from mem_efficient_blr_b200 import ops
    N, I, O, b, R = 320, 512, 768, 4, 128
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.bfloat16, seed=6)
    xd, Ud, Vtd, Sd = _cuda(x, U, Vt, S)
    ops.clear_coupling_cache()
    K.bk.blast_torch_layout(xd, Ud, Vtd, Sd)  # scratch buffers at their final size, and one cache entry
    torch.cuda.synchronize()
    entries = len(ops._coupling)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        K.bk.blast_torch_layout(xd, Ud, Vtd, Sd)
        torch.cuda.synchronize()
        ops.clear_coupling_cache()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            out = K.bk.blast_torch_layout(xd, Ud, Vtd, Sd)
    assert len(ops._coupling) == 0 and entries == 1
    Sd.mul_(2.0)
    g.replay()
    assert _err(out, orc.blast(x, U, Vt, S * 2.0)[0]) < TOL
    ops.clear_coupling_cache()


def test_coupling_entry_points_check_their_arguments(K):
    from mem_efficient_blr_b200 import _lib as L
    lib = L.load()
    assert lib.blr_blast_coupling_bytes(16, 16, 1024) == 1024 * 16 * 16 * 16 * 2
    assert lib.blr_blast_coupling_bytes(16, 4, 1032) == 1032 * 8 * 4 * 16 * 2   # R % 16 != 0: groups of 8 ranks
    assert lib.blr_blast_coupling_bytes(32, 32, 1024) == 0 and lib.blr_blast_coupling_bytes(4, 4, 100) == 0
    S = torch.randn(4, 4, 128, device=DEV, dtype=torch.float16)
    need = lib.blr_blast_coupling_bytes(4, 4, 128)
    E = torch.empty(need, dtype=torch.uint8, device=DEV)
    st = L.stream_ptr(S.device)
    args = (S.data_ptr(), 4 * 128, 128, 1, 4, 4)
    assert lib.blr_blast_expand_coupling(*args, 128, 0, E.data_ptr(), need - 1, st) == -4  # BLR_ERR_WORKSPACE
    assert lib.blr_blast_expand_coupling(*args, 100, 0, E.data_ptr(), need, st) == -6  # BLR_ERR_UNSUPPORTED
    assert lib.blr_blast_expand_coupling(None, *args[1:], 128, 0, E.data_ptr(), need, st) == -1  # BLR_ERR_ARG
    assert lib.blr_blast_expand_coupling(*args, 128, 0, E.data_ptr(), need, st) == 0
    torch.cuda.synchronize()


# ------------------------------------------------------------------------- many tokens: passes over parts of the batch
def test_token_counts_beyond_one_pass_run_as_passes_on_a_capped_workspace(K):
    """When the 16-bit intermediates of a call would outgrow L2 the call runs as passes over equal parts of the tokens;
    a token's result does not depend on which pass it is in, and the workspace stops growing."""
    from mem_efficient_blr_b200 import _lib as L
    lib = L.load()
    assert lib.blr_workspace_bytes(9000, 16, 1024) == lib.blr_workspace_bytes(3072, 16, 1024) < lib.blr_workspace_bytes(4096, 16, 1024)
    assert lib.blr_workspace_bytes(4096, 16, 1024) == lib.blr_workspace_bytes(8192, 16, 1024)
    g = torch.Generator().manual_seed(12)
    # BLAST, b = 16, R = 1024: 4096 tokens per pass at most -> 9000 tokens in three passes of 3072, 3072, 2856
    N, b, P, Q, R = 9000, 16, 16, 16, 1024
    x = torch.randn(N, b * P, generator=g).half()
    U = (torch.randn(b, Q, R, generator=g) / R ** 0.5).half()
    Vt = (torch.randn(b, R, P, generator=g) / P ** 0.5).half()
    S = (torch.rand(b, b, R, generator=g) + 0.5).half()
    xd, Ud, Vd, Sd = _cuda(x, U, Vt, S)
    whole = K.bk.blast_torch_layout(xd, Ud, Vd, Sd)
    parts = torch.cat([K.bk.blast_torch_layout(xd[i:i + 3000], Ud, Vd, Sd) for i in range(0, N, 3000)])
    torch.cuda.synchronize()
    assert torch.equal(whole, parts)
    rows = torch.cat((torch.arange(0, 40), torch.arange(3050, 3100), torch.arange(N - 40, N)))
    assert _err(whole[rows.to(DEV)], orc.blast(x[rows], U, Vt, S)[0]) < TOL
    # the same with int8 factors widened inside the GEMMs (the C entry point; 300 tokens per slice keep the same kernels)
    from mem_efficient_blr_b200 import ops
    Uq, us, Vq, vs = K.bq.quantize_blast_factors(Ud, Vd, 8)
    wq = ops.blast_wq(xd, Uq, us, Vq, vs, Sd, b * R, R, 1, 8, 0, b, P, Q, R)
    wq_parts = torch.cat([ops.blast_wq(xd[i:i + 3000], Uq, us, Vq, vs, Sd, b * R, R, 1, 8, 0, b, P, Q, R) for i in range(0, N, 3000)])
    torch.cuda.synchronize()
    assert torch.equal(wq, wq_parts)
    # Monarch, 4 blocks, rank 1024: 16384 tokens per pass at most
    N2, I2, O2, b2, rank = 20000, 256, 256, 4, 1024
    x2, w1, w2 = orc.make_monarch_inputs(N2, I2, O2, b2, rank, torch.float16, seed=3)
    x2d, w1d, w2d = _cuda(x2.reshape(N2, I2), w1, w2)
    whole2 = K.mk.monarch_torch_layout(x2d, w1d, w2d)
    parts2 = torch.cat([K.mk.monarch_torch_layout(x2d[i:i + 5000], w1d, w2d) for i in range(0, N2, 5000)])
    torch.cuda.synchronize()
    assert torch.equal(whole2, parts2)
    rows2 = torch.cat((torch.arange(0, 40), torch.arange(N2 - 40, N2)))
    assert _err(whole2[rows2.to(DEV)], orc.monarch(x2.reshape(N2, I2)[rows2], w1, w2)[0]) < TOL


# ------------------------------------------------------------------------- bias and residual in the last GEMM's epilogue
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [16, 8])
@pytest.mark.parametrize("shape", [(17, 512, 768, 4, 128), (64, 4096, 4096, 16, 1024), (65, 768, 2304, 16, 256),
                                   (300, 512, 288, 4, 128), (2048, 4096, 4096, 16, 1024)])
def test_bias_and_residual_added_by_the_pipeline(K, shape, bits, dtype):
    """Above 16 tokens the fused call runs the layers through the pipeline and the last GEMM adds bias and residual
    (both orientations of the tile, ragged output blocks, 16-bit and quantised factors); against the oracle plus the
    additions in fp32."""
    from mem_efficient_blr_b200 import ops
    N, I, O, b, R = shape
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, dtype, seed=N + bits)
    g = torch.Generator().manual_seed(N)
    bias = torch.randn(O, generator=g).to(dtype)
    res = torch.randn(N, O, generator=g).to(dtype)
    x2 = x.reshape(N, I)
    if bits == 16:
        ref = orc.blast(x, U, Vt, S)[0].reshape(N, O)
        layers = [tuple(_cuda(U, Vt, S))]
    else:
        Uq, us = orc.quantize_sym(U, bits)
        Vq, vs = orc.quantize_sym(Vt, bits)
        ref = orc.blast_wq(x, Uq, us, Vq, vs, S, bits)[0].reshape(N, O)
        layers = [tuple(_cuda(Uq, us, Vq, vs, S))]
    xd, bd, rd = _cuda(x2, bias, res)
    P, Q = I // b, O // b
    outs = ops.blast_multi(xd, layers, bits, 0, b, P, Q, R, None, [bd], [rd])
    if bits != 16 and N > 384:
        assert outs is None   # (the widening route serves those; nothing fused)
        return
    only_bias = ops.blast_multi(xd, layers, bits, 0, b, P, Q, R, None, [bd], None)[0]
    assert _err(only_bias, ref + bias.float()) < TOL
    if N <= 64 or N > 512:
        assert outs is None   # (residuals are fused only where that is faster than torch's add: 65..512 tokens)
        # the C entry point itself serves them all the same
        import mem_efficient_blr_b200.blast_kernels as bk
        keep = ops.blast_multi
        try:
            ops.blast_multi = lambda *a, **k: None
            unfused = bk.blast_multi_torch_layout(xd, layers, None, [bd], [rd])[0] if bits == 16 else \
                K.bq.blast_wq_multi(xd, layers, bits, 0, None, [bd], [rd])[0]
        finally:
            ops.blast_multi = keep
        assert _err(unfused, ref + bias.float() + res.float()) < TOL
        return
    assert outs is not None and len(outs) == 1
    assert _err(outs[0], ref + bias.float() + res.float()) < TOL
    # a residual view with a longer row stride and an odd start (no 16-byte pieces)
    wide = torch.zeros(N, O + 9, dtype=dtype, device=DEV)
    wide[:, 1:O + 1] = rd
    got = ops.blast_multi(xd, layers, bits, 0, b, P, Q, R, None, None, [wide[:, 1:O + 1]])[0]
    assert _err(got, ref + res.float()) < TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("act", ["gelu", "gelu_tanh"])
@pytest.mark.parametrize("shape,bits", [((40, 512, 768, 4, 128), 16), ((197, 768, 3072, 16, 288), 16), ((300, 1152, 4608, 9, 256), 16),
                                        ((130, 512, 768, 4, 128), 8)])
def test_output_activation_in_the_epilogue(K, shape, bits, act, dtype):
    """gelu(result + bias) (+ residual) by the last GEMM's epilogue above 16 tokens, against the oracle and torch's GELU in
    fp32; up to 16 tokens the wrappers apply torch's activation."""
    from mem_efficient_blr_b200 import ops
    N, I, O, b, R = shape
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, dtype, seed=N)
    g = torch.Generator().manual_seed(N + 1)
    bias = torch.randn(O, generator=g).to(dtype)
    res = torch.randn(N, O, generator=g).to(dtype)
    if bits == 16:
        lin = orc.blast(x, U, Vt, S)[0].reshape(N, O)
        layers = [tuple(_cuda(U, Vt, S))]
    else:
        Uq, us = orc.quantize_sym(U, bits)
        Vq, vs = orc.quantize_sym(Vt, bits)
        lin = orc.blast_wq(x, Uq, us, Vq, vs, S, bits)[0].reshape(N, O)
        layers = [tuple(_cuda(Uq, us, Vq, vs, S))]
    gelu = lambda t: torch.nn.functional.gelu(t, approximate="tanh" if act == "gelu_tanh" else "none")
    xd, bd, rd = _cuda(x.reshape(N, I), bias, res)
    P, Q = I // b, O // b
    got = ops.blast_multi(xd, layers, bits, 0, b, P, Q, R, None, [bd], None, act)
    assert got is not None and _err(got[0], gelu(lin + bias.float())) < TOL
    if 64 < N <= 512:
        got = ops.blast_multi(xd, layers, bits, 0, b, P, Q, R, None, [bd], [rd], act)
        assert got is not None and _err(got[0], gelu(lin + bias.float()) + res.float()) < TOL
    no_bias = ops.blast_multi(xd, layers, bits, 0, b, P, Q, R, None, None, None, act)
    assert no_bias is not None and _err(no_bias[0], gelu(lin)) < TOL
    # the reference-facing wrapper, also at a decode size (torch's activation there)
    wrap = (lambda t: K.bk.blast_multi_torch_layout(t, layers, biases=[bd], out_act=act)[0]) if bits == 16 else \
        (lambda t: K.bq.blast_wq_multi(t, layers, bits, 0, biases=[bd], out_act=act)[0])
    assert _err(wrap(xd), gelu(lin + bias.float())) < TOL
    assert _err(wrap(xd[:5]), gelu(lin[:5] + bias.float())) < TOL
