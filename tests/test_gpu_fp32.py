"""GPU parity of the fp32 verification entry points (the `_fp32` functions) against the CPU oracle.

These kernels use plain fp32 FMAs, so the bound is the reference's own: allclose(atol=1e-1, rtol=0)
on randn data (utils.py:35-44), and a relative Frobenius error of 1e-5.
"""
import pytest
import torch

from oracle import blr_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import mem_efficient_blr_b200.blast_kernels as bk
    import mem_efficient_blr_b200.dense_kernels as dk
    import mem_efficient_blr_b200.low_rank_kernels as lk
    import mem_efficient_blr_b200.monarch_kernels as mk

    class NS:
        pass

    ns = NS()
    ns.bk, ns.dk, ns.lk, ns.mk = bk, dk, lk, mk
    return ns


def _close(got, ref):
    torch.cuda.synchronize()
    g = got.float().cpu()
    assert g.shape == ref.shape
    assert torch.allclose(g, ref, atol=1e-1, rtol=0)
    assert orc.rel_fro(g, ref) < 1e-5


def test_blast_fp32_returns_out_z_y_like_the_reference(K):
    g = torch.Generator().manual_seed(0)
    b, P, Q, R = 4, 24, 40, 32
    x = torch.randn(2, 5, b * P, generator=g)
    U, Vt, S = torch.randn(b, Q, R, generator=g), torch.randn(b, R, P, generator=g), torch.randn(b, b, R, generator=g)
    out, z, y = orc.blast(x, U, Vt, S)
    Up, Vp, Sp = orc.blast_to_partial_layout(U, Vt, S)
    for fn in (K.bk.triton_blast_partial_fp32, K.bk.triton_blast_partial_grouped_fp32,
               K.bk.triton_blast_partial_grouped_persistent_fp32, K.bk.triton_blast_full_fp32):
        o, zz, yy = fn(x.to(DEV), Up.to(DEV), Vp.to(DEV), Sp.to(DEV))
        _close(o, out); _close(zz, z); _close(yy, y)
    Ub, Vb, Sb = orc.blast_to_bmm_layout(U, Vt, S)
    o, zz, yy = K.bk.triton_blast_bmm_fp32(x.to(DEV), Ub.to(DEV), Vb.to(DEV), Sb.to(DEV))
    _close(o, out)
    _close(zz, z.transpose(1, 2))      # (b, R, N) like blast_kernels.py:3024-3041
    _close(yy, y.permute(2, 0, 1))     # (R, b, N)


def test_monarch_fp32_variants(K):
    x, w1_t, w2_t = orc.make_monarch_inputs(6, 64, 96, 4, 16, torch.float32, seed=1)
    out2, _, out1, _ = orc.monarch(x, w1_t, w2_t)
    w1k = orc.monarch_w1_to_kernel_layout(w1_t).to(DEV)
    r = K.mk.triton_monarch_right_fp32(x.to(DEV), w1k, w2_t.to(DEV))
    _close(r[0], out2); _close(r[1], out1)
    r = K.mk.triton_monarch_right_ideal_fp32(x.to(DEV), w1k, w2_t.to(DEV))
    _close(r[1], out1)                 # what the reference's harness verifies (layer.py:235-237)
    _close(r[0], orc.monarch_ideal_order(out2, 4))
    r = K.mk.triton_monarch_right_left_fp32(x.to(DEV), w1k, orc.monarch_w2_to_left_layout(w2_t).to(DEV))
    _close(r[0], out2); _close(r[2], out1)


def test_low_rank_and_dense_fp32(K):
    x, Vt, Ut = orc.make_low_rank_inputs(5, 72, 56, 24, torch.float32, seed=2)
    ref, z = orc.low_rank(x, Vt, Ut)
    y, zz = K.lk.triton_low_rank_fp32(x.to(DEV), Vt.t().contiguous().to(DEV), Ut.t().contiguous().to(DEV))
    _close(y, ref.reshape(5, 56)); _close(zz, z.reshape(5, 24))
    x, Wt = orc.make_dense_inputs(5, 72, 56, torch.float32, seed=3)
    _close(K.dk.triton_dense_fp32(x.to(DEV), Wt.t().contiguous().to(DEV)), orc.dense(x, Wt).reshape(5, 56))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_load_store_probes_write_what_the_reference_probes_write(dtype):
    """triton_low_rank_load_store_* stores the index of the 64-wide output tile (low_rank_kernels.py:229-234),
    triton_dense_load_store_* stores zeros (dense_kernels.py:222-227); both return the 2-D (N, O) shape."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import mem_efficient_blr_b200.dense_kernels as dk
    import mem_efficient_blr_b200.low_rank_kernels as lk
    x = torch.randn(2, 5, 256, device="cuda:0", dtype=dtype)
    a, b = torch.randn(256, 64, device="cuda:0", dtype=dtype), torch.randn(64, 200, device="cuda:0", dtype=dtype)
    f = lk.triton_low_rank_load_store_fp32 if dtype == torch.float32 else lk.triton_low_rank_load_store_fp16
    y = f(x, a, b)
    torch.cuda.synchronize()
    assert y.shape == (10, 200) and y.dtype == dtype
    assert torch.equal(y.float().cpu(), (torch.arange(200) // 64).float().expand(10, 200))
    w = torch.randn(256, 200, device="cuda:0", dtype=dtype)
    g = dk.triton_dense_load_store_fp32 if dtype == torch.float32 else dk.triton_dense_load_store_fp16
    y = g(x, w)
    torch.cuda.synchronize()
    assert y.shape == (10, 200) and float(y.abs().max()) == 0.0
