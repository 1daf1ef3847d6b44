"""The small kernels of the decode step (RMSNorm, rotary embedding + cache append, one-token attention) against plain
PyTorch fp32 references of the same ops on the same 16-bit inputs.  Tolerance: one 16-bit rounding of the result
(relative Frobenius error 2e-3 for fp16, 1e-2 for bf16)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tol(dtype):
    return 2e-3 if dtype == torch.float16 else 1e-2


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from mem_efficient_blr_b200 import ops as o
    return o


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,d", [(1, 4096), (5, 512), (33, 768)])
def test_rmsnorm(ops, rows, d, dtype):
    g = torch.Generator().manual_seed(rows + d)
    x = (torch.randn(rows, d, generator=g) * 3).to(dtype)
    w = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    v = x.float()
    ref = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    got = ops.rmsnorm(x.to(DEV), w.to(DEV), 1e-5)
    assert got.dtype == dtype and _rel(got.float().cpu(), ref) < _tol(dtype)
    # a strided view (every second row of a wider buffer) and leading batch dims
    wide = torch.zeros(rows, 2, d, dtype=dtype)
    wide[:, 0] = x
    got2 = ops.rmsnorm(wide.to(DEV)[:, 0], w.to(DEV), 1e-5)
    assert torch.equal(got2, got)
    got3 = ops.rmsnorm(x.to(DEV).view(1, rows, d), w.to(DEV), 1e-5)
    assert got3.shape == (1, rows, d) and torch.equal(got3[0], got)


def _rope_ref(t, cos, sin):
    t1, t2 = t.float().chunk(2, dim=-1)
    return torch.cat((t1 * cos - t2 * sin, t2 * cos + t1 * sin), dim=-1)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,T,H,hd,S", [(1, 1, 32, 128, 64), (3, 1, 8, 64, 12), (2, 5, 4, 64, 16)])
def test_rope_append(ops, B, T, H, hd, S, dtype):
    g = torch.Generator().manual_seed(B * 100 + T)
    q, k, v = (torch.randn(B, T, H * hd, generator=g).to(dtype) for _ in range(3))
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    ang = torch.outer(torch.arange(S, dtype=torch.float32), inv)
    cos, sin = ang.cos(), ang.sin()
    pos = torch.randperm(S, generator=g)[:T].sort().values
    kc = torch.randn(B, H, S, hd, generator=g).to(dtype)
    vc = torch.randn(B, H, S, hd, generator=g).to(dtype)
    # reference: (B, H, T, hd) views, rotation by the angles of the slots, index_copy into the caches
    c, s_ = cos[pos], sin[pos]
    qh, kh, vh = (t.view(B, T, H, hd).transpose(1, 2) for t in (q, k, v))
    q_ref, k_ref = _rope_ref(qh, c, s_), _rope_ref(kh, c, s_)
    kc_ref, vc_ref = kc.float().clone(), vc.float().clone()
    kc_ref.index_copy_(2, pos, k_ref)
    vc_ref.index_copy_(2, pos, vh.float())
    qd, kd, vd = (t.to(DEV).view(B * T, H * hd) for t in (q, k, v))
    kcd, vcd = kc.to(DEV), vc.to(DEV)
    out = ops.rope_append(qd, kd, vd, cos.to(DEV), sin.to(DEV), pos.to(DEV), kcd, vcd, T)
    torch.cuda.synchronize()
    assert out.data_ptr() == qd.data_ptr()
    assert _rel(qd.view(B, T, H, hd).transpose(1, 2).float().cpu(), q_ref) < _tol(dtype)
    assert _rel(kcd.float().cpu(), kc_ref) < _tol(dtype)
    assert torch.equal(vcd.float().cpu(), vc_ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,hd,S,n_keys", [(1, 32, 128, 2048, -1), (3, 8, 64, 12, -1), (2, 4, 128, 300, 257), (64, 4, 64, 128, -1),
                                             (1, 2, 256, 70, 1)])
def test_attention_decode(ops, B, H, hd, S, n_keys, dtype):
    g = torch.Generator().manual_seed(S + B)
    q = torch.randn(B, H * hd, generator=g).to(dtype)
    kc = torch.randn(B, H, S, hd, generator=g).to(dtype)
    vc = torch.randn(B, H, S, hd, generator=g).to(dtype)
    n = S if n_keys < 0 else n_keys
    ref = F.scaled_dot_product_attention(q.float().view(B, H, 1, hd), kc.float()[:, :, :n], vc.float()[:, :, :n]).reshape(B, H * hd)
    got = ops.attention_decode(q.to(DEV), kc.to(DEV), vc.to(DEV), n_keys)
    torch.cuda.synchronize()
    assert got.dtype == dtype and _rel(got.float().cpu(), ref) < _tol(dtype)


def test_argument_errors(ops):
    x = torch.zeros(2, 12, dtype=torch.float16, device=DEV)   # 12 is not a multiple of 8
    with pytest.raises(RuntimeError):
        ops.rmsnorm(x, torch.ones(12, dtype=torch.float16, device=DEV), 1e-5)
    with pytest.raises(RuntimeError):   # CPU tensors: no fallback
        ops.rmsnorm(torch.zeros(2, 16, dtype=torch.float16), torch.ones(16, dtype=torch.float16), 1e-5)


def test_fused_decode_step_equals_the_module_by_module_step():
    """The decoder's fused decode path (these kernels) against the same step through the torch modules."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from mem_efficient_blr_b200 import networks as nw
    shape = nw.LlamaShape(layers=2, d=512, heads=8, ffn=1024, vocab=384, b=16, rank_attn=64, rank_mlp=96)
    B, T = 3, 9
    ids = torch.randint(0, shape.vocab, (B, T), generator=torch.Generator().manual_seed(1)).to(DEV)
    outs = []
    for fused in (True, False):
        m = nw.LlamaDecoder(shape, "blast", batch=B, cache_len=T, device=DEV, dtype=torch.float16, seed=3)
        m.fused_decode = fused
        m.prefill(ids[:, :T - 1])
        outs.append(m.decode_step(ids[:, T - 1:], torch.tensor([T - 1], device=DEV)).float().cpu())
    assert _rel(outs[0], outs[1]) < 5e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("affine", [True, False])
@pytest.mark.parametrize("rows,d", [(1, 768), (13, 1152), (197, 768), (1000, 2048), (9, 8)])
def test_layernorm(ops, rows, d, affine, dtype):
    """A warp per row, the row in registers: against F.layer_norm in fp32 on the same 16-bit inputs (rows with an
    offset mean, so that a one-pass variance would lose digits), with and without weight / bias, strided rows."""
    g = torch.Generator().manual_seed(rows + d)
    x = (torch.randn(rows, d, generator=g) * 2 + 5).to(dtype)
    w = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype) if affine else None
    b = (0.1 * torch.randn(d, generator=g)).to(dtype) if affine else None
    ref = F.layer_norm(x.float(), (d,), None if w is None else w.float(), None if b is None else b.float(), 1e-6)
    got = ops.layernorm(x.to(DEV), None if w is None else w.to(DEV), None if b is None else b.to(DEV), 1e-6)
    assert got.dtype == dtype and got.shape == x.shape and _rel(got.float().cpu(), ref) < _tol(dtype)
    wide = torch.zeros(rows, 2, d, dtype=dtype)
    wide[:, 0] = x
    got2 = ops.layernorm(wide.to(DEV)[:, 0], None if w is None else w.to(DEV), None if b is None else b.to(DEV), 1e-6)
    assert _rel(got2.float().cpu(), ref) < _tol(dtype)
    got3 = ops.layernorm(x.to(DEV).view(1, rows, d), None if w is None else w.to(DEV), None if b is None else b.to(DEV), 1e-6)
    assert got3.shape == (1, rows, d) and _rel(got3.float().cpu().view(rows, d), ref) < _tol(dtype)


def test_layernorm_refuses_rows_a_warp_cannot_hold(ops):
    x = torch.randn(4, 4096, device=DEV, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="d <= 2048"):
        ops.layernorm(x, None, None, 1e-6)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,T,d", [(1, 256, 1152), (3, 16, 144), (5, 7, 2048)])
def test_layernorm_modulate_and_gated_add(ops, B, T, d, dtype):
    """norm(x) * (1 + scale) + shift with one (shift, scale) row per image taken as column slices of a wider matrix, and
    x + gate * y, against fp32 PyTorch on the same 16-bit inputs."""
    g = torch.Generator().manual_seed(B * T + d)
    x = (torch.randn(B, T, d, generator=g) + 2).to(dtype)
    y = torch.randn(B, T, d, generator=g).to(dtype)
    mod = torch.randn(B, 3 * d, generator=g).to(dtype)       # shift | scale | gate as an adaLN linear emits them
    xd, yd, md = x.to(DEV), y.to(DEV), mod.to(DEV)
    shift, scale, gate = md.chunk(3, dim=1)
    sf, cf, gf = (t.float() for t in mod.chunk(3, dim=1))
    ref = F.layer_norm(x.float(), (d,), None, None, 1e-6) * (1 + cf.unsqueeze(1)) + sf.unsqueeze(1)
    got = ops.layernorm_modulate(xd, shift, scale, 1e-6)
    assert got.shape == x.shape and got.dtype == dtype and _rel(got.float().cpu(), ref) < _tol(dtype)
    ref2 = x.float() + gf.unsqueeze(1) * y.float()
    got2 = ops.gated_add(xd, gate, yd)
    assert got2.shape == x.shape and _rel(got2.float().cpu(), ref2) < _tol(dtype)
