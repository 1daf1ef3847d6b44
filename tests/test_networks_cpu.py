"""Host-side logic of the network glue (mem_efficient_blr_b200/networks.py) with dense linears on CPU: the static
key/value cache, the rotary embedding and the prefill / decode split must agree with each other."""
import torch

from mem_efficient_blr_b200 import networks as nw


def _small():
    return nw.LlamaShape(layers=2, d=64, heads=4, ffn=128, vocab=97, b=4, rank_attn=16, rank_mlp=16)


def test_decode_step_continues_a_prefill():
    """Prefill of T - 1 tokens followed by one decode step at slot T - 1 of a cache of length T gives the logits of a
    prefill of all T tokens."""
    T, B = 9, 3
    ids = torch.randint(0, 97, (B, T), generator=torch.Generator().manual_seed(1))
    full = nw.LlamaDecoder(_small(), "dense", batch=B, cache_len=T, device="cpu", dtype=torch.float32, seed=3)
    want = full.prefill(ids)
    step = nw.LlamaDecoder(_small(), "dense", batch=B, cache_len=T, device="cpu", dtype=torch.float32, seed=3)
    step.prefill(ids[:, :T - 1])
    got = step.decode_step(ids[:, T - 1:], torch.tensor([T - 1]))
    assert got.shape == (B, 97)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)
    # the caches of the two runs hold the same keys and values
    for a, b in zip(full.kcache + full.vcache, step.kcache + step.vcache):
        assert torch.allclose(a, b, atol=1e-5)


def test_same_seed_gives_same_network_and_structured_list():
    a = nw.LlamaDecoder(_small(), "dense", batch=1, cache_len=4, device="cpu", dtype=torch.float32, seed=5)
    b = nw.LlamaDecoder(_small(), "dense", batch=1, cache_len=4, device="cpu", dtype=torch.float32, seed=5)
    for pa, pb in zip(a.parameters(), b.parameters()):
        assert torch.equal(pa, pb)
    assert len(a.structured_linears()) == 2 * 7


def test_vit_shapes_and_rank_rule():
    s = nw.ViTShape()
    # ranks chosen for about half of the dense parameters: R (I + O + b^2) ~ I O / 2, multiples of 16
    for name, (i, o) in {"qkv": (768, 2304), "intermediate": (768, 3072), "output": (3072, 768)}.items():
        r = s.ranks[name]
        assert r % 16 == 0 and 0.45 < r * (i + o + s.b ** 2) / (i * o) < 0.55
    small = nw.ViTShape(layers=1, d=64, heads=4, mlp=128, image=32, patch=16, b=4, ranks={"qkv": 16, "intermediate": 16, "output": 16})
    m = nw.ViTEncoder(small, "dense", device="cpu", dtype=torch.float32)
    out = m(torch.randn(2, 3, 32, 32))
    assert out.shape == (2, 5, 64) and len(m.structured_linears()) == 3


def test_ideal_order_index_and_dense_folding_on_cpu():
    """The block-major (right_ideal) order against the oracle's re-ordering, and a dense layer that absorbs it."""
    from mem_efficient_blr_b200 import monarch_kernels as mk
    from oracle import blr_oracle as orc
    b, S, O = 4, 6, 5
    g = torch.Generator().manual_seed(0)
    y_int = torch.randn(3, S * b, generator=g)
    y_ideal = orc.monarch_ideal_order(y_int, b)
    idx = mk.ideal_order_index(S * b, b)
    assert torch.equal(y_ideal[..., idx], y_int)
    W = torch.randn(O, S * b, generator=g)
    Wf = mk.fold_ideal_order_into_dense(W, b)
    assert torch.allclose(y_ideal @ Wf.T, y_int @ W.T, atol=1e-6)
