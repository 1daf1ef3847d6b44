"""Network level on the GPU: a small Llama-shaped decoder and a small ViT-shaped encoder whose structured linears run
this package's kernels, against the same networks on CPU in fp32 whose structured linears call the oracle
(same seeds, same 16-bit-rounded parameters).  Bound: relative Frobenius error of the logits / features <= 1e-2."""
import pytest
import torch

from oracle import blr_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-2


def _round_params_like(model, dtype):
    """fp32 twin: every parameter rounded through the 16-bit type the GPU model stores."""
    with torch.no_grad():
        for p in list(model.parameters()) + list(model.buffers()):
            if p.is_floating_point():
                p.copy_(p.to(dtype).float())


def _oracle_linears(nw, model, bits):
    """Swaps the forward of every structured linear of the CPU twin for the oracle's BLAST."""
    for m in model.structured_linears():
        assert isinstance(m, nw.BlastTorchLinear)
        if bits == 16:
            m.forward = (lambda x, m=m: orc.blast(x, m.U, m.Vt, m.S)[0] + (0 if m.bias is None else m.bias))
        else:
            Uq, us = orc.quantize_sym(m.U.data.half(), bits)
            Vq, vs = orc.quantize_sym(m.Vt.data.half(), bits)
            m.forward = (lambda x, m=m, q=(Uq, us, Vq, vs): orc.blast_wq(x, *q, m.S, bits)[0] + (0 if m.bias is None else m.bias))


@pytest.mark.parametrize("method,bits", [("blast", 16), ("blast_int8", 8)])
def test_llama_shaped_decoder_matches_oracle_backed_twin(method, bits):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from mem_efficient_blr_b200 import networks as nw
    shape = nw.LlamaShape(layers=2, d=512, heads=8, ffn=1024, vocab=384, b=16, rank_attn=64, rank_mlp=96)
    B, T = 3, 12
    ids = torch.randint(0, shape.vocab, (B, T), generator=torch.Generator().manual_seed(5))
    gpu = nw.LlamaDecoder(shape, method, batch=B, cache_len=T, device=DEV, dtype=torch.float16, seed=11)
    cpu = nw.LlamaDecoder(shape, "blast", batch=B, cache_len=T, device="cpu", dtype=torch.float32, seed=11)
    _round_params_like(cpu, torch.float16)
    _oracle_linears(nw, cpu, bits)
    # prefill of T - 1 tokens (tensor-core pipeline: 33 rows per linear), then one decode step (3 rows: decode kernels)
    want_p, got_p = cpu.prefill(ids[:, :T - 1]), gpu.prefill(ids[:, :T - 1].to(DEV))
    want_d = cpu.decode_step(ids[:, T - 1:], torch.tensor([T - 1]))
    got_d = gpu.decode_step(ids[:, T - 1:].to(DEV), torch.tensor([T - 1], device=DEV))
    torch.cuda.synchronize()
    assert orc.rel_fro(got_p.float().cpu(), want_p) < TOL
    assert orc.rel_fro(got_d.float().cpu(), want_d) < TOL
    # the decode step replayed from a CUDA graph gives the same logits
    step = nw.GraphedCall(gpu.decode_step, ids[:, T - 1:].to(DEV), torch.tensor([T - 1], device=DEV))
    again = step(ids[:, T - 1:].to(DEV), torch.tensor([T - 1], device=DEV))
    torch.cuda.synchronize()
    assert orc.rel_fro(again.float().cpu(), got_d.float().cpu()) < 1e-3
    # the same step with the package's own attention kernel instead of torch's
    for layer in gpu.layers:
        layer.fused_attention_max_batch = B
    own = gpu.decode_step(ids[:, T - 1:].to(DEV), torch.tensor([T - 1], device=DEV))
    torch.cuda.synchronize()
    assert orc.rel_fro(own.float().cpu(), want_d) < TOL


def test_vit_shaped_encoder_matches_oracle_backed_twin():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from mem_efficient_blr_b200 import networks as nw
    shape = nw.ViTShape(layers=2, d=256, heads=4, mlp=512, image=64, patch=16, b=16,
                        ranks={"qkv": 32, "intermediate": 48, "output": 48})
    img = torch.randn(2, 3, 64, 64, generator=torch.Generator().manual_seed(2))
    gpu = nw.ViTEncoder(shape, "blast", device=DEV, dtype=torch.float16, seed=4)
    cpu = nw.ViTEncoder(shape, "blast", device="cpu", dtype=torch.float32, seed=4)
    # the twin's unseeded pieces (patch convolution, layer norms) take the GPU model's values
    cpu.load_state_dict({k: v.float().cpu() for k, v in gpu.state_dict().items()})
    _round_params_like(cpu, torch.float16)
    _oracle_linears(nw, cpu, 16)
    got = gpu(img.to(DEV, torch.float16))
    torch.cuda.synchronize()
    want = cpu(img.half().float())
    assert got.shape == (2, 17, 256)
    assert orc.rel_fro(got.float().cpu(), want) < TOL


def test_dit_shaped_denoiser_matches_oracle_backed_twin():
    """DiT block structure (adaLN-Zero modulation from one conditioning token per image, attention, tanh-GELU MLP) with
    the reference's swap list (qkv, fc1, adaLN linear; b = 9 blocks) against the twin on the oracle's BLAST."""
    from mem_efficient_blr_b200 import networks as nw
    shape = nw.DiTShape(layers=2, d=144, heads=4, mlp=288, latent=8, patch=2, channels=4, classes=10, b=9, freq=32,
                        ranks={"qkv": 32, "fc1": 24, "adaln": 16})
    g = torch.Generator().manual_seed(3)
    lat = torch.randn(3, 4, 8, 8, generator=g)
    t = torch.tensor([5.0, 400.0, 999.0])
    y = torch.tensor([0, 7, 10])
    gpu = nw.DiTDenoiser(shape, "blast", device=DEV, dtype=torch.float16, seed=4)
    cpu = nw.DiTDenoiser(shape, "blast", device="cpu", dtype=torch.float32, seed=4)
    cpu.load_state_dict({k: v.float().cpu() for k, v in gpu.state_dict().items()})
    _round_params_like(cpu, torch.float16)
    cpu.freqs.copy_(gpu.freqs.cpu())   # the fp32 frequency table is not a 16-bit weight: undo its rounding
    _oracle_linears(nw, cpu, 16)
    got = gpu(lat.to(DEV, torch.float16), t.to(DEV), y.to(DEV))
    torch.cuda.synchronize()
    want = cpu(lat.half().float(), t, y)
    assert got.shape == (3, 8, 8, 8)
    assert orc.rel_fro(got.float().cpu(), want) < TOL


# ------------------------------------------------------------------------------------------------ packed-weight files
@pytest.mark.parametrize("bits", [8, 4])
def test_packed_weight_file_rebuilds_the_quantised_decoder(tmp_path, bits):
    """16-bit decoder -> packer (device quantiser) -> file -> skeleton built without random numbers or 16-bit factors
    -> the same logits, bit for bit, as the decoder quantised in memory; the file holds the quantised layers only."""
    import os
    from mem_efficient_blr_b200 import networks as nw, packed
    shape = nw.LlamaShape(layers=2, d=256, heads=4, ffn=512, vocab=1000, b=4, rank_attn=64, rank_mlp=128)
    method = f"blast_int{bits}"
    src = nw.LlamaDecoder(shape, "blast", batch=2, cache_len=32, seed=11)
    want_model = nw.LlamaDecoder(shape, method, batch=2, cache_len=32, seed=11)
    tensors, layers = packed.pack_module(src, bits)
    assert len(layers) == 2 * 7 and all(v["kind"] == "blast_wq" and v["bits"] == bits for v in layers.values())
    assert not any(k.endswith((".U", ".Vt")) for k in tensors)
    path = os.path.join(tmp_path, "decoder.blrpack")
    size = packed.save_packed(path, tensors, layers, {"shape": vars(shape), "method": method})
    dense16 = sum(p.numel() * p.element_size() for p in src.parameters())
    assert size < dense16                      # the quantised factors are smaller than the 16-bit ones
    del src, tensors
    with nw.empty_init():
        got_model = nw.LlamaDecoder(shape, method, batch=2, cache_len=32, seed=0)
    meta = packed.load_packed_into(got_model, path)
    assert meta["method"] == method and meta["shape"]["rank_mlp"] == 128
    ids = torch.randint(0, shape.vocab, (2, 20), device="cuda")
    want, got = want_model.prefill(ids), got_model.prefill(ids)
    nxt = torch.randint(0, shape.vocab, (2, 1), device="cuda")
    pos = torch.tensor([20], device="cuda")
    want2, got2 = want_model.decode_step(nxt, pos), got_model.decode_step(nxt, pos)
    torch.cuda.synchronize()
    assert torch.equal(want, got) and torch.equal(want2, got2)
    # and back to the torch layout: the widened factors are what blr_dequantize_sym gives
    from mem_efficient_blr_b200 import ops
    loaded, layers2, _ = packed.load_packed(path, "cuda")
    state = packed.unpack_to_torch_layout(dict(loaded), layers2)
    p0 = "layers.0.q_proj" if "layers.0.q_proj" in layers2 else sorted(layers2)[0]
    U = ops.dequantize_sym(loaded[p0 + ".Uq"], loaded[p0 + ".u_scale"], bits, 0, torch.float16)
    assert torch.equal(state[p0 + ".U"], U) and p0 + ".Uq" not in state


# ------------------------------------------------------------------------------------------------ right_ideal chaining
@pytest.mark.parametrize("n", [1, 16, 200])
@pytest.mark.parametrize("chain", ["ideal", "interleaved"])
def test_monarch_swiglu_chained_on_the_ideal_order(chain, n):
    """gate / up in the reference's right_ideal order feeding down directly, against the oracle composition; and the
    dense layer with folded input columns that consumes the same activations."""
    from mem_efficient_blr_b200 import networks as nw, monarch_kernels as mk
    d, ffn, b, rank = 512, 1024, 4, 128
    g = torch.Generator().manual_seed(5)
    m = nw.MonarchSwiGLU(d, ffn, b, rank, chain, generator=g)
    x = torch.randn(n, d, generator=g).half()
    cpu = lambda t: t.detach().float().cpu()
    gate = orc.monarch(x, cpu(m.gate_w1), cpu(m.gate_w2))[0]
    up = orc.monarch(x, cpu(m.up_w1), cpu(m.up_w2))[0]
    if chain == "ideal":
        gate, up = orc.monarch_ideal_order(gate, b), orc.monarch_ideal_order(up, b)
    act = (torch.nn.functional.silu(gate.half().float()) * up.half().float()).half()
    ref = orc.monarch(act, cpu(m.down_w1), cpu(m.down_w2))[0]
    got = m(x.cuda())
    torch.cuda.synchronize()
    assert orc.rel_fro(got.float().cpu(), ref) < 1e-2
    if chain == "ideal":
        # a dense consumer absorbs the order by a column permutation
        W = (torch.randn(d, ffn, generator=g) / ffn ** 0.5).half()
        y_ideal = mk.monarch_torch_layout(x.cuda(), m.gate_w1, m.gate_w2, ideal=True)
        y_int = mk.monarch_torch_layout(x.cuda(), m.gate_w1, m.gate_w2)
        a = torch.nn.functional.linear(y_ideal, mk.fold_ideal_order_into_dense(W.cuda(), b))
        bb = torch.nn.functional.linear(y_int, W.cuda())
        torch.cuda.synchronize()
        assert orc.rel_fro(a.float().cpu(), bb.float().cpu()) < 2e-3
