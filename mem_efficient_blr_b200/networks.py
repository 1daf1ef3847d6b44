"""Network-level glue around the structured linears: a Llama-7B-shaped decoder, a ViT-B/16-shaped encoder and a
DiT-XL/2-shaped denoiser.

The reference times whole HuggingFace models whose nn.Linear layers were swapped for its structured modules
(models/llama7b.py:24-92, models/vit_b_patch16_224.py:69-131, utils.py:46-116).  No checkpoint or tokenizer can be
fetched here, so the networks are built from the shapes alone with random weights: the same layer list, the same
linears swapped (Llama: q/k/v/o and gate/up/down of every layer, lm_head stays dense; ViT: fused qkv, intermediate
and output of every layer, the attention output projection stays dense), and around them plain PyTorch - RMSNorm /
LayerNorm, rotary embedding, `scaled_dot_product_attention`, SwiGLU / GELU.  Those surrounding pieces are
placeholders for what a serving stack would fuse; the structured linears are what this package is about.

Decode runs against a static key/value cache (one write position per step, attention over the whole cache), so a
step has fixed shapes and can be captured in a CUDA graph (`GraphedCall`).
"""
from __future__ import annotations

import contextlib
import math
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import blast_kernels as bk
from . import blast_sym_quant_kernels as bq


# ------------------------------------------------------------------------------------------------ structured linears
_EMPTY_INIT = False


@contextlib.contextmanager
def empty_init():
    """Inside this context the networks and layers of this module are built with uninitialised weights (no random
    numbers, and quantised layers without their 16-bit factors ever existing): the skeleton for
    packed.load_packed_into."""
    global _EMPTY_INIT
    keep, _EMPTY_INIT = _EMPTY_INIT, True
    try:
        yield
    finally:
        _EMPTY_INIT = keep


class BlastTorchLinear(nn.Module):
    """BLAST linear on the torch layouts U (b,Q,R), Vt (b,R,P), S (b,b,R) (torch_funcs/blast_funcs.py:3-47), with a
    variance-preserving random init: x ~ N(0,1) gives out ~ N(0,1) (Vt ~ N(0,1/P), S ~ U(0.5,1.5), U ~ N(0,1/(R b E[S^2])))."""

    def __init__(self, in_features, out_features, b, rank, bias=False, device="cuda", dtype=torch.float16, generator=None):
        super().__init__()
        assert in_features % b == 0 and out_features % b == 0
        self.in_features, self.out_features, self.b, self.rank = in_features, out_features, b, rank
        P, Q = in_features // b, out_features // b
        g = generator
        gd = g.device if g is not None else "cpu"   # a CUDA generator fills the factors on the device (large models)
        if _EMPTY_INIT:
            for name, shp in (("U", (b, Q, rank)), ("Vt", (b, rank, P)), ("S", (b, b, rank))):
                setattr(self, name, nn.Parameter(torch.empty(shp, device=device, dtype=dtype), requires_grad=False))
            self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype), requires_grad=False) if bias else None
            return
        rn = lambda *s: torch.randn(*s, generator=g, device=gd)
        self.U = nn.Parameter((rn(b, Q, rank) / math.sqrt(rank * b * 13.0 / 12.0)).to(device=device, dtype=dtype), requires_grad=False)
        self.Vt = nn.Parameter((rn(b, rank, P) / math.sqrt(P)).to(device=device, dtype=dtype), requires_grad=False)
        self.S = nn.Parameter((torch.rand(b, b, rank, generator=g, device=gd) + 0.5).to(device=device, dtype=dtype), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype), requires_grad=False) if bias else None

    def forward(self, x, out_act=None):
        """out_act ("gelu" | "gelu_tanh"): the activation that follows the layer, applied in the kernels' epilogue where
        the fused call applies."""
        if self.bias is not None or out_act is not None:   # (bias and activation in the kernels' epilogue where the fused call applies)
            return bk.blast_multi_torch_layout(x, [(self.U, self.Vt, self.S)], biases=[self.bias], out_act=out_act)[0]
        return bk.blast_torch_layout(x, self.U, self.Vt, self.S)

    def U_device_ok(self) -> bool:
        return self.U.is_cuda

    def quantized(self, bits: int, group: int = 0) -> "BlastQuantLinear":
        return BlastQuantLinear(self, bits, group)


class BlastQuantLinear(nn.Module):
    """The same layer with int8 / packed-int4 factors and fp16 scales (the format of blr_blast_wq)."""

    def __init__(self, src: Optional[BlastTorchLinear], bits: int, group: int = 0):
        super().__init__()
        self.bits, self.group = bits, group
        if src is None:
            return   # BlastQuantLinear.empty fills the rest
        self.in_features, self.out_features, self.b, self.rank = src.in_features, src.out_features, src.b, src.rank
        Uq, us, Vq, vs = bq.quantize_blast_factors(src.U.data, src.Vt.data, bits, group)
        for name, t in (("Uq", Uq), ("u_scale", us), ("Vq", Vq), ("v_scale", vs), ("S", src.S.data)):
            self.register_buffer(name, t)
        self.bias = src.bias

    @classmethod
    def empty(cls, in_features, out_features, b, rank, bits, group=0, bias=False, device="cuda", dtype=torch.float16):
        """The layer with uninitialised buffers of the right shapes (to be filled from a packed-weight file)."""
        m = cls(None, bits, group)
        m.in_features, m.out_features, m.b, m.rank = in_features, out_features, b, rank
        P, Q, per = in_features // b, out_features // b, (1 if bits == 8 else 2)
        e = lambda shp, dt: torch.empty(shp, device=device, dtype=dt)
        m.register_buffer("Uq", e((b, Q, rank // per), torch.int8 if bits == 8 else torch.uint8))
        m.register_buffer("u_scale", e((b, Q) if group == 0 else (b, Q, rank // group), torch.float16))
        m.register_buffer("Vq", e((b, rank, P // per), torch.int8 if bits == 8 else torch.uint8))
        m.register_buffer("v_scale", e((b, rank) if group == 0 else (b, rank, P // group), torch.float16))
        m.register_buffer("S", e((b, b, rank), dtype))
        m.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype), requires_grad=False) if bias else None
        return m

    def U_device_ok(self) -> bool:
        return self.Uq.is_cuda

    def forward(self, x, out_act=None):
        if self.bias is not None or out_act is not None:
            return bq.blast_wq_multi(x, [(self.Uq, self.u_scale, self.Vq, self.v_scale, self.S)], self.bits, self.group,
                                     biases=[self.bias], out_act=out_act)[0]
        return bq.blast_wq(x, self.Uq, self.u_scale, self.Vq, self.v_scale, self.S, self.bits, self.group)


def make_linear(method: str, in_features: int, out_features: int, b: int, rank: int, bias: bool, device, dtype, generator):
    """method: 'blast' (16-bit factors), 'blast_int8', 'blast_int4', or 'dense' (nn.Linear, the unstructured bar)."""
    if method == "dense":
        lin = nn.Linear(in_features, out_features, bias=bias, device=device, dtype=dtype)
        gd = generator.device if generator is not None else "cpu"
        if _EMPTY_INIT:
            return lin.requires_grad_(False)
        with torch.no_grad():
            lin.weight.copy_((torch.randn(out_features, in_features, generator=generator, device=gd) / math.sqrt(in_features)).to(dtype))
            if bias:
                lin.bias.zero_()
        return lin.requires_grad_(False)
    if _EMPTY_INIT and method in ("blast_int8", "blast_int4"):
        return BlastQuantLinear.empty(in_features, out_features, b, rank, 8 if method == "blast_int8" else 4, 0, bias, device, dtype)
    base = BlastTorchLinear(in_features, out_features, b, rank, bias, device, dtype, generator)
    if method == "blast":
        return base
    if method in ("blast_int8", "blast_int4"):
        return base.quantized(8 if method == "blast_int8" else 4)
    raise ValueError(f"unknown method {method!r}")


def linear_act(m, x, act: str):
    """act(m(x)) for act = "gelu" | "gelu_tanh": inside the layer's kernels where it is a BLAST layer of this module (and its
    forward has not been replaced), else torch's activation on the layer's result."""
    if isinstance(m, (BlastTorchLinear, BlastQuantLinear)) and "forward" not in vars(m) and m.U_device_ok():
        return m(x, out_act=act)
    return F.gelu(m(x), approximate="tanh" if act == "gelu_tanh" else "none")


def structured_multi(mods, x, x_mul=None, residual=None):
    """[m(x') (+ residual) for m in mods] with x' = x, or silu(x) * x_mul: the layers of `mods` share their input.
    BLAST layers of equal shape go through the fused operators (one pair of launches at decode sizes, with the SwiGLU
    product, the bias and the residual folded in); anything else runs layer by layer."""
    res = None if residual is None else [residual] * len(mods)
    if any("forward" in vars(m) or not (isinstance(m, (BlastTorchLinear, BlastQuantLinear)) and m.U_device_ok()) for m in mods):
        pass   # replaced forward (tests put the oracle there), a dense layer or CPU tensors: layer by layer below
    elif all(isinstance(m, BlastTorchLinear) for m in mods):
        return bk.blast_multi_torch_layout(x, [(m.U, m.Vt, m.S) for m in mods], x_mul, [m.bias for m in mods], res)
    elif all(isinstance(m, BlastQuantLinear) for m in mods) and len({(m.bits, m.group) for m in mods}) == 1:
        return bq.blast_wq_multi(x, [(m.Uq, m.u_scale, m.Vq, m.v_scale, m.S) for m in mods], mods[0].bits, mods[0].group,
                                 x_mul, [m.bias for m in mods], res)
    xe = x if x_mul is None else F.silu(x) * x_mul
    return [m(xe) if residual is None else residual + m(xe) for m in mods]


class MonarchSwiGLU(nn.Module):
    """SwiGLU MLP on Monarch linears, torch layouts (w1_t (b, rank, P), w2_t (b, Qs, rank)): down(silu(gate(x)) * up(x)).
    chain = "ideal": gate and up leave their outputs in the block-major order of the reference's right_ideal variant
    (no interleave; contiguous stores) and down takes block l of that order as its input block l - the chaining of
    configs/networks/llama7b.yaml:164,180; "interleaved": every layer emits the interleaved order (the reference's
    `right`).  The two are different networks on the same factors (monarch_kernels.ideal_order_index)."""

    def __init__(self, d, ffn, b, rank, chain="ideal", device="cuda", dtype=torch.float16, generator=None):
        super().__init__()
        assert chain in ("ideal", "interleaved") and d % b == 0 and ffn % b == 0 and rank % b == 0
        self.d, self.ffn, self.b, self.rank, self.chain = d, ffn, b, rank, chain
        gd = generator.device if generator is not None else "cpu"
        rn = lambda *s: torch.randn(*s, generator=generator, device=gd)
        mk_ = lambda t: nn.Parameter(t.to(device=device, dtype=dtype), requires_grad=False)
        for name, (i_f, o_f) in (("gate", (d, ffn)), ("up", (d, ffn)), ("down", (ffn, d))):
            setattr(self, name + "_w1", mk_(rn(b, rank, i_f // b) / math.sqrt(i_f // b)))
            setattr(self, name + "_w2", mk_(rn(b, o_f // b, rank) / math.sqrt(rank)))

    def forward(self, x):
        from . import monarch_kernels as mk
        ideal = self.chain == "ideal"
        g = mk.monarch_torch_layout(x, self.gate_w1, self.gate_w2, ideal)
        u = mk.monarch_torch_layout(x, self.up_w1, self.up_w2, ideal)
        return mk.monarch_torch_layout(F.silu(g) * u, self.down_w1, self.down_w2)


# ------------------------------------------------------------------------------------------------ Llama-shaped decoder
@dataclass
class LlamaShape:
    """Llama-7B: 32 layers, d = 4096, 32 heads, FFN 11008 (SwiGLU), vocabulary 32000; BLAST b = 16 with the ranks of
    the reference's configs/networks/llama7b.yaml (q/k/v/o 1024, gate/up/down 1488: 50 % of the dense parameters)."""
    layers: int = 32
    d: int = 4096
    heads: int = 32
    ffn: int = 11008
    vocab: int = 32000
    b: int = 16
    rank_attn: int = 1024
    rank_mlp: int = 1488
    rope_theta: float = 10000.0
    eps: float = 1e-6


class RMSNorm(nn.Module):
    def __init__(self, d, eps, device, dtype):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d, device=device, dtype=dtype), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        if x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and x.shape[-1] % 8 == 0:
            from . import ops
            return ops.rmsnorm(x, self.weight, self.eps)   # one kernel instead of five element-wise ones
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return (v * self.weight.float()).to(x.dtype)


class LayerNorm(nn.LayerNorm):
    """nn.LayerNorm whose 16-bit CUDA forward is the package's kernel (a warp per row: 12.6 k rows of 768 values took
    torch's kernel 33 us, a sixth of the memory rate); anything else runs torch's."""

    def forward(self, x):
        d = x.shape[-1]
        if x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and d % 8 == 0 and d <= 2048 and len(self.normalized_shape) == 1 \
                and not torch.compiler.is_compiling():
            from . import ops
            return ops.layernorm(x, self.weight, self.bias, self.eps)
        return super().forward(x)


def _rope(q, k, cos, sin):
    """q, k (B, H, T, hd); cos, sin (T, hd/2): rotate pairs (first half, second half) like HF's Llama."""
    def rot(t):
        t1, t2 = t.float().chunk(2, dim=-1)
        return torch.cat((t1 * cos - t2 * sin, t2 * cos + t1 * sin), dim=-1).to(t.dtype)
    return rot(q), rot(k)


class LlamaLayer(nn.Module):
    def __init__(self, shape: LlamaShape, method: str, device, dtype, generator):
        super().__init__()
        s, mk = shape, lambda i, o, r: make_linear(method, i, o, shape.b, r, False, device, dtype, generator)
        self.heads, self.hd = s.heads, s.d // s.heads
        # Batches up to this size use the package's attention kernel (ops.attention_decode), larger ones torch's
        # scaled_dot_product_attention.  Measured through the whole decode step at 2048 keys (ms, torch | package):
        # batch 1 3.08 | 3.23, 4: 3.94 | 4.28, 16: 7.34 | 8.56, 64: 15.5 | 18.0 - torch's flash-decoding kernel streams the
        # cache at 6.3 - 7.3 TB/s, the package's at 4.4 - 5.7: the library kernel serves every batch size.
        self.fused_attention_max_batch = 0
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = (mk(s.d, s.d, s.rank_attn) for _ in range(4))
        self.gate_proj, self.up_proj = mk(s.d, s.ffn, s.rank_mlp), mk(s.d, s.ffn, s.rank_mlp)
        self.down_proj = mk(s.ffn, s.d, s.rank_mlp)
        self.input_layernorm = RMSNorm(s.d, s.eps, device, dtype)
        self.post_attention_layernorm = RMSNorm(s.d, s.eps, device, dtype)

    def structured(self):
        return [self.q_proj, self.k_proj, self.v_proj, self.o_proj, self.gate_proj, self.up_proj, self.down_proj]

    def _decode_fused(self, x, cos_table, sin_table, kc, vc, pos):
        """One new token per sequence on the GPU: four structured-linear calls and four small kernels (two norms,
        rotary embedding + cache append, attention over the cache) instead of some thirty element-wise launches."""
        from . import ops
        B, _, d = x.shape
        h = self.input_layernorm(x)
        q, k, v = (t.view(B, d) for t in structured_multi([self.q_proj, self.k_proj, self.v_proj], h))
        ops.rope_append(q, k, v, cos_table, sin_table, pos, kc, vc, 1)
        if B <= self.fused_attention_max_batch:
            a = ops.attention_decode(q, kc, vc)
        else:
            a = F.scaled_dot_product_attention(q.view(B, self.heads, 1, self.hd), kc, vc).view(B, d)
        (x,) = structured_multi([self.o_proj], a.view(B, 1, d), residual=x)
        h = self.post_attention_layernorm(x)
        g, u = structured_multi([self.gate_proj, self.up_proj], h)
        (x,) = structured_multi([self.down_proj], g, x_mul=u, residual=x)
        return x

    def forward(self, x, cos, sin, kc, vc, pos, causal: bool, tables=None):
        """x (B, T, d); kc, vc (B, H, S, hd) static cache; pos (T,) int64 cache slots of these tokens; cos, sin (T, hd/2)
        the angles of those slots.  causal: the T tokens are the whole sequence so far (prefill); else they attend to
        the whole cache.  tables: the full (S, hd/2) cos / sin tables, which selects the fused decode path."""
        B, T, d = x.shape
        if tables is not None and not causal:
            return self._decode_fused(x, tables[0], tables[1], kc, vc, pos)
        h = self.input_layernorm(x)
        if tables is not None:
            # prefill on the GPU (slots 0 .. T-1): one kernel rotates q in place and writes the rotated k and v into the
            # cache, whose first T slots then serve as the keys and values (torch's rotate / cat / index_copy chain was
            # about 390 us per layer at 2048 tokens, 30 % of the prefill)
            from . import ops
            q, k, v = structured_multi([self.q_proj, self.k_proj, self.v_proj], h)
            ops.rope_append(q.view(B * T, d), k.view(B * T, d), v.view(B * T, d), tables[0], tables[1], pos, kc, vc, T)
            a = F.scaled_dot_product_attention(q.view(B, T, self.heads, self.hd).transpose(1, 2), kc[:, :, :T], vc[:, :, :T], is_causal=True)
        else:
            q, k, v = (t.view(B, T, self.heads, self.hd).transpose(1, 2) for t in
                       structured_multi([self.q_proj, self.k_proj, self.v_proj], h))
            q, k = _rope(q, k, cos, sin)
            kc.index_copy_(2, pos, k)
            vc.index_copy_(2, pos, v)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True) if causal else F.scaled_dot_product_attention(q, kc, vc)
        (x,) = structured_multi([self.o_proj], a.transpose(1, 2).reshape(B, T, -1), residual=x)
        h = self.post_attention_layernorm(x)
        g, u = structured_multi([self.gate_proj, self.up_proj], h)
        (x,) = structured_multi([self.down_proj], g, x_mul=u, residual=x)   # down(silu(gate) * up) + x
        return x


class LlamaDecoder(nn.Module):
    """Decoder of the shape above with a static cache for `cache_len` positions and `batch` sequences."""

    def __init__(self, shape: LlamaShape, method: str, batch: int, cache_len: int, device="cuda", dtype=torch.float16, seed=0,
                 init_on_device: bool = False):
        super().__init__()
        g = torch.Generator(device=device if init_on_device else "cpu").manual_seed(seed)
        self.shape, self.method, self.batch, self.cache_len = shape, method, batch, cache_len
        self.fused_decode = True   # False: prefill and decode step run torch modules around the linears (no rotary / cache / norm-fusing kernels)
        self.embed_tokens = nn.Embedding(shape.vocab, shape.d, device=device, dtype=dtype)
        with torch.no_grad():
            if not _EMPTY_INIT:
                self.embed_tokens.weight.copy_(torch.randn(shape.vocab, shape.d, generator=g, device=g.device).to(dtype))
        self.embed_tokens.requires_grad_(False)
        self.layers = nn.ModuleList(LlamaLayer(shape, method, device, dtype, g) for _ in range(shape.layers))
        self.norm = RMSNorm(shape.d, shape.eps, device, dtype)
        self.lm_head = make_linear("dense", shape.d, shape.vocab, 0, 0, False, device, dtype, g)
        hd = shape.d // shape.heads
        inv = 1.0 / (shape.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
        ang = torch.outer(torch.arange(cache_len, dtype=torch.float32), inv)
        self.register_buffer("cos", ang.cos().to(device), persistent=False)
        self.register_buffer("sin", ang.sin().to(device), persistent=False)
        self.kcache = [torch.zeros(batch, shape.heads, cache_len, hd, device=device, dtype=dtype) for _ in range(shape.layers)]
        self.vcache = [torch.zeros(batch, shape.heads, cache_len, hd, device=device, dtype=dtype) for _ in range(shape.layers)]

    def structured_linears(self):
        return [m for layer in self.layers for m in layer.structured()]

    def _run(self, ids, pos, causal):
        x = self.embed_tokens(ids)
        B = ids.shape[0]   # a smaller batch than the cache was built for uses the first B sequences' slots
        # one new token per sequence on the GPU with 16-bit activations takes the fused decode path
        hd = self.shape.d // self.shape.heads
        kernels = x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and hd in (8, 16, 32, 64, 128, 256) and self.fused_decode
        # one new token per sequence: the fused decode step; a prefill (the whole sequence so far, slots 0 .. T-1): the rotary
        # / cache kernel in front of torch's causal attention
        fused = kernels and ((not causal and ids.shape[1] == 1) or causal)
        tables = (self.cos, self.sin) if fused else None
        cos, sin = (None, None) if fused else (self.cos.index_select(0, pos), self.sin.index_select(0, pos))
        for i, layer in enumerate(self.layers):
            x = layer(x, cos, sin, self.kcache[i][:B], self.vcache[i][:B], pos, causal, tables)
        return self.lm_head(self.norm(x[:, -1]))

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """ids (B, T), T <= cache_len: fills cache slots 0..T-1, returns the logits of the last position (B, vocab)."""
        pos = torch.arange(ids.shape[1], device=ids.device)
        return self._run(ids, pos, True)

    @torch.no_grad()
    def decode_step(self, ids: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """ids (B, 1): one new token per sequence, written to cache slot pos (1,) and attending to the whole cache
        (slots beyond the sequence's length must hold real keys: the benchmark decodes at a full cache)."""
        return self._run(ids, pos, False)


# ------------------------------------------------------------------------------------------------ ViT-shaped encoder
@dataclass
class ViTShape:
    """ViT-B/16 at 224 x 224: 12 layers, d = 768, 12 heads, MLP 3072, 196 patches + class token = 197 tokens.
    BLAST b = 16 with ranks for 50 % of the dense parameters: R (I + O + b^2) = I O / 2."""
    layers: int = 12
    d: int = 768
    heads: int = 12
    mlp: int = 3072
    image: int = 224
    patch: int = 16
    b: int = 16
    eps: float = 1e-12
    ranks: dict = field(default_factory=lambda: {"qkv": 256, "intermediate": 288, "output": 288})


class ViTLayer(nn.Module):
    def __init__(self, shape: ViTShape, method: str, device, dtype, generator):
        super().__init__()
        s = shape
        mk = lambda i, o, r: make_linear(method, i, o, s.b, r, True, device, dtype, generator)
        self.heads = s.heads
        self.qkv = mk(s.d, 3 * s.d, s.ranks["qkv"])                 # fused like fuse_qkv_in_vit (vit_b_patch16_224.py:14-66)
        self.attn_out = make_linear("dense", s.d, s.d, 0, 0, True, device, dtype, generator)  # skipped by the reference's swap
        self.intermediate = mk(s.d, s.mlp, s.ranks["intermediate"])
        self.output = mk(s.mlp, s.d, s.ranks["output"])
        self.ln1 = LayerNorm(s.d, eps=s.eps, device=device, dtype=dtype).requires_grad_(False)
        self.ln2 = LayerNorm(s.d, eps=s.eps, device=device, dtype=dtype).requires_grad_(False)

    def structured(self):
        return [self.qkv, self.intermediate, self.output]

    def forward(self, x):
        B, T, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v)
        x = x + self.attn_out(a.transpose(1, 2).reshape(B, T, d))
        return x + self.output(linear_act(self.intermediate, self.ln2(x), "gelu"))


class ViTEncoder(nn.Module):
    def __init__(self, shape: ViTShape, method: str, device="cuda", dtype=torch.float16, seed=0, init_on_device: bool = False):
        super().__init__()
        g = torch.Generator(device=device if init_on_device else "cpu").manual_seed(seed)
        s = shape
        self.shape, self.method = shape, method
        self.patch = nn.Conv2d(3, s.d, s.patch, s.patch, device=device, dtype=dtype).requires_grad_(False)
        ntok = (s.image // s.patch) ** 2 + 1
        self.cls = nn.Parameter((torch.randn(1, 1, s.d, generator=g, device=g.device) * 0.02).to(device=device, dtype=dtype), requires_grad=False)
        self.posemb = nn.Parameter((torch.randn(1, ntok, s.d, generator=g, device=g.device) * 0.02).to(device=device, dtype=dtype), requires_grad=False)
        self.layers = nn.ModuleList(ViTLayer(s, method, device, dtype, g) for _ in range(s.layers))
        self.ln = LayerNorm(s.d, eps=s.eps, device=device, dtype=dtype).requires_grad_(False)

    def structured_linears(self):
        return [m for layer in self.layers for m in layer.structured()]

    @torch.no_grad()
    def forward(self, images: torch.Tensor) -> torch.Tensor:
        """images (B, 3, 224, 224) -> features (B, 197, d)."""
        # the patch embedding as one GEMM over unfolded patches (the convolution's weights, viewed (d, 3 p p)): the strided
        # convolution took 0.48 ms at batch 64 with its layout changes, a twentieth of the whole forward
        B, C, H, W = images.shape
        p = self.shape.patch
        x = images.view(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // p) * (W // p), C * p * p)
        x = F.linear(x, self.patch.weight.view(self.patch.weight.shape[0], -1), self.patch.bias)
        # class token and position embedding written straight into the token stream: one add over the patch rows instead
        # of a concatenation (62 us at batch 64) followed by an add
        tok = torch.empty(B, x.shape[1] + 1, x.shape[2], device=x.device, dtype=x.dtype)
        tok[:, :1] = self.cls + self.posemb[:, :1]
        torch.add(x, self.posemb[:, 1:], out=tok[:, 1:])
        x = tok
        for layer in self.layers:
            x = layer(x)
        return self.ln(x)


# ------------------------------------------------------------------------------------------------ DiT-shaped denoiser
@dataclass
class DiTShape:
    """DiT-XL/2 on 32 x 32 x 4 latents (256 x 256 images): 28 blocks, d = 1152, 16 heads, MLP 4608, patch 2 -> 256
    tokens, 1000 classes, adaLN-Zero conditioning on timestep + class.  Structured linears and their BLAST settings as
    in the reference's configs/networks/dit_xl.yaml: attn.qkv (rank 384), mlp.fc1 (256), adaLN_modulation.1 (256),
    all with b = 9; attn.proj and mlp.fc2 stay dense."""
    layers: int = 28
    d: int = 1152
    heads: int = 16
    mlp: int = 4608
    latent: int = 32
    patch: int = 2
    channels: int = 4
    classes: int = 1000
    b: int = 9
    freq: int = 256
    eps: float = 1e-6
    ranks: dict = field(default_factory=lambda: {"qkv": 384, "fc1": 256, "adaln": 256})


def _modulate(x, shift, scale):
    """x * (1 + scale) + shift with shift, scale (B, d) broadcast over the tokens: one small add and one fused multiply-add."""
    return torch.addcmul(shift.unsqueeze(1), x, (scale + 1).unsqueeze(1))


class DiTBlock(nn.Module):
    """x <- x + gate_a * attn(mod(norm(x))), x <- x + gate_m * mlp(mod(norm(x))); the six modulation vectors come
    from one linear on silu(c), c (B, d) the conditioning of the image (one token per image: a decode-size call)."""

    def __init__(self, shape: DiTShape, method: str, device, dtype, generator):
        super().__init__()
        s = shape
        mk = lambda i, o, r: make_linear(method, i, o, s.b, r, True, device, dtype, generator)
        dense = lambda i, o: make_linear("dense", i, o, 0, 0, True, device, dtype, generator)
        self.heads = s.heads
        self.qkv = mk(s.d, 3 * s.d, s.ranks["qkv"])
        self.proj = dense(s.d, s.d)
        self.fc1 = mk(s.d, s.mlp, s.ranks["fc1"])
        self.fc2 = dense(s.mlp, s.d)
        self.adaln = mk(s.d, 6 * s.d, s.ranks["adaln"])
        self.norm1 = LayerNorm(s.d, eps=s.eps, elementwise_affine=False, device=device, dtype=dtype)
        self.norm2 = LayerNorm(s.d, eps=s.eps, elementwise_affine=False, device=device, dtype=dtype)

    def structured(self):
        return [self.qkv, self.fc1, self.adaln]

    def forward(self, x, c):
        B, T, d = x.shape
        sa, ca, ga, sm, cm, gm = self.adaln(F.silu(c)).chunk(6, dim=1)
        # 16-bit tensors on the GPU: norm + modulation in one kernel and the gated residuals in another (torch's broadcast
        # element-wise kernels ran at 1 TB/s: a quarter of the denoiser's time at batch 64)
        fast = x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and d % 8 == 0 and d <= 2048 and not torch.compiler.is_compiling()
        if fast:
            from . import ops
            mod = lambda norm, t, shift, scale: ops.layernorm_modulate(t, shift, scale, norm.eps)
            gated = ops.gated_add
        else:
            mod = lambda norm, t, shift, scale: _modulate(norm(t), shift, scale)
            gated = lambda t, gate, y: torch.addcmul(t, gate.unsqueeze(1), y)
        q, k, v = self.qkv(mod(self.norm1, x, sa, ca)).view(B, T, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v)
        x = gated(x, ga, self.proj(a.transpose(1, 2).reshape(B, T, d)))
        return gated(x, gm, self.fc2(linear_act(self.fc1, mod(self.norm2, x, sm, cm), "gelu_tanh")))


class DiTDenoiser(nn.Module):
    """Latents (B, C, H, W), timesteps (B,), class labels (B,) -> (B, 2C, H, W) (noise and variance channels).  Patch
    embedding, positional embedding, timestep MLP on sinusoidal features, class embedding, the blocks, and an
    adaLN-modulated linear back to patches.  Random weights of the shape (no checkpoint can be fetched here)."""

    def __init__(self, shape: DiTShape, method: str, device="cuda", dtype=torch.float16, seed=0, init_on_device: bool = False):
        super().__init__()
        g = torch.Generator(device=device if init_on_device else "cpu").manual_seed(seed)
        s = shape
        self.shape, self.method = shape, method
        self.x_embed = nn.Conv2d(s.channels, s.d, s.patch, s.patch, device=device, dtype=dtype).requires_grad_(False)
        ntok = (s.latent // s.patch) ** 2
        self.posemb = nn.Parameter((torch.randn(1, ntok, s.d, generator=g, device=g.device) * 0.02).to(device=device, dtype=dtype), requires_grad=False)
        dense = lambda i, o: make_linear("dense", i, o, 0, 0, True, device, dtype, g)
        self.t_fc1, self.t_fc2 = dense(s.freq, s.d), dense(s.d, s.d)
        self.y_embed = nn.Embedding(s.classes + 1, s.d, device=device, dtype=dtype).requires_grad_(False)
        self.blocks = nn.ModuleList(DiTBlock(s, method, device, dtype, g) for _ in range(s.layers))
        self.final_norm = LayerNorm(s.d, eps=s.eps, elementwise_affine=False, device=device, dtype=dtype)
        self.final_adaln = dense(s.d, 2 * s.d)
        self.final = dense(s.d, s.patch * s.patch * 2 * s.channels)
        half = s.freq // 2
        self.register_buffer("freqs", torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32) / half).to(device), persistent=False)

    def structured_linears(self):
        return [m for blk in self.blocks for m in blk.structured()]

    @torch.no_grad()
    def forward(self, latents: torch.Tensor, t: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        s = self.shape
        B = latents.shape[0]
        # patch embedding as a GEMM over unfolded patches, which also leaves x token-major and contiguous (the transposed
        # view of a convolution's output made every element-wise kernel after it a strided one and every norm a copy)
        C, p = s.channels, s.patch
        hh = s.latent // p
        x = latents.view(B, C, hh, p, hh, p).permute(0, 2, 4, 1, 3, 5).reshape(B, hh * hh, C * p * p)
        x = F.linear(x, self.x_embed.weight.view(self.x_embed.weight.shape[0], -1), self.x_embed.bias) + self.posemb
        ang = t.float()[:, None] * self.freqs[None]
        temb = torch.cat((ang.cos(), ang.sin()), dim=-1).to(x.dtype)
        c = self.t_fc2(F.silu(self.t_fc1(temb))) + self.y_embed(y)
        for blk in self.blocks:
            x = blk(x, c)
        shift, scale = self.final_adaln(F.silu(c)).chunk(2, dim=1)
        x = self.final(_modulate(self.final_norm(x), shift, scale))
        # patches back to the image grid: (B, h, w, p, p, C) -> (B, C, h p, w p)
        h = s.latent // s.patch
        x = x.view(B, h, h, s.patch, s.patch, 2 * s.channels).permute(0, 5, 1, 3, 2, 4)
        return x.reshape(B, 2 * s.channels, h * s.patch, h * s.patch)


# ------------------------------------------------------------------------------------------------ CUDA-graph replay
class GraphedCall:
    """Captures `fn(*static_inputs)` once in a CUDA graph and replays it; inputs are updated by copying into the
    static tensors.  The structured operators launch on the current stream from caller-provided tensors and their
    per-stream workspace exists after the warm-up calls, so a capture contains no allocation of theirs."""

    def __init__(self, fn, *static_inputs, warmup: int = 2):
        self.fn, self.inputs = fn, static_inputs
        self.stream = torch.cuda.Stream()
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                self.out = fn(*static_inputs)
            self.stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                self.out = fn(*static_inputs)
        torch.cuda.current_stream().wait_stream(self.stream)

    def __call__(self, *new_inputs):
        for dst, src in zip(self.inputs, new_inputs):
            dst.copy_(src)
        self.graph.replay()
        return self.out
