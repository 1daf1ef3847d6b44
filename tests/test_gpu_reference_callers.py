"""The reference's own callers, unmodified, driven against this package (GPU).

oracle/_ref/ holds a byte-for-byte copy of the reference's models/wrappers.py, utils.py, layer.py, torch_funcs/ and
configs/ (made by oracle/make_ref.py).  These tests import them from there and only change *dotted function paths*:
wherever the reference's YAML or call site names `triton_funcs.<module>.<function>`, they name
`mem_efficient_blr_b200.<module>.<function>`.  Skipped when the copy is absent.
"""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")
PKG = "mem_efficient_blr_b200"


@pytest.fixture()
def ref(monkeypatch):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    if not os.path.isfile(os.path.join(REF, "models", "wrappers.py")):
        pytest.skip("oracle/_ref is absent: run `python oracle/make_ref.py <reference checkout>`")
    monkeypatch.syspath_prepend(REF)
    monkeypatch.chdir(REF)   # layer.py reads ./configs/config.yaml
    for name in ("utils", "models", "models.wrappers", "layer", "torch_funcs", "torch_funcs.blast_funcs"):
        sys.modules.pop(name, None)
    yield REF
    for name in list(sys.modules):
        if name in ("utils", "layer") or name.startswith("models") or name.startswith("torch_funcs"):
            sys.modules.pop(name, None)


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm())


def test_reference_wrapper_modules_on_this_package(ref):
    """models/wrappers.py classes with func_path -> this package, against the same classes with func_path ->
    torch_funcs.* (on CPU, fp32) after converting the parameters between the layouts (layer.py:191-226, 250-267)."""
    import models.wrappers as RW
    torch.manual_seed(0)
    x = torch.randn(2, 5, 512, dtype=torch.bfloat16)
    sc = lambda m: [p.data.mul_(0.05) for p in m.parameters()]

    def torch_twin(cls, *args, **kw):
        return cls(*args, device="cpu", dtype=torch.float32, **kw)

    for fn in ("triton_blast_partial_grouped_fp16", "triton_blast_bmm_fp16"):
        ours = RW.BlastLinear(512, 768, 4, 64, f"{PKG}.blast_kernels.{fn}", DEV, torch.bfloat16, bias=True)
        sc(ours)
        twin = torch_twin(RW.BlastLinear, 512, 768, 4, 64, "torch_funcs.blast_funcs.torch_blast_baseline", bias=True)
        U, V, S = (t.detach().float().cpu() for t in (ours.U, ours.V, ours.S))
        if "bmm" in fn:   # U (b,Q,R), V (b,P,R), S (R,b_out,b_in)
            twin.U.data, twin.V.data, twin.S.data = U, V.transpose(1, 2).contiguous(), S.permute(1, 2, 0).contiguous()
        else:             # U (b,R,Q), V (b,P,R), S (b_in,b_out,R)
            twin.U.data, twin.V.data, twin.S.data = U.transpose(1, 2).contiguous(), V.transpose(1, 2).contiguous(), S.transpose(0, 1).contiguous()
        twin.bias.data = ours.bias.detach().float().cpu()
        with torch.no_grad():
            got, want = ours(x.to(DEV)), twin(x.float())
        assert got.shape == want.shape and _rel(got, want) < 1e-2, fn

    ours = RW.LowRankLinear(512, 768, 64, f"{PKG}.low_rank_kernels.triton_low_rank_fp16", DEV, torch.bfloat16, bias=False)
    sc(ours)
    twin = torch_twin(RW.LowRankLinear, 512, 768, 64, "torch_funcs.low_rank_funcs.torch_low_rank_baseline", bias=False)
    twin.V.data, twin.U.data = ours.V.detach().float().cpu().t().contiguous(), ours.U.detach().float().cpu().t().contiguous()
    with torch.no_grad():
        got, want = ours(x.to(DEV)), twin(x.float())
    assert _rel(got, want.reshape(got.shape)) < 1e-2

    ours = RW.DenseLinear(512, 768, f"{PKG}.dense_kernels.triton_dense_fp16", DEV, torch.bfloat16, bias=False)
    sc(ours)
    twin = torch_twin(RW.DenseLinear, 512, 768, "torch_funcs.dense_funcs.torch_dense_baseline", bias=False)
    twin.W.data = ours.W.detach().float().cpu().t().contiguous()
    with torch.no_grad():
        got, want = ours(x.to(DEV)), twin(x.float())
    assert _rel(got, want.reshape(got.shape)) < 1e-2

    # Monarch: w1 (b,P,rank) in the harness' regrouped column order (layer.py:221-224), w2 (b,Q,rank)
    b, rank = 4, 64
    ours = RW.MonarchLinear(512, 768, b, rank, f"{PKG}.monarch_kernels.triton_monarch_right_fp16", DEV, torch.bfloat16, bias=False)
    sc(ours)
    twin = torch_twin(RW.MonarchLinear, 512, 768, b, rank, "torch_funcs.monarch_funcs.torch_monarch_baseline", bias=False)
    w1k = ours.w1_bfly.detach().float().cpu()                       # column l*per + jj holds torch column jj*b + l
    w1t = w1k.view(b, 512 // b, b, rank // b).permute(0, 1, 3, 2).reshape(b, 512 // b, rank).transpose(1, 2).contiguous()
    twin.w1_bfly.data, twin.w2_bfly.data = w1t, ours.w2_bfly.detach().float().cpu()
    with torch.no_grad():
        got, want = ours(x.to(DEV)), twin(x.float())
    assert _rel(got, want) < 1e-2


def test_reference_layer_swap_on_this_package(ref):
    """utils.replace_linear_with_custom (utils.py:46-116) with `func` paths into this package, on a block whose layer
    names follow the Llama keys of configs/networks/llama7b.yaml; the repository's mirror of it must swap the same layers."""
    import utils as RU
    import torch.nn as nn
    from mem_efficient_blr_b200 import wrappers as W

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp = nn.ModuleDict({"gate_proj": nn.Linear(512, 1024, bias=False), "up_proj": nn.Linear(512, 1024, bias=False),
                                      "down_proj": nn.Linear(1024, 512, bias=False)})
            self.head = nn.Linear(512, 64)

        def forward(self, x):
            return self.head(self.mlp["down_proj"](torch.nn.functional.silu(self.mlp["gate_proj"](x)) * self.mlp["up_proj"](x)))

    cfg = {k: {"b": 4, "rank": 64, "func": f"{PKG}.blast_kernels.triton_blast_partial_grouped_fp16", "compile": False}
           for k in ("mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")}
    a, b_ = Block().to(DEV, torch.bfloat16), Block().to(DEV, torch.bfloat16)
    RU.replace_linear_with_custom(a, cfg, "blast")
    n = W.replace_linear_with_custom(b_, cfg, "blast")
    assert n == 3
    for (na, ma), (nb, mb) in zip(a.named_modules(), b_.named_modules()):
        assert na == nb and type(ma).__name__ == type(mb).__name__
    assert type(a.mlp["up_proj"]).__name__ == "BlastLinear" and isinstance(a.head, nn.Linear)
    for m in a.modules():
        if type(m).__name__ == "BlastLinear":
            for p in m.parameters():
                p.data.mul_(0.05)
    with torch.no_grad():
        out = a(torch.randn(3, 512, device=DEV, dtype=torch.bfloat16))
    torch.cuda.synchronize()
    assert out.shape == (3, 64) and bool(torch.isfinite(out.float()).all())


def test_reference_layer_verify_on_this_package(ref, tmp_path):
    """layer.Layer.verify (layer.py:185-278) on the reference's llama7b q/k/v/o YAML with only the `triton_funcs.`
    prefixes changed (and torch.compile of the torch path switched off to keep the test short): every fp32 operator
    of this package must come out as MATCH under the reference's own comparison (do_verify, atol = 1e-1)."""
    import yaml
    from utils import VerificationStatus

    def edited(rel):
        with open(os.path.join(ref, rel)) as f:
            cfg = yaml.safe_load(f.read().replace("triton_funcs.", f"{PKG}."))
        for key in ("torch_blast", "torch_monarch", "torch_low_rank", "torch_dense"):
            if key in cfg:
                cfg[key]["compile"] = False
        return cfg

    # layer.py merges ./configs/config.yaml (relative to the working directory) under the layer's YAML
    (tmp_path / "configs").mkdir()
    (tmp_path / "configs" / "config.yaml").write_text(yaml.safe_dump(edited(os.path.join("configs", "config.yaml"))))
    cfg = edited(os.path.join("configs", "layers", "llama7b.qkvo_proj.yaml"))
    cfg["num_seq"], cfg["num_batches"] = 64, 1
    # the shipped YAMLs list no low-rank / dense verify functions; the schema has the keys (layer.py:104-133), so name
    # this package's functions there and let the reference's comparison run on them too
    for fam in ("low_rank", "dense"):
        cfg[f"triton_{fam}_verify"] = {"funcs": [f"{PKG}.{fam}_kernels.triton_{fam}_fp32"]}
        cfg[f"triton_{fam}_benchmark"] = {"funcs": [f"{PKG}.{fam}_kernels.triton_{fam}_fp16"]}
    path = tmp_path / "layer.yaml"
    path.write_text(yaml.safe_dump(cfg))
    os.chdir(tmp_path)   # (the fixture's monkeypatch.chdir restores the directory afterwards)
    from layer import Layer
    layer = Layer(str(path))
    torch.manual_seed(3)
    layer.verify("all")
    torch.cuda.synchronize()
    for name in ("triton_blast", "triton_monarch", "triton_low_rank", "triton_dense"):
        status = getattr(layer, f"{name}_verification_status")
        funcs = getattr(layer, f"{name}_verify")
        assert funcs and status, name
        for fn, st in zip(funcs, status):
            assert st == VerificationStatus.MATCH, (fn.__name__, st)
