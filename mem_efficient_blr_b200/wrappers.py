"""nn.Module wrappers with the reference's constructor signatures (models/wrappers.py:5-181).

`func_path` is a dotted path to an operator function; like the reference, the parameter layouts are
chosen from substrings of the function name ("triton" / "torch", "bmm", "left"), parameters are
`torch.randn`, and `forward` adds the bias in place.  The default `func_path`s point at this package.
`QuantBlastLinear` is the weight-quantised module, which the reference does not have.
"""
from __future__ import annotations

import importlib

import torch
import torch.nn as nn

_PKG = __name__.rsplit(".", 1)[0]


def _resolve(func_path: str):
    module_name, func_name = func_path.rsplit(".", 1)
    return func_name, getattr(importlib.import_module(module_name), func_name)


class _Base(nn.Module):
    def _bias(self, bias, device, dtype):
        if bias:
            self.bias = nn.Parameter(torch.randn(self.out_features, device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)

    def _finish(self, x, out):
        if self.bias is not None:
            out += self.bias.to(x.dtype)
        return out


class BlastLinear(_Base):
    """Mirror of BlastLinear (models/wrappers.py:131-181)."""

    def __init__(self, in_features, out_features, b, rank, func_path=f"{_PKG}.blast_kernels.triton_blast_partial_grouped_fp16",
                 device="cuda", dtype=torch.bfloat16, bias=True, is_compiled=False):
        super().__init__()
        assert in_features % b == 0 and out_features % b == 0
        self.in_features, self.out_features, self.b, self.rank = in_features, out_features, b, rank
        self.func_name, self.func = _resolve(func_path)
        if is_compiled:
            self.func = torch.compile(self.func)
        P, Q = in_features // b, out_features // b
        kw = dict(device=device, dtype=dtype)
        if "triton" in self.func_name:
            if "bmm" in self.func_name:
                shapes = ((b, Q, rank), (b, P, rank), (rank, b, b))
            else:
                shapes = ((b, rank, Q), (b, P, rank), (b, b, rank))
        elif "torch" in self.func_name:
            shapes = ((b, Q, rank), (b, rank, P), (b, b, rank))
        else:
            raise ValueError("function name must contain 'triton' or 'torch' (the reference picks layouts from it)")
        self.U, self.V, self.S = (nn.Parameter(torch.randn(s, **kw)) for s in shapes)
        self._bias(bias, device, dtype)

    def forward(self, x):
        out = self.func(x, self.U, self.V, self.S)
        if isinstance(out, tuple):
            out = out[0]
        return self._finish(x, out)

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"rank={self.rank}, b={self.b}, func={self.func_name}")


class MonarchLinear(_Base):
    """Mirror of MonarchLinear (models/wrappers.py:5-52)."""

    def __init__(self, in_features, out_features, b, rank, func_path=f"{_PKG}.monarch_kernels.triton_monarch_right_fp16",
                 device="cuda", dtype=torch.bfloat16, bias=True, is_compiled=False):
        super().__init__()
        assert in_features % b == 0 and out_features % b == 0
        assert rank % b == 0
        self.in_features, self.out_features, self.b, self.rank = in_features, out_features, b, rank
        self.func_name, self.func = _resolve(func_path)
        if is_compiled:
            self.func = torch.compile(self.func)
        P, Q = in_features // b, out_features // b
        kw = dict(device=device, dtype=dtype)
        if "triton" in self.func_name:
            self.w1_bfly = nn.Parameter(torch.randn((b, P, rank), **kw))
            self.w2_bfly = nn.Parameter(torch.randn((b, rank, Q) if "left" in self.func_name else (b, Q, rank), **kw))
        elif "torch" in self.func_name:
            self.w1_bfly = nn.Parameter(torch.randn((b, rank, P), **kw))
            self.w2_bfly = nn.Parameter(torch.randn((b, Q, rank), **kw))
        else:
            raise ValueError("function name must contain 'triton' or 'torch'")
        self._bias(bias, device, dtype)

    def forward(self, x):
        out = self.func(x, self.w1_bfly, self.w2_bfly)
        if isinstance(out, tuple):
            out = out[0]
        return self._finish(x, out)


class LowRankLinear(_Base):
    """Mirror of LowRankLinear (models/wrappers.py:54-92); like the reference, a 2-D result gets the bias too."""

    def __init__(self, in_features, out_features, rank, func_path=f"{_PKG}.low_rank_kernels.triton_low_rank_fp16",
                 device="cuda", dtype=torch.bfloat16, bias=True, is_compiled=False):
        super().__init__()
        self.in_features, self.out_features, self.rank = in_features, out_features, rank
        self.func_name, self.func = _resolve(func_path)
        if is_compiled:
            self.func = torch.compile(self.func)
        kw = dict(device=device, dtype=dtype)
        if "triton" in self.func_name:
            self.V = nn.Parameter(torch.randn((in_features, rank), **kw))
            self.U = nn.Parameter(torch.randn((rank, out_features), **kw))
        else:
            self.V = nn.Parameter(torch.randn((rank, in_features), **kw))
            self.U = nn.Parameter(torch.randn((out_features, rank), **kw))
        self._bias(bias, device, dtype)

    def forward(self, x):
        out = self.func(x, self.V, self.U)
        if isinstance(out, tuple):
            out = out[0]
        return self._finish(x, out)


class DenseLinear(_Base):
    """Mirror of DenseLinear (models/wrappers.py:94-129)."""

    def __init__(self, in_features, out_features, func_path=f"{_PKG}.dense_kernels.triton_dense_fp16", device="cuda",
                 dtype=torch.bfloat16, bias=True, is_compiled=False):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.func_name, self.func = _resolve(func_path)
        if is_compiled:
            self.func = torch.compile(self.func)
        kw = dict(device=device, dtype=dtype)
        shape = (in_features, out_features) if "triton" in self.func_name else (out_features, in_features)
        self.W = nn.Parameter(torch.randn(shape, **kw))
        self._bias(bias, device, dtype)

    def forward(self, x):
        return self._finish(x, self.func(x, self.W))


class QuantBlastLinear(_Base):
    """BLAST linear with int8 / packed-int4 factors (up to 16 tokens per call).  Built from torch-layout
    16-bit factors U (b,Q,R), Vt (b,R,P), S (b,b,R); one scale per output channel, or per 128 contraction indices
    with group = 128; no counterpart in the reference."""

    def __init__(self, U: torch.Tensor, Vt: torch.Tensor, S: torch.Tensor, bits: int = 8, bias: torch.Tensor | None = None,
                 group: int = 0):
        super().__init__()
        from . import blast_sym_quant_kernels as bq
        self.bits, self.group = bits, group
        b, Q, R = U.shape
        self.in_features, self.out_features, self.b, self.rank = b * Vt.shape[2], b * Q, b, R
        Uq, us, Vq, vs = bq.quantize_blast_factors(U, Vt, bits, group)
        for name, t in (("Uq", Uq), ("u_scale", us), ("Vq", Vq), ("v_scale", vs), ("S", S.contiguous())):
            self.register_buffer(name, t)
        self.bias = None if bias is None else nn.Parameter(bias)
        self._op = bq.blast_wq

    def forward(self, x):
        return self._finish(x, self._op(x, self.Uq, self.u_scale, self.Vq, self.v_scale, self.S, self.bits, self.group))


def replace_linear_with_factory(module: nn.Module, key: str, factory) -> int:
    """Swaps every nn.Linear whose qualified name contains `key` for `factory(in_features, out_features, bias)`.
    Returns the count."""
    n = 0
    for name, child in list(module.named_modules()):
        if key in name and isinstance(child, nn.Linear):
            parent = module
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            setattr(parent, parts[-1], factory(child.in_features, child.out_features, child.bias is not None))
            n += 1
    return n


def _conv1d_type():
    try:  # HuggingFace's GPT-2 style linear (weight stored transposed); optional
        from transformers.pytorch_utils import Conv1D
        return Conv1D
    except Exception:
        return ()


def replace_linear_with_custom(model: nn.Module, layer_configs: dict, method: str, skip_keys=None) -> int:
    """Mirror of utils.replace_linear_with_custom (utils.py:46-116), same arguments: for every (key, config) of
    `layer_configs`, each nn.Linear (or HF Conv1D) whose qualified name contains `key` - and none of `skip_keys` -
    becomes the structured module of `method` ("blast", "blast_sym_quant", "monarch", "low_rank", "dense") built from
    config["b"], config["rank"], config["func"] (dotted path of the operator function) and config.get("compile").
    Device, dtype and the presence of a bias follow the replaced layer.  Returns the number of layers replaced."""
    conv1d = _conv1d_type()
    skip_keys = skip_keys or []
    count = 0
    for name, module in list(model.named_modules()):
        is_lin, is_c1d = isinstance(module, nn.Linear), bool(conv1d) and isinstance(module, conv1d)
        if not (is_lin or is_c1d):
            continue
        for key, config in layer_configs.items():
            if key not in name or any(skip in name for skip in skip_keys):
                continue
            i_f, o_f = (module.in_features, module.out_features) if is_lin else (module.nx, module.nf)
            common = dict(func_path=config["func"], device=module.weight.device, dtype=module.weight.dtype,
                          bias=module.bias is not None, is_compiled=config.get("compile", False))
            if method in ("blast", "blast_sym_quant"):
                new_layer = BlastLinear(i_f, o_f, config["b"], config["rank"], **common)
            elif method == "monarch":
                new_layer = MonarchLinear(i_f, o_f, config["b"], config["rank"], **common)
            elif method == "low_rank":
                new_layer = LowRankLinear(i_f, o_f, config["rank"], **common)
            elif method == "dense":
                new_layer = DenseLinear(i_f, o_f, **common)
            else:
                raise ValueError(f"unknown method {method!r}")
            parent = model
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            setattr(parent, parts[-1], new_layer)
            count += 1
            break
    return count
