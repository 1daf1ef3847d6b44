"""Packed-weight files for networks on structured linears, and the packer that makes them.

The reference keeps no weight format of its own: its replaced linears are filled with ``torch.randn`` and the rest comes
from Hugging Face checkpoints (models/wrappers.py:151-163, models/llama7b.py:63-69).  A deployment of the quantised
layers needs one, because the layer that is served (int8 / packed-int4 factors + fp16 scales, the operands of
``blr_blast_wq``) is not the layer that was trained (16-bit U, Vt, S), and a 7B-class network should reach the device
without its 16-bit factors ever being resident.

File layout (little endian)::

    0     8 bytes   magic  b"BLRPACK1"
    8     8 bytes   n = length of the header in bytes (uint64)
    16    n bytes   header, UTF-8 JSON: {"format": 1, "tensors": {name: {dtype, shape, offset, nbytes}},
                                         "layers": {prefix: {kind, bits, group, in_features, out_features, b, rank, bias}},
                                         "meta": {...}}
    ...             tensor data; every tensor starts at a multiple of 256 bytes from the start of the file (`offset`),
                    stored contiguously in the byte order of the device kernels (int4: two weights per byte, the even
                    contraction index in the low nibble)

so that a loader can map the file and hand each tensor to the device with one copy.  A layer `prefix` of kind
``blast_wq`` owns the tensors ``prefix.Uq``, ``prefix.u_scale``, ``prefix.Vq``, ``prefix.v_scale``, ``prefix.S`` (and
``prefix.bias``); kind ``blast`` owns ``prefix.U``, ``prefix.Vt``, ``prefix.S`` in the torch layout of
torch_funcs/blast_funcs.py:3-47.  Every other parameter or buffer of a packed module is stored under its state-dict name.
"""
from __future__ import annotations

import json
import mmap
import os
from typing import Dict, Optional, Tuple

import numpy as np
import torch

MAGIC = b"BLRPACK1"
ALIGN = 256
FORMAT = 1

_DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32, "int8": torch.int8,
           "uint8": torch.uint8, "int32": torch.int32, "int64": torch.int64}
_NAMES = {v: k for k, v in _DTYPES.items()}


def _round_up(n: int, a: int = ALIGN) -> int:
    return (n + a - 1) // a * a


# ------------------------------------------------------------------------------------------------ packer
def pack_blast_factors(U: torch.Tensor, Vt: torch.Tensor, S: torch.Tensor, bits: int, group: int = 0,
                       bias: Optional[torch.Tensor] = None) -> Tuple[Dict[str, torch.Tensor], dict]:
    """Torch-layout factors U (b,Q,R), Vt (b,R,P), S (b,b,R) -> (tensors of one layer, its header entry).
    bits = 16 keeps the factors; 8 | 4 quantises them with the device quantiser (``blr_quantize_sym``: the factors must
    be CUDA tensors, there is no CPU implementation)."""
    b, Q, R = U.shape
    P = Vt.shape[-1]
    assert tuple(Vt.shape) == (b, R, P) and tuple(S.shape) == (b, b, R) and bits in (16, 8, 4)
    info = {"bits": bits, "group": group, "in_features": b * P, "out_features": b * Q, "b": b, "rank": R, "bias": bias is not None}
    if bits == 16:
        out = {"U": U.contiguous(), "Vt": Vt.contiguous(), "S": S.contiguous()}
        info["kind"] = "blast"
    else:
        from . import ops
        Uq, us = ops.quantize_sym(U.contiguous(), bits, group)
        Vq, vs = ops.quantize_sym(Vt.contiguous(), bits, group)
        out = {"Uq": Uq, "u_scale": us, "Vq": Vq, "v_scale": vs, "S": S.contiguous()}
        info["kind"] = "blast_wq"
    if bias is not None:
        out["bias"] = bias.contiguous()
    return out, info


def pack_module(model: torch.nn.Module, bits: int = 0, group: int = 0) -> Tuple[Dict[str, torch.Tensor], dict]:
    """Everything a module needs to be rebuilt: its structured linears as packed layers, the rest of its state dict
    as it is.  bits = 0 keeps every layer in the form it has (16-bit layers stay 16-bit, quantised ones quantised);
    8 | 4 quantises the 16-bit BLAST layers on the way."""
    from .networks import BlastQuantLinear, BlastTorchLinear
    tensors: Dict[str, torch.Tensor] = {}
    layers: Dict[str, dict] = {}
    owned = set()
    for prefix, m in model.named_modules():
        if isinstance(m, BlastTorchLinear):
            t, info = pack_blast_factors(m.U.data, m.Vt.data, m.S.data, bits if bits else 16, group,
                                         None if m.bias is None else m.bias.data)
            owned.update(f"{prefix}.{k}" for k in ("U", "Vt", "S", "bias"))
        elif isinstance(m, BlastQuantLinear):
            t = {k: getattr(m, k) for k in ("Uq", "u_scale", "Vq", "v_scale", "S")}
            if m.bias is not None:
                t["bias"] = m.bias.data
            info = {"kind": "blast_wq", "bits": m.bits, "group": m.group, "in_features": m.in_features,
                    "out_features": m.out_features, "b": m.b, "rank": m.rank, "bias": m.bias is not None}
            owned.update(f"{prefix}.{k}" for k in ("Uq", "u_scale", "Vq", "v_scale", "S", "bias"))
        else:
            continue
        layers[prefix] = info
        tensors.update({f"{prefix}.{k}": v for k, v in t.items()})
    for name, v in model.state_dict().items():
        if name not in owned:
            tensors[name] = v
    return tensors, layers


def pack_torch_state_dict(state: Dict[str, torch.Tensor], bits: int, group: int = 0) -> Tuple[Dict[str, torch.Tensor], dict]:
    """The offline packer: a torch-layout state dict (``<prefix>.U``, ``<prefix>.Vt``, ``<prefix>.S`` [, ``<prefix>.bias``]
    per BLAST layer, anything else passed through) -> packed tensors + layer table, quantised to `bits`."""
    tensors: Dict[str, torch.Tensor] = {}
    layers: Dict[str, dict] = {}
    prefixes = sorted({k[:-2] for k in state if k.endswith(".U") and k[:-2] + ".Vt" in state and k[:-2] + ".S" in state})
    owned = set()
    for p in prefixes:
        t, info = pack_blast_factors(state[p + ".U"], state[p + ".Vt"], state[p + ".S"], bits, group, state.get(p + ".bias"))
        layers[p] = info
        tensors.update({f"{p}.{k}": v for k, v in t.items()})
        owned.update(p + s for s in (".U", ".Vt", ".S", ".bias"))
    tensors.update({k: v for k, v in state.items() if k not in owned})
    return tensors, layers


def unpack_to_torch_layout(tensors: Dict[str, torch.Tensor], layers: dict, dtype: torch.dtype = torch.float16) -> Dict[str, torch.Tensor]:
    """The inverse direction: packed layers -> a torch-layout state dict (quantised factors widened to `dtype` with
    ``blr_dequantize_sym``: q * scale rounded once, the weights the kernels multiply with)."""
    from . import ops
    out = {k: v for k, v in tensors.items()}
    for p, info in layers.items():
        if info["kind"] != "blast_wq":
            continue
        for q, s, name in (("Uq", "u_scale", "U"), ("Vq", "v_scale", "Vt")):
            out[f"{p}.{name}"] = ops.dequantize_sym(out.pop(f"{p}.{q}"), out.pop(f"{p}.{s}"), info["bits"], info["group"], dtype)
    return out


# ------------------------------------------------------------------------------------------------ file
def save_packed(path: str, tensors: Dict[str, torch.Tensor], layers: dict, meta: Optional[dict] = None) -> int:
    """Writes the file described in the module docstring; returns its size in bytes."""
    entries = {}
    for name, t in tensors.items():
        assert t.dtype in _NAMES, f"{name}: dtype {t.dtype} has no place in the format"
        entries[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "offset": 0, "nbytes": t.numel() * t.element_size()}

    def header_bytes() -> bytes:
        return json.dumps({"format": FORMAT, "tensors": entries, "layers": layers, "meta": meta or {}}, sort_keys=True).encode()

    # offsets depend on the header's length, which depends on the offsets' digits: reserve room for the widest numbers
    for e in entries.values():
        e["offset"] = 1 << 62
    start = _round_up(16 + len(header_bytes()))
    pos = start
    for e in entries.values():
        e["offset"] = pos
        pos = _round_up(pos + e["nbytes"])
    head = header_bytes()
    assert 16 + len(head) <= start
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(len(head).to_bytes(8, "little"))
        f.write(head)
        for name, t in tensors.items():
            f.seek(entries[name]["offset"])
            c = t.detach().contiguous().cpu()
            f.write(c.view(torch.uint8).numpy().tobytes() if c.numel() else b"")
        f.truncate(pos)
    return pos


def read_header(path: str) -> dict:
    with open(path, "rb") as f:
        assert f.read(8) == MAGIC, f"{path} is not a packed-weight file"
        n = int.from_bytes(f.read(8), "little")
        head = json.loads(f.read(n).decode())
    assert head.get("format") == FORMAT, f"unknown format {head.get('format')}"
    return head


def load_packed(path: str, device="cpu") -> Tuple[Dict[str, torch.Tensor], dict, dict]:
    """Maps the file and returns (tensors on `device`, layer table, meta).  Each tensor reaches the device with one copy
    from the mapping; on the CPU the tensors are private copies (the mapping is closed on return)."""
    head = read_header(path)
    size = os.path.getsize(path)
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as f, mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY) as mm:
        for name, e in head["tensors"].items():
            assert e["offset"] % ALIGN == 0 and e["offset"] + e["nbytes"] <= size, f"{name}: entry outside the file"
            dt = _DTYPES[e["dtype"]]
            if e["nbytes"] == 0:
                out[name] = torch.empty(e["shape"], dtype=dt, device=device)
                continue
            # (a private copy-on-write mapping: nothing is written, the buffer only has to be writable for numpy -> torch)
            raw = np.frombuffer(mm, dtype=np.uint8, count=e["nbytes"], offset=e["offset"])
            t = torch.from_numpy(raw)
            out[name] = (t.clone() if torch.device(device).type == "cpu" else t.to(device)).view(dt).reshape(e["shape"])
            del raw, t
    return out, head["layers"], head["meta"]


def load_packed_into(model: torch.nn.Module, path: str) -> dict:
    """Fills a module built with the same structure (networks.empty_init() builds one without random numbers and without
    16-bit factors) from a packed-weight file: structured layers take their packed tensors, which must match in kind,
    shape and bit width; everything else goes through load_state_dict.  Returns the file's meta."""
    from .networks import BlastQuantLinear, BlastTorchLinear
    dev = next(iter(model.state_dict().values())).device
    tensors, layers, meta = load_packed(path, dev)
    mods = dict(model.named_modules())
    owned = set()
    for prefix, info in layers.items():
        m = mods.get(prefix)
        want = BlastQuantLinear if info["kind"] == "blast_wq" else BlastTorchLinear
        assert isinstance(m, want), f"{prefix}: the file holds a {info['kind']} layer, the module is {type(m).__name__}"
        assert (m.in_features, m.out_features, m.b, m.rank) == (info["in_features"], info["out_features"], info["b"], info["rank"]), \
            f"{prefix}: shape mismatch"
        if info["kind"] == "blast_wq":
            assert (m.bits, m.group) == (info["bits"], info["group"]), f"{prefix}: bit width or scale group mismatch"
        names = ("Uq", "u_scale", "Vq", "v_scale", "S") if info["kind"] == "blast_wq" else ("U", "Vt", "S")
        for k in names + (("bias",) if info["bias"] else ()):
            dst = getattr(m, k)
            src = tensors[f"{prefix}.{k}"]
            assert dst.shape == src.shape and dst.dtype == src.dtype, f"{prefix}.{k}: {tuple(src.shape)} {src.dtype} does not fit"
            dst.data.copy_(src)
            owned.add(f"{prefix}.{k}")
    rest = {k: v for k, v in tensors.items() if k not in owned}
    missing = [k for k in model.state_dict() if k not in owned and k not in rest]
    assert not missing, f"the file lacks {missing[:4]}"
    model.load_state_dict(rest, strict=False)
    return meta
