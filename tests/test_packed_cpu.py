"""The packed-weight file format on the CPU: layout, alignment, round trip (no device arithmetic involved)."""
import json
import os

import pytest
import torch

from mem_efficient_blr_b200 import packed


def _tensors():
    g = torch.Generator().manual_seed(3)
    return {
        "layers.0.q.Uq": torch.randint(-127, 128, (4, 48, 64), generator=g, dtype=torch.int8),
        "layers.0.q.u_scale": torch.rand(4, 48, generator=g).half(),
        "layers.0.q.Vq": torch.randint(0, 256, (4, 64, 16), generator=g, dtype=torch.int32).to(torch.uint8),
        "layers.0.q.v_scale": torch.rand(4, 64, 1, generator=g).half(),
        "layers.0.q.S": torch.rand(4, 4, 64, generator=g).bfloat16(),
        "norm.weight": torch.ones(7, dtype=torch.float32),
        "odd": torch.arange(13, dtype=torch.int64),
        "nothing": torch.empty(0, 5, dtype=torch.float16),
    }


def test_file_layout_and_round_trip(tmp_path):
    t = _tensors()
    layers = {"layers.0.q": {"kind": "blast_wq", "bits": 8, "group": 0, "in_features": 128, "out_features": 192, "b": 4,
                             "rank": 64, "bias": False}}
    path = os.path.join(tmp_path, "w.blrpack")
    size = packed.save_packed(path, t, layers, {"note": "unit test"})
    assert size == os.path.getsize(path) and size % packed.ALIGN == 0
    raw = open(path, "rb").read()
    assert raw[:8] == b"BLRPACK1"
    n = int.from_bytes(raw[8:16], "little")
    head = json.loads(raw[16:16 + n])
    assert head["format"] == 1 and head["layers"] == layers and head["meta"] == {"note": "unit test"}
    spans = sorted((e["offset"], e["offset"] + e["nbytes"]) for e in head["tensors"].values())
    assert spans[0][0] >= 16 + n
    for (a0, a1), (b0, _) in zip(spans, spans[1:]):
        assert a0 % packed.ALIGN == 0 and a1 <= b0          # aligned, no overlap
    # the bytes of a tensor are its contiguous storage
    e = head["tensors"]["odd"]
    assert raw[e["offset"]:e["offset"] + e["nbytes"]] == t["odd"].numpy().tobytes()
    got, layers2, meta = packed.load_packed(path)
    assert layers2 == layers and meta == {"note": "unit test"} and set(got) == set(t)
    for k in t:
        assert got[k].dtype == t[k].dtype and got[k].shape == t[k].shape and torch.equal(got[k], t[k]), k
    assert packed.read_header(path)["tensors"].keys() == head["tensors"].keys()


def test_rejects_foreign_and_truncated_files(tmp_path):
    bad = os.path.join(tmp_path, "bad")
    open(bad, "wb").write(b"not a packed file at all")
    with pytest.raises(AssertionError, match="not a packed-weight file"):
        packed.load_packed(bad)
    path = os.path.join(tmp_path, "w.blrpack")
    packed.save_packed(path, _tensors(), {})
    cut = os.path.join(tmp_path, "cut")
    open(cut, "wb").write(open(path, "rb").read()[:-300])
    with pytest.raises(AssertionError, match="outside the file"):
        packed.load_packed(cut)


def test_bits16_packing_keeps_the_torch_layout():
    g = torch.Generator().manual_seed(1)
    U, Vt, S = torch.randn(4, 6, 8, generator=g).half(), torch.randn(4, 8, 5, generator=g).half(), torch.rand(4, 4, 8, generator=g).half()
    state = {"mlp.up.U": U, "mlp.up.Vt": Vt, "mlp.up.S": S, "mlp.up.bias": torch.zeros(24).half(), "norm.weight": torch.ones(3)}
    tensors, layers = packed.pack_torch_state_dict(state, 16)
    assert layers == {"mlp.up": {"kind": "blast", "bits": 16, "group": 0, "in_features": 20, "out_features": 24, "b": 4, "rank": 8,
                                 "bias": True}}
    assert set(tensors) == set(state) and all(torch.equal(tensors[k], state[k]) for k in state)
    assert all(torch.equal(v, state[k]) for k, v in packed.unpack_to_torch_layout(tensors, layers).items())
