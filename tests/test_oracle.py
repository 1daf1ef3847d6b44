"""Pins the CPU oracle against golden vectors produced by the reference's own torch functions."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import blr_oracle as orc

TOL = 2e-6  # fp32 einsum vs fp32 bmm: differences are summation order only


def _load(path):
    return {k: torch.from_numpy(v) for k, v in np.load(path).items()}


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_blast_matches_reference_golden(golden_dir, tag):
    g = _load(os.path.join(golden_dir, f"blast_{tag}.npz"))
    out, z, y = orc.blast(g["x"], g["U"], g["Vt"], g["S"])
    assert out.shape == g["out"].shape
    assert orc.rel_fro(out, g["out"]) < TOL
    assert orc.rel_fro(z, g["z"]) < TOL
    assert orc.rel_fro(y, g["y"]) < TOL
    out_b, z_b, y_b = orc.blast_bmm(g["x"], g["U"], g["Vt"], g["S"].permute(2, 0, 1).contiguous())
    assert z_b.shape == g["z_bmm"].shape
    assert orc.rel_fro(out_b, g["out_bmm"]) < TOL
    assert orc.rel_fro(z_b, g["z_bmm"]) < TOL
    assert orc.rel_fro(y_b, g["y_bmm"]) < TOL


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_monarch_matches_reference_golden(golden_dir, tag):
    g = _load(os.path.join(golden_dir, f"monarch_{tag}.npz"))
    out2, pre2, out1, pre1 = orc.monarch(g["x"], g["w1_t"], g["w2_t"])
    for got, key in ((out2, "out2"), (pre2, "pre_out2"), (out1, "out1"), (pre1, "pre_out1")):
        assert got.shape == g[key].shape, key
        assert orc.rel_fro(got, g[key]) < TOL, key


def test_low_rank_and_dense_match_reference_golden(golden_dir):
    g = _load(os.path.join(golden_dir, "low_rank_a.npz"))
    out, _ = orc.low_rank(g["x"], g["Vt"], g["Ut"])
    assert orc.rel_fro(out, g["out"]) < TOL
    g = _load(os.path.join(golden_dir, "dense_a.npz"))
    assert orc.rel_fro(orc.dense(g["x"], g["Wt"]), g["out"]) < TOL


def test_all_golden_files_are_covered(golden_dir):
    names = sorted(os.path.basename(p) for p in glob.glob(os.path.join(golden_dir, "*.npz")))
    assert names == ["blast_a.npz", "blast_b.npz", "blast_c.npz", "dense_a.npz", "low_rank_a.npz",
                     "monarch_a.npz", "monarch_b.npz", "monarch_c.npz"]


def test_monarch_kernel_layout_is_a_column_regrouping():
    b, rank, P = 4, 8, 3
    w1_t = torch.arange(b * rank * P, dtype=torch.float32).reshape(b, rank, P)
    w = orc.monarch_w1_to_kernel_layout(w1_t)
    per = rank // b
    for l in range(b):
        for jj in range(per):
            assert torch.equal(w[:, :, l * per + jj], w1_t[:, jj * b + l, :])


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("group", [0, 16])
def test_quantiser_roundtrip_and_bounds(bits, group):
    g = torch.Generator().manual_seed(5)
    w = torch.randn(3, 7, 64, generator=g)
    w[1, 2] = 0.0  # an all-zero channel must not divide by zero
    q, s = orc.quantize_sym(w, bits, group)
    qmax = 127 if bits == 8 else 7
    qi = orc.unpack_int4(q) if bits == 4 else q
    assert qi.dtype == torch.int8 and int(qi.abs().max()) <= qmax
    assert s.dtype == torch.float16
    if bits == 4:
        assert q.dtype == torch.uint8 and q.shape[-1] == 32
        assert torch.equal(orc.pack_int4(qi), q)  # pack -> unpack -> pack is bit exact
    wd = orc.dequantize_sym(q, s, bits, group)
    # symmetric rounding error is at most half a step (plus the fp16 rounding of the scale)
    step = s.float().unsqueeze(-1) if group == 0 else s.float().repeat_interleave(group, dim=-1)
    step = step if group else step.expand_as(w)
    assert torch.all((wd - w).abs() <= 0.51 * step.reshape(w.shape) + 1e-6)
    assert torch.all(wd[1, 2] == 0)


def test_act_int8_intermediates_are_integers():
    x, U, Vt, S = orc.make_blast_inputs(4, 64, 96, 4, 16, torch.bfloat16, seed=3)
    out, z8, y8 = orc.blast_act_int8(x, U, Vt, S)
    assert z8.dtype == torch.int8 and y8.dtype == torch.int8 and out.shape == (1, 4, 96)
