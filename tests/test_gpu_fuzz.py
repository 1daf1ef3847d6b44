"""Seeded random shapes against the oracle: decode sizes (cluster and grid-wide kernels) and a few prefill sizes.

The hand-picked shapes of the other GPU tests follow the reference's configurations; these cover what lies between
them: odd block counts, ranks that are not multiples of a K-chunk, ragged last slices and row groups.
"""
import random

import pytest
import torch

from oracle import blr_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-2


def _cases(seed, count, n_choices, quantised):
    rng = random.Random(seed)
    out = []
    while len(out) < count:
        b = rng.choice([2, 3, 4, 6, 8, 9, 12, 16])
        step = 32 if quantised else 8      # int4 rows need 32 elements per 16 bytes
        P = rng.randrange(step, 320 + 1, step)
        Q = rng.randrange(8, 320 + 1, 8)
        R = rng.randrange(step, 640 + 1, step)
        N = rng.choice(n_choices)
        out.append((N, b * P, b * Q, b, R))
    return out


@pytest.mark.parametrize("case", _cases(1, 24, [1, 2, 3, 5, 8, 9, 13, 16], False))
def test_blast_random_decode_shapes(case):
    import mem_efficient_blr_b200.blast_kernels as bk
    from mem_efficient_blr_b200 import _lib
    N, I, O, b, R = case
    dtype = torch.float16 if (I + O + R) % 16 == 0 else torch.bfloat16
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, dtype, seed=I + O + R + N)
    ref, _, _ = orc.blast(x, U, Vt, S)
    got = bk.blast_torch_layout(x.to(DEV), U.to(DEV), Vt.to(DEV), S.to(DEV))
    torch.cuda.synchronize()
    _lib.workspace_status(torch.device(DEV))
    assert orc.rel_fro(got.float().cpu(), ref) < TOL, case
    Up, Vp, Sp = orc.blast_to_partial_layout(U, Vt, S)
    got = bk.triton_blast_partial_grouped_fp16(x.to(DEV), Up.to(DEV), Vp.to(DEV), Sp.to(DEV))
    torch.cuda.synchronize()
    assert orc.rel_fro(got.float().cpu(), ref) < TOL, case


@pytest.mark.parametrize("case", _cases(2, 16, [1, 4, 7, 8, 12, 16], True))
def test_blast_wq_random_decode_shapes(case):
    import mem_efficient_blr_b200.blast_sym_quant_kernels as bq
    from mem_efficient_blr_b200 import _lib
    N, I, O, b, R = case
    bits = 8 if (I // b) % 64 else 4
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=I + O + R + N)
    Uq, us = orc.quantize_sym(U, bits)
    Vq, vs = orc.quantize_sym(Vt, bits)
    ref, _, _ = orc.blast_wq(x, Uq, us, Vq, vs, S, bits)
    got = bq.blast_wq(x.to(DEV), Uq.to(DEV), us.to(DEV), Vq.to(DEV), vs.to(DEV), S.to(DEV), bits)
    torch.cuda.synchronize()
    _lib.workspace_status(torch.device(DEV))
    assert orc.rel_fro(got.float().cpu(), ref) < TOL, (case, bits)


@pytest.mark.parametrize("case", _cases(3, 8, [17, 40, 64, 65, 130, 300], False))
def test_blast_random_prefill_shapes(case):
    import mem_efficient_blr_b200.blast_kernels as bk
    N, I, O, b, R = case
    x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.bfloat16, seed=I + O + R + N)
    ref, _, _ = orc.blast(x, U, Vt, S)
    got = bk.blast_torch_layout(x.to(DEV), U.to(DEV), Vt.to(DEV), S.to(DEV))
    torch.cuda.synchronize()
    assert orc.rel_fro(got.float().cpu(), ref) < TOL, case


@pytest.mark.parametrize("case", _cases(4, 10, [1, 3, 8, 11, 16, 33, 200], False))
def test_low_rank_and_monarch_random_shapes(case):
    import mem_efficient_blr_b200.low_rank_kernels as lk
    import mem_efficient_blr_b200.monarch_kernels as mk
    N, I, O, b, R = case
    x, Vt, Ut = orc.make_low_rank_inputs(N, I, O, R, torch.float16, seed=I + O + N)
    ref, _ = orc.low_rank(x, Vt, Ut)
    got = lk.low_rank_torch_layout(x.to(DEV), Vt.to(DEV), Ut.to(DEV))
    torch.cuda.synchronize()
    assert orc.rel_fro(got.float().cpu(), ref) < TOL, case
    rank = (R + b * 8 - 1) // (b * 8) * (b * 8)  # Monarch needs rank % b == 0, and rank / b rows of 16 bytes
    x, w1_t, w2_t = orc.make_monarch_inputs(N, I, O, b, rank, torch.float16, seed=I + O + N)
    ref = orc.monarch(x, w1_t, w2_t)[0]
    got = mk.monarch_torch_layout(x.to(DEV), w1_t.to(DEV), w2_t.to(DEV))
    torch.cuda.synchronize()
    assert orc.rel_fro(got.float().cpu(), ref) < TOL, (case, rank)


@pytest.mark.parametrize("seed", range(6))
def test_grouped_scales_and_block_slices_random(seed):
    import mem_efficient_blr_b200.blast_kernels as bk
    import mem_efficient_blr_b200.blast_sym_quant_kernels as bq
    rng = random.Random(100 + seed)
    b = rng.choice([2, 4, 8, 16])
    P, R = 128 * rng.randrange(1, 3), 128 * rng.randrange(1, 5)
    Q = rng.randrange(8, 200, 8)
    N = rng.choice([1, 6, 8, 10, 16])
    bits = rng.choice([8, 4])
    x, U, Vt, S = orc.make_blast_inputs(N, b * P, b * Q, b, R, torch.float16, seed=seed)
    Uq, us = orc.quantize_sym(U, bits, 128)
    Vq, vs = orc.quantize_sym(Vt, bits, 128)
    ref, _, _ = orc.blast_wq(x, Uq, us, Vq, vs, S, bits, 128)
    got = bq.blast_wq(x.to(DEV), Uq.to(DEV), us.to(DEV), Vq.to(DEV), vs.to(DEV), S.to(DEV), bits, 128)
    torch.cuda.synchronize()
    assert orc.rel_fro(got.float().cpu(), ref) < TOL, (N, b, P, Q, R, bits)
    # a slice of the output blocks (what one rank of a block-sharded layer computes)
    lo = rng.randrange(0, b)
    hi = rng.randrange(lo + 1, b + 1)
    full, _, _ = orc.blast(x, U, Vt, S)
    got = bk.blast_output_blocks(x.to(DEV), U[lo:hi].contiguous().to(DEV), Vt.to(DEV), S[lo:hi].contiguous().to(DEV))
    torch.cuda.synchronize()
    assert orc.rel_fro(got.float().cpu(), full[..., lo * Q:hi * Q]) < TOL, (N, b, lo, hi)
