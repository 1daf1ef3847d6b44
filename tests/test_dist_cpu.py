"""World-size-2 gloo tests (CPU) of the multi-GPU host logic: token slicing and BLAST output-block sharding.
The compute function is the oracle here; on GPUs it is the CUDA operator (tests/test_gpu_modules.py)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import blr_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mem_efficient_blr_b200 import dist as bd
        x, U, Vt, S = orc.make_blast_inputs(5, 64, 96, 4, 16, torch.float32, seed=3)
        ref, _, _ = orc.blast(x, U, Vt, S)

        # --- output-block sharding: every rank must end up with the full row
        Ul, Sl = bd.shard_blast_factors(U, S, rank, world)

        def compute(xx, Uloc, Vt_, Sloc):
            y = torch.einsum("njp,jrp->jnr", xx.reshape(-1, 4, 16), Vt_)
            z = torch.einsum("ijr,jnr->inr", Sloc, y)
            return torch.einsum("inr,iqr->niq", z, Uloc).reshape(*xx.shape[:-1], -1)

        out = bd.blast_row_block_parallel(x, Ul, Vt, Sl, compute)
        ok1 = out.shape == ref.shape and orc.rel_fro(out, ref) < 1e-6

        # --- token data parallelism with a ragged split (5 tokens over 2 ranks) and gather
        full = bd.data_parallel_apply(x, lambda t: orc.blast(t, U, Vt, S)[0], gather=True)
        ok2 = full.shape == (5, 96) and orc.rel_fro(full, ref.reshape(5, 96)) < 1e-6
        lo, hi = bd.token_slice(5, rank, world)
        ok3 = (hi - lo) == (3 if rank == 0 else 2)

        # --- fewer tokens than ranks: one rank's slice is empty, the gathered result is still complete
        x1 = x.reshape(5, 64)[:1]
        one = bd.data_parallel_apply(x1, lambda t: orc.blast(t, U, Vt, S)[0] if t.shape[0] else t.new_empty((0, 96)), gather=True)
        ok3 = ok3 and one.shape == (1, 96) and orc.rel_fro(one, ref.reshape(5, 96)[:1]) < 1e-6
        q.put((rank, ok1, ok2, ok3))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_and_gather():
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    for r in results:
        assert r[1] and r[2] and r[3], r


def test_slices_are_balanced_and_exhaustive():
    from mem_efficient_blr_b200 import dist as bd
    for n in (1, 5, 16, 197, 2048):
        for w in (1, 2, 4, 8):
            spans = [bd.token_slice(n, r, w) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b_[0] for a, b_ in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    assert bd.block_slice(16, 3, 8) == (6, 8)
    with pytest.raises(ValueError):
        bd.block_slice(3, 0, 2)


def test_roofline_model_matches_the_headline_table():
    from mem_efficient_blr_b200 import roofline as rf
    from mem_efficient_blr_b200.device import Device
    nbytes, flops = rf.triton_blast_full_mem_flops(1, 4096, 1024, 11008, 16, 16, 2)
    assert abs(nbytes - 31.49e6) < 0.02e6 and flops == 2 * 1024 * (4096 + 11008 + 256)
    nbytes, flops = rf.triton_blast_full_mem_flops(2048, 4096, 1024, 11008, 16, 16, 2)
    assert abs(nbytes - 93.32e6) < 0.05e6 and abs(flops - 64.42e9) < 0.02e9
    nbytes, _ = rf.blast_wq_mem_flops(1, 4096, 1024, 11008, 16, 8)
    assert abs(nbytes - (16.02e6 + 55e3)) < 0.03e6
    d = Device("B200")
    assert d.break_point > 100
    t = rf.roofline_time_us(*rf.triton_blast_full_mem_flops(2048, 4096, 1024, 11008, 16, 16, 2), d)
    assert t["bound"] == "tensor"
    assert Device("A40").peak_performance == 149.7e12
    with pytest.raises(ValueError):
        Device("nope")
