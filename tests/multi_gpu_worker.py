"""Worker of tests/test_gpu_multi.py: one process per GPU under torchrun (NCCL).

Checks, on real GPUs, the two ways the path shards: BLAST by output block with one all_gather along the feature
axis (this package's kernels on a slice of the blocks), and token-batch data parallelism with a gathered result.
Every rank compares what it assembled with the CPU oracle on the same seeded inputs and prints one line.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import blr_oracle as orc  # noqa: E402

TOL = 1e-2


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import mem_efficient_blr_b200.blast_kernels as bk
    from mem_efficient_blr_b200 import _lib
    from mem_efficient_blr_b200 import dist as bd

    worst = 0.0
    for N, I, O, b, R in [(1, 4096, 11008, 16, 1024), (16, 4096, 11008, 16, 1024), (130, 1024, 1536, 8, 256)]:
        x, U, Vt, S = orc.make_blast_inputs(N, I, O, b, R, torch.float16, seed=7 + N)  # same on every rank
        ref, _, _ = orc.blast(x, U, Vt, S)
        xd, Ud, Vd, Sd = x.to(dev), U.to(dev), Vt.to(dev), S.to(dev)
        # (1) output-block sharding: this rank's U_i, S_i; all of V; gather along features
        Ul, Sl = bd.shard_blast_factors(Ud, Sd, rank, world)
        got = bd.blast_row_block_parallel(xd, Ul.contiguous(), Vd, Sl.contiguous(), bk.blast_output_blocks)
        torch.cuda.synchronize()
        _lib.workspace_status(dev)
        e1 = orc.rel_fro(got.float().cpu(), ref)
        # (2) token slices, gathered
        got2 = bd.data_parallel_apply(xd, lambda xs: bk.blast_torch_layout(xs, Ud, Vd, Sd), gather=True)
        torch.cuda.synchronize()
        _lib.workspace_status(dev)
        e2 = orc.rel_fro(got2.float().cpu(), ref.reshape(-1, ref.shape[-1]))
        worst = max(worst, e1, e2)
        assert got.shape == ref.shape and e1 < TOL, f"rank {rank}: block sharding N={N}: {e1}"
        assert e2 < TOL, f"rank {rank}: token sharding N={N}: {e2}"
    print(f"MULTI_GPU_OK rank {rank}/{world} worst_rel_fro {worst:.2e}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
