"""Multi-GPU helpers: token-batch data parallelism and BLAST output-block sharding.

The path shards two ways (neither exists in the reference, which runs on one GPU, layer.py:186):
  * by tokens: rows of x are independent, factors are replicated, no collective in the forward pass;
  * by BLAST output block i: rank g owns U[i], S[i, :, :] for its blocks, streams all of V (the first stage is
    replicated: at decode sizes that costs less than exchanging y), produces out[:, i*Q:(i+1)*Q] for its blocks,
    and one all_gather along the feature axis assembles the row.
The compute function is injected, so the partition / gather logic is testable on CPU ranks (gloo).
"""
from __future__ import annotations

from typing import Callable, Tuple

import torch
import torch.distributed as dist


def token_slice(n_tokens: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, balanced slice [lo, hi) of the tokens for `rank`."""
    base, rem = divmod(n_tokens, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def block_slice(b: int, rank: int, world: int) -> Tuple[int, int]:
    """Output blocks [lo, hi) owned by `rank`; the block count must divide evenly."""
    if b % world != 0:
        raise ValueError(f"{b} output blocks do not divide over {world} ranks")
    per = b // world
    return rank * per, (rank + 1) * per


def shard_blast_factors(U: torch.Tensor, S: torch.Tensor, rank: int, world: int):
    """torch-layout U (b,Q,R), S (b_out,b_in,R) -> this rank's (U[lo:hi], S[lo:hi]) (views, no copy)."""
    lo, hi = block_slice(U.shape[0], rank, world)
    return U[lo:hi], S[lo:hi]


def blast_row_block_parallel(x: torch.Tensor, U_local: torch.Tensor, Vt: torch.Tensor, S_local: torch.Tensor,
                             compute: Callable, group=None) -> torch.Tensor:
    """out (..., b*Q) from a rank-local slice of the output blocks.

    `compute(x, U_local, Vt, S_local)` must return this rank's (..., b_local*Q) columns; on GPUs it is an operator
    of this package that accepts b_out != b_in, on CPU ranks a reference function.  The slices are gathered with
    one all_gather (NCCL over NVLink on GPUs) and concatenated along the feature axis."""
    world = dist.get_world_size(group)
    local = compute(x, U_local, Vt, S_local).contiguous()
    if world == 1:
        return local
    # one collective into a (world, N, width) buffer; rank g's columns are out[:, g*width:(g+1)*width]
    lead, width = local.shape[:-1], local.shape[-1]
    flat = local.reshape(-1, width)
    gathered = torch.empty((world, flat.shape[0], width), dtype=local.dtype, device=local.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(gathered, flat, group=group)
    else:  # gloo (CPU ranks in the tests) gathers into a list of views of the same buffer
        dist.all_gather(list(gathered.unbind(0)), flat, group=group)
    if flat.shape[0] == 1:   # one token: the gathered buffer already is the row
        return gathered.reshape(*lead, world * width)
    return gathered.permute(1, 0, 2).reshape(*lead, world * width)


def data_parallel_apply(x: torch.Tensor, fn: Callable, group=None, gather: bool = False) -> torch.Tensor:
    """Applies fn to this rank's token slice of x (..., I) flattened over the leading dims.  With gather=True
    every rank receives the full (N, O) result (ragged slices are padded for the all_gather)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    x2 = x.reshape(-1, x.shape[-1])
    lo, hi = token_slice(x2.shape[0], rank, world)
    out = fn(x2[lo:hi])
    if not gather or world == 1:
        return out
    width = out.shape[-1]
    most = -(-x2.shape[0] // world)
    pad = torch.zeros((most, width), dtype=out.dtype, device=out.device)
    pad[: hi - lo] = out
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    rows = []
    for r in range(world):
        a, b_ = token_slice(x2.shape[0], r, world)
        rows.append(parts[r][: b_ - a])
    return torch.cat(rows, dim=0)
