"""Generate golden vectors by running the reference's own PyTorch functions on seeded inputs.

Run in a container where the reference checkout is mounted:
    python tests/golden/make_golden.py /path/to/reference
It imports ``torch_funcs.*`` from that checkout (unmodified), evaluates them in fp32 on CPU and
writes inputs + outputs to ``tests/golden/*.npz``.  The fixtures are small (a few hundred KB)
and committed; nothing at test time reads the reference checkout.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from torch_funcs.blast_funcs import torch_blast_baseline, torch_blast_bmm
    from torch_funcs.monarch_funcs import torch_monarch_baseline
    from torch_funcs.low_rank_funcs import torch_low_rank_baseline
    from torch_funcs.dense_funcs import torch_dense_baseline

    def save(name, **arrs):
        np.savez_compressed(os.path.join(HERE, name), **{k: v.numpy() for k, v in arrs.items()})
        print("wrote", name, {k: tuple(v.shape) for k, v in arrs.items()})

    # BLAST: (b, P, Q, R, lead) including b=3 (the reference's ViT setting), ragged Q, N=1
    for tag, (b, P, Q, R, lead) in {
        "a": (4, 16, 24, 32, (2, 5)),
        "b": (3, 8, 16, 8, (1, 1)),
        "c": (16, 8, 43, 16, (1, 17)),
    }.items():
        g = torch.Generator().manual_seed(100 + ord(tag))
        x = torch.randn(*lead, b * P, generator=g)
        U = torch.randn(b, Q, R, generator=g)
        Vt = torch.randn(b, R, P, generator=g)
        S = torch.randn(b, b, R, generator=g)
        out, z, y = torch_blast_baseline(x, U, Vt, S)
        out_b, z_b, y_b = torch_blast_bmm(x, U, Vt, S.permute(2, 0, 1).contiguous())
        save(f"blast_{tag}.npz", x=x, U=U, Vt=Vt, S=S, out=out, z=z, y=y,
             out_bmm=out_b, z_bmm=z_b.contiguous(), y_bmm=y_b)

    # Monarch: (k=l=b, rank, P, Sdim, lead) and one rectangular case k != l
    for tag, (k, l, q, p, s, lead) in {
        "a": (4, 4, 8, 6, 5, (2, 3)),
        "b": (16, 16, 32, 4, 3, (1, 7)),
        "c": (2, 4, 8, 5, 3, (1, 4)),     # l*r == k*q with r = 4
    }.items():
        g = torch.Generator().manual_seed(200 + ord(tag))
        r = k * q // l
        x = torch.randn(*lead, k * p, generator=g)
        w1 = torch.randn(k, q, p, generator=g)
        w2 = torch.randn(l, s, r, generator=g)
        out2, pre2, out1, pre1 = torch_monarch_baseline(x, w1, w2)
        save(f"monarch_{tag}.npz", x=x, w1_t=w1, w2_t=w2, out2=out2, pre_out2=pre2,
             out1=out1.contiguous(), pre_out1=pre1)

    g = torch.Generator().manual_seed(300)
    x = torch.randn(2, 3, 40, generator=g)
    Vt = torch.randn(12, 40, generator=g)
    Ut = torch.randn(28, 12, generator=g)
    save("low_rank_a.npz", x=x, Vt=Vt, Ut=Ut, out=torch_low_rank_baseline(x, Vt, Ut))
    Wt = torch.randn(28, 40, generator=g)
    save("dense_a.npz", x=x, Wt=Wt, out=torch_dense_baseline(x, Wt))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
