#!/usr/bin/env python
"""Benchmark of the structured-matmul hot path on B200.

Headline workload (the configuration the metric is quoted on): symmetric-quantised BLAST decode on the
Llama-7B gate_proj shape, 4096 -> 11008, b = 16, R = 1024, int8 and packed-int4 factors with fp16
per-channel scales, token counts 1, 4 and 16.  One *pass* runs every (bits, N) point once over a
rotating set of weight replicas whose total footprint exceeds the L2 cache, so every launch streams
its weights from HBM; one *step* is PASSES_PER_STEP passes (so that the timed region lasts about a second
and the clock sampler sees it).  The metric is algorithmic bytes per second (weights + scales + S + x + out
of every launch, divided by device time), summed over ranks.

Beside the headline the same JSON line carries, in top-level keys: the per-point times with the dense fp16
cuBLAS bar (`sweep`), the layer sweep over all Llama-7B projections and operator families (`layer_sweep`), a
Llama-7B-shaped decoder with BLAST linears - prefill at 2048 tokens and decode at batch 1/4/16/64 against a
2048-token cache, 16-bit and int8 factors - a ViT-B/16-shaped encoder and a DiT-XL/2-shaped denoiser (`llama7b_blast`,
`vit_b16_blast`, `dit_xl2_blast`),
and, on more than one GPU, BLAST sharded by output block with an all-gather (`row_block_sharding`).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--quick]

With N > 1 launch under torchrun; every rank runs the same workload on its own GPU (independent
token batches, replicated weights: weak scaling, no collective in the data path of the headline).
`--impl reference` times the reference's own torch path (torch_funcs/blast_funcs.py, copied unmodified under
oracle/_ref/ by oracle/make_ref.py; the oracle's restatement if that copy is absent) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

I_F, O_F, B_BLK, RANK = 4096, 11008, 16, 1024
P_BLK, Q_BLK = I_F // B_BLK, O_F // B_BLK
POINTS = [(8, 1), (8, 4), (8, 16), (4, 1), (4, 4), (4, 16)]  # (bits, tokens)
L2_BYTES = 126 * 2 ** 20
PASSES_PER_STEP = 25
# Which kernels serve a point of the headline workload (the library's dispatch for this layer): up to 4 tokens the
# two-launch path (two kernels per call), above it the cluster kernel (one).
GROUPS = {"two_launch": ("blr_blast_front_kernel+blr_blast_back_kernel (+blr_blast_fx_kernel above 2 tokens)", 2),
          "cluster": ("blr_blast_cluster_kernel", 1)}


def launches_of(bits: int, n: int) -> int:
    """Kernel launches of one call of a point: front + back, and above 2 tokens the conversion of x ahead of them
    (blr_blast_fx_kernel)."""
    return 3 if n > 2 else 2


def group_of(bits: int, n: int) -> str:
    """Kernel group the library's dispatch picks for a point: every point of the workload takes the two-launch path."""
    return "two_launch"


def algorithmic_bytes(bits: int, n: int) -> float:
    """bytes = wb*R*(I+O) + 2*b^2*R + 2*N*(I+O) + scale bytes, wb = bits/8."""
    return bits / 8 * RANK * (I_F + O_F) + 2 * B_BLK * B_BLK * RANK + 2 * n * (I_F + O_F) + 2 * (B_BLK * Q_BLK + B_BLK * RANK)


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def ncu_traffic(group: str):
    """dram read + write bytes of one call of the group from the ncu capture summarised under profiles/ (None if absent)."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            d = json.load(f)[group]
        return float(d["bytes_per_call"]), d["note"]
    except Exception:
        return None, "no capture on file"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


def workload_config():
    return {"workload": "symmetric-quantised BLAST decode, Llama-7B gate_proj 4096->11008, b=16, R=1024, "
                        "int8 and packed-int4 factors with fp16 per-channel scales, tokens 1/4/16 (one launch per point per replica)",
            "in_features": I_F, "out_features": O_F, "blocks": B_BLK, "rank": RANK,
            "points": [f"int{b}/N={n}" for b, n in POINTS],
            "passes_per_step": PASSES_PER_STEP,
            "l2_policy": "weights rotate over replicas whose footprint exceeds L2 (inputs larger than L2)"}


# ------------------------------------------------------------------------------------------ reference arm (CPU)
def cpu_blast_function():
    """The reference's torch_blast_baseline from the unmodified copy under oracle/_ref/ ("reference"), else the oracle's
    restatement of it ("port")."""
    from oracle import make_ref
    if make_ref.available():
        sys.path.insert(0, make_ref.import_path())
        try:
            from torch_funcs.blast_funcs import torch_blast_baseline
            return torch_blast_baseline, "reference"
        finally:
            sys.path.pop(0)
    from oracle import blr_oracle as orc
    return orc.blast, "port"


class CpuWorkload:
    """The headline points on dequantised fp32 factors for the CPU function (the reference has no weight-quantised path)."""

    def __init__(self, threads: int):
        from oracle import blr_oracle as orc
        torch.set_num_threads(threads)
        self.fn, self.kind = cpu_blast_function()
        x16, U, Vt, S = orc.make_blast_inputs(16, I_F, O_F, B_BLK, RANK, torch.float16, seed=0)
        self.S = S.float()
        self.x = {n: x16[:, :n].float() for n in (1, 4, 16)}
        self.f = {}
        for bits in (8, 4):
            Uq, us = orc.quantize_sym(U, bits)
            Vq, vs = orc.quantize_sym(Vt, bits)
            self.f[bits] = (orc.dequantize_sym(Uq, us, bits), orc.dequantize_sym(Vq, vs, bits))

    def step(self):
        """One call per (bits, tokens) point; returns seconds per point."""
        t = {}
        for bits, n in POINTS:
            Ud, Vd = self.f[bits]
            t0 = time.perf_counter()
            self.fn(self.x[n], Ud, Vd, self.S)
            t[(bits, n)] = time.perf_counter() - t0
        return t


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    t0 = time.perf_counter()
    wl = CpuWorkload(threads)
    for _ in range(args.warmup):
        wl.step()
    steps = [wl.step() for _ in range(args.steps)]
    per_point = {p: statistics.median(s[p] for s in steps) for p in POINTS}
    step_s = sum(sum(s.values()) for s in steps) / len(steps)
    total_bytes = sum(algorithmic_bytes(b, n) for b, n in POINTS)
    value = total_bytes / step_s / 1e9
    line = {
        "impl": "reference", "metric": "blast_wq_decode_algorithmic_GBps", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": wl.kind,
                         "sample": "a step = one call per (bits, tokens) point of torch_blast_baseline "
                                   "(torch_funcs/blast_funcs.py:3-47) on dequantised fp32 factors, all host cores"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "us_per_layer": {f"int{b}_n{n}": per_point[(b, n)] * 1e6 for b, n in POINTS},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ GPU helpers
class GraphTimer:
    def __init__(self):
        self.side = torch.cuda.Stream()

    def capture(self, fn):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self.side):
            with torch.cuda.graph(g, stream=self.side):
                fn()
        torch.cuda.synchronize()
        return g

    def us_per_call(self, fns, reps=10):
        """Mean device time of one call of a list of callables captured back to back in one graph."""
        g = self.capture(lambda: [f() for f in fns])
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b_.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b_) * 1e3 / (reps * len(fns))


def graphed_ms(fn, reps=5):
    """Milliseconds per replay of fn captured in a CUDA graph; NaN where the capture fails."""
    try:
        g = GraphTimer().capture(fn)
        return time_ms(g.replay, reps, warm=2)
    except Exception:
        return float("nan")


def time_ms(fn, reps, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b_.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b_) / reps


def max_over_ranks(dist, dev, values):
    if dist is None:
        return values
    t = torch.tensor(values, device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


# ------------------------------------------------------------------------------------------ network level
def llama_leg(dev, rank, world, dist, quick):
    """Llama-7B-shaped decoder, every attention / MLP linear a BLAST linear (b = 16, ranks 1024 / 1488): prefill at 2048
    tokens (16-bit factors) and decode at batch 1/4/16/64 against a full 2048-token cache (16-bit and int8 factors),
    each decode step replayed from a CUDA graph.  Token batches are independent per rank (data parallel): tokens/s
    are summed over ranks, times are the maximum over ranks."""
    from mem_efficient_blr_b200 import networks as nw
    shape = nw.LlamaShape(layers=4) if quick else nw.LlamaShape()
    batches = (1, 16) if quick else (1, 4, 16, 64)
    cache = 2048
    peak_hbm, _, _ = measured_peaks()
    out = {"shape": {"layers": shape.layers, "d": shape.d, "heads": shape.heads, "ffn": shape.ffn, "vocab": shape.vocab,
                     "blast_b": shape.b, "rank_attn": shape.rank_attn, "rank_mlp": shape.rank_mlp},
           "kv_cache_tokens": cache, "dtype": "f16", "parallelism": f"dp{world} (token batches per rank)"}
    gt = GraphTimer()
    for method in ("blast", "blast_int8"):
        torch.cuda.empty_cache()
        model = nw.LlamaDecoder(shape, method, batch=max(batches), cache_len=cache, device=dev, dtype=torch.float16,
                                seed=rank, init_on_device=True)
        for kc, vc in zip(model.kcache, model.vcache):
            kc.normal_(0, 0.5)
            vc.normal_(0, 0.5)
        wbytes = sum(p.numel() * p.element_size() for m in model.structured_linears() for p in list(m.parameters()) + list(m.buffers()))
        res = {"structured_weight_bytes": wbytes, "weight_streaming_floor_ms": wbytes / (peak_hbm * 1e9) * 1e3, "decode": {}}
        lin = model.structured_linears()
        for B in batches:
            ids = torch.randint(0, shape.vocab, (B, 1), device=dev)
            pos = torch.tensor([cache - 1], device=dev)
            step = nw.GraphedCall(model.decode_step, ids, pos)
            ms = time_ms(step.graph.replay, 10, warm=3)
            # the structured linears of the same step alone, same graph technique: their share of the step
            xin = {m.in_features: torch.randn(B, m.in_features, device=dev, dtype=torch.float16) for m in lin}
            g = gt.capture(lambda: [m(xin[m.in_features]) for m in lin])
            ms_lin = time_ms(g.replay, 10, warm=3)
            ms, ms_lin = max_over_ranks(dist, dev, [ms, ms_lin])
            res["decode"][f"batch{B}"] = {"ms_per_token_step": ms, "tokens_per_s": world * B / (ms * 1e-3),
                                          "structured_linears_ms": ms_lin, "structured_linears_share": ms_lin / ms}
            del step, g
        if method == "blast":
            T = 512 if quick else 2048
            ids = torch.randint(0, shape.vocab, (1, T), device=dev)
            ms = time_ms(lambda: model.prefill(ids), 3, warm=2)
            xin = {m.in_features: torch.randn(T, m.in_features, device=dev, dtype=torch.float16) for m in lin}
            ms_lin = time_ms(lambda: [m(xin[m.in_features]) for m in lin], 3, warm=2)
            ms, ms_lin = max_over_ranks(dist, dev, [ms, ms_lin])
            res["prefill"] = {"tokens": T, "ms": ms, "tokens_per_s": world * T / (ms * 1e-3), "structured_linears_ms": ms_lin,
                              "structured_linears_share": ms_lin / ms}
        out[method] = res
        del model, lin
    torch.cuda.empty_cache()
    return out


def vit_leg(dev, rank, world, dist, quick):
    """ViT-B/16-shaped encoder (197 tokens per image), fused qkv / intermediate / output linears as BLAST b = 16 with
    about half of the dense parameters; images per second at several batch sizes, independent batches per rank."""
    from mem_efficient_blr_b200 import networks as nw
    shape = nw.ViTShape()
    model = nw.ViTEncoder(shape, "blast", device=dev, dtype=torch.float16, seed=rank, init_on_device=True)
    out = {"shape": {"layers": shape.layers, "d": shape.d, "heads": shape.heads, "mlp": shape.mlp, "tokens": 197,
                     "blast_b": shape.b, "ranks": shape.ranks}, "dtype": "f16", "parallelism": f"dp{world} (image batches per rank)"}
    for B in ((1, 32) if quick else (1, 16, 64, 256)):
        img = torch.randn(B, 3, shape.image, shape.image, device=dev, dtype=torch.float16)
        ms = time_ms(lambda: model(img), 5, warm=2)
        ms_g = graphed_ms(lambda: model(img))   # the same forward replayed from a CUDA graph: device time without launch work
        ms, ms_g = max_over_ranks(dist, dev, [ms, ms_g])
        out[f"batch{B}"] = {"ms": ms, "images_per_s": world * B / (ms * 1e-3), "tokens_per_s": world * B * 197 / (ms * 1e-3),
                            "ms_graph": ms_g, "images_per_s_graph": world * B / (ms_g * 1e-3)}
    del model
    torch.cuda.empty_cache()
    return out


def dit_leg(dev, rank, world, dist, quick):
    """DiT-XL/2-shaped denoiser (256 tokens per 32 x 32 x 4 latent), attn.qkv / mlp.fc1 / adaLN linear as BLAST b = 9 with
    the ranks of the reference's configs/networks/dit_xl.yaml; denoising steps (forward passes) per second at several
    batch sizes, independent batches per rank."""
    from mem_efficient_blr_b200 import networks as nw
    shape = nw.DiTShape()
    model = nw.DiTDenoiser(shape, "blast", device=dev, dtype=torch.float16, seed=rank, init_on_device=True)
    out = {"shape": {"layers": shape.layers, "d": shape.d, "heads": shape.heads, "mlp": shape.mlp, "tokens": 256,
                     "blast_b": shape.b, "ranks": shape.ranks}, "dtype": "f16", "parallelism": f"dp{world} (latent batches per rank)"}
    for B in ((1, 16) if quick else (1, 8, 64)):
        lat = torch.randn(B, shape.channels, shape.latent, shape.latent, device=dev, dtype=torch.float16)
        t = torch.randint(0, 1000, (B,), device=dev)
        y = torch.randint(0, shape.classes, (B,), device=dev)
        ms = time_ms(lambda: model(lat, t, y), 5, warm=2)
        ms_g = graphed_ms(lambda: model(lat, t, y))
        ms, ms_g = max_over_ranks(dist, dev, [ms, ms_g])
        out[f"batch{B}"] = {"ms": ms, "latents_per_s": world * B / (ms * 1e-3), "tokens_per_s": world * B * 256 / (ms * 1e-3),
                            "ms_graph": ms_g, "latents_per_s_graph": world * B / (ms_g * 1e-3)}
    del model
    torch.cuda.empty_cache()
    return out


def network_step_case(case, dev):
    """Small case for a profiler launch list of one network step: 'step:llama:BATCH[:METHOD]' (four decoder layers, one
    decode step against a full 2048-token cache), 'step:vit:BATCH' and 'step:dit:BATCH' (four layers, one forward).
    Three warm-up steps, then one step between cudaProfilerStart / Stop (ncu --profile-from-start off)."""
    from mem_efficient_blr_b200 import networks as nw, _lib
    parts = case.split(":")
    kind, B = parts[1], int(parts[2])
    if kind == "llama":
        shape = nw.LlamaShape(layers=4)
        model = nw.LlamaDecoder(shape, parts[3] if len(parts) > 3 else "blast", batch=B, cache_len=2048, device=dev,
                                dtype=torch.float16, seed=0, init_on_device=True)
        ids, pos = torch.randint(0, shape.vocab, (B, 1), device=dev), torch.tensor([2047], device=dev)
        step = lambda: model.decode_step(ids, pos)
    elif kind == "vit":
        shape = nw.ViTShape(layers=4)
        model = nw.ViTEncoder(shape, "blast", device=dev, dtype=torch.float16, seed=0, init_on_device=True)
        img = torch.randn(B, 3, shape.image, shape.image, device=dev, dtype=torch.float16)
        step = lambda: model(img)
    elif kind == "dit":
        shape = nw.DiTShape(layers=4)
        model = nw.DiTDenoiser(shape, "blast", device=dev, dtype=torch.float16, seed=0, init_on_device=True)
        lat = torch.randn(B, shape.channels, shape.latent, shape.latent, device=dev, dtype=torch.float16)
        t, y = torch.randint(0, 1000, (B,), device=dev), torch.randint(0, shape.classes, (B,), device=dev)
        step = lambda: model(lat, t, y)
    else:
        raise SystemExit(f"unknown network case {case!r}")
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    _lib.workspace_status(dev)
    print(json.dumps({"ncu_case": case, "steps": 1}))


def sharding_leg(dev, rank, world, dist):
    """BLAST sharded by output block over the ranks (gate_proj shape with the 50 %-parameter rank): every rank holds
    b / world blocks of U and S and all of V, computes its columns, and one NCCL all_gather along the feature axis
    assembles the row.  Microseconds per layer including the gather, against the whole layer on one GPU; the gathered
    result is checked against the unsharded one on every rank."""
    import mem_efficient_blr_b200.blast_kernels as bk
    from mem_efficient_blr_b200 import dist as bd
    R = 1488
    g = torch.Generator(device=dev).manual_seed(7)   # same factors on every rank
    U = (torch.randn(B_BLK, Q_BLK, R, generator=g, device=dev) / R ** 0.5).half()
    Vt = (torch.randn(B_BLK, R, P_BLK, generator=g, device=dev) / P_BLK ** 0.5).half()
    S = (torch.rand(B_BLK, B_BLK, R, generator=g, device=dev) + 0.5).half()
    Ul, Sl = (t.contiguous() for t in bd.shard_blast_factors(U, S, rank, world))
    out = {"layer": f"BLAST {I_F}->{O_F}, b={B_BLK}, R={R}, fp16", "ranks": world, "blocks_per_rank": B_BLK // world}
    for n in (1, 16, 2048):
        x = torch.randn(n, I_F, generator=g, device=dev).half()
        full = bk.blast_torch_layout(x, U, Vt, S)
        got = bd.blast_row_block_parallel(x, Ul, Vt, Sl, bk.blast_output_blocks)
        torch.cuda.synchronize()
        err = float((got.float() - full.float()).norm() / full.float().norm())
        if not err < 1e-3:
            raise SystemExit(f"rank {rank}: row-block sharding disagrees with the unsharded layer at {n} tokens: {err}")
        dist.barrier()
        us_full = time_ms(lambda: bk.blast_torch_layout(x, U, Vt, S), 50, warm=5) * 1e3
        us_local = time_ms(lambda: bk.blast_output_blocks(x, Ul, Vt, Sl), 50, warm=5) * 1e3
        dist.barrier()
        us_shard = time_ms(lambda: bd.blast_row_block_parallel(x, Ul, Vt, Sl, bk.blast_output_blocks), 50, warm=5) * 1e3
        # the same call replayed from a CUDA graph (kernels and the NCCL collective captured together): what a
        # decode step that is itself a graph pays, without the host's launch work
        us_graph = None
        try:
            dist.barrier()
            gcall = GraphTimer().capture(lambda: bd.blast_row_block_parallel(x, Ul, Vt, Sl, bk.blast_output_blocks))
            dist.barrier()
            us_graph = time_ms(gcall.replay, 50, warm=5) * 1e3
        except Exception as e:   # a collective that cannot be captured on this stack: report the eager figure only
            us_graph = float("nan")
            out.setdefault("graph_capture_error", repr(e)[:200])
        us_full, us_local, us_shard, us_graph = max_over_ranks(dist, dev, [us_full, us_local, us_shard, us_graph])
        best = us_graph if us_graph == us_graph else us_shard
        out[f"n{n}"] = {"us_one_gpu": us_full, "us_local_part": us_local, "us_sharded_with_gather": us_shard,
                        "us_sharded_with_gather_graph": us_graph, "speedup": us_full / best,
                        "efficiency": us_full / best / world, "rel_err_vs_unsharded": err}
    return out


def layer_sweep(dev, quick):
    """Every operator family at the three Llama-7B linear shapes (Monarch with 4 blocks, BLAST with 16), fp16, tokens
    1 / 16 / 128 / 2048, ranks for about half of the dense parameters; roofline = max(bytes / HBM, flops / tensor)."""
    import mem_efficient_blr_b200.blast_kernels as bk
    import mem_efficient_blr_b200.dense_kernels as dk
    import mem_efficient_blr_b200.low_rank_kernels as lk
    import mem_efficient_blr_b200.monarch_kernels as mk
    peak_hbm, peak_tf, _ = measured_peaks()
    gt = GraphTimer()

    def point(kind, i_f, o_f, r, n):
        xn = torch.randn(n, i_f, device=dev, dtype=torch.float16)
        h = lambda *shape, fan: torch.randn(*shape, device=dev, dtype=torch.float16) / fan ** 0.5
        if kind == "blast":
            wbytes, flops = 2 * r * (i_f + o_f) + 2 * B_BLK * B_BLK * r, 2 * n * r * (i_f + o_f + B_BLK * B_BLK)
            mk_one = lambda: (h(B_BLK, o_f // B_BLK, r, fan=r), h(B_BLK, r, i_f // B_BLK, fan=i_f // B_BLK),
                              torch.rand(B_BLK, B_BLK, r, device=dev, dtype=torch.float16) + 0.5)
            call = lambda f: bk.blast_torch_layout(xn, *f)
        elif kind in ("monarch", "monarch_ideal"):
            # monarch_ideal: the output stays in the block-major order of the reference's right_ideal variant
            wbytes, flops = 2 * r * (i_f + o_f), 2 * n * r * (i_f + o_f)
            mk_one = lambda: (h(4, r, i_f // 4, fan=i_f // 4), h(4, o_f // 4, r, fan=r))
            call = lambda f: mk.monarch_torch_layout(xn, *f, ideal=(kind == "monarch_ideal"))
        elif kind == "low_rank":
            wbytes, flops = 2 * r * (i_f + o_f), 2 * n * r * (i_f + o_f)
            mk_one = lambda: (h(r, i_f, fan=i_f), h(o_f, r, fan=r))
            call = lambda f: lk.low_rank_torch_layout(xn, *f)
        else:
            wbytes, flops = 2 * i_f * o_f, 2 * n * i_f * o_f
            mk_one = lambda: (h(o_f, i_f, fan=i_f),)
            call = lambda f: dk.dense_torch_layout(xn, *f)
        nrep = int(2 * L2_BYTES // wbytes) + 1
        sets = [mk_one() for _ in range(nrep)]
        us = gt.us_per_call([(lambda f=f: call(f)) for f in sets], reps=5)
        nbytes = wbytes + 2 * n * (i_f + o_f)
        roof = max(nbytes / (peak_hbm * 1e9), flops / (peak_tf * 1e12)) * 1e6
        return {"us_per_layer": round(us, 2), "roofline_us": round(roof, 2), "frac": round(roof / us, 3)}

    res = {}
    tokens = (1, 2048) if quick else (1, 16, 128, 2048)
    for lname, i_f, o_f, ranks in (("qkvo_4096x4096", 4096, 4096, {"blast": 1024, "monarch": 1024, "low_rank": 1024}),
                                   ("gate_4096x11008", 4096, 11008, {"blast": 1488, "monarch": 1536, "low_rank": 1024}),
                                   ("down_11008x4096", 11008, 4096, {"blast": 1488, "monarch": 1536, "low_rank": 1024})):
        kinds = ("blast", "monarch", "low_rank", "dense") + (("monarch_ideal",) if lname.startswith("gate") else ())
        for kind in kinds:
            for n in tokens:
                res[f"{lname}/{kind}/n{n}"] = point(kind, i_f, o_f, ranks.get(kind.split("_ideal")[0], 0), n)
                torch.cuda.empty_cache()
    # SwiGLU MLP on Monarch linears (4 blocks, rank 1536): gate / up in the ideal order feeding down directly (the
    # reference's configs/networks/llama7b.yaml:164,180) against every layer interleaving its output
    from mem_efficient_blr_b200 import networks as nw
    nrep = int(2 * L2_BYTES // (3 * 2 * 1536 * (4096 + 11008))) + 1
    for chain in ("ideal", "interleaved"):
        mods = [nw.MonarchSwiGLU(4096, 11008, 4, 1536, chain, device=dev, generator=torch.Generator(device=dev).manual_seed(i))
                for i in range(nrep)]
        for n in tokens:
            xn = torch.randn(n, 4096, device=dev, dtype=torch.float16)
            us = gt.us_per_call([(lambda m=m: m(xn)) for m in mods], reps=5)
            res[f"monarch_swiglu_mlp/{chain}/n{n}"] = {"us_per_mlp": round(us, 2)}
        del mods
        torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------------ our arm (GPU)
def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    import mem_efficient_blr_b200.blast_kernels as bk
    import mem_efficient_blr_b200.blast_sym_quant_kernels as bq
    from mem_efficient_blr_b200 import _lib

    if args.ncu_case.startswith("step:"):
        network_step_case(args.ncu_case, dev)
        return

    # ---- synthetic factors with the headline configuration's distributions:
    # U, Vt ~ N(0, 1/sqrt(fan_in)), S ~ U(0.5, 1.5), x ~ N(0, 1), fp16, seeded per rank
    g = torch.Generator().manual_seed(rank)
    U = (torch.randn(B_BLK, Q_BLK, RANK, generator=g) / RANK ** 0.5).half()
    Vt = (torch.randn(B_BLK, RANK, P_BLK, generator=g) / P_BLK ** 0.5).half()
    S = (torch.rand(B_BLK, B_BLK, RANK, generator=g) + 0.5).half()
    x16 = torch.randn(1, 16, I_F, generator=g).half()
    Ud, Vd, Sd = U.to(dev), Vt.to(dev), S.to(dev)
    reps = {}
    for bits in (8, 4):
        q = bq.quantize_blast_factors(Ud, Vd, bits)
        per = sum(t.numel() * t.element_size() for t in q)
        nrep = int(2 * L2_BYTES // per) + 1
        reps[bits] = [tuple(t.clone() for t in q) for _ in range(nrep)]
    xs = {n: x16[0, :n].contiguous().to(dev) for n in (1, 4, 16)}
    xs_host = {n: x16[0, :n].contiguous().pin_memory() for n in (1, 4, 16)}
    outs_host = {n: torch.empty(n, O_F, dtype=torch.float16).pin_memory() for n in (1, 4, 16)}

    def launch_points(group=None):
        calls = 0
        for bits, n in POINTS:
            if group is not None and group_of(bits, n) != group:
                continue
            for q in reps[bits]:
                bq.blast_wq(xs[n], q[0], q[1], q[2], q[3], Sd, bits)
                calls += 1
        return calls

    if args.ncu_case.startswith("p16:"):
        # small case for a profiler capture of the tensor-core pipeline: the 16-bit layer on N tokens, three calls
        n = int(args.ncu_case.split(":")[1])
        xn = torch.randn(n, I_F, device=dev, dtype=torch.float16)
        for _ in range(3):
            bk.blast_torch_layout(xn, Ud, Vd, Sd)
        torch.cuda.synchronize()
        _lib.workspace_status(dev)
        print(json.dumps({"ncu_case": args.ncu_case, "calls": 3}))
        return
    if args.ncu_case:
        # small case for a profiler capture: a few eager calls of one point over distinct replicas
        bits, n = (int(t) for t in args.ncu_case.split(":"))
        xn = xs[n] if n in xs else torch.randn(n, I_F, device=dev, dtype=torch.float16)
        for q in reps[bits][:6]:
            bq.blast_wq(xn, q[0], q[1], q[2], q[3], Sd, bits)
        torch.cuda.synchronize()
        _lib.workspace_status(dev)
        print(json.dumps({"ncu_case": args.ncu_case, "calls": 6}))
        return

    groups = sorted({group_of(b, n) for b, n in POINTS})
    calls = {k: launch_points(k) for k in groups}
    torch.cuda.synchronize()
    kbytes = {k: sum(algorithmic_bytes(b, n) * len(reps[b]) for b, n in POINTS if group_of(b, n) == k) for k in groups}
    bytes_per_pass = sum(kbytes.values())
    launches_per_pass = sum(len(reps[b]) * launches_of(b, n) for b, n in POINTS)

    # ---- capture one pass in CUDA graphs (the per-launch host work would otherwise bound the rate): one graph per
    # kernel group, replayed back to back, with an event between them so that each group's time is known
    gt = GraphTimer()
    graphs = {k: gt.capture(lambda k=k: launch_points(k)) for k in groups}

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def one_step(ev=None):
        for ps in range(PASSES_PER_STEP):
            for i, k in enumerate(groups):
                if ev is not None and ps == 0:
                    ev[i].record()
                graphs[k].replay()
            if ev is not None and ps == 0:
                ev[len(groups)].record()

    for _ in range(max(args.warmup, 3)):
        one_step()
    barrier()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(groups) + 1)] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        barrier()
        t_begin.record()
        for st in range(args.steps):
            one_step(ev[st])
        t_end.record()
        barrier()
    step_ms = t_begin.elapsed_time(t_end) / args.steps
    # time of each group inside the first pass of every step (events on the launching stream)
    group_ms = {k: sum(ev[st][i].elapsed_time(ev[st][i + 1]) for st in range(args.steps)) / args.steps for i, k in enumerate(groups)}
    _lib.workspace_status(dev)
    vals = max_over_ranks(dist, dev, [step_ms] + [group_ms[k] for k in groups])
    step_ms, group_ms = vals[0], {k: vals[i + 1] for i, k in enumerate(groups)}
    value = world * bytes_per_pass * PASSES_PER_STEP / (step_ms * 1e-3) / 1e9

    peak_hbm, peak_tf, peak_kind = measured_peaks()
    # ---- per-point detail (separate timed loops, same graph technique) with the dense fp16 cuBLAS bar of the layer
    sweep = {}
    if rank == 0:
        Ws = [torch.randn(O_F, I_F, device=dev, dtype=torch.float16) / 64 for _ in range(4)]
        dense_us = {}
        for n in (1, 4, 16):
            xn = xs[n]
            dense_us[n] = gt.us_per_call([(lambda w=w: torch.nn.functional.linear(xn, w)) for w in Ws])
        del Ws
        for bits, n in POINTS:
            us = gt.us_per_call([(lambda q=q: bq.blast_wq(xs[n], q[0], q[1], q[2], q[3], Sd, bits)) for q in reps[bits]])
            nb = algorithmic_bytes(bits, n)
            sweep[f"int{bits}_n{n}"] = {"us_per_layer": us, "GBps": nb / us / 1e3, "roofline_us": nb / (peak_hbm * 1e3),
                                        "frac": nb / (peak_hbm * 1e3) / us, "dense_fp16_cublas_us": dense_us[n],
                                        "speedup_vs_dense_fp16_cublas": dense_us[n] / us,
                                        "speedup_target": 3.9 if bits == 8 else 7.6}
        # the 16-bit layer at decode and prefill sizes
        Us = [Ud.clone() for _ in range(9)]  # 9 x 31 MB of fp16 factors > 2 x L2
        Vs = [Vd.clone() for _ in range(9)]
        for n in (1, 4, 16, 128, 2048):
            xn = torch.randn(n, I_F, device=dev, dtype=torch.float16)
            us = gt.us_per_call([(lambda u=u, v=v: bk.blast_torch_layout(xn, u, v, Sd)) for u, v in zip(Us, Vs)])
            nbytes = 2 * RANK * (I_F + O_F) + 2 * B_BLK * B_BLK * RANK + 2 * n * (I_F + O_F)
            flops = 2 * n * RANK * (I_F + O_F + B_BLK * B_BLK)
            roof = max(nbytes / (peak_hbm * 1e9), flops / (peak_tf * 1e12)) * 1e6
            sweep[f"fp16_n{n}"] = {"us_per_layer": us, "roofline_us": roof, "frac": roof / us,
                                   "TFLOPs": flops / us / 1e6, "GBps": nbytes / us / 1e3}
        del Us, Vs
        torch.cuda.empty_cache()

    lsweep = layer_sweep(dev, args.quick) if rank == 0 and not args.no_context else None

    # ---- end to end through the public host-buffer operator: x in pinned host memory, result back in pinned host
    # memory, every call (one library call enqueues copy-in, kernel and copy-out; its copy streams let consecutive
    # calls overlap).  The step ends when the last result has arrived in host memory.
    host_calls = {bits: [bq.BlastWqHostCall(q[0], q[1], q[2], q[3], Sd, bits) for q in reps[bits]] for bits in reps}

    def e2e_pass():
        for bits, n in POINTS:
            for call in host_calls[bits]:
                call(xs_host[n], outs_host[n])
        bq.host_flush(dev)

    e2e_passes = 5
    for _ in range(2):
        e2e_pass()
    barrier()
    # the host path must deliver what the device path computes (last call of a pass: int4, 16 tokens, last replica)
    q = reps[4][-1]
    want = bq.blast_wq(xs[16], q[0], q[1], q[2], q[3], Sd, 4).float().cpu()
    err = float((outs_host[16].float() - want).norm() / want.norm())
    if not err < 1e-3:
        raise SystemExit(f"host-buffer path disagrees with the device path: relative error {err}")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_passes):
        e2e_pass()
    e1.record()
    barrier()
    (e2e_ms,) = max_over_ranks(dist, dev, [e0.elapsed_time(e1) / e2e_passes])
    h2d = sum(2 * n * I_F * len(reps[b]) for b, n in POINTS) * PASSES_PER_STEP
    d2h = sum(2 * n * O_F * len(reps[b]) for b, n in POINTS) * PASSES_PER_STEP
    del host_calls, reps
    torch.cuda.empty_cache()

    # ---- network level and sharding (all ranks take part; rank 0 reports)
    llama = vit = dit = shard = None
    if not args.no_context:
        llama = llama_leg(dev, rank, world, dist, args.quick)
        vit = vit_leg(dev, rank, world, dist, args.quick)
        dit = dit_leg(dev, rank, world, dist, args.quick)
        if world > 1 and B_BLK % world == 0:
            shard = sharding_leg(dev, rank, world, dist)

    if rank == 0:
        per_group = {}
        for k in groups:
            ach = kbytes[k] / (group_ms[k] * 1e-3) / 1e9
            per_group[k] = {"kernels": GROUPS[k][0], "calls_per_pass": calls[k], "launches_per_call": launches_per_pass / sum(calls.values()),
                            "share": group_ms[k] / sum(group_ms.values()), "us_per_call": group_ms[k] * 1e3 / calls[k],
                            "algorithmic_bytes_per_call": kbytes[k] / calls[k], "achieved": ach, "frac": ach / peak_hbm}
        top = max(groups, key=lambda k: group_ms[k])
        traffic, traffic_note = ncu_traffic(top)
        cpu = None
        if world == 1:
            threads = os.cpu_count() or 1
            wl = CpuWorkload(threads)
            wl.step()
            steps = [wl.step() for _ in range(5)]
            cpu_s = sum(sum(s.values()) for s in steps) / len(steps)
            cpu = {"value": sum(algorithmic_bytes(b, n) for b, n in POINTS) / cpu_s / 1e9, "unit": "GB/s", "cores": threads,
                   "kind": wl.kind, "sample": "5 timed calls per (bits, tokens) point of torch_blast_baseline "
                                              "(torch_funcs/blast_funcs.py:3-47) on dequantised fp32 factors, all host cores"}
        line = {
            "metric": "blast_wq_decode_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 activations, s8/s4 weights, s32/f32 accumulate",
            "data": "synthetic",
            "config": workload_config(),
            "gpu_launches": launches_per_pass * PASSES_PER_STEP * args.steps,
            "us_per_layer_mean": step_ms * 1e3 / (sum(calls.values()) * PASSES_PER_STEP),
            "roofline": {"bound": "hbm", "achieved": per_group[top]["achieved"], "peak": peak_hbm, "unit": "GB/s",
                         "frac": per_group[top]["frac"], "peak_kind": peak_kind, "traffic": traffic, "traffic_note": traffic_note,
                         "kernel": GROUPS[top][0], "whole_step_frac": value / world / peak_hbm, "groups": per_group},
            "e2e": {"value": world * bytes_per_pass / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms * PASSES_PER_STEP},
            "cpu_baseline": cpu,
            "clocks": clk.summary(),
            "sweep": sweep,
            "llama7b_blast": llama,
            "vit_b16_blast": vit,
            "dit_xl2_blast": dit,
            "row_block_sharding": shard,
            "layer_sweep": lsweep,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-context", action="store_true", help="headline only: skip the layer sweep, the networks and the sharding leg")
    ap.add_argument("--quick", action="store_true", help="smaller network legs (4 decoder layers, fewer batch sizes) and a two-point layer sweep")
    ap.add_argument("--ncu-case", default="", help="BITS:TOKENS, e.g. 8:16 - run six eager calls of one point and exit (for profiler captures); "
                                                  "p16:TOKENS - three calls of the 16-bit layer on that many tokens; "
                                                  "step:llama:BATCH[:METHOD] | step:vit:BATCH | step:dit:BATCH - one step of a "
                                                  "four-layer network between cudaProfilerStart / Stop")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
