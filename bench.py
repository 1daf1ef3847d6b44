#!/usr/bin/env python
"""Benchmark of the structured-matmul hot path on B200.

Headline workload (the configuration the metric is quoted on): symmetric-quantised BLAST decode on the
Llama-7B gate_proj shape, 4096 -> 11008, b = 16, R = 1024, int8 and packed-int4 factors with fp16
per-channel scales, token counts 1, 4 and 16.  One *step* runs every (bits, N) point once over a
rotating set of weight replicas whose total footprint exceeds the L2 cache, so every launch streams
its weights from HBM.  The metric is algorithmic bytes per second (weights + scales + S + x + out of
every launch, divided by device time), summed over ranks.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

With N > 1 launch under torchrun; every rank runs the same workload on its own GPU (independent
token batches, replicated weights: weak scaling, no collective in the data path).
`--impl reference` times the CPU restatement of the reference's torch path on the host cores.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one launch from ncu captures (profiles/): the cluster kernel on
# int8 factors and 1 token, the grid-wide streaming kernel on int8 factors and 16 tokens
NCU_TRAFFIC = {"blr_blast_cluster_kernel": (16.474e6, "int8/N=1"), "blr_stream_kernel": (16.249e6, "int8/N=16")}
CLUSTER_MAX_TOKENS = 16  # BLAST calls with up to 16 tokens run blr_blast_cluster_kernel on this layer's shape


def algorithmic_bytes(bits: int, n: int) -> float:
    """bytes = wb*R*(I+O) + 2*b^2*R + 2*N*(I+O) + scale bytes, wb = bits/8."""
    return bits / 8 * RANK * (I_F + O_F) + 2 * B_BLK * B_BLK * RANK + 2 * n * (I_F + O_F) + 2 * (B_BLK * Q_BLK + B_BLK * RANK)


def peak_hbm_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


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


# ------------------------------------------------------------------------------------------ reference arm (CPU)
def cpu_reference_times(threads: int, iters: int):
    """Times the CPU restatement of torch_blast_baseline (fp32, dequantised factors) per (bits, N) point."""
    from oracle import blr_oracle as orc
    torch.set_num_threads(threads)
    out = {}
    x16, U, Vt, S = orc.make_blast_inputs(16, I_F, O_F, B_BLK, RANK, torch.float16, seed=0)
    for bits in (8, 4):
        Uq, us = orc.quantize_sym(U, bits)
        Vq, vs = orc.quantize_sym(Vt, bits)
        Ud, Vd = orc.dequantize_sym(Uq, us, bits), orc.dequantize_sym(Vq, vs, bits)
        Sf = S.float()
        for n in (1, 4, 16):
            x = x16[:, :n].float()
            orc.blast(x, Ud, Vd, Sf)
            ts = []
            for _ in range(iters):
                t0 = time.perf_counter()
                orc.blast(x, Ud, Vd, Sf)
                ts.append(time.perf_counter() - t0)
            out[(bits, n)] = statistics.median(ts)
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    iters = max(3, min(10, args.steps))
    # warm-up happens inside cpu_reference_times (one untimed call per point)
    t0 = time.perf_counter()
    times = cpu_reference_times(threads, iters)
    total_bytes = sum(algorithmic_bytes(b, n) for b, n in POINTS)
    step_s = sum(times[p] for p in POINTS)
    value = total_bytes / step_s / 1e9
    line = {
        "impl": "reference", "metric": "blast_wq_decode_algorithmic_GBps", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": iters, "warmup": 1, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(1),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{iters} timed calls per (bits, tokens) point of the CPU restatement of torch_blast_baseline "
                                   "on dequantised fp32 factors (the reference has no weight-quantised path)"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "us_per_layer": {f"int{b}_n{n}": times[(b, n)] * 1e6 for b, n in POINTS},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


def workload_config(replicas_note):
    return {"workload": "symmetric-quantised BLAST decode, Llama-7B gate_proj 4096->11008, b=16, R=1024, "
                        "int8 and packed-int4 factors with fp16 per-channel scales, tokens 1/4/16 (one launch per point per replica)",
            "in_features": I_F, "out_features": O_F, "blocks": B_BLK, "rank": RANK,
            "points": [f"int{b}/N={n}" for b, n in POINTS],
            "l2_policy": "weights rotate over replicas whose footprint exceeds L2 (inputs larger than L2)",
            "replicas": replicas_note}


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

    import mem_efficient_blr_b200.blast_sym_quant_kernels as bq
    from mem_efficient_blr_b200 import _lib

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

    def kernel_of(n):
        return "blr_blast_cluster_kernel" if n <= CLUSTER_MAX_TOKENS else "blr_stream_kernel"

    KERNELS = sorted({kernel_of(n) for _, n in POINTS})

    def launch_points(kernel=None):
        count = 0
        for bits, n in POINTS:
            if kernel is not None and kernel_of(n) != kernel:
                continue
            for q in reps[bits]:
                bq.blast_wq(xs[n], q[0], q[1], q[2], q[3], Sd, bits)
                count += 1
        return count

    if args.ncu_case.startswith("p16:"):
        # small case for a profiler capture of the tensor-core pipeline: the 16-bit layer on N tokens, three calls
        import mem_efficient_blr_b200.blast_kernels as bk
        n = int(args.ncu_case.split(":")[1])
        xn = torch.randn(n, I_F, device=dev, dtype=torch.float16)
        for _ in range(3):
            bk.blast_torch_layout(xn, Ud, Vd, Sd)
        torch.cuda.synchronize()
        _lib.workspace_status(dev)
        print(json.dumps({"ncu_case": args.ncu_case, "calls": 3}))
        return
    if args.ncu_case:
        # small case for a profiler capture: a few eager launches of one point over distinct replicas
        bits, n = (int(t) for t in args.ncu_case.split(":"))
        for q in reps[bits][:6]:
            bq.blast_wq(xs[n], q[0], q[1], q[2], q[3], Sd, bits)
        torch.cuda.synchronize()
        _lib.workspace_status(dev)
        print(json.dumps({"ncu_case": args.ncu_case, "launches": 6}))
        return

    launches = {k: launch_points(k) for k in KERNELS}
    launches_per_step = sum(launches.values())
    torch.cuda.synchronize()
    kbytes = {k: sum(algorithmic_bytes(b, n) * len(reps[b]) for b, n in POINTS if kernel_of(n) == k) for k in KERNELS}
    bytes_per_step = sum(kbytes.values())

    # ---- capture one step in CUDA graphs (the per-launch host work would otherwise bound the rate): one graph
    # per kernel, replayed back to back, with an event between them so that each kernel's time is known
    side = torch.cuda.Stream()
    graphs = {}
    with torch.cuda.stream(side):
        for k in KERNELS:
            launch_points(k)
            torch.cuda.synchronize()
            graphs[k] = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graphs[k], stream=side):
                launch_points(k)
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        for k in KERNELS:
            graphs[k].replay()
    barrier()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(KERNELS) + 1)] for _ in range(args.steps)]
    with ClockSampler(local) as clk:
        barrier()
        for st in range(args.steps):
            ev[st][0].record()
            for i, k in enumerate(KERNELS):
                graphs[k].replay()
                ev[st][i + 1].record()
        barrier()
    step_ms = ev[0][0].elapsed_time(ev[-1][-1]) / args.steps
    kernel_ms = {k: sum(ev[st][i].elapsed_time(ev[st][i + 1]) for st in range(args.steps)) / args.steps
                 for i, k in enumerate(KERNELS)}
    _lib.workspace_status(dev)
    if dist is not None:
        t = torch.tensor([step_ms] + [kernel_ms[k] for k in KERNELS], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms = float(t[0].item())
        kernel_ms = {k: float(t[i + 1].item()) for i, k in enumerate(KERNELS)}
    value = world * bytes_per_step / (step_ms * 1e-3) / 1e9

    # ---- per-point detail (separate timed loops, same graph technique)
    sweep = {}
    if rank == 0:
        for bits, n in POINTS:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    for q in reps[bits]:
                        bq.blast_wq(xs[n], q[0], q[1], q[2], q[3], Sd, bits)
            torch.cuda.synchronize()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                g.replay()
            b_.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b_) * 1e3 / (10 * len(reps[bits]))
            sweep[f"int{bits}_n{n}"] = {"us_per_layer": us, "GBps": algorithmic_bytes(bits, n) / us / 1e3}

    # ---- context (not part of the headline): the 16-bit layer at decode and prefill sizes, and the dense fp16
    # cuBLAS bar of the same layer that the quantised decode is meant to beat
    context = {}
    if rank == 0 and not args.no_context:
        import mem_efficient_blr_b200.blast_kernels as bk

        def graph_time(fns, reps=10):
            for f in fns:
                f()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    for f in fns:
                        f()
            torch.cuda.synchronize()
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

        peak_hbm, _ = peak_hbm_gbs()
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peak_tf = float(json.load(f)["bf16_tflops"])
        except Exception:
            peak_tf = 1590.0
        nrep16 = 9  # 9 x 31 MB of fp16 factors > 2 x L2
        Us = [Ud.clone() for _ in range(nrep16)]
        Vs = [Vd.clone() for _ in range(nrep16)]
        Ws = [torch.randn(O_F, I_F, device=dev, dtype=torch.float16) / 64 for _ in range(4)]
        for n in (1, 4, 16, 128, 2048):
            xn = torch.randn(n, I_F, device=dev, dtype=torch.float16)
            us = graph_time([(lambda u=u, v=v: bk.blast_torch_layout(xn, u, v, Sd)) for u, v in zip(Us, Vs)])
            nbytes = 2 * RANK * (I_F + O_F) + 2 * B_BLK * B_BLK * RANK + 2 * n * (I_F + O_F)
            flops = 2 * n * RANK * (I_F + O_F + B_BLK * B_BLK)
            roof = max(nbytes / (peak_hbm * 1e9), flops / (peak_tf * 1e12)) * 1e6
            entry = {"us_per_layer": us, "roofline_us": roof, "frac": roof / us}
            if n <= 16:
                entry["dense_fp16_cublas_us"] = graph_time([(lambda w=w: torch.nn.functional.linear(xn, w)) for w in Ws])
            context[f"blast_fp16_n{n}"] = entry
        for key, v in sweep.items():
            n = int(key.split("_n")[1])
            v["speedup_vs_dense_fp16_cublas"] = context[f"blast_fp16_n{n}"]["dense_fp16_cublas_us"] / v["us_per_layer"]
        del Us, Vs, Ws

        # Network-level context: the 224 structured linears of one Llama-7B-BLAST decode step (32 layers x
        # q/k/v/o 4096->4096 R=1024 and gate/up/down R=1488, b=16, as in the reference's
        # configs/networks/llama7b.yaml), every layer with its own random factors (6.6 GB in fp16, far beyond L2),
        # chained in one CUDA graph.  Attention, norms and the SwiGLU product are not part of the path and not run.
        def linear_chain(bits):
            shapes = [(4096, 4096, 1024)] * 4 + [(4096, 11008, 1488)] * 2 + [(11008, 4096, 1488)]
            layers, nbytes = [], 0
            for _ in range(32):
                for (i_f, o_f, r) in shapes:
                    p_, q_ = i_f // B_BLK, o_f // B_BLK
                    u = torch.randn(B_BLK, q_, r, device=dev, dtype=torch.float16) / r ** 0.5
                    v = torch.randn(B_BLK, r, p_, device=dev, dtype=torch.float16) / p_ ** 0.5
                    s_ = torch.rand(B_BLK, B_BLK, r, device=dev, dtype=torch.float16) + 0.5
                    wb = 2 if bits == 16 else bits / 8
                    nbytes += wb * r * (i_f + o_f) + 2 * B_BLK * B_BLK * r + 2 * (i_f + o_f)
                    if bits == 16:
                        layers.append((i_f, (u, v, s_)))
                    else:
                        layers.append((i_f, (*bq.quantize_blast_factors(u, v, bits), s_)))
                        del u, v
            xin = {4096: torch.randn(1, 4096, device=dev, dtype=torch.float16),
                   11008: torch.randn(1, 11008, device=dev, dtype=torch.float16)}

            def step():
                for i_f, f in layers:
                    if bits == 16:
                        bk.blast_torch_layout(xin[i_f], *f)
                    else:
                        bq.blast_wq(xin[i_f], f[0], f[1], f[2], f[3], f[4], bits)
            us = graph_time([step], reps=5)
            floor = nbytes / (peak_hbm * 1e9) * 1e6
            return {"us_per_token_step": us, "tokens_per_s_batch1": 1e6 / us, "linears": len(layers),
                    "weight_streaming_floor_us": floor, "frac": floor / us}

        # Layer sweep: every operator family at the three Llama-7B linear shapes, 1 token and 2048 tokens, fp16,
        # ranks from the reference's 50 %-parameter configurations; roofline = max(bytes / HBM, flops / tensor).
        import mem_efficient_blr_b200.dense_kernels as dk
        import mem_efficient_blr_b200.low_rank_kernels as lk
        import mem_efficient_blr_b200.monarch_kernels as mk

        def sweep_point(kind, i_f, o_f, r, n):
            xn = torch.randn(n, i_f, device=dev, dtype=torch.float16)
            h = lambda *shape, fan: torch.randn(*shape, device=dev, dtype=torch.float16) / fan ** 0.5
            if kind == "blast":
                wbytes = 2 * r * (i_f + o_f) + 2 * B_BLK * B_BLK * r
                flops = 2 * n * r * (i_f + o_f + B_BLK * B_BLK)
                mk_one = lambda: (h(B_BLK, o_f // B_BLK, r, fan=r), h(B_BLK, r, i_f // B_BLK, fan=i_f // B_BLK),
                                  torch.rand(B_BLK, B_BLK, r, device=dev, dtype=torch.float16) + 0.5)
                call = lambda f: bk.blast_torch_layout(xn, *f)
            elif kind == "monarch":
                wbytes = 2 * r * (i_f + o_f)
                flops = 2 * n * r * (i_f + o_f)
                mk_one = lambda: (h(B_BLK, r, i_f // B_BLK, fan=i_f // B_BLK), h(B_BLK, o_f // B_BLK, r, fan=r))
                call = lambda f: mk.monarch_torch_layout(xn, *f)
            elif kind == "low_rank":
                wbytes = 2 * r * (i_f + o_f)
                flops = 2 * n * r * (i_f + o_f)
                mk_one = lambda: (h(r, i_f, fan=i_f), h(o_f, r, fan=r))
                call = lambda f: lk.low_rank_torch_layout(xn, *f)
            else:
                wbytes = 2 * i_f * o_f
                flops = 2 * n * i_f * o_f
                mk_one = lambda: (h(o_f, i_f, fan=i_f),)
                call = lambda f: dk.dense_torch_layout(xn, *f)
            nrep = int(2 * L2_BYTES // wbytes) + 1
            sets = [mk_one() for _ in range(nrep)]
            us = graph_time([(lambda f=f: call(f)) for f in sets], reps=5)
            nbytes = wbytes + 2 * n * (i_f + o_f)
            roof = max(nbytes / (peak_hbm * 1e9), flops / (peak_tf * 1e12)) * 1e6
            return {"us_per_layer": us, "roofline_us": roof, "frac": roof / us}

        layer_sweep = {}
        for lname, i_f, o_f, ranks in (("qkvo_4096x4096", 4096, 4096, {"blast": 1024, "monarch": 1024, "low_rank": 1024}),
                                       ("gate_4096x11008", 4096, 11008, {"blast": 1488, "monarch": 1536, "low_rank": 1024}),
                                       ("down_11008x4096", 11008, 4096, {"blast": 1488, "monarch": 1536, "low_rank": 1024})):
            for kind in ("blast", "monarch", "low_rank", "dense"):
                for n in (1, 2048):
                    layer_sweep[f"{lname}/{kind}/n{n}"] = sweep_point(kind, i_f, o_f, ranks.get(kind, 0), n)
                    torch.cuda.empty_cache()
        context["layer_sweep_fp16"] = layer_sweep

        context["llama7b_blast_linears_decode_fp16"] = linear_chain(16)
        context["llama7b_blast_linears_decode_int8"] = linear_chain(8)
        torch.cuda.empty_cache()

    # ---- end to end through the public host-buffer operator: x in pinned host memory, result back in pinned host
    # memory, every launch (one library call enqueues copy-in, kernel and copy-out; its copy streams let consecutive
    # calls overlap).  The step ends when the last result has arrived in host memory.
    host_calls = {bits: [bq.BlastWqHostCall(q[0], q[1], q[2], q[3], Sd, bits) for q in reps[bits]] for bits in reps}

    def e2e_step():
        for bits, n in POINTS:
            for call in host_calls[bits]:
                call(xs_host[n], outs_host[n])
        bq.host_flush(dev)

    e2e_steps = max(2, min(args.steps, 5))
    for _ in range(2):
        e2e_step()
    barrier()
    # the host path must deliver what the device path computes (last call of a step: int4, 16 tokens, last replica)
    q = reps[4][-1]
    want = bq.blast_wq(xs[16], q[0], q[1], q[2], q[3], Sd, 4).float().cpu()
    err = float((outs_host[16].float() - want).norm() / want.norm())
    if not err < 1e-3:
        raise SystemExit(f"host-buffer path disagrees with the device path: relative error {err}")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    if dist is not None:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    h2d = sum(2 * n * I_F * len(reps[b]) for b, n in POINTS)
    d2h = sum(2 * n * O_F * len(reps[b]) for b, n in POINTS)

    if rank == 0:
        peak, peak_kind = peak_hbm_gbs()
        # roofline of the kernel with the largest share of the timed region (per GPU): algorithmic bytes of its
        # launches / their device time; the other kernel is listed beside it
        per_kernel = {}
        for k in KERNELS:
            ach = kbytes[k] / (kernel_ms[k] * 1e-3) / 1e9
            per_kernel[k] = {"launches_per_step": launches[k], "share": kernel_ms[k] / sum(kernel_ms.values()),
                             "us_per_launch": kernel_ms[k] * 1e3 / launches[k],
                             "algorithmic_bytes_per_launch": kbytes[k] / launches[k], "achieved": ach, "frac": ach / peak}
        top = max(KERNELS, key=lambda k: kernel_ms[k])
        achieved = per_kernel[top]["achieved"]
        cpu = None
        if world == 1:
            threads = os.cpu_count() or 1
            times = cpu_reference_times(threads, 5)
            cpu_s = sum(times[p] for p in POINTS)
            cpu = {"value": sum(algorithmic_bytes(b, n) for b, n in POINTS) / cpu_s / 1e9, "unit": "GB/s", "cores": threads,
                   "kind": "port", "sample": "5 timed calls per (bits, tokens) point of the CPU restatement of "
                                             "torch_blast_baseline on dequantised fp32 factors"}
        line = {
            "metric": "blast_wq_decode_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 activations, s8/s4 weights, f32 accumulate",
            "data": "synthetic",
            "config": workload_config({f"int{b}": len(reps[b]) for b in (8, 4)}),
            "gpu_launches": launches_per_step * args.steps,
            "us_per_layer_mean": step_ms * 1e3 / launches_per_step,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "traffic": NCU_TRAFFIC[top][0], "kernel": top,
                         "traffic_note": f"dram read+write bytes of one {NCU_TRAFFIC[top][1]} launch from an ncu capture "
                                         "(profiles/); algorithmic bytes of that point: "
                                         f"{algorithmic_bytes(8, 1 if top == 'blr_blast_cluster_kernel' else 16):.0f}",
                         "kernels": per_kernel},
            "e2e": {"value": world * bytes_per_step / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
            "cpu_baseline": cpu,
            "clocks": clk.summary(),
            "sweep": sweep,
            "context": context,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-context", action="store_true", help="skip the informational 16-bit / cuBLAS measurements")
    ap.add_argument("--ncu-case", default="", help="BITS:TOKENS, e.g. 8:16 - run six eager launches of one point and exit (for profiler captures); "
                                                  "p16:TOKENS - three calls of the 16-bit layer on that many tokens")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
