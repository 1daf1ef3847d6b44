"""Analytic bytes / FLOPs per operator and roofline times.

The `*_mem_flops` functions keep the reference's names and formulas (roofline.py:7-99) so its name-based lookup
(`<function name minus its last suffix>_mem_flops`, roofline.py:136-142) keeps working; every function of this
package is fully fused, so the BLAST families all map to the fused count (`triton_blast_full_mem_flops`,
roofline.py:59-63).  Plotting is left to the caller (matplotlib is not a dependency here).
"""
from __future__ import annotations

from .device import Device


def triton_low_rank_mem_flops(n, i, r, o, num_bytes_per_element):
    return (i * r + r * o + n * o + n * i) * num_bytes_per_element, n * r * (i + o) * 2


def triton_dense_mem_flops(n, i, o, num_bytes_per_element):
    return (n * i + i * o + n * o) * num_bytes_per_element, n * i * o * 2


def triton_blast_full_mem_flops(n, i, r, o, b1, b2, num_bytes_per_element):
    return (n * i + b1 * b2 * r + i * r + r * o + n * o) * num_bytes_per_element, n * r * (i + o + b1 * b2) * 2


triton_blast_partial_mem_flops = triton_blast_full_mem_flops
triton_blast_partial_grouped_mem_flops = triton_blast_full_mem_flops
triton_blast_partial_grouped_persistent_mem_flops = triton_blast_full_mem_flops
triton_blast_bmm_mem_flops = triton_blast_full_mem_flops
triton_blast_bmm_int8_mem_flops = triton_blast_full_mem_flops


def blast_wq_mem_flops(n, i, r, o, b, bits, act_bytes=2):
    """Weight-quantised BLAST: factors at bits/8 bytes, fp16 scales per output channel, S and activations 16-bit."""
    w = r * (i + o) * bits / 8 + 2 * (o + b * r)
    return w + (b * b * r + n * (i + o)) * act_bytes, n * r * (i + o + b * b) * 2


def triton_monarch_right_ideal_mem_flops(n, i, r, o, b, num_bytes_per_element):
    """Fused count: the intermediate stays on chip (r is the per-factor rank)."""
    return (n * i + i * r + r * o + n * o) * num_bytes_per_element, n * r * (i + o) * 2


triton_monarch_right_mem_flops = triton_monarch_right_ideal_mem_flops
triton_monarch_right_left_mem_flops = triton_monarch_right_ideal_mem_flops


def roofline_time_us(mem_bytes: float, flops: float, device: Device) -> dict:
    t_mem = mem_bytes / device.memory_bandwidth * 1e6
    t_cmp = flops / device.peak_performance * 1e6
    return {"t_mem_us": t_mem, "t_cmp_us": t_cmp, "roofline_us": max(t_mem, t_cmp), "bound": "hbm" if t_mem >= t_cmp else "tensor",
            "intensity": flops / mem_bytes}
