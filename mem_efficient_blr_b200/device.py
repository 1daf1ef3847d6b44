"""Device table for the roofline model; the reference's Device (device.py:1-24) plus a B200 entry."""
from __future__ import annotations


class Device:
    """`memory_bandwidth` (bytes/s) and `peak_performance` (FLOP/s) override the table entry, e.g. with figures
    measured on the machine at hand (a STREAM-style copy and a dense bf16 GEMM)."""

    def __init__(self, name: str, memory_bandwidth: float | None = None, peak_performance: float | None = None):
        self.name = name
        if name == "A40":                       # device.py:5-7
            self.memory_bandwidth = 696 * 2 ** 30
            self.peak_performance = 149.7e12
        elif name == "Jetson Orin Nano 8GB":    # device.py:8-10
            self.memory_bandwidth = 68.29 * 2 ** 30
            self.peak_performance = 10e12
        elif name == "B200":                    # nominal: 7.7 TB/s HBM3e, 2.25 PFLOP/s dense bf16
            self.memory_bandwidth = 7.7e12
            self.peak_performance = 2.25e15
        else:
            raise ValueError("Name not supported in Device class")
        self.measured = memory_bandwidth is not None or peak_performance is not None
        if memory_bandwidth is not None:
            self.memory_bandwidth = float(memory_bandwidth)
        if peak_performance is not None:
            self.peak_performance = float(peak_performance)
        self.break_point = self.peak_performance / self.memory_bandwidth

    def __repr__(self):
        return (f"Device {self.name}: {self.memory_bandwidth / 1e9:.1f} GB/s, {self.peak_performance / 1e12:.1f} TFLOP/s, "
                f"break point {self.break_point:.1f} FLOP/B")
