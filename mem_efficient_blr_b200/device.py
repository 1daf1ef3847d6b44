"""Device table for the roofline model; the reference's Device (device.py:1-24) plus a B200 entry."""
from __future__ import annotations

import json
import os

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Device:
    def __init__(self, name: str):
        self.name = name
        if name == "A40":                       # device.py:5-7
            self.memory_bandwidth = 696 * 2 ** 30
            self.peak_performance = 149.7e12
        elif name == "Jetson Orin Nano 8GB":    # device.py:8-10
            self.memory_bandwidth = 68.29 * 2 ** 30
            self.peak_performance = 10e12
        elif name == "B200":
            # nominal: 7.7 TB/s HBM3e, 2.25 PFLOP/s dense bf16; replaced by the figures measured on the
            # machine (MEASURED_PEAKS.json at the repository root) when that file is present
            self.memory_bandwidth = 7.7e12
            self.peak_performance = 2.25e15
            try:
                with open(os.path.join(_ROOT, "MEASURED_PEAKS.json")) as f:
                    m = json.load(f)
                self.memory_bandwidth = float(m["hbm_gbs"]) * 1e9
                self.peak_performance = float(m["bf16_tflops"]) * 1e12
                self.measured = True
            except Exception:
                self.measured = False
        else:
            raise ValueError("Name not supported in Device class")
        self.break_point = self.peak_performance / self.memory_bandwidth

    def __repr__(self):
        return (f"Device {self.name}: {self.memory_bandwidth / 1e9:.1f} GB/s, {self.peak_performance / 1e12:.1f} TFLOP/s, "
                f"break point {self.break_point:.1f} FLOP/B")
