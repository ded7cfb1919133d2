"""The device limits a profile is read against.

Measured on the machine where one was taken (a plain copy's bytes per second, the library matrix
product's bfloat16 rate in a burst and sustained), from a JSON file named by ``ROCML_B200_PEAKS`` or
lying at the root of the checkout as ``MEASURED_PEAKS.json``; otherwise an earlier measurement of a
B200, marked as a fallback.  The reference keeps its two constants in source
(rocml/src/profile/roofline.rs:15,42); a measured file is used here because one is at hand.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# 148 multiprocessors x 128 fused multiply-adds a clock x 2 x 1.965 GHz: the CUDA cores' nominal
# 32-bit rate (nobody measured it here; the 32-bit path is read against it)
NOMINAL_F32_TFLOPS = 74.4


@dataclass(frozen=True)
class Peaks:
    hbm_gbs: float
    bf16_tflops: float
    bf16_tflops_sustained: float
    f32_tflops: float
    source: str                 # "measured" or "fallback"

    def flops_per_sec(self, dtype: str, sustained: bool = False) -> float:
        if dtype == "float32":
            return self.f32_tflops * 1e12
        return (self.bf16_tflops_sustained if sustained else self.bf16_tflops) * 1e12

    @property
    def bytes_per_sec(self) -> float:
        return self.hbm_gbs * 1e9


def load_peaks(path: Optional[str] = None) -> Peaks:
    here = os.path.dirname(os.path.abspath(__file__))
    candidates = [path, os.environ.get("ROCML_B200_PEAKS"),
                  os.path.join(os.path.dirname(os.path.dirname(here)), "MEASURED_PEAKS.json")]
    for cand in candidates:
        if cand and os.path.isfile(cand):
            try:
                with open(cand) as f:
                    d = json.load(f)
                burst = float(d["bf16_tflops"])
                return Peaks(float(d["hbm_gbs"]), burst, float(d.get("bf16_tflops_sustained", burst)),
                             NOMINAL_F32_TFLOPS, "measured")
            except (OSError, ValueError, KeyError, TypeError):
                continue
    return Peaks(FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, 1400.0, NOMINAL_F32_TFLOPS, "fallback")
