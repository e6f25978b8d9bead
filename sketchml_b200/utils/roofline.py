"""Roofline arithmetic against the measured peaks of this machine pool."""
from __future__ import annotations

import json
import os
from pathlib import Path

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
NVLINK_GBS_MEASURED = 770.0   # peer copy, per direction per GPU
NVLINK_GBS_NOMINAL = 900.0


def load_peaks() -> dict:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        d["source"] = "measured"
        return d
    return dict(FALLBACK)


def roofline_fraction(hbm_bytes: float, seconds: float, nvlink_bytes: float = 0.0) -> dict:
    """Achieved fraction of the slower of (HBM bytes at the measured copy bandwidth) and
    (bytes that must cross NVLink at the measured per-direction link bandwidth)."""
    peaks = load_peaks()
    t_hbm = hbm_bytes / (peaks["hbm_gbs"] * 1e9)
    t_link = nvlink_bytes / (NVLINK_GBS_MEASURED * 1e9)
    target = max(t_hbm, t_link)
    return {"target_s": target, "achieved_s": seconds, "fraction": target / seconds if seconds > 0 else 0.0,
            "bound": "nvlink" if t_link > t_hbm else "hbm", "denominator": peaks["source"],
            "hbm_gbs_achieved": hbm_bytes / seconds / 1e9 if seconds > 0 else 0.0}
