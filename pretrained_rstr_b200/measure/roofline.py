"""Peaks, clocks and the arithmetic of the rooflines.

Peaks come from ``MEASURED_PEAKS.json`` beside ``bench.py`` when that file exists (a copy
bandwidth and a cuBLAS bf16 rate measured on the machine), else from an earlier
measurement on the same kind of GPU; the record says which ("measured" or "fallback")."""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import threading

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SMALL = dict(n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257, n_positions=1024)
SIZES = {
    "small": SMALL,
    "medium": dict(n_layer=24, n_embd=1024, n_head=16, n_inner=4096, vocab_size=50257, n_positions=1024),
    "xl": dict(n_layer=48, n_embd=1600, n_head=25, n_inner=6400, vocab_size=50257, n_positions=1024),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as fh:
                raw = json.load(fh)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self.index = index

    def _run(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                     "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(float(parts[0]))
                    self.max_mhz = float(parts[1])
                    for name, val in zip(names, parts[2:6]):
                        if val.lower().startswith("active"):
                            self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def model_bytes(cfg, dtype_bytes=2):
    d, f, L, V = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"], cfg["vocab_size"]
    per_layer = (d * 3 * d + d * d + d * f + f * d) * dtype_bytes + (3 * d + d + f + d + 4 * d) * 4
    return L * per_layer + V * d * dtype_bytes + 2 * d * 4


def kv_bytes_per_token(cfg, dtype_bytes=2):
    return 2 * cfg["n_layer"] * cfg["n_embd"] * dtype_bytes


def prefill_flops(cfg, n_prompts, prompt_len):
    d, f, L, V = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"], cfg["vocab_size"]
    t = n_prompts * prompt_len
    gemm = 2 * t * (d * 3 * d + d * d + 2 * d * f) * L
    attn = L * n_prompts * 4 * d * (prompt_len * (prompt_len + 1) // 2)
    head = 2 * n_prompts * d * V
    return gemm + attn + head




def quantiles(ms):
    """min / median / p95 / max of a series, the reference's own summary of a run
    (``src/pretrained/continuation/benchmark.clj:180-224``)."""
    if not ms:
        return None
    s = sorted(ms)
    p95 = s[min(len(s) - 1, int(round(0.95 * (len(s) - 1))))]
    return {"min": round(s[0], 4), "median": round(statistics.median(s), 4), "p95": round(p95, 4),
            "max": round(s[-1], 4), "n": len(s)}
