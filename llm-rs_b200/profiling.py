"""Where a step's time goes: every kernel class timed with CUDA events, with the bytes it has to move and the
flops it has to do, and what fraction of the device's peaks that is.

The reference's counterpart is its tracing (``RUST_LOG``, the dump of the first operators of a pass,
llm-core/src/backends/candle.rs:1102-1109) and the timings its command-line tools print
(llm-cli/src/bin/run_model.rs:131-150). Here ``Profiler`` wraps the kernel entry points of ``ops`` while it is
active: every call is bracketed by two CUDA events on the launching stream and by an NVTX range (so that a
timeline tool shows the same names), and classed by kernel and shape. It is meant for eager steps (a replayed
CUDA graph launches nothing through ``ops``): the callers switch graphs off while they profile. Timings taken
this way are serialised launch by launch; they show shares and per-kernel rooflines, not the step's time.

    with Profiler(hbm_gbs=6550, tflops=1660) as prof:
        runner.step(entries)
    print(prof.report())
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Tuple

import torch

from . import ops


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if isinstance(t, torch.Tensor))


# What each wrapped entry point must read and write at the least (bytes) and compute (flops), from its arguments.
def _cost_gemm(x, w, *a, **k) -> Tuple[str, int, float]:
    tokens, K = x.shape
    n = w.size(0)
    width = n // 2 if k.get("epilogue") == "silu_mul" else n
    return f"{n}x{K}", _nbytes(x, w) + tokens * width * 2, 2.0 * tokens * n * K


def _cost_qkv(x, w, q_out, *a, **k):
    tokens, K = x.shape
    return f"{w.size(0)}x{K}", _nbytes(x, w) + tokens * w.size(0) * 2, 2.0 * tokens * w.size(0) * K


def _cost_gemm_f32(x, w, *a, **k):
    return f"{w.size(0)}x{w.size(1)}", _nbytes(x, w) + x.size(0) * w.size(0) * 4, 2.0 * x.size(0) * w.size(0) * w.size(1)


def _cost_library(x, w, *a, **k):
    return f"{w.size(0)}x{w.size(1)}", _nbytes(x, w) + x.size(0) * w.size(0) * 2, 2.0 * x.size(0) * w.size(0) * w.size(1)


def _cost_attn_decode(q, out, cache, dec_reqs, n_dec, q_start, cached_len, block_table, scratch, max_splits, split_keys,
                      n_q_heads, n_kv_heads, head_dim, page_size, window, scale, **k):
    # The keys are counted on the device and read when the report is made: a read here would make the host wait for
    # the device, and the next launch's preparation on the host would then show up as that kernel's time.
    keys = (cached_len[dec_reqs[:n_dec].long()] + 1).clamp(max=window if window > 0 else 1 << 30).sum()
    per_key, fixed = 2 * n_kv_heads * head_dim * cache.element_size(), _nbytes(q, out)
    return (f"{n_dec} requests", lambda: int(keys) * per_key + fixed, lambda: 4.0 * int(keys) * n_q_heads * head_dim)


def _cost_attn_prefill(q, out, cache, tiles, n_tiles, q_start, n_new, cached_len, block_table, n_q_heads, n_kv_heads,
                       head_dim, page_size, window, scale, **k):
    n, c = n_new.double(), cached_len.double()
    pairs = (n * c + n * (n + 1) / 2).sum()             # (query, key) pairs a causal portion sees
    keys, tokens = (n + c).sum(), int(q.size(0))
    per_key, fixed = 2 * n_kv_heads * head_dim * cache.element_size(), _nbytes(q, out)
    return (f"{tokens} tokens", lambda: int(float(keys) * per_key) + fixed,
            lambda: 4.0 * float(pairs) * n_q_heads * head_dim)


def _cost_rows(*tensors_from):
    def cost(*a, **k):
        ts = [a[i] for i in tensors_from if i < len(a) and isinstance(a[i], torch.Tensor)]
        return "", 2 * _nbytes(*ts), 0.0
    return cost


WRAPPED: Dict[str, Callable] = {
    "gemm_bf16": _cost_gemm, "gemm_qkv_rope": _cost_qkv, "gemm_f32": _cost_gemm_f32, "library_gemm": _cost_library,
    "attn_decode": _cost_attn_decode, "attn_prefill": _cost_attn_prefill,
    "add_rmsnorm": _cost_rows(0), "embedding": lambda table, ids, *a, **k: ("", ids.numel() * table.size(1) * (table.element_size() + 4), 0.0),
    "silu_mul": _cost_rows(0), "qk_norm_rope_kvwrite": _cost_rows(0, 1, 2), "residual_add": _cost_rows(0, 1),
    "argmax": _cost_rows(0), "sample": _cost_rows(0), "scatter_tokens": _cost_rows(0),
}


def device_peaks() -> Tuple[float, float]:
    """(GB/s, TFLOP/s) to report against: what a file MEASURED_PEAKS.json in the working directory or beside the
    package says (keys hbm_gbs, bf16_tflops), else the nominal figures of a B200 (7,700 GB/s, 2,250 TFLOP/s)."""
    import json
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    for path in ("MEASURED_PEAKS.json", os.path.join(here, "..", "MEASURED_PEAKS.json")):
        try:
            with open(path) as f:
                m = json.load(f)
            return float(m["hbm_gbs"]), float(m["bf16_tflops"])
        except (OSError, ValueError, KeyError):
            continue
    return 7700.0, 2250.0


class Profiler:
    """Times every call of the wrapped ``ops`` entry points while active (see the module's head)."""

    def __init__(self, hbm_gbs: float, tflops: float, nvtx: bool = True):
        self.hbm_gbs, self.tflops, self.nvtx = float(hbm_gbs), float(tflops), nvtx
        self._saved: Dict[str, Callable] = {}
        self._calls: List[tuple] = []      # (class, bytes, flops, start event, end event); bytes and flops may be callables

    def __enter__(self):
        for name, cost in WRAPPED.items():
            real = getattr(ops, name)
            self._saved[name] = real
            setattr(ops, name, self._wrap(name, real, cost))
        return self

    def __exit__(self, *exc):
        for name, real in self._saved.items():
            setattr(ops, name, real)
        self._saved.clear()
        return False

    def _wrap(self, name, real, cost):
        def timed(*a, **k):
            label, nbytes, flops = cost(*a, **k)
            if name == "gemm_bf16" and k.get("epilogue", "store") != "store":
                label += " " + k["epilogue"]
            cls = f"{name}[{label}]" if label else name
            if self.nvtx:
                torch.cuda.nvtx.range_push(cls)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            try:
                return real(*a, **k)
            finally:
                end.record()
                if self.nvtx:
                    torch.cuda.nvtx.range_pop()
                self._calls.append((cls, nbytes, flops, start, end))
        return timed

    def classes(self) -> List[dict]:
        """Per kernel class: calls, total and mean microseconds, bytes and flops per call, achieved GB/s and
        TFLOP/s and the larger of the two fractions of peak (which bound applies)."""
        torch.cuda.synchronize()
        agg: Dict[str, List[float]] = {}
        for cls, nbytes, flops, start, end in self._calls:
            a = agg.setdefault(cls, [0, 0.0, 0.0, 0.0])
            a[0] += 1
            a[1] += start.elapsed_time(end) * 1e3
            a[2] += int(nbytes() if callable(nbytes) else nbytes)      # (counted on the device: see _cost_attn_decode)
            a[3] += float(flops() if callable(flops) else flops)
        total = sum(a[1] for a in agg.values()) or 1.0
        rows = []
        for cls, (n, us, nbytes, flops) in agg.items():
            gbs, tf = nbytes / us / 1e3, flops / us / 1e6
            f_mem, f_math = gbs / self.hbm_gbs, tf / self.tflops
            rows.append({"class": cls, "calls": n, "us_total": round(us, 1), "us_each": round(us / n, 2),
                         "share": round(us / total, 4), "bytes_each": int(nbytes / n), "flops_each": flops / n,
                         "gb_s": round(gbs, 1), "tflop_s": round(tf, 2), "bound": "hbm" if f_mem >= f_math else "tensor",
                         "frac": round(max(f_mem, f_math), 4)})
        return sorted(rows, key=lambda r: -r["us_total"])

    def report(self) -> str:
        rows = self.classes()
        lines = [f"{'share':>6} {'us total':>10} {'calls':>6} {'us each':>9} {'MB each':>9} {'GFLOP each':>11} "
                 f"{'GB/s':>8} {'TFLOP/s':>8} {'of peak':>8}  kernel class",
                 f"(peaks: {self.hbm_gbs:.0f} GB/s, {self.tflops:.0f} TFLOP/s; serialised launches, CUDA events: where the "
                 f"device waited for the host to prepare a launch, that wait counts, so kernels of tens of us read high)"]
        for r in rows:
            lines.append(f"{100 * r['share']:5.1f}% {r['us_total']:10.1f} {r['calls']:6d} {r['us_each']:9.2f} "
                         f"{r['bytes_each'] / 1e6:9.2f} {r['flops_each'] / 1e9:11.3f} {r['gb_s']:8.1f} {r['tflop_s']:8.2f} "
                         f"{r['frac']:7.3f}{'m' if r['bound'] == 'hbm' else 't'}  {r['class']}")
        return "\n".join(lines)
