#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second and prefill throughput
at the layer sizes of Qwen3-8B with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--context C]

A "step" is one decode step of the whole batch. The default is batch 8 at a context of
4,096 tokens per request. One JSON line is printed:

  value          decoded tokens per second, timed on the device with CUDA events around K
                 steps of the step function (given tokens, no host round trip per step)
  e2e            the same through ``Engine.step()``: every step copies that step's index
                 arrays from pinned host memory and reads the sampled tokens back
  prefill        one prompt of 2,048 tokens: tokens/s, milliseconds, fraction of the
                 bf16 peak (flops of the step / time / peak)
  roofline       decode: bytes the step must read (every weight once, the cache of the
                 live requests) / time, against the measured HBM copy bandwidth
  points         decode tokens per second at batch 1 and 64

The K timed steps run back to back as five runs of K/5 steps with a CUDA event between them: ``value`` and
``ms_per_step`` are the median run's, ``repeats`` gives the runs' spread and the mean over all K steps.
Fractions are given against two denominators: the peaks measured on this pool (MEASURED_PEAKS.json beside
this file when present, else 6.65 TB/s and 1.59 PFLOP/s) and the nominal figures of the part (7.7 TB/s,
2.25 PFLOP/s dense bf16). Only N = 1 is supported: the engine is a single-GPU engine.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=False,
    max_position_embeddings=40960, hidden_act="silu", eos_token_id=151645)
FULL_LAYERS = 36
PREFILL_TOKENS = 2048
# Two further workloads, run through the engine's public API from host token ids to host tokens
# (``--workload``): a mixed load on the layer sizes of Qwen3-14B and a memory stress on those of Qwen3-32B.
QWEN3_14B = dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
WORKLOADS = {
    "mixed14b": dict(model="Qwen3-14B shape", cfg=QWEN3_14B, seed=3, requests=32, prompt_lo=128, prompt_hi=3072,
                     new_tokens=256, temperature=0.8, prefill_chunk=512),
    "stress32b": dict(model="Qwen3-32B shape", cfg=QWEN3_32B, seed=4, requests=16, prompt_lo=8192, prompt_hi=8192,
                      new_tokens=512, temperature=0.0, prefill_chunk=512),
}


NOMINAL = {"hbm_gbs": 7700.0, "bf16_tflops": 2250.0}     # HBM3e of the HGX B200, dense bfloat16
REPEATS = 5


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    try:
        with open(path) as f:
            m = json.load(f)
        out["hbm_gbs"] = float(m.get("hbm_gbs", out["hbm_gbs"]))
        out["bf16_tflops"] = float(m.get("bf16_tflops", out["bf16_tflops"]))
        if "bf16_tflops_sustained" in m:
            out["bf16_tflops_sustained"] = float(m["bf16_tflops_sustained"])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            cols = [c.strip() for c in line.split(",")]
            if len(cols) < 7:
                continue
            try:
                sm.append(float(cols[0]))
                mx.append(float(cols[1]))
            except ValueError:
                continue
            for name, val in zip(names, cols[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_bytes_per_decode_step(cfg, n_layers, batch, context, kv_bytes=2, w_bytes=2):
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = ((nq + 2 * nkv) * d * H + H * nq * d + 3 * H * I) * w_bytes + (2 * H + 2 * d) * 4
    weights = n_layers * per_layer + V * H * w_bytes + H * 4 + batch * H * w_bytes
    cache = batch * context * 2 * nkv * d * kv_bytes * n_layers
    return weights + cache


def prefill_flops(cfg, n_layers, tokens):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer_params = (nq + 2 * nkv) * d * H + H * nq * d + 3 * H * I
    linear = 2.0 * tokens * n_layers * per_layer_params + 2.0 * V * H  # head on the last position only
    attention = 2.0 * tokens * tokens * nq * d * n_layers              # causal: half of 4*T^2*d per head
    return linear + attention


def run_workload(args):
    """A whole serving run through ``Engine``: requests in, tokens out, scheduler, chunked prefill
    beside decoding, sampling, preemption if the pool is made small. Prints one JSON line."""
    import numpy as np
    import torch
    import llm_rs_b200  # noqa: F401
    from llm_rs_b200 import ops
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import Engine, EngineConfig, ModelRunner
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import DecoderModel
    from llm_rs_b200.sampling import SamplingParams
    from llm_rs_b200.weights import random_tensors

    w = WORKLOADS[args.workload]
    torch.cuda.set_device(0)
    layers = args.layers if args.layers != FULL_LAYERS else w["cfg"]["num_hidden_layers"]
    raw = dict(w["cfg"], num_hidden_layers=layers)
    cfg = Qwen3Config.from_dict(raw)
    spec = build_spec(cfg)
    page = 16
    rng = np.random.default_rng(w["seed"])
    lens = rng.integers(w["prompt_lo"], w["prompt_hi"] + 1, w["requests"]).tolist()
    need_tokens = sum(-(-(n + w["new_tokens"]) // page) * page for n in lens)
    pool_tokens = args.pool_tokens or need_tokens + 64 * page
    t0 = time.time()
    tensors = random_tensors(DecoderModel(spec).weight_specs(), seed=w["seed"], sigma=0.02, dtype=torch.bfloat16,
                             device="cuda:0")
    runner = ModelRunner(spec, tensors, torch.bfloat16, "cuda:0", max_tokens=pool_tokens, page_size=page,
                         max_requests=w["requests"] + 1)
    del tensors
    torch.cuda.empty_cache()
    runner.use_graphs = not args.no_graphs
    print(f"[bench] {w['model']}: model on device in {time.time() - t0:.1f} s, "
          f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB allocated, pool of {pool_tokens} tokens "
          f"({need_tokens} needed to hold every request whole)", file=sys.stderr, flush=True)
    engine = Engine(EngineConfig(model_path="", block_pool_size=pool_tokens // page, page_size=page,
                                 max_requests=w["requests"] + 1, max_tokens_per_step=2048,
                                 prefill_chunk=w["prefill_chunk"], cuda_graphs=not args.no_graphs), runner=runner)
    sp = SamplingParams(temperature=w["temperature"], max_new_tokens=w["new_tokens"], ignore_eos=True, seed=7)

    def run_once():
        for n in lens:
            engine.add_request(rng.integers(0, cfg.vocab_size, n).tolist(), sp)
        stats0 = dict(engine.stats)
        pre0 = engine.scheduler.stats["preemptions"]
        launches0 = ops.launch_count
        torch.cuda.synchronize()
        t_start = time.perf_counter()
        got, first = 0, None
        while engine.has_work():
            for _, tok, _ in engine.step():
                if tok is not None:
                    got += 1
                    if first is None:
                        first = time.perf_counter() - t_start
        torch.cuda.synchronize()
        dt = time.perf_counter() - t_start
        st = {k: engine.stats[k] - stats0[k] for k in stats0 if k != "max_step_tokens"}
        return dt, got, first, st, engine.scheduler.stats["preemptions"] - pre0, ops.launch_count - launches0

    cold = run_once()               # warm-up: graph captures, workspace, first-call set-up
    print(f"[bench] first run (with graph captures and first-call set-up): {cold[0]:.2f} s, "
          f"{len(runner._graphs)} captured steps", file=sys.stderr, flush=True)
    sampler = ClockSampler()
    sampler.start()
    dt, got, first, st, preempt, launches = run_once()
    clocks = sampler.stop()
    engine.check_kernels()
    runner.manager.check_invariants()
    result = {
        "metric": f"{w['model']} bf16 serving run: {w['requests']} requests, prompts {w['prompt_lo']}-{w['prompt_hi']} "
                  f"tokens, {w['new_tokens']} new tokens each",
        "value": round(got / dt, 2), "unit": "generated tokens/s", "n_gpus": 1, "impl": "ours", "dtype": "bf16",
        "data": f"synthetic: random weights (seed {w['seed']}), uniform-random token ids",
        "seconds": round(dt, 3), "generated_tokens": got, "prompt_tokens": int(sum(lens)),
        "all_tokens_per_s": round((got + sum(lens)) / dt, 1), "first_token_s": round(first or 0.0, 4),
        "steps": st, "preemptions": preempt, "gpu_launches_eager": launches,
        "config": {"model": w["model"], "layers": layers, "layers_full": w["cfg"]["num_hidden_layers"],
                   "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "requests": w["requests"], "pool_tokens": pool_tokens, "page_size": page,
                   "prefill_chunk": w["prefill_chunk"], "max_tokens_per_step": 2048,
                   "temperature": w["temperature"], "cuda_graphs": not args.no_graphs},
        "clocks": clocks,
    }
    print(json.dumps(result))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than 36 only where memory or time needs it")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="length of the timed prompt (the contract's figure is the default, 2,048)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step by itself "
                    "(for a profiler's launch list)")
    ap.add_argument("--profile", action="store_true", help="instead of the benchmark: time every kernel class of one "
                    "decode step and of the prefill with CUDA events (eager launches, NVTX ranges) and print a table "
                    "with bytes, flops and the fraction of the peaks to standard error, the rows as JSON to standard output")
    ap.add_argument("--workload", default="decode", choices=["decode", *WORKLOADS],
                    help="decode: the benchmark contract (default). mixed14b / stress32b: a whole serving run "
                    "through the engine on the layer sizes of Qwen3-14B / Qwen3-32B")
    ap.add_argument("--pool-tokens", type=int, default=0, help="size of the cache pool of a --workload run in "
                    "tokens (default: what holds every request whole); smaller makes the scheduler preempt")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "mashriram/llm-rs is a Rust workspace (cargo, candle, cubecl); no Rust toolchain or "
                          "vendored crates offline, pip cannot install it"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload != "decode":
        return run_workload(args)
    W = max(3, args.warmup)
    K = max(1, args.steps)

    import numpy as np
    import torch
    import llm_rs_b200
    from llm_rs_b200 import ops
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import Engine, EngineConfig, ModelRunner, StepEntry
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import DecoderModel
    from llm_rs_b200.sampling import SamplingParams
    from llm_rs_b200.weights import random_tensors

    torch.cuda.set_device(0)
    pk = peaks()
    raw = dict(QWEN3_8B, num_hidden_layers=args.layers)
    cfg = Qwen3Config.from_dict(raw)
    spec = build_spec(cfg)
    page = 16
    ctx = args.context
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    pool_tokens = max_batch * (ctx + 64) + args.prefill_tokens + 64
    t0 = time.time()
    tensors = random_tensors(DecoderModel(spec).weight_specs(), seed=2, sigma=0.02, dtype=torch.bfloat16,
                             device="cuda:0")
    runner = ModelRunner(spec, tensors, torch.bfloat16, "cuda:0", max_tokens=pool_tokens, page_size=page,
                         max_requests=max_batch + 1)
    del tensors
    torch.cuda.empty_cache()
    # Keys and values of the context are random numbers: the decode step reads the same bytes
    # whatever they hold, and random values keep the softmax from degenerating.
    for kv in runner.storage.kv:
        for i in range(kv.size(0)):
            kv[i].normal_(0.0, 1.0)
    runner.use_graphs = not args.no_graphs
    print(f"[bench] model on device in {time.time() - t0:.1f} s, "
          f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB allocated", file=sys.stderr, flush=True)
    rng = np.random.default_rng(0)
    V = cfg.vocab_size

    def fill_context(ids, n_tokens):
        """Give each request ``n_tokens`` of (random) cached context without running a prefill."""
        for rid in ids:
            runner.manager.admit(rid)
            runner.manager.reserve(rid, n_tokens)
            runner.manager.commit(rid, n_tokens)

    def timed_decode(batch, steps, warmup, sampler=None):
        ids = [f"d{batch}_{i}" for i in range(batch)]
        fill_context(ids, ctx - warmup - steps)
        toks = rng.integers(0, V, (warmup + steps, batch)).tolist()
        out = torch.empty((batch,), dtype=torch.int32, device="cuda:0")
        if sampler:
            sampler.start()       # nvidia-smi needs a moment to deliver its first sample
        for s in range(warmup):
            logits = runner.step([StepEntry(r, [toks[s][i]], [0]) for i, r in enumerate(ids)])
            ops.argmax(logits, out)
        torch.cuda.synchronize()
        launches0 = ops.launch_count
        # The steps run back to back; an event after every run of steps // REPEATS steps gives the runs' times.
        runs = min(REPEATS, steps)
        marks = [warmup + (steps * r) // runs for r in range(runs + 1)]
        events = [torch.cuda.Event(enable_timing=True) for _ in marks]
        events[0].record()
        at = 1
        for s in range(warmup, warmup + steps):
            logits = runner.step([StepEntry(r, [toks[s][i]], [0]) for i, r in enumerate(ids)])
            ops.argmax(logits, out)
            if s + 1 == marks[at]:
                events[at].record()
                at += 1
        torch.cuda.synchronize()
        clocks = sampler.stop() if sampler else None
        per_run = [events[r].elapsed_time(events[r + 1]) / (marks[r + 1] - marks[r]) for r in range(runs)]
        spread = {"runs": runs, "median_ms": round(statistics.median(per_run), 4), "min_ms": round(min(per_run), 4),
                  "max_ms": round(max(per_run), 4), "mean_ms": round(events[0].elapsed_time(events[-1]) / steps, 4)}
        for rid in ids:
            runner.release(rid)
        return statistics.median(per_run), clocks, ops.launch_count - launches0, spread

    # Kernels of ours in one captured decode step (a replay launches all of them again).
    def kernels_per_decode_step(batch):
        ids = [f"k{i}" for i in range(batch)]
        fill_context(ids, 64)
        runner.use_graphs = False
        n0 = ops.launch_count
        runner.step([StepEntry(r, [1], [0]) for r in ids])
        n = ops.launch_count - n0
        runner.use_graphs = not args.no_graphs
        for rid in ids:
            runner.release(rid)
        return n

    if args.profile:
        from llm_rs_b200.profiling import Profiler
        runner.use_graphs = False
        ids = [f"q{i}" for i in range(args.batch)]
        fill_context(ids, ctx - 8)
        step = lambda: ops.argmax(runner.step([StepEntry(r, [int(rng.integers(0, V))], [0]) for r in ids]))
        for _ in range(3):
            step()
        out = {}
        with Profiler(pk["hbm_gbs"], pk["bf16_tflops"]) as prof:
            for _ in range(3):
                step()
        print(f"[profile] decode step, batch {args.batch}, context {ctx}, {args.layers} layers (3 steps):\n" + prof.report(),
              file=sys.stderr)
        out["decode"] = prof.classes()
        for rid in ids:
            runner.release(rid)
        prompt = rng.integers(0, V, args.prefill_tokens).tolist()
        runner.step([StepEntry("p", prompt, [len(prompt) - 1])])
        runner.release("p")
        with Profiler(pk["hbm_gbs"], pk["bf16_tflops"]) as prof:
            runner.step([StepEntry("p", prompt, [len(prompt) - 1])])
        print(f"[profile] prefill of {len(prompt)} tokens:\n" + prof.report(), file=sys.stderr)
        out["prefill"] = prof.classes()
        print(json.dumps({"profile": out, "peaks": pk, "layers": args.layers, "batch": args.batch, "context": ctx}))
        return 0

    per_step_kernels = kernels_per_decode_step(args.batch)
    ms, clocks, eager_launches, spread = timed_decode(args.batch, K, W, ClockSampler())
    value = args.batch / (ms / 1e3)
    step_bytes = model_bytes_per_decode_step(raw, args.layers, args.batch, ctx)
    achieved = step_bytes / (ms / 1e3) / 1e9
    result = {
        "metric": "Qwen3-8B bf16 decode tok/s @ batch 8, context 4096 (random weights)",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 2), uniform-random token ids, random cache contents",
        "impl": "ours",
        "config": {
            "model": "Qwen3-8B shape", "layers": args.layers, "layers_full": FULL_LAYERS, "hidden": cfg.hidden_size,
            "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": args.batch,
            "seq_len": ctx, "page_size": page, "kv_dtype": "bf16", "parallelism": "single GPU",
            "cuda_graphs": not args.no_graphs, "l2": "inputs larger than L2 (weights 15 GB per step)",
            "peaks": pk["source"]},
        "clocks": clocks,
        # One replay of a captured step launches every kernel of the step; argmax is launched eagerly.
        "gpu_launches": (per_step_kernels * K if not args.no_graphs else 0) + eager_launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"],
                     "nominal_peak": NOMINAL["hbm_gbs"], "frac_nominal": round(achieved / NOMINAL["hbm_gbs"], 4)},
        "repeats": spread,
    }

    if not args.no_points:
        points = {}
        for b in (1, 64):
            try:
                ms_b, _, _, _ = timed_decode(b, max(10, K // 2), W)
                points[f"decode_b{b}"] = round(b / (ms_b / 1e3), 2)
            except Exception as e:  # a point that fails must not lose the headline
                points[f"decode_b{b}"] = None
                print(f"[bench] decode at batch {b} failed: {e}", file=sys.stderr)
        result["points"] = points

    if not args.no_prefill:
        try:
            n_prompt = args.prefill_tokens
            prompt = rng.integers(0, V, n_prompt).tolist()
            times = []
            for it in range(REPEATS + 1):        # the first run is warm-up; the median of the others counts
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                runner.step([StepEntry("p", prompt, [n_prompt - 1])])
                end.record()
                torch.cuda.synchronize()
                runner.release("p")
                if it >= 1:
                    times.append(start.elapsed_time(end))
            pms = statistics.median(times)
            fl = prefill_flops(raw, args.layers, n_prompt)
            result["prefill"] = {"value": round(n_prompt / (pms / 1e3), 1), "tokens": n_prompt,
                                 "ms": round(pms, 3), "min_ms": round(min(times), 3), "max_ms": round(max(times), 3),
                                 "frac": round(fl / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4), "of": pk["source"],
                                 "frac_sustained": round(fl / (pms / 1e3) / (pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) * 1e12), 4),
                                 "frac_nominal": round(fl / (pms / 1e3) / (NOMINAL["bf16_tflops"] * 1e12), 4)}
        except Exception as e:
            result["prefill"] = None
            print(f"[bench] prefill failed: {e}", file=sys.stderr)

    if not args.no_e2e:
        try:
            engine = Engine(EngineConfig(model_path="", block_pool_size=pool_tokens // page, page_size=page,
                                         max_requests=max_batch + 1, max_tokens_per_step=2048, prefill_chunk=512),
                            runner=runner)
            # Prompts are prefilled four at a time, so some requests start decoding several steps
            # before the others, and results are read one step late: give every request enough
            # tokens to decode through the whole timed region, inside the context length.
            # (the prompts of the whole batch take batch * context / 2048 steps to prefill)
            spare = -(-(args.batch * ctx) // 2048) + 2 * (-(-(ctx) // 512)) + 8
            sp = SamplingParams(temperature=0.0, max_new_tokens=W + K + spare, ignore_eos=True)
            plen = ctx - (W + K + spare) - 2
            rids = [engine.add_request(rng.integers(0, V, plen).tolist(), sp) for _ in range(args.batch)]
            while any(engine.requests[r].remaining > 1 or not engine.requests[r].output for r in rids):
                engine.step()   # prefill of the prompts, not timed
            for _ in range(W):
                engine.step()
            torch.cuda.synchronize()
            h2d0, d2h0 = runner.h2d_bytes, engine.d2h_bytes
            graphs0, pre0 = len(runner._graphs), engine.scheduler.stats["preemptions"]
            t_start = time.perf_counter()
            got = 0
            for _ in range(K):
                got += sum(1 for _, tok, _ in engine.step() if tok is not None)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t_start
            print(f"[bench] e2e: {got} tokens in {K} steps, {len(runner._graphs) - graphs0} graphs captured and "
                  f"{engine.scheduler.stats['preemptions'] - pre0} preemptions inside the timed region",
                  file=sys.stderr, flush=True)
            result["e2e"] = {"value": round(got / dt, 2), "unit": "tokens/s",
                             "h2d_bytes_per_step": (runner.h2d_bytes - h2d0) // K,
                             "d2h_bytes_per_step": (engine.d2h_bytes - d2h0) // K, "ms_per_step": round(dt / K * 1e3, 4)}
            while engine.has_work():
                engine.step()
        except Exception as e:
            result["e2e"] = None
            print(f"[bench] e2e failed: {e}", file=sys.stderr)

    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
