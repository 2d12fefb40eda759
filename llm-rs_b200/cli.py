"""Command line in the manner of the reference's binaries.

``run_model`` (llm-cli/src/bin/run_model.rs:9-35) takes --model-path, --prompt,
--temperature (0.0), --top-p (1.0), --repetition-penalty (1.0) and prints time to first
token, prefill and decode tokens per second (run_model.rs:131-150); ``benchmark_speed``
(llm-cli/src/bin/benchmark_speed.rs:9-26) adds --max-new-tokens (50). Both exist here
with those names, meanings and defaults. Prompts are token ids (--prompt-ids, or a
random prompt of --prompt-len tokens): the engine depends on no tokenizer, so
--tokenizer-path and a text --prompt are accepted only where the ``tokenizers`` package
and a tokenizer file are at hand. ``random_model`` writes a model folder with random
weights from a config.json and a seed.

    python -m llm_rs_b200.cli run_model --model-path DIR --prompt-ids 1,2,3
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List


def _prompt_ids(args, vocab: int) -> List[int]:
    if args.prompt_ids:
        return [int(t) for t in args.prompt_ids.split(",") if t.strip()]
    if args.prompt is not None and args.tokenizer_path:
        try:
            from tokenizers import Tokenizer
        except ImportError:
            raise SystemExit("--prompt needs the `tokenizers` package; pass --prompt-ids instead")
        return Tokenizer.from_file(args.tokenizer_path).encode(args.prompt).ids
    import numpy as np
    rng = np.random.default_rng(args.prompt_seed)
    return rng.integers(0, vocab, args.prompt_len).tolist()


def _add_common(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model-path", required=True, help="folder with config.json and *.safetensors")
    p.add_argument("--tokenizer-path", default=None, help="tokenizer.json (optional; only for --prompt text)")
    p.add_argument("--prompt", default=None, help="prompt text (needs --tokenizer-path)")
    p.add_argument("--prompt-ids", default=None, help="prompt as comma-separated token ids")
    p.add_argument("--prompt-len", type=int, default=16, help="length of a random prompt when no prompt is given")
    p.add_argument("--prompt-seed", type=int, default=0)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--block-pool-size", type=int, default=1024, help="pages in the cache pool")
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--seed", type=int, default=0, help="seed of the sampler's draws")
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--profile", action="store_true", help="time every kernel class with CUDA events (steps launched "
                   "kernel by kernel instead of from CUDA graphs) and print their shares, bytes, flops and fractions "
                   "of the device's peaks after the run")


def _run(args, max_new_tokens: int, temperature: float, top_p: float, repetition_penalty: float, top_k: int = 0):
    from .engine import Engine, EngineConfig
    from .sampling import SamplingParams
    t0 = time.time()
    profile = getattr(args, "profile", False)
    engine = Engine(EngineConfig(model_path=args.model_path, block_pool_size=args.block_pool_size,
                                 page_size=args.page_size, dtype=args.dtype, cuda_graphs=not profile,
                                 async_steps=not profile))
    spec = engine.runner.spec
    print(f"Model loaded in {time.time() - t0:.2f}s (vocab_size: {spec.vocab_size}, hidden_dim: {spec.hidden_size})")
    prompt = _prompt_ids(args, spec.vocab_size)
    params = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k,
                            repetition_penalty=repetition_penalty, max_new_tokens=max_new_tokens,
                            seed=args.seed, ignore_eos=args.ignore_eos)
    import torch
    profiler = None
    if profile:
        from .profiling import Profiler, device_peaks
        profiler = Profiler(*device_peaks()).__enter__()
    rid = engine.add_request(prompt, params)
    start = time.time()
    first = last = None
    tokens: List[int] = []
    while engine.has_work():
        for r, tok, fin in engine.step():
            if r == rid and tok is not None:
                torch.cuda.synchronize()
                now = time.time()
                first = first or now
                last = now
                tokens.append(tok)
    if profiler is not None:
        profiler.__exit__(None, None, None)
        print(profiler.report())
    print("Generated token ids:", ",".join(str(t) for t in tokens))
    print(f"Finish reason: {engine.finish_reason(rid)}")
    if first is not None:
        ttft = first - start
        print(f"TTFT: {ttft * 1e3:.2f} ms")
        print(f"Prefill: {len(prompt) / max(ttft, 1e-9):.2f} tok/s ({len(prompt)} tokens)")
        if len(tokens) > 1:
            print(f"Decode: {(len(tokens) - 1) / max(last - first, 1e-9):.2f} tok/s ({len(tokens)} tokens)")
        print(f"Overall: {len(tokens) / max(last - start, 1e-9):.2f} tok/s")
    return tokens


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llm_rs_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    p = sub.add_parser("run_model", help="generate from one prompt and print timings")
    _add_common(p)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--repetition-penalty", type=float, default=1.0)
    p.add_argument("--max-new-tokens", type=int, default=50)

    p = sub.add_parser("benchmark_speed", help="greedy generation of --max-new-tokens tokens with timings")
    _add_common(p)
    p.add_argument("--max-new-tokens", type=int, default=50)

    p = sub.add_parser("random_model", help="write a model folder with random weights")
    p.add_argument("--config", required=True, help="a config.json of a registered architecture")
    p.add_argument("--out", required=True, help="folder to write config.json and model.safetensors into")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--sigma", type=float, default=0.02, help="standard deviation of matrices and embeddings")
    p.add_argument("--norm-jitter", type=float, default=0.0, help="norm weights are 1 + N(0, this)")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")

    args = ap.parse_args(argv)
    if args.command == "run_model":
        _run(args, args.max_new_tokens, args.temperature, args.top_p, args.repetition_penalty, args.top_k)
    elif args.command == "benchmark_speed":
        _run(args, args.max_new_tokens, 0.0, 1.0, 1.0)
    elif args.command == "random_model":
        import torch
        from .config import resolve_architecture
        from .weights import write_random_model
        with open(args.config) as f:
            raw = json.load(f)
        cfg = resolve_architecture(raw).config_cls.from_dict(raw)
        write_random_model(args.out, cfg, seed=args.seed, sigma=args.sigma, norm_jitter=args.norm_jitter,
                           dtype=getattr(torch, args.dtype))
        print(f"wrote {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
