"""Replay on the GPU against the plain implementation: whole, tail one by one, portions
of changing size, and mixed batches with so few pages that they are used again; in
float32 and in bfloat16; for three tiny configurations and one with heads of 128 elements (at
two page sizes), the size at which the bfloat16 engine takes its tcgen05 kernels."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as RU
from tiny_configs import TINY, write_tiny_model

pytestmark = pytest.mark.gpu

# float32: the engine and the float64 plain implementation differ by float32 rounding only.
TOL_F32 = 1e-4
# bfloat16: activations between kernels carry 8 bits of mantissa; measured differences on
# these models are a few 1e-3 of the logits' spread, so 2 % of the largest logit is a
# bound that a wrong key, page or position (errors of the order of the logits) cannot meet.
TOL_BF16_REL = 0.02

LENGTHS = {"A": [5, 17, 33, 64, 100, 161], "B": [1, 9, 40, 77, 128, 200], "C": [3, 30, 48, 65, 97, 150],
           "D": [40, 130, 300, 520, 257], "E": [40, 130, 300, 520, 257], "F": [2, 19, 70, 131, 260],
           "G": [4, 31, 66, 129, 200]}
MODES = ["whole", "tail", "portions", "mixed"]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    folder = tmp_path_factory.mktemp("models")
    out = {}
    for name in TINY:
        path = write_tiny_model(name, str(folder))
        cfg, w = P.load_model_dir(path)
        rng = np.random.default_rng(100 + ord(name))
        reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate(LENGTHS[name])}
        ref = {r: P.forward(cfg, w, toks).numpy() for r, toks in reqs.items()}
        out[name] = (path, cfg, reqs, ref)
    return out


def _steps(mode, reqs):
    return {"whole": RU.whole, "tail": RU.tail_one_by_one, "portions": RU.portions, "mixed": RU.mixed}[mode](reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", list(TINY))
def test_replay_matches_plain(models, name, mode, dtype):
    from llm_rs_b200.engine import ModelRunner
    path, cfg, reqs, ref = models[name]
    steps = _steps(mode, reqs)
    page = TINY[name][3]
    runner = ModelRunner.from_model_dir(path, dtype=getattr(torch, dtype), max_tokens=RU.live_token_peak(steps),
                                        page_size=page, max_requests=4)
    used_before = runner.manager.free_pages(0)
    got = RU.run_steps(runner, steps)
    assert runner.manager.free_pages(0) == used_before, "pages were lost"
    worst, where, n = RU.max_diff(got, ref)
    assert n == sum(len(t) for t in reqs.values())
    scale = max(float(np.abs(r).max()) for r in ref.values())
    tol = TOL_F32 if dtype == "float32" else TOL_BF16_REL * scale
    assert worst <= tol, f"{name} {mode} {dtype}: max |diff| {worst:.3e} at {where} (tolerance {tol:.3e})"


@pytest.mark.parametrize("name", ["A", "C"])
def test_pages_are_used_again(models, name):
    """In the mixed trace the pool is so small that later requests get pages that earlier ones held."""
    from llm_rs_b200.engine import ModelRunner
    path, cfg, reqs, ref = models[name]
    steps = RU.mixed(reqs)
    runner = ModelRunner.from_model_dir(path, dtype=torch.float32, max_tokens=RU.live_token_peak(steps),
                                        page_size=TINY[name][3], max_requests=4)
    seen, reused = {}, False
    from llm_rs_b200.engine import StepEntry
    for st in steps:
        runner.step([StepEntry(e["id"], e["tokens"], []) for e in st["entries"]])
        for e in st["entries"]:
            for page in runner.manager.table(e["id"], 0):
                if page >= 0 and seen.setdefault(page, e["id"]) != e["id"]:
                    reused = True
        for r in st["end"]:
            runner.release(r)
    assert reused


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    """bin/trace_run end to end: the JSON protocol, the files it writes, 'done' lines."""
    path, cfg, reqs, ref = models["B"]
    steps = RU.mixed(reqs, seed=3)
    out_dir = tmp_path / "out"
    lines = [json.dumps({"step": i, **st}) for i, st in enumerate(steps)]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", dtype,
         "--out", str(out_dir), "--max-tokens", str(RU.live_token_peak(steps)), "--page-size", "16"],
        input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    at, worst = {}, 0.0
    V = cfg["vocab_size"]
    for i, st in enumerate(steps):
        data = np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(-1, V)
        k = 0
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                worst = max(worst, float(np.abs(data[k] - ref[e["id"]][base + w]).max()))
                k += 1
            at[e["id"]] = base + len(e["tokens"])
        assert k == data.shape[0]
    scale = max(float(np.abs(r).max()) for r in ref.values())
    assert worst <= (TOL_F32 if dtype == "float32" else TOL_BF16_REL * scale), worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [11, 12, 13])
@pytest.mark.parametrize("name", ["C", "D", "E", "F"])
def test_mixed_replay_with_other_cuts(models, name, seed, dtype):
    """The mixed trace again with other seeds, portion sizes from 2 to 300 tokens (longer than C's window, long
    enough for the tcgen05 attention of D and E), other tail lengths and two or three live requests."""
    from llm_rs_b200.engine import ModelRunner
    path, cfg, reqs, ref = models[name]
    rng = np.random.default_rng(seed)
    sizes = tuple(int(x) for x in rng.choice([2, 3, 7, 16, 31, 33, 64, 65, 128, 129, 200, 300], size=6, replace=False))
    steps = RU.mixed(reqs, seed=seed, max_live=int(rng.integers(2, 5)), decode_tail=int(rng.integers(1, 40)), sizes=sizes)
    runner = ModelRunner.from_model_dir(path, dtype=getattr(torch, dtype), max_tokens=RU.live_token_peak(steps),
                                        page_size=TINY[name][3], max_requests=4)
    runner.use_graphs = bool(seed % 2)
    got = RU.run_steps(runner, steps)
    worst, where, n = RU.max_diff(got, ref)
    assert n == sum(len(t) for t in reqs.values())
    scale = max(float(np.abs(r).max()) for r in ref.values())
    tol = TOL_F32 if dtype == "float32" else TOL_BF16_REL * scale
    assert worst <= tol, f"{name} seed {seed} sizes {sizes} {dtype}: max |diff| {worst:.3e} at {where} (tolerance {tol:.3e})"
    assert all(p.free_pages() == p.capacity for p in runner.manager.pools)
