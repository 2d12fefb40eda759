"""Schedules that the replay tests do not reach, each against the plain implementation: decode steps of 17
to 64 requests with CUDA graphs (the products leave the few-token kernel, the keys are cut into two waves
or into more splits than a cluster merges), mixed steps whose prompt portions are long enough for the
tcgen05 attention kernel, preemption in bfloat16 and with a window group under graphs, and requests
that end at an EOS token while the next step is already queued."""
import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as RU
from tiny_configs import TINY, write_tiny_model

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    folder = str(tmp_path_factory.mktemp("models"))
    out = {}
    for name in ("A", "C", "D", "E"):
        path = write_tiny_model(name, folder)
        out[name] = (path, *P.load_model_dir(path))
    return out


def _tol(dtype, ref):
    return 1e-4 if dtype == torch.float32 else 0.02 * float(np.abs(ref).max())


# -- decode steps of many requests under graphs --------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name,batch,context,split_keys", [
    ("D", 17, 40, 0), ("D", 24, 700, 0), ("E", 64, 150, 0), ("E", 64, 500, 0), ("D", 3, 1900, 0), ("E", 20, 1000, 0),
    ("D", 3, 1900, 64),        # 30 splits: more than a cluster merges, so the second kernel combines them
    ("E", 33, 900, 128)])
def test_decode_steps_of_many_requests_with_graphs(models, name, batch, context, split_keys, dtype):
    """``batch`` requests (a few distinct sequences at different lengths, so the batch is ragged) decode 6
    tokens each, one step per token, graphs on. ``split_keys`` > 0 fixes the cut of the keys."""
    import dataclasses
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import ModelRunner, StepEntry
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import DecoderModel, PartSpec
    from llm_rs_b200.weights import load_weights
    path, cfg, w = models[name]
    page = TINY[name][3]
    rng = np.random.default_rng(batch * 1000 + context)
    n_dec = 6
    # A few distinct sequences (the plain forward is the slow part); requests cycle through them at
    # different lengths, so the batch is ragged.
    base = [rng.integers(0, cfg["vocab_size"], context + n_dec).tolist() for _ in range(3)]
    refs = [P.forward(cfg, w, s).numpy() for s in base]
    lens = [max(2, context - 7 * (r % 5)) for r in range(batch)]
    spec = build_spec(Qwen3Config.from_dict(cfg))
    if split_keys:
        spec = dataclasses.replace(spec, layers=tuple(
            dataclasses.replace(l, mixer=PartSpec(l.mixer.kind, {**l.mixer.params, "split_keys": split_keys}))
            for l in spec.layers))
    tensors = load_weights(path, DecoderModel(spec).weight_specs(), dtype, torch.device(DEV))
    runner = ModelRunner(spec, tensors, dtype, DEV, max_tokens=batch * (-(-(context + n_dec) // 64) * 64),
                         page_size=page, max_requests=batch)
    runner.use_graphs = True
    for r in range(batch):
        runner.step([StepEntry(r, base[r % 3][:lens[r]], [])])
    worst = 0.0
    for i in range(n_dec):
        rows = runner.step([StepEntry(r, [base[r % 3][lens[r] + i]], [0]) for r in range(batch)]).float().cpu().numpy()
        for r in range(batch):
            worst = max(worst, float(np.abs(rows[r] - refs[r % 3][lens[r] + i]).max()))
    assert runner._graphs, "the decode steps were not captured"
    tol = _tol(dtype, np.stack(refs))
    assert worst <= tol, (name, batch, context, dtype, worst, tol)
    from llm_rs_b200 import ops
    ops.check_tc_error(torch.device(DEV))
    ops.check_attention_error()


# -- long portions beside decode tokens -----------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["D", "E"])
def test_mixed_steps_with_long_portions(models, name, dtype, monkeypatch):
    """Portions of 128 to 300 tokens beside single decoded tokens of other requests: in bfloat16 the
    long portions take the tcgen05 attention kernel inside the mixed step (checked by counting)."""
    from llm_rs_b200 import ops
    from llm_rs_b200.engine import ModelRunner
    path, cfg, w = models[name]
    rng = np.random.default_rng(17)
    reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate((700, 450, 333, 900, 150, 520))}
    ref = {r: P.forward(cfg, w, t).numpy() for r, t in reqs.items()}
    steps = RU.mixed(reqs, seed=9, sizes=(128, 150, 200, 257, 300), decode_tail=20)
    assert any(len(e["tokens"]) >= 128 for st in steps for e in st["entries"]
               if any(len(o["tokens"]) == 1 for o in st["entries"]))
    took_tc, real = [], ops.attn_prefill
    monkeypatch.setattr(ops, "attn_prefill", lambda *a, **k: (took_tc.append(bool(k.get("prefer_tc"))), real(*a, **k))[1])
    runner = ModelRunner.from_model_dir(path, dtype=dtype, max_tokens=RU.live_token_peak(steps),
                                        page_size=TINY[name][3], max_requests=4)
    got = RU.run_steps(runner, steps)
    worst, where, n = RU.max_diff(got, ref)
    assert n == sum(len(t) for t in reqs.values())
    tol = _tol(dtype, np.concatenate(list(ref.values())))
    assert worst <= tol, (name, dtype, worst, where, tol)
    assert any(took_tc), "no step had portions long enough for the tcgen05 attention kernel"
    ops.check_attention_error()


# -- preemption -----------------------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", [("A", "bfloat16"), ("C", "float32"), ("C", "bfloat16"), ("D", "bfloat16")])
def test_preemption_in_bfloat16_and_with_a_window_group(models, name, dtype):
    """A pool too small for all requests at once, CUDA graphs on, steps queued ahead: requests are
    preempted and recomputed, and each still gets the tokens it would get alone."""
    from llm_rs_b200.engine import Engine, EngineConfig
    from llm_rs_b200.sampling import SamplingParams
    path, cfg, w = models[name]
    rng = np.random.default_rng(23)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (30, 41, 30, 25)]
    sp = SamplingParams(temperature=0.0, max_new_tokens=28, ignore_eos=True)
    e = Engine(EngineConfig(model_path=path, block_pool_size=9, page_size=16, dtype=dtype, max_requests=4,
                            max_tokens_per_step=64, prefill_chunk=32, cuda_graphs=True, async_steps=True))
    got = e.generate(prompts, sp)
    assert e.scheduler.stats["preemptions"] >= 1
    gap = 1e-4 if dtype == "float32" else 0.05
    for p, g in zip(prompts, got):
        assert len(g) == 28 and P.greedy_gap(cfg, w, p, g) < gap
    e.runner.manager.check_invariants()
    assert not e.runner.manager.requests
    assert all(e.runner.manager.free_pages(g) == 9 for g in range(len(e.runner.manager.groups)))


# -- EOS with a step queued ahead ------------------------------------------------------------------
@pytest.mark.parametrize("graphs", [False, True])
def test_requests_end_at_eos_under_async_steps(models, graphs, tmp_path):
    """The EOS id is chosen from the plain implementation's own greedy output, so every request is known to
    reach it; the engine (float32, steps queued one ahead) must stop there, emit the EOS token, drop the one
    token that was already in flight, and give every page back."""
    import json
    import os
    import shutil
    from llm_rs_b200.engine import Engine, EngineConfig
    from llm_rs_b200.sampling import SamplingParams
    path, cfg, w = models["A"]
    rng = np.random.default_rng(31)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (6, 19, 33)]
    plain = [P.greedy_generate(cfg, w, p, 14) for p in prompts]
    # The token that request 0 generates fifth ends every request that generates it.
    eos = plain[0][4]
    want = []
    for g in plain:
        want.append(g[:g.index(eos) + 1] if eos in g else g)
    assert len(want[0]) <= 5
    folder = str(tmp_path / "with_eos")
    shutil.copytree(path, folder)
    raw = json.load(open(os.path.join(folder, "config.json")))
    raw["eos_token_id"] = int(eos)
    json.dump(raw, open(os.path.join(folder, "config.json"), "w"))
    e = Engine(EngineConfig(model_path=folder, block_pool_size=32, page_size=16, dtype="float32", max_requests=4,
                            max_tokens_per_step=64, prefill_chunk=16, cuda_graphs=graphs, async_steps=True))
    ids = [e.add_request(p, SamplingParams(temperature=0.0, max_new_tokens=14)) for p in prompts]
    while e.has_work():
        e.step()
    for rid, g in zip(ids, want):
        assert e.requests[rid].output == g
        assert e.finish_reason(rid) == ("stop" if g[-1] == eos else "length")
    assert not e.runner.manager.requests and e.runner.manager.free_pages(0) == 32


# -- a kernel that gives up fails the step it is in ---------------------------------------------------
def test_kernel_error_surfaces_with_the_steps_tokens(models):
    """The tcgen05 product kernel is made to give up on a wait (its producer leaves out a copy, the limit is
    1,024 polls) during one decode step of a running engine: that step's call or the next raises, every
    running request ends with ``error_step_failed``, all pages come back, and the engine serves new requests
    afterwards with the right tokens."""
    from llm_rs_b200 import ops
    from llm_rs_b200.engine import Engine, EngineConfig
    from llm_rs_b200.sampling import SamplingParams
    path, cfg, w = models["D"]
    rng = np.random.default_rng(41)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (20, 33)]
    e = Engine(EngineConfig(model_path=path, block_pool_size=32, page_size=16, dtype="bfloat16", max_requests=4,
                            max_tokens_per_step=64, prefill_chunk=64, cuda_graphs=False, async_steps=True))
    ids = [e.add_request(p, SamplingParams(temperature=0.0, max_new_tokens=40, ignore_eos=True)) for p in prompts]
    for _ in range(4):
        e.step()
    assert all(e.requests[i].output for i in ids)
    ops.set_tc_wait_limit(1 << 10)
    ops.test_skip_copy(gemm_k_block=1)
    try:
        with pytest.raises(ops.KernelError, match="gave up waiting"):
            for _ in range(3):          # the failing step's tokens are read one call later
                e.step()
    finally:
        ops.test_skip_copy()
        ops.set_tc_wait_limit(0)
    torch.cuda.synchronize()
    ops.tc_error_flag(DEV).zero_()      # steps that were queued behind the failing one set it again
    assert all(e.finish_reason(i) == "error_step_failed" for i in ids)
    assert not e.runner.manager.requests and e.runner.manager.free_pages(0) == 32
    assert not e.has_work()
    got = e.generate([prompts[0]], SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True))[0]
    assert P.greedy_gap(cfg, w, prompts[0], got) < 0.05


# -- a model whose layers all look through a window: the pool does not bound the context --------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_all_window_model_runs_far_beyond_its_pool(models, dtype, tmp_path):
    """Every layer sees the last 24 keys only, so pages behind the window go back while the request runs: a
    sequence of 500 tokens runs through a pool of 160, in portions and then token by token."""
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import ModelRunner
    from llm_rs_b200.weights import write_random_model
    from tiny_configs import TINY_C
    raw = dict(TINY_C, use_sliding_window=True, sliding_window=24, max_window_layers=0, no_rope_layers=[False] * 4)
    path = write_random_model(str(tmp_path / "all_window"), Qwen3Config.from_dict(raw), seed=8, sigma=0.05, norm_jitter=0.1)
    cfg, w = P.load_model_dir(path)
    assert P.layer_windows(cfg) == [24] * 4
    toks = np.random.default_rng(3).integers(0, cfg["vocab_size"], 500).tolist()
    ref = {"a": P.forward(cfg, w, toks).numpy()}
    runner = ModelRunner.from_model_dir(path, dtype=dtype, max_tokens=160, page_size=16, max_requests=2)
    assert runner.max_positions == cfg["max_position_embeddings"] > 160
    steps = RU.portions({"a": toks[:300]}, sizes=(7, 2, 13, 5, 2, 31, 3, 17, 2, 64))
    steps[-1]["end"] = []
    steps += [{"entries": [{"id": "a", "tokens": [t], "want": [0]}], "end": []} for t in toks[300:]]
    steps[-1]["end"] = ["a"]
    got = RU.run_steps(runner, steps)
    worst, where, n = RU.max_diff(got, ref)
    assert n == 500
    assert worst <= _tol(dtype, ref["a"]), (worst, where)
    assert runner.manager.free_pages(0) == 10


# -- random workloads through the whole engine ------------------------------------------------------
@pytest.mark.parametrize("name,seed", [("A", 0), ("A", 1), ("C", 2), ("C", 3), ("D", 4)])
def test_random_workloads_through_the_engine(models, name, seed):
    """Requests of random lengths arrive while others run, in a pool so small that the scheduler preempts, with
    CUDA graphs and queued steps on: every request still gets exactly the greedy tokens of the plain
    implementation (float32), whatever was batched with it, preempted around it or recomputed."""
    from llm_rs_b200.engine import Engine, EngineConfig
    from llm_rs_b200.sampling import SamplingParams
    path, cfg, w = models[name]
    rng = np.random.default_rng(1000 + seed)
    n_req = 10
    prompts = [rng.integers(0, cfg["vocab_size"], int(rng.integers(1, 70))).tolist() for _ in range(n_req)]
    new = [int(rng.integers(1, 18)) for _ in range(n_req)]
    arrive = sorted(int(rng.integers(0, 25)) for _ in range(n_req))      # the engine step at which each is submitted
    e = Engine(EngineConfig(model_path=path, block_pool_size=12, page_size=16, dtype="float32", max_requests=4,
                            max_tokens_per_step=int(rng.choice([24, 40, 64])), prefill_chunk=int(rng.choice([8, 16, 32])),
                            cuda_graphs=True, async_steps=True))
    ids, step = {}, 0
    while len(ids) < n_req or e.has_work():
        for i in range(n_req):
            if i not in ids and arrive[i] <= step:
                ids[i] = e.add_request(prompts[i], SamplingParams(temperature=0.0, max_new_tokens=new[i], ignore_eos=True))
        e.step()
        step += 1
        assert step < 3000
        e.runner.manager.check_invariants()
    for i in range(n_req):
        got = e.requests[ids[i]].output
        assert len(got) == new[i], (i, e.finish_reason(ids[i]))
        assert P.greedy_gap(cfg, w, prompts[i], got) < 1e-4, (name, seed, i)
    assert not e.runner.manager.requests
    assert all(e.runner.manager.free_pages(g) == 12 for g in range(len(e.runner.manager.groups)))
    _PREEMPTIONS.append(e.scheduler.stats["preemptions"])


_PREEMPTIONS = []


def test_random_workloads_did_preempt():
    """The pools above are meant to be too small: at least one of the runs must have preempted."""
    if not _PREEMPTIONS:
        pytest.skip("the random workloads did not run in this session")
    assert sum(_PREEMPTIONS) >= 1, _PREEMPTIONS
