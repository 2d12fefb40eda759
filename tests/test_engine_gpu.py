"""The engine above the step function, and the generality of the parts: generation through
the entry point, long decoding, the first tokens of a sequence, parts alone, a run order
that names a layer twice and lets a layer read another's cache, tensors stored in 32-bit,
and a toy mixer with state of its own that is defined here and plugged in."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as RU
from tiny_configs import TINY, TINY_A, TINY_B, write_tiny_model

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return str(tmp_path_factory.mktemp("models"))


@pytest.fixture(scope="module")
def models(folder):
    out = {}
    for name in TINY:
        path = write_tiny_model(name, folder)
        out[name] = (path, *P.load_model_dir(path))
    return out


# -- generation through the entry point ------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(models, name, dtype, graphs):
    from llm_rs_b200.engine import Engine, EngineConfig
    from llm_rs_b200.sampling import SamplingParams
    path, cfg, w = models[name]
    rng = np.random.default_rng(7)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (3, 40, 17, 70)]
    engine = Engine(EngineConfig(model_path=path, block_pool_size=64, page_size=TINY[name][3], dtype=dtype,
                                 max_requests=4, max_tokens_per_step=48, prefill_chunk=32, cuda_graphs=graphs))
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True))
    assert [len(g) for g in got] == [12] * 4
    if dtype == "float32":
        for p, g in zip(prompts, got):
            assert P.greedy_gap(cfg, w, p, g) < 1e-4        # the plain implementation's own choice (or an exact tie)
    else:
        for p, g in zip(prompts, got):
            assert P.greedy_gap(cfg, w, p, g) < 0.05
    assert not engine.runner.manager.requests
    engine.runner.manager.check_invariants()


def test_reference_style_entry_points(models):
    from llm_rs_b200.engine import (ChatRequest, EngineConfig, create_engine, destroy_engine, poll_token,
                                    send_request)
    path, cfg, w = models["A"]
    engine = create_engine(EngineConfig(model_path=path, block_pool_size=32, dtype="float32"))
    a = send_request(engine, ChatRequest(prompt=[5, 6, 7], temperature=0.0, max_tokens=5))
    b = send_request(engine, ChatRequest(prompt=[9, 1], temperature=0.9, top_p=0.9, max_tokens=3, seed=4))
    assert a != 0 and b != 0 and a != b
    toks = []
    while True:
        r = poll_token(engine, a)
        toks.append(r.token)
        if r.is_eos:
            break
    eos = cfg["eos_token_id"]
    assert len(toks) == 5 or toks[-1] == eos
    want = P.greedy_generate(cfg, w, [5, 6, 7], len(toks))
    assert toks == want
    n = 0
    while not poll_token(engine, b).is_eos:
        n += 1
    assert n <= 2
    destroy_engine(engine)
    assert not engine.runner.manager.requests


def test_temperature_sampling_is_seeded_and_batch_independent(models):
    from llm_rs_b200.engine import Engine, EngineConfig
    from llm_rs_b200.sampling import SamplingParams
    path, cfg, w = models["B"]
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (9, 40, 77)]
    sp = [SamplingParams(temperature=0.7, seed=7, max_new_tokens=10, ignore_eos=True),
          SamplingParams(temperature=1.0, top_k=20, top_p=0.9, repetition_penalty=1.2, seed=8, max_new_tokens=10,
                         ignore_eos=True),
          SamplingParams(temperature=0.0, max_new_tokens=10, ignore_eos=True)]

    def run(order, budget):
        e = Engine(EngineConfig(model_path=path, block_pool_size=128, page_size=8, dtype="float32", max_requests=4,
                                max_tokens_per_step=budget, prefill_chunk=32))
        ids = {}
        for i in order:
            # Request ids feed the draws: give each prompt the same id whatever the order.
            e._ids = iter([i + 1])
            ids[i] = e.add_request(prompts[i], sp[i])
        while e.has_work():
            e.step()
        return [e.requests[ids[i]].output for i in range(3)]
    a = run([0, 1, 2], 64)
    b = run([2, 1, 0], 17)          # other order, other cuts: same tokens
    assert a == b
    # Every sampled token is the plain sampler's choice on the engine's own float32 logits at that place
    # (taken by feeding prompt + output back through the step function), with the request's history.
    from llm_rs_b200.engine import ModelRunner, StepEntry
    runner = ModelRunner.from_model_dir(path, dtype=torch.float32, max_tokens=256, page_size=8, max_requests=2)
    for i, (prompt, out, p) in enumerate(zip(prompts, a, sp)):
        seq = prompt + out
        rows = runner.step([StepEntry("t", seq[:-1], list(range(len(prompt) - 1, len(seq) - 1)))]).cpu().numpy()
        runner.release("t")
        for j, tok in enumerate(out):
            want = P.sample(rows[j], p.temperature, p.top_k, p.top_p, p.repetition_penalty, seq[:len(prompt) + j],
                            seed=p.seed, request_id=i + 1, index=j)
            if want != tok:
                # The draw may fall within float32 rounding of a boundary between two tokens.
                probs = P.kept_probabilities(rows[j], p.temperature, p.top_k, p.top_p, p.repetition_penalty,
                                             seq[:len(prompt) + j]) if p.temperature > 1e-5 else None
                assert probs is not None, (i, j, tok, want)
                cum, u = np.cumsum(probs), P.uniform(p.seed, i + 1, j)
                assert (cum[tok - 1] if tok else 0.0) - 1e-5 <= u * cum[-1] <= cum[tok] + 1e-5, (i, j, tok, want)
    # And the first one also follows the plain sampler on the plain logits.
    logits = P.forward(cfg, w, prompts[0])[-1].numpy()
    probs = P.kept_probabilities(logits, 0.7)
    u = P.uniform(7, 1, 0)
    cum = np.cumsum(probs)
    tok = a[0][0]
    assert (cum[tok - 1] if tok else 0.0) - 1e-4 <= u <= cum[tok] + 1e-4


def test_out_of_pages_preempts_and_still_finishes(models):
    """A pool too small for all requests at once: the engine preempts, recomputes, and every
    request gets exactly the tokens it would get alone."""
    from llm_rs_b200.engine import Engine, EngineConfig
    from llm_rs_b200.sampling import SamplingParams
    path, cfg, w = models["A"]
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (30, 30, 30)]
    sp = SamplingParams(temperature=0.0, max_new_tokens=24, ignore_eos=True)
    e = Engine(EngineConfig(model_path=path, block_pool_size=8, page_size=16, dtype="float32", max_requests=4,
                            max_tokens_per_step=64, prefill_chunk=32))     # 128 tokens of cache for 3 x 54
    got = e.generate(prompts, sp)
    assert e.scheduler.stats["preemptions"] >= 1
    for p, g in zip(prompts, got):
        assert len(g) == 24 and P.greedy_gap(cfg, w, p, g) < 1e-4
    assert e.runner.manager.free_pages(0) == 8


# -- long decoding, first tokens ---------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding(models, dtype):
    """600 tokens decoded one by one after a short prompt (many pages, many splits), against the whole sequence."""
    from llm_rs_b200.engine import ModelRunner, StepEntry
    path, cfg, w = models["B"]
    toks = np.random.default_rng(5).integers(0, cfg["vocab_size"], 640).tolist()
    ref = P.forward(cfg, w, toks).numpy()
    runner = ModelRunner.from_model_dir(path, dtype=dtype, max_tokens=704, page_size=8, max_requests=2)
    runner.use_graphs = True
    runner.step([StepEntry("r", toks[:40], [])])
    worst = 0.0
    for i in range(40, 640):
        row = runner.step([StepEntry("r", [toks[i]], [0])]).float().cpu().numpy()[0]
        worst = max(worst, float(np.abs(row - ref[i]).max()))
    tol = 1e-4 if dtype == torch.float32 else 0.02 * float(np.abs(ref).max())
    assert worst <= tol, worst


def test_captured_steps_are_bounded_and_evicted(models):
    """Decode steps of changing batch size with room for two captured steps only: steps whose graph
    was evicted are captured again and give the same logits."""
    from llm_rs_b200.engine import ModelRunner, StepEntry
    path, cfg, w = models["A"]
    rng = np.random.default_rng(11)
    seqs = [rng.integers(0, cfg["vocab_size"], 30).tolist() for _ in range(4)]
    refs = [P.forward(cfg, w, s).numpy() for s in seqs]
    runner = ModelRunner.from_model_dir(path, dtype=torch.float32, max_tokens=512, page_size=16, max_requests=4)
    runner.use_graphs = True
    runner.max_graphs = 2
    for r, s in enumerate(seqs):
        runner.step([StepEntry(r, s[:10], [])])
    worst = 0.0
    for i in range(10, 30):
        live = [r for r in range(4) if (i + r) % 4 != 0] or [0]      # batch sizes 3 and 4 in turn, varying members
        batches = [live[:n] for n in (len(live), 2, 1)] if i % 3 == 0 else [live]
        done = set()
        for batch in batches:
            batch = [r for r in batch if r not in done]
            if not batch:
                continue
            rows = runner.step([StepEntry(r, [seqs[r][i]], [0]) for r in batch]).cpu().numpy()
            for k, r in enumerate(batch):
                worst = max(worst, float(np.abs(rows[k] - refs[r][i]).max()))
                done.add(r)
        for r in range(4):
            if r not in done:
                runner.step([StepEntry(r, [seqs[r][i]], [])])
    assert len(runner._graphs) <= 2
    assert worst <= 1e-4, worst


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(TINY))
def test_first_tokens(models, name, dtype):
    """Sequences of 1, 2 and 3 tokens, fed whole and token by token from position 0."""
    from llm_rs_b200.engine import ModelRunner, StepEntry
    path, cfg, w = models[name]
    runner = ModelRunner.from_model_dir(path, dtype=dtype, max_tokens=256, page_size=TINY[name][3], max_requests=4)
    tol = 1e-4 if dtype == torch.float32 else 0.03
    for n in (1, 2, 3):
        toks = np.random.default_rng(n).integers(0, cfg["vocab_size"], n).tolist()
        ref = P.forward(cfg, w, toks).numpy()
        whole = runner.step([StepEntry(f"w{n}", toks, list(range(n)))]).float().cpu().numpy()
        assert np.abs(whole - ref).max() <= tol
        for i, t in enumerate(toks):
            row = runner.step([StepEntry(f"s{n}", [t], [0])]).float().cpu().numpy()[0]
            assert np.abs(row - ref[i]).max() <= tol
        runner.release(f"w{n}")
        runner.release(f"s{n}")


def test_norms_spread_over_products_in_small_steps(models, monkeypatch):
    """In a bfloat16 step of few tokens the norm kernel runs for the first layer and the last norm only:
    every other norm is made by the product before it and applied by the product after it. The logits agree
    with the ones that the norm kernels give, and with the plain implementation."""
    from llm_rs_b200 import ops
    from llm_rs_b200.engine import ModelRunner, StepEntry
    from llm_rs_b200.parts import block as block_module
    path, cfg, w = models["D"]
    toks = np.random.default_rng(4).integers(0, cfg["vocab_size"], 12).tolist()
    ref = P.forward(cfg, w, toks).numpy()
    calls, real = [], ops.add_rmsnorm
    monkeypatch.setattr(ops, "add_rmsnorm", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    got = {}
    for linked in (True, False):
        monkeypatch.setattr(block_module, "LINK_NORMS", linked)
        runner = ModelRunner.from_model_dir(path, dtype=torch.bfloat16, max_tokens=256, page_size=16, max_requests=4)
        rows = []
        for i in range(0, 12, 3):
            del calls[:]
            rows.append(runner.step([StepEntry("a", toks[i:i + 3], [0, 1, 2])]).float().cpu().numpy())
            assert len(calls) == (2 if linked else 2 * cfg["num_hidden_layers"] + 1), (linked, len(calls))
        got[linked] = np.concatenate(rows)
    scale = np.abs(ref).max()
    assert np.abs(got[True] - ref).max() < 0.02 * scale
    assert np.abs(got[True] - got[False]).max() < 0.02 * scale


@pytest.mark.parametrize("hidden,heads,kv_heads,inter", [(2048, 16, 8, 6144), (2560, 32, 8, 9728), (5120, 40, 8, 17408)])
def test_layer_sizes_of_the_family_against_plain(hidden, heads, kv_heads, inter):
    """Two layers at the layer sizes of larger models of the family (heads of 128, widths that are no power
    of two): the bfloat16 engine, which takes its tcgen05 kernels with all their fused epilogues there, and
    the float32 engine on the same weights, each against the plain implementation (float64, on the device);
    prompts of three lengths in one step, then decode steps."""
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import ModelRunner, StepEntry
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import DecoderModel
    from llm_rs_b200.weights import random_tensors
    raw = dict(TINY_B, num_hidden_layers=2, hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=kv_heads,
               head_dim=128, intermediate_size=inter, vocab_size=8000, max_position_embeddings=2048, eos_token_id=1)
    spec = build_spec(Qwen3Config.from_dict(raw))
    t16 = random_tensors(DecoderModel(spec).weight_specs(), seed=5, sigma=0.02, dtype=torch.bfloat16, device=DEV)
    rng = np.random.default_rng(hidden)
    prompts = [rng.integers(0, 8000, n).tolist() for n in (100, 37, 300)]
    later = rng.integers(0, 8000, (10, 3)).tolist()
    outs = []
    for dtype, tensors in ((torch.bfloat16, t16), (torch.float32, {k: v.float() for k, v in t16.items()})):
        runner = ModelRunner(spec, tensors, dtype, DEV, max_tokens=1024, page_size=16, max_requests=4)
        rows = [runner.step([StepEntry(i, p, [len(p) - 1]) for i, p in enumerate(prompts)]).float().cpu()]
        for s in range(10):
            rows.append(runner.step([StepEntry(i, [later[s][i]], [0]) for i in range(3)]).float().cpu())
        outs.append(torch.cat(rows))
        del runner
    w64 = {k: v.double() for k, v in t16.items()}
    fulls = [P.forward(raw, w64, p + [later[k][i] for k in range(10)]) for i, p in enumerate(prompts)]
    want = torch.stack([fulls[i][len(prompts[i]) - 1 + s] for s in range(11) for i in range(3)]).float().cpu()
    scale = float(want.abs().max())
    assert float((outs[1] - want).abs().max()) <= 1e-4, float((outs[1] - want).abs().max())
    assert float((outs[0] - want).abs().max()) < 0.02 * scale, (float((outs[0] - want).abs().max()), scale)


# -- weights stored in 32-bit --------------------------------------------------------------------
def test_tensors_stored_in_32_bit_stay_32_bit(folder):
    """A folder whose matrices are float32: the bfloat16 engine keeps them (its products then
    run in true float32), so it lands closer to the plain implementation than bfloat16 weights could."""
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import ModelRunner, StepEntry
    from llm_rs_b200.weights import write_random_model
    path = write_random_model(folder + "/f32", Qwen3Config.from_dict(TINY_B), seed=3, sigma=0.03, norm_jitter=0.1,
                              dtype=torch.float32)
    cfg, w = P.load_model_dir(path)
    toks = np.random.default_rng(0).integers(0, cfg["vocab_size"], 50).tolist()
    ref = P.forward(cfg, w, toks).numpy()
    runner = ModelRunner.from_model_dir(path, dtype=torch.bfloat16, max_tokens=128, page_size=8)
    assert runner.model.blocks[0].feed_forward.down.weight.dtype == torch.float32
    got = runner.step([StepEntry("a", toks, list(range(50)))]).float().cpu().numpy()
    assert np.abs(got - ref).max() < 0.02 * np.abs(ref).max()
    r32 = ModelRunner.from_model_dir(path, dtype=torch.float32, max_tokens=128, page_size=8)
    got32 = r32.step([StepEntry("a", toks, list(range(50)))]).float().cpu().numpy()
    assert np.abs(got32 - ref).max() < 1e-4


# -- parts alone -----------------------------------------------------------------------------------
def _runtime(dtype, max_positions=128):
    from llm_rs_b200.parts import Runtime
    return Runtime(torch.device(DEV), dtype, max_positions)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_part_rmsnorm_and_swiglu_alone(dtype):
    from llm_rs_b200.parts import PartSpec, build
    torch.manual_seed(0)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    norm = build("norm", PartSpec("rmsnorm", {"dim": 72, "eps": 2e-6, "name": "n.weight"}), prefix="x.")
    assert [s.name for s in norm.weight_specs()] == ["x.n.weight"]
    wn = 1 + 0.1 * torch.randn(72)
    norm.bind({"x.n.weight": wn.to(DEV)}, _runtime(dtype))
    h = torch.randn(5, 72, device=DEV)
    y = norm.forward(h.clone(), None)
    assert torch.allclose(y.double().cpu(), P.rms_norm(h.double().cpu(), wn.double(), 2e-6), **tol)

    ffn = build("feed_forward", PartSpec("swiglu", {"hidden_size": 72, "intermediate_size": 200, "names": {
        "gate": "gate_proj", "up": "up_proj", "down": "down_proj"}}), prefix="m.")
    assert sorted(s.name for s in ffn.weight_specs()) == ["m.down_proj.weight", "m.gate_proj.weight", "m.up_proj.weight"]
    ws = {s.name: (torch.randn(s.shape) * 0.1).to(dtype).to(DEV) for s in ffn.weight_specs()}
    ffn.bind(ws, _runtime(dtype))
    x = torch.randn(5, 72).to(dtype)
    want = P.swiglu(x.double(), {k: v.double().cpu() for k, v in ws.items()}, "m.")
    assert torch.allclose(ffn.forward(x.to(DEV), None).double().cpu(), want, **tol)


def test_part_rotary_table():
    from llm_rs_b200.parts import PartSpec, build
    rope = build("position", PartSpec("rope_half", {"head_dim": 32, "theta": 5e5, "rotary_dim": 16}))
    rope.bind({}, _runtime(torch.float32, 300))
    table = rope.rotation_table().cpu().double()
    ang = P.rope_angles(range(300), 16, 5e5, torch.float64)
    assert table.shape == (300, 8, 2)
    assert torch.allclose(table[..., 0], ang.cos(), atol=1e-7) and torch.allclose(table[..., 1], ang.sin(), atol=1e-7)
    assert build("position", PartSpec("none", {"head_dim": 32})).rotation_table() is None


def test_decode_attention_split_choice():
    """The cut of the keys for decode attention: multiples of 64 keys, and among the cuts of up to 16 splits
    (which the kernel's cluster merges) the one with the least waves x (keys + fixed cost), waves counted
    against what the device really holds in clusters of that size; more splits only for few requests
    with long contexts."""
    from llm_rs_b200 import ops
    from llm_rs_b200.parts import PartSpec, build
    from llm_rs_b200.parts.attention import CAPACITY_USED, FIXED_KEYS, MAX_CLUSTER
    att = build("mixer", PartSpec("gqa_attention", {
        "hidden_size": 1024, "n_heads": 32, "n_kv_heads": 8, "head_dim": 128,
        "position": PartSpec("none", {"head_dim": 128})}))
    q = torch.empty(1, 1, dtype=torch.bfloat16, device=DEV)
    held = {s: int(CAPACITY_USED * ops.attn_decode_capacity(128, s, 4, DEV)) for s in range(1, MAX_CLUSTER + 1)}
    assert all(128 <= held[s] <= 2 * 148 for s in held)
    for length in (100, 4096, 5000, 32768):
        for n in range(1, 41):
            keys, ring = att._choose_split(n, length, q)
            splits = -(-length // keys)
            assert keys % 64 == 0 and keys >= 128 and ring in (2, 3)
            if ring == 2:       # the kernel of which three blocks fit an SM: only where it saves a wave
                light = int(CAPACITY_USED * ops.attn_decode_capacity(128, splits, 4, DEV, light=True))
                assert light > held[splits] and -(-(splits * n * 8) // light) < -(-(splits * n * 8) // held[splits])
                continue
            costs = {}
            for s in range(1, MAX_CLUSTER + 1):
                k = max(-(-(-(-length // s)) // 64) * 64, 128)
                real = -(-length // k)
                costs.setdefault(real, -(-(real * n * 8) // held[real]) * (k + FIXED_KEYS))
            if splits <= MAX_CLUSTER:
                assert costs[splits] == min(costs.values()), (length, n, keys, costs)
            else:
                assert n * 8 * 2 * MAX_CLUSTER <= ops.attn_decode_capacity(128, 1, 4, DEV) and length > MAX_CLUSTER * 1024, (length, n, keys)


# -- run order: a layer named twice, a layer that reads another's cache ----------------------------
def _plain_with_run_order(cfg, w, toks, order):
    """The plain forward with an explicit run order [(layer, cache_of)]: an entry that reads
    another entry's cache attends with ITS queries over THAT entry's keys and values."""
    h = P.embedding(w["model.embed_tokens.weight"], toks)
    pos = list(range(len(toks)))
    eps = cfg["rms_norm_eps"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    kv = {}
    for s, (layer, cache_of) in enumerate(order):
        p = f"model.layers.{layer}."
        x = P.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        T = x.shape[0]
        ang = P.rope_angles(pos, d, cfg["rope_theta"], x.dtype)
        q = P.rotate_half(P.rms_norm(P.linear(x, w[p + "self_attn.q_proj.weight"]).reshape(T, nq, d),
                                     w[p + "self_attn.q_norm.weight"], eps), ang)
        if cache_of is None:
            k = P.rotate_half(P.rms_norm(P.linear(x, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, d),
                                         w[p + "self_attn.k_norm.weight"], eps), ang)
            v = P.linear(x, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, d)
            kv[s] = (k, v)
        else:
            k, v = kv[cache_of]
        h = h + P.linear(P.attention(q, k, v), w[p + "self_attn.o_proj.weight"])
        h = h + P.swiglu(P.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    h = P.rms_norm(h, w["model.norm.weight"], eps)
    return P.linear(h, w["lm_head.weight"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_run_order_with_repeated_layer_and_shared_cache(models, dtype):
    import dataclasses
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import ModelRunner, StepEntry
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import DecoderModel, RunStep
    from llm_rs_b200.weights import load_weights
    path, cfg, w = models["B"]
    spec = build_spec(Qwen3Config.from_dict(cfg))
    # layer 0, layer 1, layer 1 again (own cache), layer 2 reading entry 1's cache, layer 0 again
    order = [(0, None), (1, None), (1, None), (2, 1), (0, None)]
    spec = dataclasses.replace(spec, run_order=tuple(RunStep(l, c) for l, c in order))
    tensors = load_weights(path, DecoderModel(spec).weight_specs(), dtype, torch.device(DEV))
    runner = ModelRunner(spec, tensors, dtype, DEV, max_tokens=256, page_size=8, max_requests=2)
    assert len(runner.storage.groups) == 1 and len(runner.storage.groups[0].entries) == 4   # four caches for five entries
    toks = np.random.default_rng(2).integers(0, cfg["vocab_size"], 70).tolist()
    ref = _plain_with_run_order(cfg, w, toks, order).numpy()
    steps = RU.portions({"a": toks}, sizes=(9, 2, 30, 1, 1, 1, 5, 64))
    got = RU.run_steps(runner, steps)
    worst, where, n = RU.max_diff(got, {"a": ref})
    assert n == 70
    assert worst <= (1e-4 if dtype == torch.float32 else 0.02 * float(np.abs(ref).max())), (worst, where)


# -- a toy mixer with state of its own, defined here ------------------------------------------------
def test_toy_mixer_with_state_plugs_in(models):
    """A mixer that keeps a running mean of its inputs per request (fixed-size state, no pages)
    is registered from this file, built into a model beside attention layers, and stepped in
    portions and mixed batches; the framework's files are not touched."""
    import dataclasses
    from llm_rs_b200 import ops
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import ModelRunner, StepEntry
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import (DecoderModel, Mixer, PartSpec, StateNeed, WeightSpec, register, unregister)
    from llm_rs_b200.weights import load_weights

    @register("mixer", "toy_running_mean", replace=True)
    class RunningMean(Mixer):
        """out_t = W * mean(x_0..x_t) per request; state = (sum of inputs, count)."""
        graph_safe = False          # plans on the host every step

        def __init__(self, hidden_size, prefix=""):
            self.hidden_size, self.prefix = hidden_size, prefix

        def weight_specs(self):
            return [WeightSpec(self.prefix + "mix.weight", (self.hidden_size, self.hidden_size))]

        def state_need(self):
            return StateNeed({"sum": (self.hidden_size,), "count": (1,)})

        def bind(self, tensors, runtime):
            self.w = tensors[self.prefix + "mix.weight"].float()
            self.dtype = runtime.act_dtype

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            for r in range(ctx.n_requests):
                a, n, slot = ctx.host_q_start[r], ctx.host_n_new[r], ctx.host_slot_ids[r]
                xs = x[a:a + n].float()
                run = cache.state["sum"][slot] + torch.cumsum(xs, 0)
                cnt = cache.state["count"][slot] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)[:, None]
                out[a:a + n] = ((run / cnt) @ self.w.t()).to(x.dtype)
                cache.state["sum"][slot] = run[-1]
                cache.state["count"][slot] = cnt[-1]
            return out

    try:
        path, cfg, w = models["A"]
        spec = build_spec(Qwen3Config.from_dict(cfg))
        toy = dataclasses.replace(spec.layers[1], mixer=PartSpec("toy_running_mean", {"hidden_size": 64}),
                                  mixer_scope="toy.")
        spec = dataclasses.replace(spec, layers=(spec.layers[0], toy))
        model = DecoderModel(spec)
        names = [s.name for s in model.weight_specs()]
        assert "model.layers.1.toy.mix.weight" in names and "model.layers.1.self_attn.q_proj.weight" not in names
        # The folder has no toy weight: take the real tensors by name and add one.
        from llm_rs_b200.weights import open_model_files
        f = open_model_files(path)[0]
        tensors = {n: f.tensor(n).float().to(DEV) for n in names if n in f.names()}
        torch.manual_seed(0)
        mixw = torch.randn(64, 64) * 0.05
        tensors["model.layers.1.toy.mix.weight"] = mixw.to(DEV)
        runner = ModelRunner(spec, tensors, torch.float32, DEV, max_tokens=256, page_size=16, max_requests=3)
        assert runner.storage.state[1]["sum"].shape == (3, 64) and not runner.storage.state[0]
        assert len(runner.storage.groups[0].entries) == 1           # only the attention layer has pages

        def plain(toks):
            h = P.embedding(w["model.embed_tokens.weight"], toks)
            h = P.decoder_layer(h, w, 0, cfg, list(range(len(toks))), 0)
            x = P.rms_norm(h, w["model.layers.1.input_layernorm.weight"], cfg["rms_norm_eps"])
            mean = torch.cumsum(x, 0) / torch.arange(1, len(toks) + 1, dtype=torch.float64)[:, None]
            h = h + mean @ mixw.double().t()
            h = h + P.swiglu(P.rms_norm(h, w["model.layers.1.post_attention_layernorm.weight"], cfg["rms_norm_eps"]),
                             w, "model.layers.1.mlp.")
            return P.linear(P.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]), w["model.embed_tokens.weight"])

        rng = np.random.default_rng(4)
        reqs = {f"r{i}": rng.integers(0, 256, n).tolist() for i, n in enumerate((50, 23, 64, 9))}
        ref = {r: plain(t).numpy() for r, t in reqs.items()}
        got = RU.run_steps(runner, RU.mixed(reqs, seed=1, max_live=3))
        worst, where, n = RU.max_diff(got, ref)
        assert n == sum(len(t) for t in reqs.values()) and worst < 1e-4, (worst, where)
    finally:
        unregister("mixer", "toy_running_mean")


# -- the same toy kept on the device: CUDA graphs, and a warm-up that must not count twice -----------
def test_toy_stateful_mixer_under_cuda_graphs(models):
    """A mixer with per-request state that it updates on the device (nothing of its step is planned on the host):
    its decode steps are captured in CUDA graphs like anyone's. The step that captures a graph runs the model
    twice (once to size the workspace, once as the first replay); the state must move once."""
    import dataclasses
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import ModelRunner, StepEntry
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import DecoderModel, Mixer, PartSpec, StateNeed, WeightSpec, register, unregister
    from llm_rs_b200.weights import open_model_files

    @register("mixer", "toy_running_mean_device", replace=True)
    class RunningMeanOnDevice(Mixer):
        """out_t = W * mean(x_0..x_t) per request; state = (sum of inputs, count). Steps of single tokens touch
        the device only (index arithmetic on the step's device arrays); longer portions loop on the host, which
        is fine outside a graph (only steps of single tokens are captured)."""

        def __init__(self, hidden_size, prefix=""):
            self.hidden_size, self.prefix = hidden_size, prefix

        def weight_specs(self):
            return [WeightSpec(self.prefix + "mix.weight", (self.hidden_size, self.hidden_size))]

        def state_need(self):
            return StateNeed({"sum": (self.hidden_size,), "count": (1,)})

        def bind(self, tensors, runtime):
            self.w = tensors[self.prefix + "mix.weight"].float()

        def forward(self, x, ctx, cache):
            total, count = cache.state["sum"], cache.state["count"]
            if ctx.n_tokens == ctx.n_requests:                  # one token per request: request r is row r
                slots = ctx.slot_ids.long()
                total.index_add_(0, slots, x.float())
                count.index_add_(0, slots, torch.ones_like(x[:, :1], dtype=torch.float32))
                return ((total[slots] / count[slots]) @ self.w.t()).to(x.dtype)
            out = torch.empty_like(x)
            for r in range(ctx.n_requests):
                a, n, slot = ctx.host_q_start[r], ctx.host_n_new[r], ctx.host_slot_ids[r]
                run = total[slot] + torch.cumsum(x[a:a + n].float(), 0)
                cnt = count[slot] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)[:, None]
                out[a:a + n] = ((run / cnt) @ self.w.t()).to(x.dtype)
                total[slot], count[slot] = run[-1], cnt[-1]
            return out

    try:
        path, cfg, w = models["A"]
        spec = build_spec(Qwen3Config.from_dict(cfg))
        toy = dataclasses.replace(spec.layers[1], mixer=PartSpec("toy_running_mean_device", {"hidden_size": 64}),
                                  mixer_scope="toy.")
        spec = dataclasses.replace(spec, layers=(spec.layers[0], toy))
        names = [s.name for s in DecoderModel(spec).weight_specs()]
        f = open_model_files(path)[0]
        tensors = {n: f.tensor(n).float().to(DEV) for n in names if n in f.names()}
        mixw = torch.randn(64, 64, generator=torch.Generator().manual_seed(1)) * 0.05
        tensors["model.layers.1.toy.mix.weight"] = mixw.to(DEV)
        runner = ModelRunner(spec, tensors, torch.float32, DEV, max_tokens=512, page_size=16, max_requests=4)
        runner.use_graphs = True
        assert runner._graph_safe

        def plain(toks):
            h = P.embedding(w["model.embed_tokens.weight"], toks)
            h = P.decoder_layer(h, w, 0, cfg, list(range(len(toks))), 0)
            x = P.rms_norm(h, w["model.layers.1.input_layernorm.weight"], cfg["rms_norm_eps"])
            mean = torch.cumsum(x, 0) / torch.arange(1, len(toks) + 1, dtype=torch.float64)[:, None]
            h = h + mean @ mixw.double().t()
            h = h + P.swiglu(P.rms_norm(h, w["model.layers.1.post_attention_layernorm.weight"], cfg["rms_norm_eps"]),
                             w, "model.layers.1.mlp.")
            return P.linear(P.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]), w["model.embed_tokens.weight"])

        rng = np.random.default_rng(6)
        seqs = [rng.integers(0, 256, 40).tolist() for _ in range(3)]
        refs = [plain(s).numpy() for s in seqs]
        for r, s in enumerate(seqs):
            runner.step([StepEntry(r, s[:9 + r], [])])
        worst = 0.0
        # Every request decodes every token; the batch's make-up changes, so that graphs of several sizes are
        # captured, each at a step whose state must not move twice.
        at = [9, 10, 11]
        step = 0
        while min(at) < 40:
            live = [r for r in range(3) if at[r] < 40 and (step % 4 != r)]
            if live:
                rows = runner.step([StepEntry(r, [seqs[r][at[r]]], [0]) for r in live]).cpu().numpy()
                for k, r in enumerate(live):
                    worst = max(worst, float(np.abs(rows[k] - refs[r][at[r]]).max()))
                    at[r] += 1
            step += 1
        assert len(runner._graphs) >= 2, "the decode steps were not captured"
        assert worst < 1e-4, worst
    finally:
        unregister("mixer", "toy_running_mean_device")


# -- a toy mixer that caches one latent row per token and plans its step on the host ------------------
def test_toy_latent_cache_mixer_with_a_plan(models):
    """A mixer that stores ONE row of 24 numbers per token in the paged cache (one head, one plane: neither
    keys and values nor equal widths) and mixes by a causal mean over the cached rows. Where a token's row goes
    and which rows a token reads is planned on the host once per step (``plan``) and reaches ``forward`` as
    device arrays. Registered from this file; storage, cache manager, packer and runner are not touched."""
    import dataclasses
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import ModelRunner
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import CacheNeed, DecoderModel, Mixer, PartSpec, Plan, WeightSpec, register, unregister
    from llm_rs_b200.weights import open_model_files
    L = 24

    @register("mixer", "toy_latent_mean", replace=True)
    class LatentMean(Mixer):
        """latent_t = W_in x_t is cached; out_t = W_out mean(latent_0..latent_t)."""

        def __init__(self, hidden_size, latent, prefix=""):
            self.H, self.L, self.prefix = hidden_size, latent, prefix

        def weight_specs(self):
            return [WeightSpec(self.prefix + "in.weight", (self.L, self.H)), WeightSpec(self.prefix + "out.weight", (self.H, self.L))]

        def bind(self, tensors, runtime):
            self.w_in, self.w_out = tensors[self.prefix + "in.weight"].float(), tensors[self.prefix + "out.weight"].float()

        def cache_need(self):
            return CacheNeed("full", n_kv_heads=1, head_dim=self.L, planes=(self.L,))

        def plan_key(self):
            return ("toy_latent_mean", self.cache_need().group_key())

        def plan(self, step):
            # Flat row index (page * page_size + place) of every new token, and of every row each request reads.
            table, P_ = step.table_of(self.cache_need()), step.page_size
            write, read, read_start = [], [], [0]
            for r in range(step.n_requests):
                c, n = int(step.cached_len[r]), int(step.n_new[r])
                pos = np.arange(c + n)
                rows = table[r, pos // P_].astype(np.int64) * P_ + pos % P_
                write.append(rows[c:])
                read.append(rows)
                read_start.append(read_start[-1] + c + n)
            return Plan(arrays={"write": np.concatenate(write).astype(np.int32), "read": np.concatenate(read).astype(np.int32),
                                "read_start": np.asarray(read_start, np.int32)},
                        values={"n_read": read_start[-1]})

        def forward(self, x, ctx, cache):
            plan = ctx.plan(self.plan_key())
            rows = cache.planes[0]                         # [pages, 1, page_size, L]: a view into the pool
            assert cache.kv is None and rows.shape[1:] == (1, cache.page_size, self.L)
            pages, place = plan.arrays["write"].long() // cache.page_size, plan.arrays["write"].long() % cache.page_size
            rows[pages, 0, place] = (x.float() @ self.w_in.t()).to(rows.dtype)
            rd = plan.arrays["read"].long()
            seen = rows[rd // cache.page_size, 0, rd % cache.page_size].float()      # [n_read, L]
            out = torch.empty((ctx.n_tokens, self.H), dtype=torch.float32, device=x.device)
            starts = plan.arrays["read_start"].tolist()
            for r in range(ctx.n_requests):
                a, n, c = ctx.host_q_start[r], ctx.host_n_new[r], ctx.host_cached_len[r]
                mine = seen[starts[r]:starts[r + 1]]
                mean = torch.cumsum(mine, 0)[c:] / torch.arange(c + 1, c + n + 1, device=x.device)[:, None]
                out[a:a + n] = mean @ self.w_out.t()
            return out.to(x.dtype)

        graph_safe = False      # forward reads host lists

    try:
        path, cfg, w = models["A"]
        spec = build_spec(Qwen3Config.from_dict(cfg))
        toy = dataclasses.replace(spec.layers[1], mixer=PartSpec("toy_latent_mean", {"hidden_size": 64, "latent": L}),
                                  mixer_scope="toy.")
        spec = dataclasses.replace(spec, layers=(spec.layers[0], toy))
        names = [s.name for s in DecoderModel(spec).weight_specs()]
        f = open_model_files(path)[0]
        tensors = {n: f.tensor(n).float().to(DEV) for n in names if n in f.names()}
        g = torch.Generator().manual_seed(2)
        w_in, w_out = torch.randn(L, 64, generator=g) * 0.2, torch.randn(64, L, generator=g) * 0.2
        tensors["model.layers.1.toy.in.weight"], tensors["model.layers.1.toy.out.weight"] = w_in.to(DEV), w_out.to(DEV)

        def plain(toks):
            h = P.embedding(w["model.embed_tokens.weight"], toks)
            h = P.decoder_layer(h, w, 0, cfg, list(range(len(toks))), 0)
            x = P.rms_norm(h, w["model.layers.1.input_layernorm.weight"], cfg["rms_norm_eps"])
            lat = x @ w_in.double().t()
            mean = torch.cumsum(lat, 0) / torch.arange(1, len(toks) + 1, dtype=torch.float64)[:, None]
            h = h + mean @ w_out.double().t()
            h = h + P.swiglu(P.rms_norm(h, w["model.layers.1.post_attention_layernorm.weight"], cfg["rms_norm_eps"]),
                             w, "model.layers.1.mlp.")
            return P.linear(P.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]), w["model.embed_tokens.weight"])

        rng = np.random.default_rng(12)
        reqs = {f"r{i}": rng.integers(0, 256, n).tolist() for i, n in enumerate((50, 23, 64, 9, 40))}
        ref = {r: plain(t).numpy() for r, t in reqs.items()}
        steps = RU.mixed(reqs, seed=3, max_live=3)
        runner = ModelRunner(spec, tensors, torch.float32, DEV, max_tokens=RU.live_token_peak(steps), page_size=16,
                             max_requests=3)
        assert [g.need.plane_widths for g in runner.storage.groups] == [(16, 16), (L,)]
        assert runner.storage.kv[1].shape == (1, runner.storage.groups[1].n_pages, 1, 16 * L)
        got = RU.run_steps(runner, steps)
        worst, where, n = RU.max_diff(got, ref)
        assert n == sum(len(t) for t in reqs.values()) and worst < 1e-4, (worst, where)
        assert all(p.free_pages() == p.capacity for p in runner.manager.pools)
    finally:
        unregister("mixer", "toy_latent_mean")


# -- a toy feed-forward with routing, defined here ---------------------------------------------------
def test_toy_routed_feed_forward_plugs_in(models):
    """A feed-forward that sends every token to the one of three small experts its router prefers
    (router logits and probabilities in float32) is registered from this file and takes the place of
    one layer's feed-forward; cache, scheduler and the other parts do not change."""
    import dataclasses
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import ModelRunner
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import DecoderModel, FeedForward, PartSpec, WeightSpec, register, unregister
    from llm_rs_b200.weights import open_model_files
    E, I = 3, 40

    @register("feed_forward", "toy_top1_experts", replace=True)
    class Top1Experts(FeedForward):
        """out = p_e * down_e(relu(up_e x)) for e = argmax(router x), p = softmax(router x)."""

        def __init__(self, hidden_size, n_experts, expert_size, prefix=""):
            self.H, self.E, self.I, self.prefix = hidden_size, n_experts, expert_size, prefix

        def weight_specs(self):
            p = self.prefix
            return [WeightSpec(p + "router.weight", (self.E, self.H)), WeightSpec(p + "up.weight", (self.E, self.I, self.H)),
                    WeightSpec(p + "down.weight", (self.E, self.H, self.I))]

        def bind(self, tensors, runtime):
            p = self.prefix
            self.router, self.up, self.down = (tensors[p + n].float() for n in ("router.weight", "up.weight", "down.weight"))

        def forward(self, x, ctx):
            xf = x.float()
            prob = torch.softmax(xf @ self.router.t(), dim=-1)
            pick = prob.argmax(dim=-1)
            out = torch.zeros_like(xf)
            for e in range(self.E):
                rows = (pick == e).nonzero(as_tuple=True)[0]
                if rows.numel():
                    y = torch.relu(xf[rows] @ self.up[e].t()) @ self.down[e].t()
                    out[rows] = y * prob[rows, e:e + 1]
            return out.to(x.dtype)

    try:
        path, cfg, w = models["A"]
        spec = build_spec(Qwen3Config.from_dict(cfg))
        toy = dataclasses.replace(spec.layers[0], feed_forward=PartSpec(
            "toy_top1_experts", {"hidden_size": 64, "n_experts": E, "expert_size": I}), feed_forward_scope="moe.")
        spec = dataclasses.replace(spec, layers=(toy, spec.layers[1]))
        names = [s.name for s in DecoderModel(spec).weight_specs()]
        assert "model.layers.0.moe.router.weight" in names and "model.layers.0.mlp.gate_proj.weight" not in names
        f = open_model_files(path)[0]
        tensors = {n: f.tensor(n).float().to(DEV) for n in names if n in f.names()}
        g = torch.Generator().manual_seed(3)
        router, up, down = torch.randn(E, 64, generator=g), torch.randn(E, I, 64, generator=g) * 0.1, torch.randn(E, 64, I, generator=g) * 0.1
        for n, t in (("router", router), ("up", up), ("down", down)):
            tensors[f"model.layers.0.moe.{n}.weight"] = t.to(DEV)
        runner = ModelRunner(spec, tensors, torch.float32, DEV, max_tokens=256, page_size=16, max_requests=3)

        def plain(toks):
            pos = list(range(len(toks)))
            eps = cfg["rms_norm_eps"]
            h = P.embedding(w["model.embed_tokens.weight"], toks)
            h = h + P.attention_block(P.rms_norm(h, w["model.layers.0.input_layernorm.weight"], eps), w,
                                      "model.layers.0.self_attn.", cfg, pos, 0)
            x = P.rms_norm(h, w["model.layers.0.post_attention_layernorm.weight"], eps)
            prob = torch.softmax(x @ router.double().t(), dim=-1)
            pick = prob.argmax(dim=-1)
            y = torch.stack([torch.relu(x[t] @ up[int(e)].double().t()) @ down[int(e)].double().t() * prob[t, int(e)]
                             for t, e in enumerate(pick)])
            h = h + y
            h = P.decoder_layer(h, w, 1, cfg, pos, 0)
            return P.linear(P.rms_norm(h, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])

        rng = np.random.default_rng(8)
        reqs = {f"r{i}": rng.integers(0, 256, n).tolist() for i, n in enumerate((41, 17, 60))}
        ref = {r: plain(t).numpy() for r, t in reqs.items()}
        got = RU.run_steps(runner, RU.mixed(reqs, seed=2, max_live=3))
        worst, where, n = RU.max_diff(got, ref)
        assert n == sum(len(t) for t in reqs.values()) and worst < 2e-4, (worst, where)
    finally:
        unregister("feed_forward", "toy_top1_experts")


# -- toy position encodings, defined here ------------------------------------------------------------
@pytest.mark.parametrize("kind", ["toy_linear_rotation", "toy_learned_offsets"])
def test_toy_position_encodings_plug_in(models, kind):
    """Two position encodings registered from this file: a rotation with angles of its own (a table
    for the fused kernel) and learned vectors added to queries and keys (weights of its own, applied
    before the fused kernel). Only the mixer's ``position`` parameter changes."""
    import dataclasses
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.engine import ModelRunner
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import DecoderModel, PartSpec, PositionEncoding, WeightSpec, register, unregister
    from llm_rs_b200.weights import open_model_files
    d, max_pos = 16, 200

    @register("position", "toy_linear_rotation", replace=True)
    class LinearRotation(PositionEncoding):
        """Angle of pair i at position p: p * (i + 1) * step."""

        def __init__(self, head_dim, step, prefix=""):
            self.head_dim, self.step, self.rotary_dim = head_dim, step, head_dim

        def bind(self, tensors, runtime):
            ang = torch.arange(runtime.max_positions, dtype=torch.float64)[:, None] * \
                (torch.arange(1, self.head_dim // 2 + 1, dtype=torch.float64) * self.step)[None, :]
            self._table = torch.stack([ang.cos(), ang.sin()], dim=-1).float().contiguous().to(runtime.device)

        def rotation_table(self):
            return self._table

    @register("position", "toy_learned_offsets", replace=True)
    class LearnedOffsets(PositionEncoding):
        """q and k of every head get table[position] added (before the per-head norms)."""

        def __init__(self, head_dim, max_positions, prefix=""):
            self.head_dim, self.max_positions, self.prefix = head_dim, max_positions, prefix

        def weight_specs(self):
            return [WeightSpec(self.prefix + "position_table", (self.max_positions, self.head_dim))]

        def bind(self, tensors, runtime):
            self.table = tensors[self.prefix + "position_table"].to(runtime.act_dtype)

        def apply_unfused(self, q, k, positions):
            add = self.table[positions.long()]
            for t in (q, k):
                if t is not None:
                    t.view(t.size(0), -1, self.head_dim).add_(add[:, None, :])

    try:
        path, cfg, w = models["A"]
        spec = build_spec(Qwen3Config.from_dict(cfg))
        position = (PartSpec("toy_linear_rotation", {"head_dim": d, "step": 0.037}) if kind == "toy_linear_rotation"
                    else PartSpec("toy_learned_offsets", {"head_dim": d, "max_positions": max_pos}))
        layers = tuple(dataclasses.replace(l, mixer=PartSpec(l.mixer.kind, {**l.mixer.params, "position": position}))
                       for l in spec.layers)
        spec = dataclasses.replace(spec, layers=layers)
        names = [s.name for s in DecoderModel(spec).weight_specs()]
        f = open_model_files(path)[0]
        tensors = {n: f.tensor(n).float().to(DEV) for n in names if n in f.names()}
        tables = {}
        if kind == "toy_learned_offsets":
            extra = [n for n in names if n.endswith("position_table")]
            assert len(extra) == 2
            for i, n in enumerate(extra):
                tables[n] = torch.randn(max_pos, d, generator=torch.Generator().manual_seed(20 + i)) * 0.5
                tensors[n] = tables[n].to(DEV)
        runner = ModelRunner(spec, tensors, torch.float32, DEV, max_tokens=256, page_size=16, max_requests=3)

        def attention_block(x, i, pos):
            p = f"model.layers.{i}.self_attn."
            nq, nkv, eps, T = 4, 2, cfg["rms_norm_eps"], x.shape[0]
            q = P.linear(x, w[p + "q_proj.weight"]).reshape(T, nq, d)
            k = P.linear(x, w[p + "k_proj.weight"]).reshape(T, nkv, d)
            v = P.linear(x, w[p + "v_proj.weight"]).reshape(T, nkv, d)
            if kind == "toy_learned_offsets":
                add = tables[p + "position_table"].double()[pos][:, None, :]
                q, k = q + add, k + add
            q, k = P.rms_norm(q, w[p + "q_norm.weight"], eps), P.rms_norm(k, w[p + "k_norm.weight"], eps)
            if kind == "toy_linear_rotation":
                ang = torch.as_tensor(pos, dtype=torch.float64)[:, None] * (torch.arange(1, d // 2 + 1, dtype=torch.float64) * 0.037)[None, :]
                q, k = P.rotate_half(q, ang), P.rotate_half(k, ang)
            return P.linear(P.attention(q, k, v), w[p + "o_proj.weight"])

        def plain(toks):
            pos, eps = list(range(len(toks))), cfg["rms_norm_eps"]
            h = P.embedding(w["model.embed_tokens.weight"], toks)
            for i in range(2):
                pre = f"model.layers.{i}."
                h = h + attention_block(P.rms_norm(h, w[pre + "input_layernorm.weight"], eps), i, pos)
                h = h + P.swiglu(P.rms_norm(h, w[pre + "post_attention_layernorm.weight"], eps), w, pre + "mlp.")
            return P.linear(P.rms_norm(h, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])

        rng = np.random.default_rng(9)
        reqs = {f"r{i}": rng.integers(0, 256, n).tolist() for i, n in enumerate((37, 64, 12))}
        ref = {r: plain(t).numpy() for r, t in reqs.items()}
        got = RU.run_steps(runner, RU.mixed(reqs, seed=5, max_live=3))
        worst, where, n = RU.max_diff(got, ref)
        assert n == sum(len(t) for t in reqs.values()) and worst < 2e-4, (worst, where)
    finally:
        unregister("position", "toy_linear_rotation")
        unregister("position", "toy_learned_offsets")
