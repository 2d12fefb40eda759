"""The engine at the layer sizes of Qwen3-8B against the plain implementation.

Hidden 4096, 32 query heads over 8 key heads of 128, feed-forward 12288, vocabulary 151,936: the sizes of
the headline configuration, with 4 of its 36 layers so that the test fits in a minute. Random weights
(seed 2) are made on the device; the plain implementation runs on the same numbers in float64 on the
device (it is the same code as on the CPU: whole sequences, no cache). A request of 2,048 tokens and three
shorter ones are replayed whole, with the last 32 tokens one by one, in portions down to two tokens, and
mixed (four live requests, portions of up to 300 tokens beside single tokens, a pool so small that pages
change owner). float32: max |diff| <= 1e-4. bfloat16: within 2 % of the largest logit.

The reference has no such test: its only logit comparison holds two identical literals
(llm-tests/tests/mlc_parity.rs:669-679).
"""
import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as RU

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LAYERS, LAYERS_OF = 4, 36
RAW = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=LAYERS, hidden_size=4096,
           num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
           rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=False,
           max_position_embeddings=4096, hidden_act="silu", eos_token_id=151645)
LENGTHS = [2048, 611, 333, 150, 97, 260]      # six requests, four live: the last two get pages that others held
MODES = ["whole", "tail", "portions", "mixed"]


def _wanted(n):
    """Positions whose logits are compared: the first ones, the neighbours of page and tile edges, every
    53rd, and the last 40 (all that the tail and mixed traces decode one by one)."""
    s = set(range(min(n, 4))) | set(range(max(0, n - 40), n)) | set(range(0, n, 53))
    for edge in (16, 64, 128, 256, 512, 1024, 2032):
        s |= {p for p in (edge - 1, edge, edge + 1) if 0 <= p < n}
    return s


@pytest.fixture(scope="module")
def setup():
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import DecoderModel
    from llm_rs_b200.weights import random_tensors
    spec = build_spec(Qwen3Config.from_dict(RAW))
    t16 = random_tensors(DecoderModel(spec).weight_specs(), seed=2, sigma=0.02, norm_jitter=0.1,
                         dtype=torch.bfloat16, device=DEV)
    rng = np.random.default_rng(8)
    reqs = {f"r{i}": rng.integers(0, RAW["vocab_size"], n).tolist() for i, n in enumerate(LENGTHS)}
    wanted = {r: _wanted(len(t)) for r, t in reqs.items()}
    ref = {}
    w64 = {k: v.double() for k, v in t16.items()}
    for r, toks in reqs.items():
        rows = torch.as_tensor(sorted(wanted[r]), device=DEV)
        ref[r] = (dict(zip(sorted(wanted[r]), range(len(rows)))), P.forward(RAW, w64, toks)[rows].clone())
    del w64
    torch.cuda.empty_cache()
    yield spec, t16, reqs, wanted, ref
    torch.cuda.empty_cache()


def _steps(mode, reqs):
    if mode == "mixed":
        return RU.mixed(reqs, seed=4, sizes=(2, 17, 64, 130, 200, 300))
    return {"whole": RU.whole, "tail": RU.tail_one_by_one, "portions": RU.portions}[mode](reqs)


def _replay(runner, steps, ref):
    """Largest |engine - plain| over the wanted positions, where, and how many rows were compared."""
    from llm_rs_b200.engine import StepEntry
    at, worst, where, n = {}, 0.0, None, 0
    for st in steps:
        logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]])
        k = 0
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            index, rows = ref[e["id"]]
            for w in e["want"]:
                d = float((logits[k].double() - rows[index[base + w]]).abs().max())
                if not d <= worst:          # also catches NaN
                    worst, where = d, (e["id"], base + w)
                k += 1
                n += 1
            at[e["id"]] = base + len(e["tokens"])
        for r in st["end"]:
            runner.release(r)
            at.pop(r, None)
        runner.manager.check_invariants()
    return worst, where, n


@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("mode", MODES)
def test_engine_at_qwen3_8b_layer_sizes_matches_plain(setup, mode, dtype, graphs):
    """``graphs``: steps of single tokens are captured in CUDA graphs and replayed (the way the engine decodes)."""
    from llm_rs_b200.engine import ModelRunner
    spec, t16, reqs, wanted, ref = setup
    if graphs and mode in ("whole", "portions"):
        pytest.skip("no step of single tokens in this mode")
    steps = RU.want_only(_steps(mode, reqs), wanted)
    tensors = t16 if dtype == "bfloat16" else {k: v.float() for k, v in t16.items()}
    runner = ModelRunner(spec, tensors, getattr(torch, dtype), DEV, max_tokens=RU.live_token_peak(steps),
                         page_size=16, max_requests=4)
    runner.use_graphs = graphs
    free = runner.manager.free_pages(0)
    worst, where, n = _replay(runner, steps, ref)
    assert n == sum(len(w) for w in wanted.values())
    assert runner.manager.free_pages(0) == free, "pages were lost"
    assert bool(runner._graphs) == graphs
    scale = max(float(rows.abs().max()) for _, rows in ref.values())
    tol = 1e-4 if dtype == "float32" else 0.02 * scale
    assert worst <= tol, (f"{LAYERS} of {LAYERS_OF} layers, {mode}, {dtype}: max |diff| {worst:.3e} at {where} "
                          f"(tolerance {tol:.3e}, largest logit {scale:.3f})")
    from llm_rs_b200 import ops
    ops.check_tc_error(torch.device(DEV))
    ops.check_attention_error()


@pytest.mark.parametrize("mode", ["whole", "mixed"])
def test_every_product_of_large_steps_on_this_packages_kernel(setup, mode, monkeypatch):
    """Steps of 256 tokens or more with all their products on the tcgen05 kernel for many tokens (off by default
    for all but gate|up): the residual sums and the norms are then spread over the products' epilogues as in decode
    steps, and no norm kernel runs between the layers' products."""
    from llm_rs_b200 import ops
    from llm_rs_b200.engine import ModelRunner
    from llm_rs_b200.parts import linear
    monkeypatch.setattr(linear, "TC_MANY_TOKENS", 256)
    spec, t16, reqs, wanted, ref = setup
    steps = RU.want_only(_steps(mode, reqs), wanted)
    runner = ModelRunner(spec, t16, torch.bfloat16, DEV, max_tokens=RU.live_token_peak(steps), page_size=16,
                         max_requests=4)
    norms = []
    real = ops.add_rmsnorm
    monkeypatch.setattr(ops, "add_rmsnorm", lambda *a, **k: (norms.append(a[0].size(0)), real(*a, **k))[1])
    worst, where, n = _replay(runner, steps, ref)
    scale = max(float(rows.abs().max()) for _, rows in ref.values())
    assert worst <= 0.02 * scale, f"{mode}: max |diff| {worst:.3e} at {where} (largest logit {scale:.3f})"
    ops.check_tc_error(torch.device(DEV))
    if mode == "whole":      # in a large step only the first layer's input norm and the final norm are kernels
        large = sum(1 for st in steps if sum(len(e["tokens"]) for e in st["entries"]) >= 256)
        assert 0 < large < len(steps)
        assert len(norms) == 2 * large + (2 * LAYERS + 1) * (len(steps) - large), (len(norms), large, len(steps))
