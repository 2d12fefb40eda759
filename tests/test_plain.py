"""The plain implementation checked against itself (CPU): properties that the formulas
imply, so that a slip in the oracle does not go unnoticed."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from tiny_configs import write_tiny_model


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    folder = str(tmp_path_factory.mktemp("m"))
    return {n: P.load_model_dir(write_tiny_model(n, folder)) for n in "ABC"}


def test_rms_norm_formula():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = P.rms_norm(x, w, 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]], dtype=torch.float64))


def test_rotation_depends_on_relative_position_only():
    torch.manual_seed(0)
    q, k = torch.randn(1, 1, 16, dtype=torch.float64), torch.randn(1, 1, 16, dtype=torch.float64)
    def score(pq, pk):
        return float((P.rotate_half(q, P.rope_angles([pq], 16, 1e4, torch.float64))
                      * P.rotate_half(k, P.rope_angles([pk], 16, 1e4, torch.float64))).sum())
    assert abs(score(5, 2) - score(105, 102)) < 1e-9
    assert abs(score(5, 2) - score(5, 3)) > 1e-6
    x = torch.randn(1, 1, 16, dtype=torch.float64)
    assert torch.equal(P.rotate_half(x, P.rope_angles([0], 16, 1e4, torch.float64)), x)   # position 0: identity


def test_causality_and_window(models):
    cfg, w = models["C"]
    ids = np.random.default_rng(0).integers(0, cfg["vocab_size"], 60).tolist()
    full = P.forward(cfg, w, ids)
    changed = list(ids)
    changed[40] = (changed[40] + 1) % cfg["vocab_size"]
    other = P.forward(cfg, w, changed)
    assert torch.equal(full[:40], other[:40])                  # later tokens do not reach back
    assert not torch.allclose(full[40:], other[40:])
    # A window wider than the sequence is no window.
    wide = dict(cfg, sliding_window=1000)
    none = {k: v for k, v in cfg.items() if k != "layer_types"}
    none["use_sliding_window"] = False
    assert torch.allclose(P.forward(wide, w, ids), P.forward(none, w, ids), atol=1e-12)
    assert not torch.allclose(full, P.forward(none, w, ids), atol=1e-6)   # the window of 24 does cut


def test_attention_matches_a_loop():
    torch.manual_seed(1)
    T, nq, nkv, d, window = 9, 4, 2, 8, 4
    q, k, v = (torch.randn(T, n, d, dtype=torch.float64) for n in (nq, nkv, nkv))
    got = P.attention(q, k, v, window).reshape(T, nq, d)
    for t in range(T):
        for h in range(nq):
            lo = max(0, t - window + 1)
            s = torch.stack([q[t, h] @ k[j, h // 2] / math.sqrt(d) for j in range(lo, t + 1)])
            p = torch.softmax(s, 0)
            want = sum(p[j - lo] * v[j, h // 2] for j in range(lo, t + 1))
            assert torch.allclose(got[t, h], want, atol=1e-12)


def test_float32_agrees_with_float64(models):
    for name in "AB":
        cfg, w = models[name]
        ids = np.random.default_rng(1).integers(0, cfg["vocab_size"], 50).tolist()
        a = P.forward(cfg, w, ids)
        b = P.forward(cfg, {k: v.float() for k, v in w.items()}, ids)
        assert float((a - b.double()).abs().max()) < 1e-4


def test_tied_head_uses_the_embedding(models):
    cfg, w = models["A"]
    assert cfg["tie_word_embeddings"] and "lm_head.weight" not in w


def test_philox_known_answer():
    # Random123 known-answer vectors for philox4x32-10.
    assert P.philox4x32_10((0, 0), (0, 0, 0, 0)) == (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)
    assert P.philox4x32_10((0xFFFFFFFF, 0xFFFFFFFF), (0xFFFFFFFF,) * 4) == (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)
    assert P.philox4x32_10((0xA4093822, 0x299F31D0), (0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344)) == \
        (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)
    u = [P.uniform(7, r, i) for r in range(3) for i in range(50)]
    assert all(0 <= x < 1 for x in u) and len(set(u)) == len(u) and 0.3 < float(np.mean(u)) < 0.7


def test_plain_sampler_rules():
    logits = np.array([1.0, 3.0, 3.0, -2.0, 0.5])
    assert P.sample(logits, 0.0) == 1                               # first maximum
    assert P.sample(logits, 0.0, repetition_penalty=2.0, history=[1, 1]) == 2   # 3/2 < 3, penalised once
    p = P.kept_probabilities(logits, 1.0, top_k=2)
    assert np.count_nonzero(p) == 2 and abs(p.sum() - 1) < 1e-12
    p = P.kept_probabilities(logits, 1.0, top_p=0.5)
    assert np.count_nonzero(p) == 2                                 # ties at the cut-off are kept
    p = P.kept_probabilities(np.array([2.0, -1.0]), 1.0, repetition_penalty=2.0, history=[0, 1])
    q = np.exp([1.0, -2.0]); q /= q.sum()
    assert np.allclose(p, q)                                        # divide if positive, multiply if negative
    draws = [P.sample(logits, 0.7, seed=3, request_id=1, index=i) for i in range(400)]
    assert set(draws) <= {0, 1, 2, 3, 4} and draws.count(1) > 100 and draws.count(2) > 100
