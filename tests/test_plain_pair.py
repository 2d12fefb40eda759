"""The two plain implementations against each other (CPU): tests/plain_qwen3.py (PyTorch, float64, tensor algebra) and
tests/ref_cpp/plain_qwen3.cpp (C++, double, scalar loops), written separately from the reference's formulas. On four
tiny models that differ in every size and option they must agree to rounding.

Neither rests on the reference's own model code: mashriram/llm-rs is Rust on the candle crate and cannot be built here
(no Rust toolchain, no vendored crates), so there are no golden outputs of its own. Model code of other installed
libraries is deliberately not used as an oracle either: the architecture is taken from the reference's files alone.
"""
import os
import shutil
import subprocess

import numpy as np
import pytest

import plain_qwen3 as P
from tiny_configs import TINY, write_tiny_model

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def program(tmp_path_factory):
    cxx = shutil.which(os.environ.get("CXX", "g++")) or shutil.which("c++") or shutil.which("clang++")
    if cxx is None:
        pytest.skip("no C++ compiler")
    exe = str(tmp_path_factory.mktemp("ref_cpp") / "plain_qwen3")
    subprocess.run([cxx, "-O2", "-std=c++17", os.path.join(HERE, "ref_cpp", "plain_qwen3.cpp"), "-o", exe], check=True)
    return exe


def _export(cfg, w, folder):
    """The model as the C++ program reads it: a manifest and a float64 blob (written here, with numpy)."""
    L = cfg["num_hidden_layers"]
    lines = ["config layers=%d hidden=%d heads=%d kv_heads=%d head_dim=%d inter=%d vocab=%d theta=%r eps=%r tied=%d bias=%d" % (
        L, cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
        cfg["intermediate_size"], cfg["vocab_size"], float(cfg["rope_theta"]), float(cfg["rms_norm_eps"]),
        int(cfg.get("tie_word_embeddings", False)), int(cfg.get("attention_bias", False)))]
    lines.append("windows " + " ".join(str(x) for x in P.layer_windows(cfg)))
    lines.append("no_rope " + " ".join(str(int(x)) for x in (cfg.get("no_rope_layers") or [False] * L)))
    at, blobs = 0, []
    for name, t in w.items():
        a = t.double().numpy().reshape(-1)
        lines.append(f"tensor {name} {at} {a.size}")
        blobs.append(a)
        at += a.size
    manifest = os.path.join(folder, "model.manifest")
    with open(manifest, "w") as f:
        f.write("\n".join(lines) + "\n")
    np.concatenate(blobs).astype("<f8").tofile(manifest + ".bin")
    return manifest


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_two_plain_implementations_agree(program, name, tmp_path):
    path = write_tiny_model(name, str(tmp_path))
    cfg, w = P.load_model_dir(path)
    manifest = _export(cfg, w, str(tmp_path))
    n = {"A": 40, "B": 33, "C": 70, "D": 20}[name]        # C: beyond its window of 24 keys
    toks = np.random.default_rng(ord(name)).integers(0, cfg["vocab_size"], n).tolist()
    with open(tmp_path / "tokens.txt", "w") as f:
        f.write(" ".join(str(t) for t in toks))
    out = str(tmp_path / "logits.f64")
    subprocess.run([program, manifest, str(tmp_path / "tokens.txt"), out], check=True, timeout=600)
    theirs = np.fromfile(out, dtype="<f8").reshape(n, cfg["vocab_size"])
    ours = P.forward(cfg, w, toks).numpy()
    assert np.abs(ours - theirs).max() <= 1e-9 * max(1.0, np.abs(ours).max()), np.abs(ours - theirs).max()
