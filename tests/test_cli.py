"""The command line: ``random_model`` without a GPU, ``run_model`` and ``benchmark_speed`` on one."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from tiny_configs import TINY_A, TINY_B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cli(*args):
    return subprocess.run([sys.executable, "-m", "llm_rs_b200", *args], cwd=ROOT, capture_output=True, text=True,
                          timeout=600)


def test_random_model_writes_a_loadable_folder(tmp_path):
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(TINY_B))
    out = tmp_path / "model"
    done = _cli("random_model", "--config", str(cfg), "--out", str(out), "--seed", "7", "--sigma", "0.03",
                "--norm-jitter", "0.1")
    assert done.returncode == 0, done.stderr
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    conf, w = P.load_model_dir(str(out))
    assert conf["hidden_size"] == TINY_B["hidden_size"]
    assert w["model.layers.2.mlp.down_proj.weight"].shape == (TINY_B["hidden_size"], TINY_B["intermediate_size"])
    assert abs(float(w["model.embed_tokens.weight"].double().std()) - 0.03) < 0.003
    assert 0.05 < float(w["model.norm.weight"].double().std()) < 0.2
    # The same seed gives the same bytes, another seed other weights.
    again = tmp_path / "again"
    other = tmp_path / "other"
    assert _cli("random_model", "--config", str(cfg), "--out", str(again), "--seed", "7", "--sigma", "0.03",
                "--norm-jitter", "0.1").returncode == 0
    assert _cli("random_model", "--config", str(cfg), "--out", str(other), "--seed", "8").returncode == 0
    assert (out / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()
    assert (out / "model.safetensors").read_bytes() != (other / "model.safetensors").read_bytes()


def test_unknown_architecture_and_missing_options_are_refused(tmp_path):
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(dict(TINY_A, architectures=["NoSuchModel"], model_type="nosuch")))
    done = _cli("random_model", "--config", str(cfg), "--out", str(tmp_path / "m"))
    assert done.returncode != 0 and "NoSuchModel" in done.stderr
    assert _cli("run_model").returncode != 0          # --model-path is required, as in the reference


def test_option_names_and_defaults_follow_the_reference():
    """llm-cli/src/bin/run_model.rs:9-35 and benchmark_speed.rs:9-26: names, meanings, defaults."""
    text = _cli("run_model", "--help").stdout
    for option in ("--model-path", "--tokenizer-path", "--prompt", "--temperature", "--top-p", "--repetition-penalty"):
        assert option in text
    text = _cli("benchmark_speed", "--help").stdout
    assert "--max-new-tokens" in text and "--model-path" in text


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_model_generates_what_the_plain_implementation_does(tmp_path, dtype):
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(TINY_A))
    out = tmp_path / "model"
    assert _cli("random_model", "--config", str(cfg), "--out", str(out), "--seed", "3", "--sigma", "0.05",
                "--norm-jitter", "0.1").returncode == 0
    prompt = [5, 17, 3, 9, 200, 41]
    done = _cli("run_model", "--model-path", str(out), "--prompt-ids", ",".join(map(str, prompt)), "--dtype", dtype,
                "--max-new-tokens", "12", "--ignore-eos", "--page-size", "16", "--block-pool-size", "32")
    assert done.returncode == 0, done.stderr
    lines = dict(l.split(":", 1) for l in done.stdout.splitlines() if ":" in l)
    got = [int(t) for t in lines["Generated token ids"].split(",")]
    assert lines["Finish reason"].strip() == "length" and len(got) == 12
    for key in ("TTFT", "Prefill", "Decode", "Overall"):        # run_model.rs:131-150
        assert key in lines
    conf, w = P.load_model_dir(str(out))
    seq = list(prompt)
    for i, tok in enumerate(got):
        logits = P.forward(conf, w, seq)[-1]
        best = int(torch.argmax(logits))
        if tok != best:   # bfloat16 may turn a near tie the other way: the chosen token must be as good as the best
            assert dtype == "bfloat16" and float(logits[best] - logits[tok]) < 0.02 * float(logits.abs().max()), (i, tok, best)
        seq.append(tok)


@pytest.mark.gpu
def test_benchmark_speed_is_greedy_with_the_reference_default_length(tmp_path):
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(TINY_A))
    out = tmp_path / "model"
    assert _cli("random_model", "--config", str(cfg), "--out", str(out), "--seed", "3").returncode == 0
    a = _cli("benchmark_speed", "--model-path", str(out), "--prompt-len", "9", "--ignore-eos", "--block-pool-size", "32")
    b = _cli("run_model", "--model-path", str(out), "--prompt-len", "9", "--ignore-eos", "--block-pool-size", "32")
    assert a.returncode == 0 and b.returncode == 0, a.stderr + b.stderr
    ids = lambda text: [l for l in text.splitlines() if l.startswith("Generated token ids")][0]
    assert ids(a.stdout) == ids(b.stdout) and len(ids(a.stdout).split(",")) == 50      # benchmark_speed.rs:20
