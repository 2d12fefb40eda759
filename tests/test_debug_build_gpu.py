"""The debug build of the kernel library (LLMRS_DEBUG_KERNELS=1): the kernels check the page ids and token ids they
are about to use, record a bad one and go on inside their buffers. A child process (the variant is chosen at import)
replays a mixed trace on a model with a window group, where released pages (-1) sit in the block tables, and finds
no record; then it hands attention a table whose visible page is -1 and a token id beyond the vocabulary, and
finds them recorded, with nothing trapped and the context alive."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))

CHILD = r"""
import sys
sys.path[:0] = [%(root)r, %(here)r]
import math, numpy as np, torch
import plain_qwen3 as P, replay_util as RU
from tiny_configs import TINY, write_tiny_model
from llm_rs_b200 import ops
from llm_rs_b200.csrc import build
from llm_rs_b200.engine import ModelRunner
assert build.DEBUG_KERNELS and build.LIB_NAME.endswith("_debug.so")
for name, dtype in (("C", torch.float32), ("C", torch.bfloat16), ("D", torch.bfloat16)):
    path = write_tiny_model(name, %(tmp)r)
    cfg, w = P.load_model_dir(path)
    rng = np.random.default_rng(5)
    reqs = {f"r{i}": rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in enumerate((70, 33, 150, 9, 64))}
    steps = RU.mixed(reqs, seed=2, sizes=(2, 17, 40, 130))
    runner = ModelRunner.from_model_dir(path, dtype=dtype, max_tokens=RU.live_token_peak(steps), page_size=TINY[name][3], max_requests=4)
    got = RU.run_steps(runner, steps)
    ref = {r: P.forward(cfg, w, t).numpy() for r, t in reqs.items()}
    worst, where, n = RU.max_diff(got, ref)
    assert worst <= (1e-4 if dtype == torch.float32 else 0.02 * max(float(np.abs(r).max()) for r in ref.values())), (name, worst, where)
    assert ops.debug_take() is None, "a healthy replay tripped an index check"
print("replay clean")
# A table that names no page for a key the query sees: recorded, read from page 0 instead, no fault.
nq, nkv, d, page = 4, 2, 64, 16
cache = torch.randn(8, nkv, 2, page, d, device="cuda").to(torch.bfloat16)
q = torch.randn(1, nq * d, device="cuda").to(torch.bfloat16)
out = torch.empty_like(q)
table = torch.tensor([[3, -1, 5]], dtype=torch.int32, device="cuda")
one = lambda v: torch.tensor([v], dtype=torch.int32, device="cuda")
scratch = torch.empty(ops.attn_decode_scratch_floats(1, nq, d, 1), device="cuda")
ops.attn_decode(q, out, cache, one(0), 1, one(0), one(40), table, scratch, 1, 128, nq, nkv, d, page, 0, 1 / math.sqrt(d))
rec = ops.debug_take()
assert rec is not None and rec[0] == 4 and rec[1] == -1 and rec[3] >= 1, rec
assert torch.isfinite(out.float()).all()
emb = torch.randn(10, 32, device="cuda").to(torch.bfloat16)
h = ops.embedding(emb, torch.tensor([3, 99, 4], dtype=torch.int32, device="cuda"))
rec = ops.debug_take()
assert rec is not None and rec[:3] == (1, 99, 1), rec
assert ops.debug_take() is None            # reading clears
torch.cuda.synchronize()
print("checks recorded")
"""


def test_debug_build_checks_indices(tmp_path):
    env = dict(os.environ, LLMRS_DEBUG_KERNELS="1")
    code = CHILD % {"root": os.path.dirname(HERE), "here": HERE, "tmp": str(tmp_path)}
    run = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=1500)
    assert run.returncode == 0, run.stdout[-1500:] + run.stderr[-3000:]
    assert "replay clean" in run.stdout and "checks recorded" in run.stdout


def test_normal_build_says_it_checks_nothing():
    from llm_rs_b200 import ops
    with pytest.raises(ops.KernelError, match="not the debug build"):
        ops.debug_take()
