"""The engine's C entry points (csrc/capi/llm_engine.h), driven the way the reference drives its own
(tests/test_parity.py:7-27,78-93 mirrors the C structs with ctypes, creates an engine, sends two requests and
polls tokens until each ends): once through ctypes from this process, once from a plain C program that starts
its own interpreter. Both must give the plain implementation's greedy tokens. Nothing here imports the
engine's Python classes."""
import ctypes
import os
import shutil
import subprocess
import sys

import numpy as np
import pytest

import plain_qwen3 as P
from tiny_configs import write_tiny_model

pytestmark = pytest.mark.gpu


class LlmEngineConfig(ctypes.Structure):
    _fields_ = [("model_path", ctypes.c_char_p), ("block_pool_size", ctypes.c_int), ("dtype", ctypes.c_char_p),
                ("page_size", ctypes.c_int), ("max_requests", ctypes.c_int), ("cuda_graphs", ctypes.c_int)]


class LlmRequest(ctypes.Structure):
    _fields_ = [("prompt", ctypes.POINTER(ctypes.c_int32)), ("n_prompt", ctypes.c_int), ("temperature", ctypes.c_float),
                ("top_p", ctypes.c_float), ("top_k", ctypes.c_int), ("repetition_penalty", ctypes.c_float),
                ("max_tokens", ctypes.c_int), ("seed", ctypes.c_uint64), ("ignore_eos", ctypes.c_int)]


class LlmResult(ctypes.Structure):
    _fields_ = [("token", ctypes.c_int32), ("finished", ctypes.c_int), ("reason", ctypes.c_int)]


@pytest.fixture(scope="module")
def library():
    from llm_rs_b200.csrc import build
    path = build.build_engine_api()
    lib = ctypes.CDLL(path)
    lib.llm_create.restype, lib.llm_create.argtypes = ctypes.c_void_p, [ctypes.POINTER(LlmEngineConfig)]
    lib.llm_submit.restype, lib.llm_submit.argtypes = ctypes.c_uint64, [ctypes.c_void_p, ctypes.POINTER(LlmRequest)]
    lib.llm_poll.restype, lib.llm_poll.argtypes = ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(LlmResult)]
    lib.llm_step.restype, lib.llm_step.argtypes = ctypes.c_int, [ctypes.c_void_p]
    lib.llm_has_work.restype, lib.llm_has_work.argtypes = ctypes.c_int, [ctypes.c_void_p]
    lib.llm_destroy.restype, lib.llm_destroy.argtypes = ctypes.c_int, [ctypes.c_void_p]
    lib.llm_last_error.restype = ctypes.c_char_p
    return lib, path


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    path = write_tiny_model("A", str(tmp_path_factory.mktemp("capi")))
    cfg, w = P.load_model_dir(path)
    rng = np.random.default_rng(13)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (7, 21)]
    want = [P.greedy_generate(cfg, w, p, 6) for p in prompts]
    return path, cfg, prompts, want


def _request(prompt, **kw):
    arr = (ctypes.c_int32 * len(prompt))(*prompt)
    req = LlmRequest(prompt=arr, n_prompt=len(prompt), **kw)
    req._keep = arr
    return req


def test_create_submit_poll_destroy_through_ctypes(library, model):
    lib, _ = library
    path, cfg, prompts, want = model
    engine = lib.llm_create(ctypes.byref(LlmEngineConfig(model_path=path.encode(), block_pool_size=32, dtype=b"float32")))
    assert engine, lib.llm_last_error().decode()
    ids = [lib.llm_submit(engine, ctypes.byref(_request(p, max_tokens=6, ignore_eos=1))) for p in prompts]
    assert all(ids) and ids[0] != ids[1], lib.llm_last_error().decode()
    got = [[], []]
    for k in (1, 0):                                # poll the second request first: polling steps the engine for both
        res = LlmResult()
        while True:
            assert lib.llm_poll(engine, ids[k], ctypes.byref(res)) == 0, lib.llm_last_error().decode()
            got[k].append(res.token)
            if res.finished:
                assert res.reason == 2              # LLM_LENGTH
                break
    assert got == want
    assert lib.llm_has_work(engine) == 0
    # A caller that drives the loop itself: llm_step until the request's events are all there.
    rid = lib.llm_submit(engine, ctypes.byref(_request(prompts[0], max_tokens=3, ignore_eos=1)))
    steps = 0
    while lib.llm_has_work(engine) == 1:
        assert lib.llm_step(engine) >= 0, lib.llm_last_error().decode()
        steps += 1
    assert 3 <= steps <= 6
    toks, res = [], LlmResult()
    for _ in range(3):
        assert lib.llm_poll(engine, rid, ctypes.byref(res)) == 0
        toks.append(res.token)
    assert toks == want[0][:3] and res.finished
    # Errors come back as codes with a message, not as crashes.
    assert lib.llm_poll(engine, 987654, ctypes.byref(res)) != 0 and b"987654" in lib.llm_last_error()
    assert lib.llm_submit(engine, ctypes.byref(_request([10 ** 6], max_tokens=1))) == 0
    assert b"vocabulary" in lib.llm_last_error()
    assert lib.llm_destroy(engine) == 0
    assert lib.llm_create(ctypes.byref(LlmEngineConfig(model_path=b"/nonexistent/model"))) is None
    assert b"config.json" in lib.llm_last_error()


C_PROGRAM = r"""
#include <stdio.h>
#include <stdlib.h>
#include "llm_engine.h"

int main(int argc, char** argv) {
    LlmEngineConfig cfg = {0};
    cfg.model_path = argv[1];
    cfg.block_pool_size = 32;
    cfg.dtype = "float32";
    void* engine = llm_create(&cfg);
    if (!engine) { fprintf(stderr, "create: %s\n", llm_last_error()); return 1; }
    int n = argc - 2;
    int32_t* prompt = malloc(sizeof(int32_t) * n);
    for (int i = 0; i < n; ++i) prompt[i] = atoi(argv[2 + i]);
    LlmRequest req = {0};
    req.prompt = prompt; req.n_prompt = n; req.max_tokens = 6; req.ignore_eos = 1;
    uint64_t id = llm_submit(engine, &req);
    if (!id) { fprintf(stderr, "submit: %s\n", llm_last_error()); return 2; }
    LlmResult r;
    do {
        if (llm_poll(engine, id, &r) != 0) { fprintf(stderr, "poll: %s\n", llm_last_error()); return 3; }
        printf("%d\n", r.token);
    } while (!r.finished);
    if (llm_destroy(engine) != 0) return 4;
    free(prompt);
    return 0;
}
"""


def test_a_plain_c_program_gets_tokens(library, model, tmp_path):
    """No Python in the caller: the library starts the interpreter it was built against."""
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    _, lib_path = library
    path, cfg, prompts, want = model
    src = tmp_path / "main.c"
    src.write_text(C_PROGRAM)
    from llm_rs_b200.csrc import build
    exe = tmp_path / "caller"
    subprocess.run([cc, str(src), "-I", build.CAPI_DIR, "-L", os.path.dirname(lib_path), "-lllmrs_b200_engine",
                    f"-Wl,-rpath,{os.path.dirname(lib_path)}", "-o", str(exe)], check=True)
    env = {k: v for k, v in os.environ.items() if not k.startswith("PYTHON")}
    run = subprocess.run([str(exe), path, *[str(t) for t in prompts[1]]], capture_output=True, text=True, timeout=600,
                         env=env)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [int(t) for t in run.stdout.split()] == want[1]
