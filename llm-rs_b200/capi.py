"""The Python side of the engine's C entry points (``csrc/capi/llm_engine.h``): the engines that C callers
created, by handle. Every function takes and returns plain integers and floats, so that the C library needs
nothing of the interpreter but calling a function; the engine behind a handle is the package's ``Engine``,
the one every other entry point uses (llm-ffi/src/lib.rs:39-167 is the reference's counterpart).
"""
from __future__ import annotations

import ctypes
import itertools
from typing import Dict

_engines: Dict[int, object] = {}
_handles = itertools.count(1)
REASONS = {None: 0, "stop": 1, "length": 2, "error_too_long": 3, "error_step_failed": 4}


def create(model_path: str, block_pool_size: int, page_size: int, dtype: str, max_requests: int, cuda_graphs: int) -> int:
    from .engine import Engine, EngineConfig
    cfg = EngineConfig(model_path=model_path)
    if block_pool_size > 0:
        cfg.block_pool_size = block_pool_size
    if page_size > 0:
        cfg.page_size = page_size
    if dtype:
        cfg.dtype = dtype
    if max_requests > 0:
        cfg.max_requests = max_requests
    if cuda_graphs:
        cfg.cuda_graphs = cuda_graphs > 0
    handle = next(_handles)
    _engines[handle] = Engine(cfg)
    return handle


def _engine(handle: int):
    try:
        return _engines[handle]
    except KeyError:
        raise ValueError(f"no engine with handle {handle}") from None


def submit(handle: int, prompt_addr: int, n_prompt: int, temperature: float, top_p: float, repetition_penalty: float,
           top_k: int, max_tokens: int, seed: int, ignore_eos: int) -> int:
    from .sampling import SamplingParams
    prompt = list((ctypes.c_int32 * n_prompt).from_address(prompt_addr))
    params = SamplingParams(temperature=temperature, top_p=top_p or 1.0, top_k=top_k,
                            repetition_penalty=repetition_penalty or 1.0, max_new_tokens=max_tokens or 50, seed=seed,
                            ignore_eos=bool(ignore_eos))
    return _engine(handle).add_request(prompt, params)


def poll(handle: int, request_id: int) -> int:
    """The request's next event as one integer: token (low 32 bits, all ones for none), finished (bit 32),
    reason (bits 40-47). Steps the engine until the request has an event."""
    engine = _engine(handle)
    o = engine.poll(request_id)
    if o.finished:
        engine.forget(request_id)
    token = 0xFFFFFFFF if o.token is None else o.token & 0xFFFFFFFF
    return token | (int(o.finished) << 32) | (REASONS.get(o.reason, 4) << 40)


def step(handle: int) -> int:
    return len(_engine(handle).step())


def has_work(handle: int) -> int:
    return int(_engine(handle).has_work())


def destroy(handle: int) -> int:
    from .engine import destroy_engine
    engine = _engines.pop(handle, None)
    if engine is not None:
        destroy_engine(engine)
    return 0
