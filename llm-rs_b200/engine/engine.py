"""The engine a user talks to: requests in, tokens out.

Python entry point in the manner of the reference's C API (llm-ffi/src/lib.rs:39-167:
create_engine, send_request, poll_token, destroy_engine) and of its scheduler's step
(llm-scheduler/src/scheduler.rs:51: a list of (sequence id, token, finished) per step),
on token ids: the reference's FFI "tokenizes" by character code (lib.rs:102) and this
engine depends on no tokenizer.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..sampling import Sampler, SamplingParams
from ..cache import OutOfPages
from .runner import ModelRunner, StepEntry
from .scheduler import Output, Request, Scheduled, Scheduler


@dataclass
class EngineConfig:
    """``model_path`` and ``block_pool_size`` are the reference's two fields
    (llm-ffi/src/lib.rs:10-15; pool default 1024 pages as llm-cli/src/main.rs:23); the
    rest configures what the reference fixes in code or does not have."""
    model_path: str
    block_pool_size: int = 1024          # pages in the cache pool
    page_size: int = 16                  # llm-core/src/backends/candle.rs:827
    dtype: str = "bfloat16"              # "bfloat16" or "float32"
    device: str = "cuda:0"
    max_requests: int = 64               # live requests (state slots)
    max_tokens_per_step: int = 2048
    prefill_chunk: int = 512
    cuda_graphs: bool = True
    # Queue the next step on the GPU before the last one's tokens are read back (they feed
    # the next step on the device); ``step()`` then reports a step's tokens one call later.
    async_steps: bool = True


class Engine:
    def __init__(self, config: EngineConfig, runner: Optional[ModelRunner] = None):
        self.config = config
        dtype = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
                 "fp32": torch.float32}[config.dtype]
        self.runner = runner or ModelRunner.from_model_dir(
            config.model_path, dtype=dtype, device=config.device,
            max_tokens=config.block_pool_size * config.page_size, page_size=config.page_size,
            max_requests=config.max_requests)
        self.runner.use_graphs = config.cuda_graphs
        self.scheduler = Scheduler(
            self.runner.manager, self.runner.max_positions, self.runner.spec.eos_token_ids,
            max_tokens_per_step=config.max_tokens_per_step, prefill_chunk=config.prefill_chunk,
            max_requests_per_step=config.max_requests)
        self.sampler = Sampler(self.runner.device)
        self._ids = itertools.count(1)
        self.requests: Dict[int, Request] = {}
        self._events: Dict[int, List[Output]] = {}
        self._inflight = None            # the step that is queued on the GPU and not read back yet
        self._tok_bufs = [None, None]
        self._tok_flip = 0
        self.d2h_bytes = 0               # bytes read back so far: 4 per sampled token and 4 for the error word per step
        from .. import ops
        self._error_word = ops.tc_error_flag(self.runner.device)   # written by a kernel whose bounded wait ran out
        # What the steps were made of: steps of decoded tokens only, of prompt portions only, of both;
        # tokens that entered the model as prompt portions and as single decoded tokens.
        self.stats = {"steps": 0, "decode_steps": 0, "prefill_steps": 0, "mixed_steps": 0,
                      "prompt_tokens": 0, "decode_tokens": 0, "max_step_tokens": 0}

    # -- requests --------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        """Queue a request; returns its id (ids start at 1; 0 is the reference's failure value)."""
        params = params or SamplingParams()
        vocab = self.runner.spec.vocab_size
        for t in prompt_token_ids:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        rid = next(self._ids)
        req = Request(rid, [int(t) for t in prompt_token_ids], params)
        self.scheduler.add_request(req)
        self.requests[rid] = req
        self._events[rid] = []
        return rid

    # -- one step --------------------------------------------------------------------
    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    def step(self) -> List[Tuple[int, Optional[int], bool]]:
        """Run one scheduler step. Returns ``(request id, token, finished)`` for every
        request whose token became known or that ended in this call. With ``async_steps``
        the tokens of a step are reported by the NEXT call: the step is queued on the GPU,
        then the previous step's tokens are read while it runs.

        If the step function, the sampler or a kernel fails (a kernel reports through the error word
        that travels with every step's tokens), every running request ends with ``error_step_failed``,
        its pages go back, and the exception is raised (llm-scheduler/src/engine.rs:92-99). ``OutOfPages``
        from a caller who shares the cache with this engine ends nothing: the step is dropped and raised,
        and the next call schedules again."""
        try:
            return self._step()
        except OutOfPages:
            raise
        except Exception:
            # A step that was queued earlier may still be in flight: its tokens were sampled and are
            # reported, and the scheduler closes its batch, before everything is aborted.
            outs: List[Output] = []
            if self._inflight is not None:
                flight, self._inflight = self._inflight, None
                try:
                    outs += self._collect(flight)
                except Exception:
                    pass            # its tokens cannot be read either; abort_all closes its batch
            outs += self.scheduler.abort_all()
            for o in outs:
                self._events.setdefault(o.request_id, []).append(o)
            raise

    def _step(self) -> List[Tuple[int, Optional[int], bool]]:
        batch = self.scheduler.schedule()
        launched = None
        if batch:
            prev = self._inflight
            entries = []
            for s in batch:
                src = prev["row_of"][s.request.request_id] if s.pending else -1
                entries.append(StepEntry(s.request.request_id, s.tokens, [len(s.tokens) - 1] if s.sample else [],
                                         device_token=src))
            try:
                logits = self.runner.step(entries, token_source=prev["tokens"] if prev else None)
            except OutOfPages:
                self.scheduler.cancel(batch)
                raise
            sampled = [s for s in batch if s.sample]
            tokens = None
            if sampled:
                rows = [(s.request.params, s.request.request_id, len(s.request.output) + s.request.n_inflight,
                         s.request.tokens() if s.request.params.repetition_penalty != 1.0 else ())
                        for s in sampled]
                tokens = self.sampler.sample(logits, rows)
            # The step's tokens and, behind them, the kernels' error word: one pinned buffer.
            n = len(sampled)
            host = self._token_buffer(n + 1)
            if n:
                host[:n].copy_(tokens, non_blocking=True)
            host[n:].copy_(self._error_word, non_blocking=True)
            self.d2h_bytes += 4 * (n + 1)
            event = torch.cuda.Event()
            event.record()
            self.scheduler.on_launched(batch)
            n_dec = sum(1 for s in batch if len(s.tokens) == 1 and s.sample)
            n_pre = sum(len(s.tokens) for s in batch) - n_dec
            st = self.stats
            st["steps"] += 1
            st["decode_steps" if not n_pre else "prefill_steps" if not n_dec else "mixed_steps"] += 1
            st["prompt_tokens"] += n_pre
            st["decode_tokens"] += n_dec
            st["max_step_tokens"] = max(st["max_step_tokens"], n_pre + n_dec)
            launched = {"batch": batch, "tokens": tokens, "host": host, "event": event,
                        "row_of": {s.request.request_id: i for i, s in enumerate(sampled)}}
        outs: List[Output] = []
        if self._inflight is not None:
            flight, self._inflight = self._inflight, launched
            outs += self._collect(flight)
        self._inflight = launched
        # Read this step's tokens at once when the caller asked for that, or when a request
        # needs its full history on the host for the next step (repetition penalty).
        if launched is not None and (not self.config.async_steps or any(
                s.request.params.repetition_penalty != 1.0 for s in batch)):
            self._inflight = None
            outs += self._collect(launched)
        if launched is None and self._inflight is None:
            outs += self.scheduler.on_result([], {})    # requests that ended without a step
        for o in outs:
            self._events.setdefault(o.request_id, []).append(o)
        return [(o.request_id, o.token, o.finished) for o in outs]

    def _token_buffer(self, n: int) -> torch.Tensor:
        """Pinned host memory for a step's sampled tokens (two buffers: one step is in flight)."""
        self._tok_flip ^= 1
        buf = self._tok_bufs[self._tok_flip]
        if buf is None or buf.numel() < n:
            buf = torch.empty((max(n, 64),), dtype=torch.int32).pin_memory()
            self._tok_bufs[self._tok_flip] = buf
        return buf[:n]

    def _collect(self, flight) -> List[Output]:
        """Wait for a queued step's tokens and let the scheduler account for them. The kernels' error
        word came with the tokens: a kernel that gave up on a bounded wait fails this very step."""
        flight["event"].synchronize()
        values = flight["host"].tolist()
        if values[-1]:
            self._error_word.zero_()
            from ..ops import KernelError, tc_error_message
            raise KernelError(tc_error_message(values[-1]))
        sampled = {rid: values[i] for rid, i in flight["row_of"].items()}
        return self.scheduler.on_result(flight["batch"], sampled)

    def check_kernels(self) -> None:
        """Raise if a kernel with bounded waits (tcgen05 product or attention) gave up on one since the
        last check. ``step`` sees the same word with every step's tokens; this reads it on demand."""
        self.runner.check_kernels()

    # -- conveniences ----------------------------------------------------------------
    def poll(self, request_id: int) -> Output:
        """The next event of one request, stepping the engine until there is one
        (the blocking ``poll_token`` of llm-ffi/src/lib.rs:127-158)."""
        if request_id not in self._events:
            raise KeyError(f"unknown request {request_id}")
        while not self._events[request_id]:
            if not self.has_work():
                raise RuntimeError(f"request {request_id} has no further events")
            self.step()
        return self._events[request_id].pop(0)

    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> List[List[int]]:
        """Generate for a batch of prompts (token ids in, token ids out)."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while self.has_work():
            self.step()
        out = []
        for rid in ids:
            out.append(list(self.requests[rid].output))
            self.forget(rid)
        return out

    def finish_reason(self, request_id: int) -> Optional[str]:
        return self.requests[request_id].finish_reason

    def forget(self, request_id: int) -> None:
        """Drop the record of a finished request."""
        self.requests.pop(request_id, None)
        self._events.pop(request_id, None)


# -- the reference's five verbs ------------------------------------------------------------
@dataclass
class ChatRequest:
    """llm-ffi/src/lib.rs:17-23, with token ids where the reference has a prompt string.
    top_k 40 and repetition_penalty 1.1 are what the reference's ``send_request`` fixes
    (lib.rs:110-111); here they are fields with neutral defaults."""
    prompt: Sequence[int]
    temperature: float = 0.0
    top_p: float = 1.0
    max_tokens: int = 50
    top_k: int = 0
    repetition_penalty: float = 1.0
    seed: int = 0


@dataclass
class GenerationResult:
    """llm-ffi/src/lib.rs:25-29 without the text field (no tokenizer here)."""
    token: int
    is_eos: bool
    reason: Optional[str] = None


def create_engine(config: EngineConfig) -> Engine:
    return Engine(config)


def send_request(engine: Engine, request: ChatRequest) -> int:
    return engine.add_request(request.prompt, SamplingParams(
        temperature=request.temperature, top_p=request.top_p, top_k=request.top_k,
        repetition_penalty=request.repetition_penalty, max_new_tokens=request.max_tokens, seed=request.seed))


def poll_token(engine: Engine, request_id: int) -> GenerationResult:
    o = engine.poll(request_id)
    return GenerationResult(token=-1 if o.token is None else o.token, is_eos=o.finished, reason=o.reason)


def destroy_engine(engine: Engine) -> None:
    for rid in list(engine.runner.manager.requests):
        engine.runner.release(rid)
    engine.requests.clear()
