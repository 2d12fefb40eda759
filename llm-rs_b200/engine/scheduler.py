"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees. Host logic only; it decides, the step function runs.

What the reference does (llm-scheduler/src/scheduler.rs:51-190): first come first
served; a request is admitted when pages for its WHOLE prompt are free, else the queue
waits behind it; every running sequence is in every step, whole prompt or one token;
a sequence ends at the EOS token or at max_new_tokens (the last token is emitted);
when a page is missing during decoding the sequence is dropped without a word
(scheduler.rs:168-171).

What this scheduler does differently, and why:
  * a token budget per step, decoded tokens first, the rest to prompt portions in order
    of arrival (a long prompt does not stall the requests that are decoding);
  * admission needs pages for the first portion only;
  * when pages run out, the request admitted LAST is preempted: its pages go back, it
    returns to the front of the waiting queue and later recomputes prompt + generated
    tokens. Nothing is dropped. A request that cannot fit although it is alone is
    finished with reason "error_too_long".
  * a step's result may be read one step late (``on_launched`` when the step is queued on
    the GPU, ``on_result`` when its tokens are on the host): the next step is scheduled
    while the tokens of the last one are still unknown. A request whose next token is
    "in flight" is scheduled with that token taken from the device; one that will end by
    its length is not scheduled further; one that turns out to have ended at EOS has its
    last, superfluous token dropped.

The decisions are made in C++ (``csrc/host/scheduler.cpp``), which knows requests by their
lengths; this module keeps the requests' tokens and parameters, hands the library the numbers
it needs and mirrors its state into the ``Request`` objects after every call.
"""
from __future__ import annotations

from ctypes import byref, c_int, c_int32, c_int64, c_void_p
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from .. import host
from ..cache.manager import CacheManager
from ..cache.pool import check
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    request_id: int
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    n_computed: int = 0          # tokens of prompt+output whose keys and values are cached
    status: str = WAITING
    finish_reason: Optional[str] = None
    preemptions: int = 0
    n_inflight: int = 0          # tokens sampled on the device that the host has not read yet (0 or 1)

    def tokens(self) -> List[int]:
        return self.prompt + self.output

    def token_slice(self, a: int, b: int) -> List[int]:
        """Tokens a..b-1 of prompt + output without building the whole list."""
        p = len(self.prompt)
        if b <= p:
            return self.prompt[a:b]
        if a >= p:
            return self.output[a - p:b - p]
        return self.prompt[a:] + self.output[:b - p]

    @property
    def n_known(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def remaining(self) -> int:
        """Tokens whose keys and values are not computed (or queued) yet, the in-flight one included."""
        return self.n_known + self.n_inflight - self.n_computed


@dataclass
class Scheduled:
    """One request's share of the next step."""
    request: Request
    tokens: List[int]
    sample: bool                 # the last of these tokens yields the request's next token
    pending: bool = False        # the single token is the request's in-flight one (not on the host yet)


@dataclass
class Output:
    request_id: int
    token: Optional[int]
    finished: bool
    reason: Optional[str] = None


_STATUS = {0: WAITING, 1: RUNNING, 2: FINISHED}
_REASON = {0: None, 1: "stop", 2: "length", 3: "error_too_long", 4: "error_step_failed"}


class Batch(list):
    """The ``Scheduled`` entries of one step, with the library's handle of the step."""
    handle = 0


class Scheduler:
    def __init__(self, manager: CacheManager, max_positions: int, eos_token_ids: Sequence[int] = (),
                 max_tokens_per_step: int = 2048, prefill_chunk: int = 512, max_requests_per_step: int = 64):
        self.manager = manager
        self.max_positions = max_positions
        self.eos = set(eos_token_ids)
        self.max_tokens_per_step = max_tokens_per_step
        self.prefill_chunk = prefill_chunk
        self.max_requests_per_step = max_requests_per_step
        self._lib = host.lib()
        self._handle = c_void_p()
        eos = (c_int32 * max(len(self.eos), 1))(*sorted(self.eos))
        check(self._lib.llmrs_sched_create(manager._handle, max_positions, eos, len(self.eos), max_tokens_per_step,
                                           prefill_chunk, max_requests_per_step, byref(self._handle)))
        self._requests: Dict[int, Request] = {}
        self._ids = (c_int64 * 64)()
        self._fields = (c_int32 * (4 * 64))()

    def __del__(self):
        if getattr(self, "_handle", None):
            self._lib.llmrs_sched_destroy(self._handle)
            self._handle = None

    # -- plumbing --------------------------------------------------------------------
    def _buffers(self, n: int):
        if len(self._ids) < n:
            self._ids = (c_int64 * (2 * n))()
            self._fields = (c_int32 * (8 * n))()
        return self._ids, self._fields

    def _take(self, which: int) -> List[int]:
        ids, _ = self._buffers(len(self._requests) + 8)
        n = c_int()
        check(self._lib.llmrs_sched_take(self._handle, which, ids, len(ids), byref(n)))
        return list(ids[:n.value])

    def _sync(self) -> None:
        """Give back the pages of the requests that the library released, and copy the state of
        the requests it touched into their ``Request`` objects."""
        for rid in self._take(0):
            if rid in self.manager.requests:
                self.manager.release(rid)
        state = (c_int32 * 6)()
        for rid in set(self._take(1)):
            req = self._requests.get(rid)
            if req is None:
                continue
            check(self._lib.llmrs_sched_get(self._handle, rid, state))
            req.status, req.finish_reason = _STATUS[state[0]], _REASON[state[1]] if state[0] == 2 else None
            req.n_computed, req.n_inflight, req.preemptions = state[3], state[4], state[5]
            if state[0] == 2 and state[4] == 0:
                if getattr(req, "_abort_reason", None):
                    req.finish_reason = req._abort_reason
                self._lib.llmrs_sched_forget(self._handle, rid)
                del self._requests[rid]

    def _outputs(self, n: int) -> List[Output]:
        outs = []
        for i in range(n):
            rid, token, finished, reason = self._ids[i], self._fields[3 * i], self._fields[3 * i + 1], self._fields[3 * i + 2]
            if token >= 0:
                self._requests[rid].output.append(token)
            outs.append(Output(rid, token if token >= 0 else None, bool(finished), _REASON[reason]))
        return outs

    # -- intake ----------------------------------------------------------------------
    def add_request(self, request: Request) -> None:
        rid = request.request_id
        if not isinstance(rid, int) or isinstance(rid, bool) or not 0 <= rid < 2 ** 62:
            raise ValueError(f"the scheduler takes non-negative integer request ids, got {rid!r}")
        request.status = WAITING
        check(self._lib.llmrs_sched_add(self._handle, rid, len(request.prompt) + len(request.output),
                                        request.params.max_new_tokens - len(request.output),
                                        int(request.params.ignore_eos)))
        self._requests[rid] = request

    def has_work(self) -> bool:
        out = c_int()
        check(self._lib.llmrs_sched_has_work(self._handle, byref(out)))
        return bool(out.value)

    # -- views -----------------------------------------------------------------------
    @property
    def waiting(self) -> List[Request]:
        return [self._requests[i] for i in self._take(2)]

    @property
    def running(self) -> List[Request]:
        return [self._requests[i] for i in self._take(3)]

    @property
    def stats(self) -> Dict[str, int]:
        v = (c_int64 * 3)()
        check(self._lib.llmrs_sched_stats(self._handle, v))
        return {"steps": v[0], "preemptions": v[1], "tokens": v[2]}

    # -- one step --------------------------------------------------------------------
    def schedule(self) -> Batch:
        """Decide the next step's batch. May preempt (see the module's header) and may
        finish requests that can never fit; those show up in the next ``on_result``."""
        ids, fields = self._buffers(self.max_requests_per_step)
        n, handle = c_int(), c_int64()
        check(self._lib.llmrs_sched_schedule(self._handle, ids, fields, len(ids), byref(n), byref(handle)))
        batch = Batch()
        batch.handle = handle.value
        for i in range(n.value):
            req = self._requests[ids[i]]
            start, count, sample, pending = fields[4 * i], fields[4 * i + 1], fields[4 * i + 2], fields[4 * i + 3]
            tokens = [0] if pending else req.token_slice(start, start + count)
            batch.append(Scheduled(req, tokens, bool(sample), bool(pending)))
        self._sync()
        return batch

    def on_launched(self, batch: Batch) -> None:
        """The step is queued on the GPU: its tokens count as computed, its samples as in flight."""
        if not batch:
            return
        check(self._lib.llmrs_sched_on_launched(self._handle, batch.handle))
        self._sync()

    def cancel(self, batch: Batch) -> None:
        """The batch was decided but could not be queued (another user of the cache took its pages):
        forget it; its requests are scheduled again by the next call."""
        if batch:
            check(self._lib.llmrs_sched_cancel(self._handle, batch.handle))

    def on_result(self, batch, sampled: Dict[int, int]) -> List[Output]:
        """The step's tokens are on the host: ``sampled`` maps request id -> chosen token for
        the entries with ``sample``. Returns what happened, finished requests freed. An empty
        ``batch`` collects the requests that ended without a step."""
        handle = getattr(batch, "handle", 0) if batch else 0
        toks = [int(sampled[s.request.request_id]) for s in batch if s.sample] if handle else []
        arr = (c_int32 * max(len(toks), 1))(*toks)
        ids, fields = self._buffers(len(self._requests) + 8)
        n = c_int()
        check(self._lib.llmrs_sched_on_result(self._handle, handle, arr, len(toks), ids, fields, len(ids), byref(n)))
        outs = self._outputs(n.value)
        self._sync()
        return outs

    def update(self, batch, sampled: Dict[int, int]) -> List[Output]:
        """``on_launched`` and ``on_result`` in one call, for a caller that reads every step's tokens at once."""
        if batch:
            self.on_launched(batch)
        return self.on_result(batch, sampled)

    def abort_all(self, reason: str = "error_step_failed") -> List[Output]:
        """A step failed: every running request ends and frees its pages
        (llm-scheduler/src/engine.rs:92-99, scheduler.rs:193-200)."""
        ids, fields = self._buffers(len(self._requests) + 8)
        n = c_int()
        for req in self._requests.values():
            req._abort_reason = reason
        check(self._lib.llmrs_sched_abort_all(self._handle, 4, ids, fields, len(ids), byref(n)))
        outs = [Output(ids[i], None, True, reason) for i in range(n.value)]
        self._sync()
        for req in self._requests.values():
            req._abort_reason = None
        return outs
