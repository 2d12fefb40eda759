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
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence

from ..cache.manager import CacheManager
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


class Scheduler:
    def __init__(self, manager: CacheManager, max_positions: int, eos_token_ids: Sequence[int] = (),
                 max_tokens_per_step: int = 2048, prefill_chunk: int = 512, max_requests_per_step: int = 64):
        self.manager = manager
        self.max_positions = max_positions
        self.eos = set(eos_token_ids)
        self.max_tokens_per_step = max_tokens_per_step
        self.prefill_chunk = prefill_chunk
        self.max_requests_per_step = max_requests_per_step
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # in order of admission
        self.stats = {"steps": 0, "preemptions": 0, "tokens": 0}
        self._finished_early: List[Output] = []

    # -- intake ----------------------------------------------------------------------
    def add_request(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        if len(request.prompt) >= self.max_positions:
            raise ValueError(f"prompt of {len(request.prompt)} tokens leaves no room under the limit of "
                             f"{self.max_positions} positions")
        request.status = WAITING
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self._finished_early)

    # -- pages -----------------------------------------------------------------------
    def _fits(self, req: Request, n_new: int, free: List[int]) -> bool:
        live = req.request_id in self.manager.requests
        need = self.manager.pages_needed(req.request_id if live else None, n_new, 0 if not live else None)
        if all(n <= f for n, f in zip(need, free)):
            for g, n in enumerate(need):
                free[g] -= n
            return True
        return False

    def _preempt_last(self, free: List[int], keep: Optional[Request] = None) -> Optional[Request]:
        """Send the request admitted last back to the waiting queue; its pages become free."""
        if not self.running:
            return None
        victim = self.running.pop()
        if victim.request_id in self.manager.requests:
            before = [p.free_pages() for p in self.manager.pools]
            self.manager.release(victim.request_id)
            for g, pool in enumerate(self.manager.pools):
                free[g] += pool.free_pages() - before[g]
        victim.n_computed = 0
        victim.status = WAITING
        victim.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(victim)
        return victim

    def _finish(self, req: Request, reason: str) -> None:
        req.status, req.finish_reason = FINISHED, reason
        if req in self.running:
            self.running.remove(req)
        elif req in self.waiting:
            self.waiting.remove(req)   # it was preempted while its last token was in flight
        if req.request_id in self.manager.requests:
            self.manager.release(req.request_id)

    # -- one step --------------------------------------------------------------------
    def schedule(self) -> List[Scheduled]:
        """Decide the next step's batch. May preempt (see the module's header) and may
        finish requests that can never fit; those show up in the next ``update``."""
        while True:
            batch = self._try_schedule()
            if batch or not self.running:
                return batch
            # Nothing to run. Either every running request only waits for tokens that are in
            # flight, or requests are running and none could get its pages.
            stuck = [r for r in self.running if r.remaining >= 1 and not self._ends_by_length(r)]
            if not stuck:
                return batch
            if len(self.running) == 1:
                req = self.running[0]
                self._finish(req, "error_too_long")
                self._finished_early.append(Output(req.request_id, None, True, "error_too_long"))
            else:
                self._preempt_last([0] * len(self.manager.pools))

    def _try_schedule(self) -> List[Scheduled]:
        free = [p.free_pages() for p in self.manager.pools]
        budget = self.max_tokens_per_step
        batch: List[Scheduled] = []

        # 1. decoding requests, in order of admission; make room by preempting from the back
        i = 0
        while i < len(self.running) and budget >= 1 and len(batch) < self.max_requests_per_step:
            req = self.running[i]
            if req.remaining != 1 or self._ends_by_length(req):
                i += 1
                continue
            fits = self._fits(req, 1, free)
            while not fits and self.running[-1] is not req:
                self._preempt_last(free)
                fits = self._fits(req, 1, free)
            if not fits:
                break  # req is the last one running; schedule() decides what becomes of it
            if req.n_inflight:
                batch.append(Scheduled(req, [0], True, pending=True))
            else:
                batch.append(Scheduled(req, req.token_slice(req.n_known - 1, req.n_known), True))
            budget -= 1
            i += 1

        # 2. running requests that still have prompt left, in order of admission
        for req in self.running:
            if req.remaining > 1 and budget >= 1 and len(batch) < self.max_requests_per_step:
                n = min(req.n_known - req.n_computed, self.prefill_chunk, budget)   # known tokens only
                if n >= 1 and self._fits(req, n, free):
                    toks = req.token_slice(req.n_computed, req.n_computed + n)
                    batch.append(Scheduled(req, toks, req.n_computed + n == req.n_known and not req.n_inflight))
                    budget -= n

        # 3. admit from the front of the waiting queue while a slot, budget and pages last
        slots = self.manager.n_slots - len(self.manager.requests)
        while self.waiting and budget >= 1 and slots > 0 and len(batch) < self.max_requests_per_step:
            req = self.waiting[0]
            n = min(req.n_known - req.n_computed, self.prefill_chunk, budget)
            if not self._fits(req, n, free):
                if not self.running and not batch:
                    # Nothing else holds pages: this request can never start.
                    self.waiting.popleft()
                    self._finish(req, "error_too_long")
                    self._finished_early.append(Output(req.request_id, None, True, "error_too_long"))
                    continue
                break  # the queue waits behind its head (llm-scheduler/src/scheduler.rs:86-89)
            self.waiting.popleft()
            req.status = RUNNING
            self.running.append(req)
            slots -= 1
            toks = req.token_slice(req.n_computed, req.n_computed + n)
            batch.append(Scheduled(req, toks, req.n_computed + n == req.n_known and not req.n_inflight))
            budget -= n
        return batch

    def _ends_by_length(self, req: Request) -> bool:
        """True when the tokens already sampled (read or not) complete the request."""
        n_out = len(req.output) + req.n_inflight
        return n_out >= req.params.max_new_tokens or len(req.prompt) + n_out >= self.max_positions

    def on_launched(self, batch: Sequence[Scheduled]) -> None:
        """The step is queued on the GPU: its tokens count as computed, its samples as in flight."""
        self.stats["steps"] += 1
        for s in batch:
            s.request.n_computed += len(s.tokens)
            self.stats["tokens"] += len(s.tokens)
            if s.sample:
                s.request.n_inflight += 1

    def on_result(self, batch: Sequence[Scheduled], sampled: Dict[int, int]) -> List[Output]:
        """The step's tokens are on the host: ``sampled`` maps request id -> chosen token for
        the entries with ``sample``. Returns what happened, finished requests freed."""
        outputs, self._finished_early = list(self._finished_early), []
        for s in batch:
            req = s.request
            if not s.sample:
                continue
            req.n_inflight -= 1
            if req.status == FINISHED:
                continue          # it had ended at EOS one step earlier: this token is one too many
            token = int(sampled[req.request_id])
            req.output.append(token)
            reason = None
            if token in self.eos and not req.params.ignore_eos:
                reason = "stop"          # the EOS token is emitted (scheduler.rs:150-156)
            elif len(req.output) >= req.params.max_new_tokens:
                reason = "length"
            elif len(req.prompt) + len(req.output) >= self.max_positions:
                reason = "length"
            if reason:
                self._finish(req, reason)
            outputs.append(Output(req.request_id, token, reason is not None, reason))
        return outputs

    def update(self, batch: Sequence[Scheduled], sampled: Dict[int, int]) -> List[Output]:
        """``on_launched`` and ``on_result`` in one call, for a caller that reads every step's tokens at once."""
        self.on_launched(batch)
        return self.on_result(batch, sampled)

    def abort_all(self, reason: str = "error_step_failed") -> List[Output]:
        """A step failed: every running request ends and frees its pages
        (llm-scheduler/src/engine.rs:92-99, scheduler.rs:193-200)."""
        outs = []
        for req in list(self.running):
            self._finish(req, reason)
            outs.append(Output(req.request_id, None, True, reason))
        return outs
