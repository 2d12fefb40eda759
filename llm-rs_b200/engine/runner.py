"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner.step(entries)`` takes portions of prompts beside single decoded tokens, cut
anywhere, runs only those tokens (everything earlier comes from the cache) and returns
the float32 logits at the wanted places. The reference's ``forward_pass``
(llm-core/src/backends/candle.rs:1096-2031) has the same role but reshapes the flat
batch to a rectangle (candle.rs:1122-1125), so it is only right when every sequence
brings the same number of tokens, and it cannot continue a prompt; the batch here is
ragged: per token its id, position and request row, per request its cached length,
number of new tokens and block tables.
"""
from __future__ import annotations

import ctypes
import gc
import itertools
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import host
from ..cache import CacheManager, OutOfPages  # noqa: F401  (OutOfPages is what step() may raise)
from ..cache.pool import check
from ..cache.storage import CacheStorage
from ..config import load_config
from ..parts import DecoderModel, ModelSpec, Runtime
from ..parts.base import Plan, StepInfo
from ..weights import load_weights


class StepError(RuntimeError):
    pass


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them whose
    logits are wanted. ``device_token`` >= 0 says that the entry's single token is not
    known on the host yet: it is element ``device_token`` of the ``token_source`` tensor
    given to ``step`` (what an earlier step sampled), and ``tokens`` holds a placeholder."""
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    device_token: int = -1


class PlanView:
    """A mixer's plan as ``forward`` sees it: ``arrays`` on the device, ``values`` on the host."""
    __slots__ = ("arrays", "values")

    def __init__(self, arrays, values):
        self.arrays, self.values = arrays, values


class StepContext:
    """Everything a part may read about the current step. Device tensors are int32."""

    def __init__(self, runner: "ModelRunner"):
        self._runner = runner
        self._scratch_bufs = runner._scratch_bufs
        self.act_dtype = runner.act_dtype
        self.n_tokens = self.n_requests = self.n_want = 0
        self.token_ids = self.positions = self.token_req = None
        self.q_start = self.n_new = self.cached_len = self.slot_ids = None
        self.want_rows = None
        self.block_tables: List[Optional[torch.Tensor]] = []
        self.plans: Dict[Hashable, PlanView] = {}
        # Host copies, for parts that plan their work on the host.
        self.host_n_new: List[int] = []
        self.host_cached_len: List[int] = []
        self.host_q_start: List[int] = []
        self.host_slot_ids: List[int] = []
        self.request_ids: List[Hashable] = []

    def layer_cache(self, s: int):
        return self._runner.storage.layer_cache(s, self.block_tables)

    def plan(self, key) -> PlanView:
        """What the mixer with this ``plan_key()`` planned for the step (``Mixer.plan``)."""
        return self.plans[key]

    def scratch(self, name: str, n_floats: int) -> torch.Tensor:
        """Float32 workspace that lives across steps (grown when a step needs more). A step
        that is captured in a CUDA graph has workspace of its own, which never moves."""
        return self._runner._scratch(self._scratch_bufs, name, n_floats)


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class ModelRunner:
    """A model on the device with its cache; owns the step function."""

    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], act_dtype: torch.dtype, device,
                 max_tokens: int, page_size: int = 16, max_requests: int = 64):
        if not torch.cuda.is_available():
            raise StepError("no CUDA device: this engine runs on the GPU only")
        self.device = torch.device(device)
        self.act_dtype = act_dtype
        self.spec = spec
        self.page_size = page_size
        self.max_requests = max_requests
        n_pages = max(1, -(-max_tokens // page_size))
        self.model = DecoderModel(spec)
        needs = self.model.cache_needs()
        # A request can grow as far as the model allows and as its pages reach: only a group that keeps
        # every token bounds it by the pool; a window group gives pages back as it goes, state takes none.
        keeps_all = any(need is not None and need.kind != "window" for need, _ in needs)
        self.max_positions = min(spec.max_positions, n_pages * page_size) if keeps_all else spec.max_positions
        self.model.bind(tensors, Runtime(self.device, act_dtype, self.max_positions))
        self.storage = CacheStorage(needs, spec.run_order, page_size, n_pages, max_requests, act_dtype, self.device)
        self.manager = CacheManager(self.storage.groups, page_size, max_requests)
        self._scratch_bufs: Dict[str, torch.Tensor] = {}
        self._meta_host = [None, None]
        self._meta_events = [None, None]
        self._meta_flip = 0
        self.steps_run = 0
        self.h2d_bytes = 0  # bytes of index arrays copied to the device so far
        # Steps that only decode (one token per request) are captured in CUDA graphs and
        # replayed: one launch instead of some ten per layer.
        self.use_graphs = False
        # A part that plans work on the host per step sets ``graph_safe = False`` (a block's mixer, its
        # feed-forward, its norms, or the block itself).
        self._graph_safe = all(getattr(part, "graph_safe", True)
                               for b in self.model.blocks for part in [b, *getattr(b, "parts", list)()])
        # Mixers that plan per step, one per plan key, in run order (``Mixer.plan_key`` / ``Mixer.plan``).
        self._planners: "OrderedDict[Hashable, object]" = OrderedDict()
        for step in spec.run_order:
            mixer = getattr(self.model.blocks[step.layer], "mixer", None)
            key = mixer.plan_key() if mixer is not None and hasattr(mixer, "plan_key") else None
            if key is not None and key not in self._planners:
                self._planners[key] = mixer
        # Captured steps by (batch size, wanted rows, table widths, plans' shapes), least recently used first; a
        # captured step keeps its own logits and workspace, so their number is bounded.
        self._graphs: "OrderedDict[tuple, _DecodeGraph]" = OrderedDict()
        self.max_graphs = 48

    # -- construction ----------------------------------------------------------------
    @classmethod
    def from_model_dir(cls, model_dir: str, dtype: torch.dtype = torch.bfloat16, device="cuda:0", **kw):
        entry, cfg = load_config(model_dir)
        spec = entry.build_spec(cfg)
        dev = torch.device(device)
        tensors = load_weights(model_dir, DecoderModel(spec).weight_specs(), dtype, dev)
        return cls(spec, tensors, dtype, dev, **kw)

    # -- helpers ---------------------------------------------------------------------
    def _scratch(self, bufs: Dict[str, torch.Tensor], name: str, n_floats: int) -> torch.Tensor:
        buf = bufs.get(name)
        if buf is None or buf.numel() < n_floats:
            # Zeroed: kernels that keep arrival counters in their workspace expect them at zero.
            buf = torch.zeros((max(n_floats, 1),), dtype=torch.float32, device=self.device)
            bufs[name] = buf
        return buf

    def release(self, request_id: Hashable) -> None:
        """The request is finished: its pages and its slot go back."""
        self.manager.release(request_id)

    def check_kernels(self) -> None:
        """Raise if a kernel with bounded waits (the tcgen05 products and attention) gave up on one since
        the last check: what the steps since then returned is invalid. Synchronises."""
        from .. import ops
        ops.check_tc_error(self.device)
        ops.check_attention_error()

    def live_requests(self) -> List[Hashable]:
        return list(self.manager.requests)

    # -- the step --------------------------------------------------------------------
    def _plan(self, entries: Sequence[StepEntry]):
        """Check the entries, admit new requests and reserve their pages. Either all of
        it succeeds or nothing is left changed."""
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) < 1:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            if e.device_token >= 0:
                if len(e.tokens) != 1:
                    raise StepError(f"request {e.request_id!r}: a token taken from the device comes alone")
            elif min(e.tokens) < 0 or max(e.tokens) >= self.spec.vocab_size:
                raise StepError(f"a token id of request {e.request_id!r} is outside the vocabulary "
                                f"of {self.spec.vocab_size}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise StepError(f"request {e.request_id!r} wants place {w} of {len(e.tokens)} tokens")
        admitted, reserved = [], []
        try:
            for e in entries:
                if e.request_id not in self.manager.requests:
                    rec = self.manager.admit(e.request_id)
                    admitted.append(e.request_id)
                    self.storage.reset_slot(rec.slot)
                rec = self.manager.record(e.request_id)
                if rec.cached_len + len(e.tokens) > self.max_positions:
                    raise StepError(
                        f"request {e.request_id!r} would reach {rec.cached_len + len(e.tokens)} tokens; the limit "
                        f"is {self.max_positions} (max_position_embeddings and the cache pool)")
                self.manager.reserve(e.request_id, len(e.tokens))
                reserved.append(e.request_id)
        except Exception:
            for rid in reserved:
                self.manager.cancel(rid)
            for rid in admitted:
                self.manager.release(rid)
            raise
        return admitted

    def _pack(self, entries: Sequence[StepEntry], table_round: int, for_graph: bool = False) -> "_PackedStep":
        """Pack the step's index arrays into pinned host memory: the host library writes what every part
        may read (tokens, positions, request rows, per-request lengths, wanted rows, tokens still on the
        device, block tables padded to ``table_round``); then every mixer that plans (``Mixer.plan``) is asked
        once per plan key, and its arrays are appended to the same buffer."""
        R = len(entries)
        G = len(self.manager.groups)
        T = sum(len(e.tokens) for e in entries)
        numbers = np.fromiter((self.manager.record(e.request_id).number for e in entries), np.int64, R)
        n_tokens = np.fromiter((len(e.tokens) for e in entries), np.int32, R)
        tokens = np.fromiter(itertools.chain.from_iterable(e.tokens for e in entries), np.int32, T)
        n_want = np.fromiter((len(e.want) for e in entries), np.int32, R)
        want = np.fromiter(itertools.chain.from_iterable(e.want for e in entries), np.int32, int(n_want.sum()))
        device_token = np.fromiter((e.device_token for e in entries), np.int32, R)
        offsets = np.empty(host.FIRST_TABLE + G, np.int64)
        sizes = np.empty(host.FIRST_TABLE + G, np.int64)
        widths = np.empty(max(G, 1), np.int32)
        shape = np.empty(4, np.int32)
        total, written = ctypes.c_int64(), ctypes.c_int()
        flip = self._meta_flip
        self._meta_flip ^= 1
        if self._meta_events[flip] is not None:
            self._meta_events[flip].synchronize()  # the copy that last read this buffer is done
        lib = host.lib()
        need = 0
        while True:
            buf = self._meta_host[flip]
            cap = 0 if buf is None else buf.numel()
            if cap >= need:
                check(lib.llmrs_pack_step(
                    self.manager._handle, R, numbers.ctypes.data, n_tokens.ctypes.data, tokens.ctypes.data,
                    n_want.ctypes.data, want.ctypes.data, device_token.ctypes.data, table_round,
                    0 if buf is None else buf.data_ptr(), cap, offsets.ctypes.data, sizes.ctypes.data,
                    widths.ctypes.data, shape.ctypes.data, ctypes.byref(total), ctypes.byref(written)),
                    self.manager._names)
                need = total.value
                if written.value:
                    # The mixers' plans go behind the common arrays, each array at a multiple of four ints.
                    host_np = buf.numpy()
                    off, sz = offsets.tolist(), sizes.tolist()
                    plans, at = {}, need
                    if self._planners:
                        info = StepInfo(
                            n_tokens=T, n_requests=R, q_start=host_np[off[host.Q_START]:off[host.Q_START] + R],
                            n_new=host_np[off[host.N_NEW]:off[host.N_NEW] + R],
                            cached_len=host_np[off[host.CACHED_LEN]:off[host.CACHED_LEN] + R],
                            slot_ids=host_np[off[host.SLOT_IDS]:off[host.SLOT_IDS] + R],
                            block_tables=[host_np[off[host.FIRST_TABLE + g]:off[host.FIRST_TABLE + g] + sz[host.FIRST_TABLE + g]]
                                          .reshape(R, -1) for g in range(G)],
                            group_keys=[g.need.group_key() for g in self.manager.groups],
                            page_size=self.page_size, for_graph=for_graph)
                        for key, mixer in self._planners.items():
                            plan = mixer.plan(info)
                            where = {}
                            for name, arr in plan.arrays.items():
                                where[name] = (at, int(arr.size))
                                at += _round_up(max(int(arr.size), 1), 4)
                            plans[key] = (plan, where)
                    if at <= cap:
                        for plan, where in plans.values():
                            for name, (o, n) in where.items():
                                host_np[o:o + n] = plan.arrays[name].reshape(-1)
                        return _PackedStep(buf, flip, at, off, sz, widths[:G].tolist(), shape.tolist(), plans)
                    need = at
            self._meta_host[flip] = torch.empty((_round_up(need + 1024, 4096),), dtype=torch.int32).pin_memory()
            self._meta_events[flip] = None

    def _upload(self, packed: "_PackedStep", entries: Sequence[StepEntry],
                graph: Optional["_DecodeGraph"] = None) -> StepContext:
        """Copy a packed step to the device in one transfer and return the context that views
        it. With ``graph`` the arrays go into that graph's own buffer (same layout every
        time) and its context is returned."""
        total, offsets, sizes = packed.total, packed.offsets, packed.sizes
        if graph is not None:
            if graph.meta is None:
                graph.meta = torch.empty((total,), dtype=torch.int32, device=self.device)
            dev = graph.meta
            if dev.numel() != total:
                raise StepError("a captured step's layout changed")
        else:
            dev = torch.empty((total,), dtype=torch.int32, device=self.device)
        dev.copy_(packed.host[:total], non_blocking=True)
        self.h2d_bytes += total * 4
        ev = torch.cuda.Event()
        ev.record()
        self._meta_events[packed.flip] = ev
        T, R, n_want = packed.shape[:3]
        host_np = packed.host.numpy()

        def host_list(i):
            return host_np[offsets[i]:offsets[i] + sizes[i]].tolist()
        host_lists = dict(host_n_new=host_list(host.N_NEW), host_cached_len=host_list(host.CACHED_LEN),
                          host_q_start=host_list(host.Q_START), host_slot_ids=host_list(host.SLOT_IDS),
                          request_ids=[e.request_id for e in entries])
        if graph is not None and graph.ctx is not None:
            graph.ctx.__dict__.update(host_lists)
            return graph.ctx  # its device views already point into graph.meta; its plans' values are the key's

        def view(i):
            return dev[offsets[i]:offsets[i] + sizes[i]]
        ctx = StepContext(self)
        ctx.n_tokens, ctx.n_requests, ctx.n_want = T, R, n_want
        ctx.token_ids, ctx.positions, ctx.token_req = view(host.TOKEN_IDS), view(host.POSITIONS), view(host.TOKEN_REQ)
        ctx.q_start, ctx.n_new = view(host.Q_START), view(host.N_NEW)
        ctx.cached_len, ctx.slot_ids = view(host.CACHED_LEN), view(host.SLOT_IDS)
        ctx.want_rows = view(host.WANT_ROWS)
        for key, (plan, where) in packed.plans.items():
            arrays = {name: dev[o:o + n].view(plan.arrays[name].shape) for name, (o, n) in where.items()}
            ctx.plans[key] = PlanView(arrays, dict(plan.values))
        if graph is not None:
            ctx._scratch_bufs = graph.scratch
            graph.ctx = ctx
        ctx.pend_dst, ctx.pend_src = view(host.PEND_DST), view(host.PEND_SRC)
        ctx.block_tables = [view(host.FIRST_TABLE + g).view(R, -1) for g in range(len(packed.widths))]
        ctx.__dict__.update(host_lists)
        return ctx

    def _build_context(self, entries: Sequence[StepEntry], table_round: int = 8) -> StepContext:
        return self._upload(self._pack(entries, table_round), entries)

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry], token_source: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one batch. Returns float32 logits ``[wanted, vocab]`` on the device, in the
        order of the entries and of each entry's ``want`` (None if nothing is wanted).

        A request id that is not live is admitted. Raises ``OutOfPages`` (and leaves
        every request as it was) when the pool cannot hold the step's tokens.
        ``token_source`` is the int32 device tensor that entries with ``device_token``
        index (tokens sampled by a step that the host has not read back yet).
        """
        entries = list(entries)
        if token_source is None and any(e.device_token >= 0 for e in entries):
            raise StepError("an entry takes its token from the device but no token_source was given")
        admitted = self._plan(entries)
        try:
            with torch.cuda.device(self.device):
                if self.use_graphs and self._graph_safe and all(len(e.tokens) == 1 for e in entries):
                    logits = self._graph_step(entries, token_source)
                else:
                    ctx = self._build_context(entries)
                    self._feed_device_tokens(ctx, entries, token_source)
                    logits = self.model.forward(ctx)
        except Exception:
            for e in entries:
                self.manager.cancel(e.request_id)
            for rid in admitted:
                self.manager.release(rid)
            raise
        for e in entries:
            self.manager.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        return logits

    # -- captured decode steps ---------------------------------------------------------
    def _feed_device_tokens(self, ctx: StepContext, entries, token_source) -> None:
        if token_source is not None and any(e.device_token >= 0 for e in entries):
            from .. import ops
            ops.scatter_tokens(ctx.token_ids, ctx.pend_dst, token_source, ctx.pend_src)

    def _graph_step(self, entries: Sequence[StepEntry], token_source=None) -> Optional[torch.Tensor]:
        packed = self._pack(entries, GRAPH_TABLE_ROUND, for_graph=True)
        # Everything that sizes a captured launch is in the key: the batch, the wanted rows, the tables'
        # widths, and the shapes and values of the mixers' plans.
        key = (len(entries), tuple(len(e.want) for e in entries), tuple(packed.widths),
               tuple((k, plan.signature()) for k, (plan, _) in packed.plans.items()))
        graph = self._graphs.get(key)
        if graph is not None:
            self._graphs.move_to_end(key)
        if graph is None:
            graph = _DecodeGraph()
            ctx = self._upload(packed, entries, graph)
            self._feed_device_tokens(ctx, entries, token_source)
            # Warm-up: sizes the workspace. The replay below runs the same tokens again: keys and values
            # are rewritten with the same numbers, fixed-size state is put back to what it was.
            saved = self.storage.snapshot_state(ctx.host_slot_ids)
            self.model.forward(ctx)
            self.storage.restore_state(saved)
            torch.cuda.current_stream().synchronize()
            graph.graph = torch.cuda.CUDAGraph()
            # A collection that ran during the capture could destroy an older runner's graphs,
            # which CUDA does not allow while a stream is capturing: collect now, then hold off.
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph.graph):
                    graph.logits = self.model.forward(ctx)
            finally:
                if gc_was_on:
                    gc.enable()
            self._graphs[key] = graph
            if len(self._graphs) > self.max_graphs:
                torch.cuda.current_stream().synchronize()   # no replay may be running when its graph goes
                while len(self._graphs) > self.max_graphs:
                    self._graphs.popitem(last=False)        # the step replayed longest ago
        else:
            ctx = self._upload(packed, entries, graph)
            self._feed_device_tokens(ctx, entries, token_source)
        graph.graph.replay()
        return graph.logits


GRAPH_TABLE_ROUND = 64  # block-table width of a captured step, in pages


@dataclass
class _PackedStep:
    """A step's index arrays in pinned host memory, as the host library laid them out."""
    host: torch.Tensor
    flip: int
    total: int
    offsets: List[int]
    sizes: List[int]
    widths: List[int]
    shape: List[int]
    plans: Dict[Hashable, tuple] = field(default_factory=dict)   # plan key -> (Plan, {array name: (offset, size)})


class _DecodeGraph:
    """A captured decode step: its index buffer, its context, its workspace and its output."""

    def __init__(self):
        self.meta: Optional[torch.Tensor] = None
        self.ctx: Optional[StepContext] = None
        self.scratch: Dict[str, torch.Tensor] = {}
        self.graph = None
        self.logits: Optional[torch.Tensor] = None
