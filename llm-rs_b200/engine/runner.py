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

import gc
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages
from ..cache.manager import RELEASED
from ..cache.storage import CacheStorage
from ..config import load_config
from ..parts import DecoderModel, ModelSpec, Runtime
from ..weights import load_weights

PREFILL_TILE = 64  # queries per entry of the prefill attention kernels' tile list


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


class StepContext:
    """Everything a part may read about the current step. Device tensors are int32."""

    def __init__(self, runner: "ModelRunner"):
        self._runner = runner
        self._scratch_bufs = runner._scratch_bufs
        self.act_dtype = runner.act_dtype
        self.n_tokens = self.n_requests = self.n_want = 0
        self.n_prefill_tiles = self.n_decode = self.max_decode_kv_len = 0
        self.long_portions = False
        self.token_ids = self.positions = self.token_req = None
        self.q_start = self.n_new = self.cached_len = self.slot_ids = None
        self.want_rows = self.prefill_tiles = self.decode_reqs = None
        self.block_tables: List[Optional[torch.Tensor]] = []
        # Host copies, for parts that plan their work on the host.
        self.host_n_new: List[int] = []
        self.host_cached_len: List[int] = []
        self.host_q_start: List[int] = []
        self.host_slot_ids: List[int] = []
        self.request_ids: List[Hashable] = []

    def layer_cache(self, s: int):
        return self._runner.storage.layer_cache(s, self.block_tables)

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
        self.max_positions = min(spec.max_positions, n_pages * page_size)
        self.model = DecoderModel(spec)
        self.model.bind(tensors, Runtime(self.device, act_dtype, self.max_positions))
        needs = self.model.cache_needs()
        self.storage = CacheStorage(needs, spec.run_order, page_size, n_pages, max_requests, act_dtype, self.device)
        self.manager = CacheManager(self.storage.groups, page_size, max_requests)
        self._scratch_bufs: Dict[str, torch.Tensor] = {}
        self._meta_host = [None, None]
        self._meta_events = [None, None]
        self._meta_flip = 0
        self.steps_run = 0
        self.h2d_bytes = 0  # bytes of index arrays copied to the device so far
        self._table_rows: Dict[Hashable, list] = {}
        # Steps that only decode (one token per request) are captured in CUDA graphs and
        # replayed: one launch instead of some ten per layer.
        self.use_graphs = False
        # A mixer that plans work on the host per step sets ``graph_safe = False``.
        self._graph_safe = all(getattr(b.mixer, "graph_safe", True) for b in self.model.blocks
                               if hasattr(b, "mixer"))
        self._graphs: Dict[tuple, "_DecodeGraph"] = {}

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
        self._table_rows.pop(request_id, None)

    def _table_row(self, rec, g: int) -> np.ndarray:
        """The request's block table of group ``g`` as an int32 array, kept between steps and
        extended when a page is appended (rebuilt after any other change to the table)."""
        cache = self._table_rows.get(rec.request_id)
        if cache is None or cache[0] is not rec or cache[1] != rec.edits:
            cache = [rec, rec.edits, [np.empty(64, np.int32) for _ in rec.tables], [0] * len(rec.tables)]
            if len(self._table_rows) > 4 * self.max_requests:
                self._table_rows = {k: v for k, v in self._table_rows.items() if k in self.manager.requests}
            self._table_rows[rec.request_id] = cache
        table, have = rec.tables[g], cache[3][g]
        arr = cache[2][g]
        if len(table) > arr.size:
            bigger = np.empty(max(2 * arr.size, len(table)), np.int32)
            bigger[:have] = arr[:have]
            cache[2][g] = arr = bigger
        if len(table) > have:
            arr[have:len(table)] = table[have:]
        cache[3][g] = len(table)
        return arr[:len(table)]

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

    def _build_context(self, entries: Sequence[StepEntry], table_round: int = 8,
                       graph: Optional["_DecodeGraph"] = None) -> StepContext:
        """Pack the step's index arrays, copy them to the device in one transfer and
        return the context that views them. With ``graph`` the arrays go into that
        graph's own buffer (same layout every time) and its context is returned."""
        ctx = StepContext(self)
        R = len(entries)
        T = sum(len(e.tokens) for e in entries)
        recs = [self.manager.record(e.request_id) for e in entries]
        token_ids = np.empty(T, np.int32)
        positions = np.empty(T, np.int32)
        token_req = np.empty(T, np.int32)
        q_start = np.empty(R, np.int32)
        n_new = np.empty(R, np.int32)
        cached = np.empty(R, np.int32)
        slots = np.empty(R, np.int32)
        want_rows: List[int] = []
        tiles: List[int] = []
        dec: List[int] = []
        at = 0
        max_dec_kv = 0
        for r, (e, rec) in enumerate(zip(entries, recs)):
            n = len(e.tokens)
            token_ids[at:at + n] = e.tokens
            positions[at:at + n] = np.arange(rec.cached_len, rec.cached_len + n)
            token_req[at:at + n] = r
            q_start[r], n_new[r], cached[r], slots[r] = at, n, rec.cached_len, rec.slot
            want_rows.extend(at + int(w) for w in e.want)
            if n == 1:
                dec.append(r)
                max_dec_kv = max(max_dec_kv, rec.cached_len + 1)
            else:
                for off in range(0, n, PREFILL_TILE):
                    tiles.extend((r, off))
            at += n
        tables = []
        for g in range(len(self.manager.groups)):
            width = _round_up(max(len(rec.tables[g]) for rec in recs), table_round)
            tab = np.full((R, width), RELEASED, np.int32)
            for r, rec in enumerate(recs):
                row = self._table_row(rec, g)
                tab[r, :row.size] = row
            tables.append(tab)
        pend_dst = np.full(R, -1, np.int32)
        pend_src = np.zeros(R, np.int32)
        for r, e in enumerate(entries):
            if e.device_token >= 0:
                pend_dst[r], pend_src[r] = q_start[r], e.device_token
                token_ids[q_start[r]] = 0

        parts = [token_ids, positions, token_req, q_start, n_new, cached, slots,
                 np.asarray(want_rows, np.int32), np.asarray(tiles, np.int32), np.asarray(dec, np.int32),
                 pend_dst, pend_src, *[t.reshape(-1) for t in tables]]
        offsets, total = [], 0
        for p in parts:
            offsets.append(total)
            total += _round_up(max(p.size, 1), 4)
        flip = self._meta_flip
        self._meta_flip ^= 1
        if self._meta_host[flip] is None or self._meta_host[flip].numel() < total:
            self._meta_host[flip] = torch.empty((_round_up(total, 4096),), dtype=torch.int32).pin_memory()
            self._meta_events[flip] = None
        if self._meta_events[flip] is not None:
            self._meta_events[flip].synchronize()  # the copy that last read this buffer is done
        host = self._meta_host[flip]
        host_np = host.numpy()
        for p, off in zip(parts, offsets):
            host_np[off:off + p.size] = p
        if graph is not None:
            if graph.meta is None:
                graph.meta = torch.empty((total,), dtype=torch.int32, device=self.device)
            dev = graph.meta
            if dev.numel() != total:
                raise StepError("a captured step's layout changed")
        else:
            dev = torch.empty((total,), dtype=torch.int32, device=self.device)
        dev.copy_(host[:total], non_blocking=True)
        self.h2d_bytes += total * 4
        ev = torch.cuda.Event()
        ev.record()
        self._meta_events[flip] = ev
        host_lists = dict(host_n_new=[int(x) for x in n_new], host_cached_len=[int(x) for x in cached],
                          host_q_start=[int(x) for x in q_start], host_slot_ids=[int(x) for x in slots],
                          request_ids=[e.request_id for e in entries])
        if graph is not None and graph.ctx is not None:
            graph.ctx.__dict__.update(host_lists)
            return graph.ctx  # its device views already point into graph.meta

        def view(i, size):
            return dev[offsets[i]:offsets[i] + size]
        ctx.n_tokens, ctx.n_requests, ctx.n_want = T, R, len(want_rows)
        ctx.token_ids, ctx.positions, ctx.token_req = view(0, T), view(1, T), view(2, T)
        ctx.q_start, ctx.n_new, ctx.cached_len, ctx.slot_ids = view(3, R), view(4, R), view(5, R), view(6, R)
        ctx.want_rows = view(7, len(want_rows))
        ctx.n_prefill_tiles = len(tiles) // 2
        # Blocks of 128 queries pay off when the portions fill them at least half on average.
        blocks = sum(-(-int(n) // 128) for n in n_new if n > 1)
        ctx.long_portions = blocks > 0 and sum(int(n) for n in n_new if n > 1) >= 64 * blocks
        ctx.prefill_tiles = view(8, len(tiles)).view(-1, 2) if tiles else view(8, 0)
        ctx.n_decode = len(dec)
        ctx.decode_reqs = view(9, len(dec))
        ctx.max_decode_kv_len = max_dec_kv
        if graph is not None:
            # Captured launch sizes must hold for every step that replays the graph.
            ctx.max_decode_kv_len = max(t.shape[1] for t in tables) * self.page_size if tables else max_dec_kv
            ctx._scratch_bufs = graph.scratch
            graph.ctx = ctx
        ctx.pend_dst, ctx.pend_src = view(10, R), view(11, R)
        ctx.block_tables = [view(12 + g, tables[g].size).view(R, -1) for g in range(len(tables))]
        ctx.__dict__.update(host_lists)
        return ctx

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
        recs = [self.manager.record(e.request_id) for e in entries]
        widths = tuple(_round_up(max(len(rec.tables[g]) for rec in recs), GRAPH_TABLE_ROUND)
                       for g in range(len(self.manager.groups)))
        key = (len(entries), tuple(len(e.want) for e in entries), widths)
        graph = self._graphs.get(key)
        if graph is None:
            graph = _DecodeGraph()
            ctx = self._build_context(entries, GRAPH_TABLE_ROUND, graph)
            self._feed_device_tokens(ctx, entries, token_source)
            self.model.forward(ctx)  # warm-up: sizes the workspace; rewrites the same keys and values
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
        else:
            ctx = self._build_context(entries, GRAPH_TABLE_ROUND, graph)
            self._feed_device_tokens(ctx, entries, token_source)
        graph.graph.replay()
        return graph.logits


GRAPH_TABLE_ROUND = 64  # block-table width of a captured step, in pages


class _DecodeGraph:
    """A captured decode step: its index buffer, its context, its workspace and its output."""

    def __init__(self):
        self.meta: Optional[torch.Tensor] = None
        self.ctx: Optional[StepContext] = None
        self.scratch: Dict[str, torch.Tensor] = {}
        self.graph = None
        self.logits: Optional[torch.Tensor] = None
