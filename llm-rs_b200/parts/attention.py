"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

import numpy as np

from .. import host, ops
from .base import Mixer, Plan, PositionEncoding, PreNormed, Runtime, StepInfo
from .linear import Linear
from .registry import build, register
from .spec import CacheNeed, PartSpec, WeightSpec


_SM_COUNT = {}
# The tcgen05 prefill kernel for long portions (head_dim 128); LLMRS_ATTN_TC=0 keeps the mma.sync kernel.
_ATTN_TC = os.environ.get("LLMRS_ATTN_TC", "1") != "0"
# Norms, rotation and cache write as the epilogue of the q|k|v product for few tokens; LLMRS_FUSE_QKV_ROPE=0
# keeps the separate kernel.
_FUSE_QKV_ROPE = os.environ.get("LLMRS_FUSE_QKV_ROPE", "1") != "0"


# A decode attention block's fixed cost (start, merge of its warps and of the cluster) in keys' worth of
# streaming; see GQAttention._choose_split.
# The q|k|v product with norms, rotation and cache write in its epilogue is taken up to this many tokens; above, the
# library product and the rotation kernel are ahead (at 64 tokens 16 + 5 us against 24).
QKV_TC_MAX_TOKENS = int(os.environ.get("LLMRS_TC_QKV_MAX_TOKENS", "32"))
FIXED_KEYS = 192
CAPACITY_USED = 0.975   # of the blocks the device holds: 256 of 264 ran in one wave, 280 of 280 did not
MAX_CLUSTER = 16     # splits that the kernel merges itself
PREFILL_TILE = 64    # queries per entry of the prefill attention kernels' tile list


# A block of the kernel with the ring of two tiles (three blocks an SM) takes about this much longer than one of the
# usual kernel (two blocks an SM, two tiles on their way per warp): it pays only where it saves a wave.
LIGHT_COST = 1.3
# LLMRS_ATTN_LIGHT=0 never takes that kernel.
_ATTN_LIGHT = os.environ.get("LLMRS_ATTN_LIGHT", "1") != "0"


def cut_keys_and_ring(length: int, units: int, capacity, capacity_light=None):
    """``cut_keys`` for both kernels: (keys per split, ring) with ring 2 where the kernel with the ring of two tiles,
    of which the device holds ``capacity_light(cluster)`` blocks (0: no such kernel), comes out cheaper."""
    keys, cost, waves = _cut(length, units, capacity)
    if capacity_light is not None and cost is not None and waves > 1 and capacity_light(1) > 0:
        # Only where the usual kernel's blocks need more than one wave at every cut and the light kernel's fit one:
        # one wave of the usual kernel beats one of the light one (batch 8: 3.66 against 3.70 ms a step), and so do
        # its several waves the light kernel's several (batch 64, context 4,096: 9.75 against 9.93 ms).
        keys2, cost2, waves2 = _cut(length, units, capacity_light)
        if cost2 is not None and waves2 == 1 and cost2 * LIGHT_COST < cost:
            return keys2, 2
    return keys, 3


def cut_keys(length: int, units: int, capacity) -> int:
    """Keys per split for the usual kernel (see ``_cut``)."""
    return _cut(length, units, capacity)[0]


def _cut(length: int, units: int, capacity):
    """Keys per split for the tensor-core decode attention kernel: ``length`` keys at most per request,
    ``units`` (request, key head group) pairs, ``capacity(cluster)`` the blocks the device holds at a time in
    thread-block clusters of that size.

    Up to ``MAX_CLUSTER`` splits merge inside the kernel as a cluster, and the cluster's size decides how many
    blocks are held (on a B200 284 in clusters of 4, 264 in clusters of 8, ...). A step whose blocks need a
    second wave that stays nearly empty loses more than longer splits cost, so: the cut with the least
    waves x (keys per split + a block's fixed cost); the fewest splits among equals. Returns the keys per split,
    that cost and the waves (cost None: the cut for the merging kernel)."""
    best_keys, best_cost, best_real, best_waves = 0, None, 0, 0
    for splits in range(1, MAX_CLUSTER + 1):
        keys = max(-(-(-(-length // splits)) // 64) * 64, 128)
        real = -(-length // keys)
        # (a wave that fills every slot was measured slow: the neighbouring kernels' blocks hold some)
        held = max(1, int(CAPACITY_USED * capacity(real)))
        waves = -(-(real * units) // held)
        cost = waves * (keys + FIXED_KEYS)
        if best_cost is None or cost < best_cost:
            best_keys, best_cost, best_real, best_waves = keys, cost, real, waves
    if best_real == MAX_CLUSTER and best_keys > 1024 and 2 * MAX_CLUSTER * units <= capacity(1):
        # Few requests with long contexts: more, shorter splits and a second kernel that merges them.
        splits = min(64, capacity(1) // units)
        return min(max(-(-(-(-length // splits)) // 64) * 64, 128), 2048), None, 0
    return best_keys, best_cost, best_waves


def _sm_count(device) -> int:
    if device not in _SM_COUNT:
        _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[device]


@register("mixer", "gqa_attention")
class GQAttention(Mixer):
    """Attention with ``n_heads`` query heads sharing ``n_kv_heads`` key/value heads.

    In order (llm-core/src/graph/builder.rs:97-243): q, k, v projections (bias only when
    ``bias``) -> per-head RMSNorm of q and k over ``head_dim`` with a shared weight when
    ``qk_norm`` (builder.rs:123-153; its eps is the parameter ``qk_norm_eps``, where the
    reference fixes 1e-6, builder.rs:130,144) -> position encoding -> new keys and values
    into the cache -> softmax(q k^T * scale) v over the keys the query may see (causal;
    the last ``window`` keys when ``window`` > 0; llm-core/src/backends/candle.rs:1587-1640)
    -> output projection. ``scale`` defaults to 1/sqrt(head_dim) (candle.rs:1608).

    The q/k/v weights are concatenated at load so that one product makes all three. The
    output projection may add its result straight into the residual stream.

    ``names`` maps the part's roles (q, k, v, o, q_norm, k_norm) to the tensors' names after the prefix,
    without ".weight" / ".bias"; an architecture's spec builder gives the names its checkpoints use.
    """
    fuses_residual = True
    ROLES = ("q", "k", "v", "o", "q_norm", "k_norm")

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: PartSpec, qk_norm: bool = True, qk_norm_eps: float = 1e-6, bias: bool = False,
                 window: int = 0, scale: Optional[float] = None, split_keys: int = 0, names=None, prefix: str = ""):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads are no multiple of {n_kv_heads} key/value heads")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"head_dim {head_dim} is not supported: the attention kernels take multiples of 16 "
                             f"from 16 to 256")
        self.hidden_size, self.n_heads, self.n_kv_heads, self.head_dim = hidden_size, n_heads, n_kv_heads, head_dim
        self.qk_norm, self.qk_norm_eps, self.bias, self.window = qk_norm, float(qk_norm_eps), bias, int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.split_keys = int(split_keys)   # keys per split of decode attention; 0: chosen per step
        self.prefix = prefix
        self.names = {role: role for role in self.ROLES}
        self.names.update(names or {})
        if set(self.names) != set(self.ROLES):
            raise ValueError(f"names may rename {self.ROLES}, got {sorted(set(self.names) - set(self.ROLES))}")
        self.position = build("position", position, prefix=prefix)
        self.q_width, self.kv_width = n_heads * head_dim, n_kv_heads * head_dim

    # -- weights ---------------------------------------------------------------------
    def _name(self, role: str, kind: str = "weight") -> str:
        return f"{self.prefix}{self.names[role]}.{kind}"

    def weight_specs(self):
        H, nm = self.hidden_size, self._name
        specs = [WeightSpec(nm("q"), (self.q_width, H)), WeightSpec(nm("k"), (self.kv_width, H)),
                 WeightSpec(nm("v"), (self.kv_width, H)), WeightSpec(nm("o"), (H, self.q_width))]
        if self.bias:
            specs += [WeightSpec(nm("q", "bias"), (self.q_width,), role="bias"),
                      WeightSpec(nm("k", "bias"), (self.kv_width,), role="bias"),
                      WeightSpec(nm("v", "bias"), (self.kv_width,), role="bias"),
                      WeightSpec(nm("o", "bias"), (H,), role="bias", optional=True)]
        if self.qk_norm:
            specs += [WeightSpec(nm("q_norm"), (self.head_dim,), role="norm"),
                      WeightSpec(nm("k_norm"), (self.head_dim,), role="norm")]
        return specs + self.position.weight_specs()

    def bind(self, tensors, runtime: Runtime):
        nm = self._name
        self.act_dtype = runtime.act_dtype
        ws = [tensors[nm(r)] for r in "qkv"]
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        wqkv = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        bqkv = None
        if self.bias:
            bqkv = torch.cat([tensors[nm(r, "bias")].to(dt) for r in "qkv"], dim=0).contiguous()
        self.qkv_proj = Linear(wqkv, bqkv, runtime.act_dtype)
        self.qkv_proj.warms_next = False
        # The query rows alone, for run-order entries that read another entry's cache.
        self.q_proj = Linear(wqkv[: self.q_width], None if bqkv is None else bqkv[: self.q_width], runtime.act_dtype)
        self.qkv_proj.tc_max_tokens = self.q_proj.tc_max_tokens = QKV_TC_MAX_TOKENS
        self.o_proj = Linear(tensors[nm("o")], tensors.get(nm("o", "bias")), runtime.act_dtype)
        self.q_norm_w = self.k_norm_w = None
        if self.qk_norm:
            self.q_norm_w = tensors[nm("q_norm")].to(torch.float32).contiguous()
            self.k_norm_w = tensors[nm("k_norm")].to(torch.float32).contiguous()
        self.position.bind(tensors, runtime)

    def chain(self):
        # Attention runs between the two: the q|k|v product warms nothing (what follows it reads the cache), the
        # decode attention kernel warms the L2 for the output projection (see ``forward``).
        return [self.qkv_proj, self.o_proj]

    # -- cache -----------------------------------------------------------------------
    def cache_need(self):
        return CacheNeed("window" if self.window > 0 else "full", self.n_kv_heads, self.head_dim, self.window)

    # -- the step's plan ---------------------------------------------------------------
    def plan_key(self):
        return ("paged_attention", PREFILL_TILE)    # the same for every layer: one plan per step

    def plan(self, step: StepInfo) -> Plan:
        """Requests that bring one token go to the decode kernel, longer portions are cut into tiles of
        queries for the prefill kernel (the host library does it). A step that will be replayed from a CUDA
        graph sizes its decode launch by the block tables' width, which the graph's key holds, instead of the
        longest request."""
        tiles, decode, max_kv, long_portions = host.plan_paged_attention(step.n_new, step.cached_len, PREFILL_TILE)
        if step.for_graph and decode.size and step.block_tables:
            max_kv = max(t.shape[1] for t in step.block_tables) * step.page_size
        return Plan(arrays={"prefill_tiles": tiles, "decode_reqs": decode},
                    values={"n_prefill_tiles": int(tiles.shape[0]), "n_decode": int(decode.size),
                            "max_decode_kv_len": int(max_kv), "long_portions": int(long_portions)})

    def _fuses_rope(self, x, cache, cos_sin) -> bool:
        """True when the q|k|v product can take norms, rotation and cache write as its epilogue."""
        if not (_FUSE_QKV_ROPE and cache.owns and self.head_dim == 128 and x.dtype == torch.bfloat16):
            return False
        if self.qkv_proj.bias is not None or not self.qkv_proj.uses_tc(x.size(0)) or x.size(0) > 64:
            return False
        if cos_sin is None:      # no rotation at all is fine; an encoding applied outside the kernel is not
            return type(self.position).apply_unfused is PositionEncoding.apply_unfused
        return self.position.rotary_dim == 128 and cos_sin.dtype == torch.float32

    def _choose_split(self, n_decode: int, max_kv_len: int, q: torch.Tensor):
        """(Keys per split of decode attention, ring of the kernel: see ``ops.attn_decode``). The choice changes
        results by rounding only (every split is merged in float32)."""
        sms = _sm_count(q.device)
        groups = self.n_kv_heads * (-(-(self.n_heads // self.n_kv_heads) // 16))
        units = max(1, n_decode * groups)
        heads = min(16, self.n_heads // self.n_kv_heads)
        length = max(max_kv_len, 1)
        if q.dtype != torch.bfloat16 or self.head_dim > 128:
            # The generic kernel: enough blocks to fill the GPU about twice.
            keys = -(-length // max(1, (2 * sms) // units))
            return min(max(-(-keys // 64) * 64, 128), 1024), 3
        return cut_keys_and_ring(
            length, units, lambda cluster: ops.attn_decode_capacity(self.head_dim, cluster, heads, q.device),
            (lambda cluster: ops.attn_decode_capacity(self.head_dim, cluster, heads, q.device, light=True))
            if _ATTN_LIGHT else None)

    def takes_prenormed(self, n_tokens: int) -> bool:
        return self.qkv_proj.takes_prenormed(n_tokens) and self.q_proj.takes_prenormed(n_tokens)

    def emits_prenormed(self, n_tokens: int) -> bool:
        return self.o_proj.emits_prenormed(n_tokens)

    # -- step ------------------------------------------------------------------------
    def forward(self, x, ctx, cache, residual=None, next_norm=None):
        nq, nkv, d = self.n_heads, self.n_kv_heads, self.head_dim
        table = cache.block_table
        cos_sin = self.position.rotation_table()
        scale = None
        if isinstance(x, PreNormed):     # only when takes_prenormed: the products below scale their rows
            scale, xin = x.scale, x.xw
        else:
            xin = x
        if self._fuses_rope(xin, cache, cos_sin):
            # Few tokens, heads of 128: the norms, the rotation and the cache write are the epilogue of the
            # q|k|v product (one kernel less in every layer of a decode step).
            q = torch.empty((ctx.n_tokens, self.q_width), dtype=xin.dtype, device=xin.device)
            ops.gemm_qkv_rope(xin, self.qkv_proj.weight, q, cache.kv, self.q_norm_w, self.k_norm_w, cos_sin,
                              ctx.positions, ctx.token_req, table, nq, nkv, cache.page_size, self.qk_norm_eps,
                              scale=scale)
        else:
            if cache.owns:
                qkv = self.qkv_proj.forward(x)
                q = qkv[:, : self.q_width]
                k = qkv[:, self.q_width: self.q_width + self.kv_width]
                v = qkv[:, self.q_width + self.kv_width:]
            else:
                q, k, v = self.q_proj.forward(x), None, None
            if cos_sin is None:
                self.position.apply_unfused(q, k, ctx.positions)
            ops.qk_norm_rope_kvwrite(q, k, v, self.q_norm_w, self.k_norm_w, cos_sin, ctx.positions, ctx.token_req,
                                     table, cache.kv if cache.owns else None, nq, nkv, d, self.position.rotary_dim,
                                     cache.page_size, self.qk_norm_eps)
        out = torch.empty((ctx.n_tokens, self.q_width), dtype=q.dtype, device=q.device)
        plan = ctx.plan(self.plan_key())
        n_tiles, n_decode, max_kv = (plan.values[k] for k in ("n_prefill_tiles", "n_decode", "max_decode_kv_len"))
        if n_tiles:
            ops.attn_prefill(q, out, cache.kv, plan.arrays["prefill_tiles"], n_tiles, ctx.q_start, ctx.n_new,
                             ctx.cached_len, table, nq, nkv, d, cache.page_size, self.window, self.scale,
                             prefer_tc=bool(plan.values["long_portions"]) and _ATTN_TC)
        if n_decode:
            split_keys, ring = (self.split_keys, 3) if self.split_keys else self._choose_split(n_decode, max_kv, q)
            max_splits = max(1, -(-max_kv // split_keys))
            scratch = ctx.scratch("attn_decode", ops.attn_decode_scratch_floats(n_decode, nq, d, max_splits))
            # Up to eight splits form a thread-block cluster and merge inside the kernel; more are merged by
            # a second, small kernel. (Merging them in the split kernel's last block,
            # ops.attn_decode(counters=...), measured no faster inside the step and slower at batch 1.)
            # The kernel asks the start of o_proj's weights into the L2 as its blocks finish their streams; when its
            # blocks run in several waves the first to finish would ask long before the kernel ends, and the keys and
            # values still streaming would push the weights out again.
            one_wave = n_decode * nkv * max_splits <= 2 * _sm_count(q.device)
            ops.attn_decode(q, out, cache.kv, plan.arrays["decode_reqs"], n_decode, ctx.q_start, ctx.cached_len, table,
                            scratch, max_splits, split_keys, nq, nkv, d, cache.page_size, self.window, self.scale,
                            then=self.o_proj.weight if one_wave and self.o_proj.uses_tc(ctx.n_tokens) else None,
                            ring=ring if ring == 2 else 0)
        if next_norm is not None:
            return self.o_proj.forward_into_residual_for_norm(out, residual, *next_norm)
        if residual is not None:
            return self.o_proj.forward_into_residual(out, residual)
        return self.o_proj.forward(out)
