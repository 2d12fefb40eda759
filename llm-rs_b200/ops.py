"""Python face of the CUDA kernel library: each function checks its tensors and launches
one kernel (or one kernel and its combine step) on the current CUDA stream.

There is no CPU path: a tensor that is not on a CUDA device is refused, and a missing
library is an error (``csrc.build.KernelBuildError``), never a silent fallback.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

launch_count = 0  # kernels launched through this module since import (read by the benchmark)


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _lib():
    return _build.library()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    """The current CUDA stream's handle. (``torch.cuda.current_stream()`` builds a Python object every time: some
    7 us a call, 1.2 ms of the 6 ms the host needs to issue the 290 launches of a prefill step; the raw handle is
    asked for directly where this torch offers it.)"""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _check(rc: int, what: str, launches: int = 1) -> None:
    global launch_count
    if rc != 0:
        msg = _lib().llmrs_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what} failed (code {rc}): {msg}")
    launch_count += launches


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be on a CUDA device (this engine has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _row_stride(t: torch.Tensor, name: str) -> int:
    """Stride between rows of a 2-D view whose rows are dense."""
    if t.dim() != 2 or (t.size(1) > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be 2-D with dense rows, got sizes {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


def embedding(table: torch.Tensor, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]`` widened to float32 (the residual stream's type)."""
    _need(table, "table")
    _need(ids, "ids", torch.int32)
    vocab, hidden = table.shape
    n = ids.numel()
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _need(out, "out", torch.float32)
    _check(_lib().llmrs_embedding(_ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), n, hidden, vocab,
                                  _stream()), "embedding")
    return out


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                act_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``h += delta`` (when given), then ``out = h / sqrt(mean(h^2) + eps) * weight``.

    ``h`` is the float32 residual stream and is updated in place. With ``rows`` (int32
    indices) only those rows are normed, into ``out[i]``, and ``h`` is left as it is.
    """
    _need(h, "h", torch.float32)
    _need(weight, "weight", torch.float32)
    hidden = h.size(-1)
    if weight.numel() != hidden:
        raise KernelError(f"norm weight has {weight.numel()} elements, rows have {hidden}")
    if delta is not None:
        _need(delta, "delta", act_dtype)
        if delta.shape != h.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match h {tuple(h.shape)}")
    n_rows = h.size(0) if rows is None else rows.numel()
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if out is None:
        out = torch.empty((n_rows, hidden), dtype=act_dtype, device=h.device)
    _need(out, "out", act_dtype)
    _check(_lib().llmrs_add_rmsnorm(_ptr(h), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), n_rows, hidden,
                                    ctypes.c_float(eps), dtype_code(act_dtype), _stream()), "add_rmsnorm")
    return out


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """``h += delta`` in float32, in place."""
    _need(h, "h", torch.float32)
    _need(delta, "delta")
    if delta.shape != h.shape:
        raise KernelError(f"delta {tuple(delta.shape)} does not match h {tuple(h.shape)}")
    _check(_lib().llmrs_residual_add(_ptr(h), _ptr(delta), ctypes.c_longlong(h.numel()), dtype_code(delta.dtype),
                                     _stream()), "residual_add")
    return h


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, block: int = 0) -> torch.Tensor:
    """``out[t, c] = silu(gate(t, c)) * up(t, c)`` for ``gate_up`` of width 2I that holds gate and
    up in alternating runs of ``block`` columns (0: the plain layout, I gate columns then I up columns)."""
    _need(gate_up, "gate_up")
    n, two_i = gate_up.shape
    inter = two_i // 2
    block = block or inter
    if out is None:
        out = torch.empty((n, inter), dtype=gate_up.dtype, device=gate_up.device)
    _need(out, "out", gate_up.dtype)
    _check(_lib().llmrs_silu_mul(_ptr(gate_up), _ptr(out), n, inter, block, dtype_code(gate_up.dtype), _stream()),
           "silu_mul")
    return out


def gemm_f32(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """True float32 ``x @ w.T (+ bias)`` with ``w`` of shape [N, K] (FFMA, no TF32)."""
    _need(x, "x", torch.float32, contiguous=False)
    _need(w, "w", torch.float32)
    M, K = x.shape
    N = w.size(0)
    if w.size(1) != K:
        raise KernelError(f"x has {K} columns, w has {w.size(1)}")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    _need(out, "out", torch.float32, contiguous=False)
    _check(_lib().llmrs_gemm_f32(_ptr(x), ctypes.c_longlong(_row_stride(x, "x")), _ptr(w), _ptr(bias), _ptr(out),
                                 ctypes.c_longlong(_row_stride(out, "out")), M, N, K, _stream()), "gemm_f32")
    return out


def library_gemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` in bfloat16 through the library (cuBLAS via ``torch``): the products of steps with
    many tokens that this package's own kernel does not take, as the reference's projections are calls into
    its tensor library (llm-core/src/backends/candle.rs:1276-1340). The only library kernel on the product path
    (not counted in ``launch_count``, which counts this package's own kernels)."""
    if out_dtype == torch.float32:
        y = torch.mm(x, w.t(), out_dtype=torch.float32)
        if bias is not None:
            y += bias.to(torch.float32)
        return y
    return torch.nn.functional.linear(x, w, bias)


def qk_norm_rope_kvwrite(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor],
                         q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                         cos_sin: Optional[torch.Tensor], positions: torch.Tensor, token_req: torch.Tensor,
                         block_table: torch.Tensor, cache: Optional[torch.Tensor], n_q_heads: int, n_kv_heads: int,
                         head_dim: int, rotary_dim: int, page_size: int, eps: float) -> None:
    """Per-head norm and rotation of ``q`` (in place) and ``k``; ``k`` and ``v`` go to their pages.

    ``q``, ``k``, ``v`` are 2-D views with dense rows (slices of one projection output
    are fine). ``k`` = ``v`` = None: this layer reads another layer's cache and writes none.
    ``cos_sin`` is [positions, rotary_dim/2, 2] float32, or None for no rotation.
    ``cache`` is one layer's [n_pages, n_kv_heads, 2, page_size, head_dim].
    """
    _need(q, "q", contiguous=False)
    dt = q.dtype
    n = q.size(0)
    for name, t in (("k", k), ("v", v)):
        if t is not None:
            _need(t, name, dt, contiguous=False)
    if (k is None) != (v is None):
        raise KernelError("k and v must both be given or both be None")
    if k is not None:
        _need(cache, "cache", dt)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("cos_sin", cos_sin)):
        if t is not None:
            _need(t, name, torch.float32)
    if cos_sin is not None and cos_sin.size(1) * 2 != rotary_dim:
        raise KernelError(f"cos_sin table is for rotary_dim {cos_sin.size(1) * 2}, asked {rotary_dim}")
    _need(positions, "positions", torch.int32)
    _need(token_req, "token_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    _check(_lib().llmrs_qk_norm_rope_kvwrite(
        _ptr(q), ctypes.c_longlong(_row_stride(q, "q")),
        _ptr(k), ctypes.c_longlong(_row_stride(k, "k") if k is not None else 0),
        _ptr(v), ctypes.c_longlong(_row_stride(v, "v") if v is not None else 0),
        _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos_sin), _ptr(positions), _ptr(token_req), _ptr(block_table),
        block_table.size(1), _ptr(cache), n, n_q_heads, n_kv_heads, head_dim,
        rotary_dim if cos_sin is not None else 0, page_size, ctypes.c_float(eps), dtype_code(dt), _stream()),
        "qk_norm_rope_kvwrite")


def attn_prefill(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, tiles: torch.Tensor, n_tiles: int,
                 q_start: torch.Tensor, n_new: torch.Tensor, cached_len: torch.Tensor, block_table: torch.Tensor,
                 n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                 prefer_tc: bool = False) -> None:
    """Causal attention of prompt portions over the paged cache (their own keys are already written).
    ``prefer_tc`` asks for the tcgen05 kernel (blocks of 128 queries) where it applies.

    ``tiles`` is int32 [n_tiles, 2]: (request row, offset of the tile's first query in
    the request's new tokens); a tile covers 64 queries.
    """
    _need(q, "q", contiguous=False)
    _need(out, "out", q.dtype, contiguous=False)
    _need(cache, "cache", q.dtype)
    for name, t in (("tiles", tiles), ("q_start", q_start), ("n_new", n_new), ("cached_len", cached_len),
                    ("block_table", block_table)):
        _need(t, name, torch.int32)
    _check(_lib().llmrs_attn_prefill(
        _ptr(q), ctypes.c_longlong(_row_stride(q, "q")), _ptr(out), ctypes.c_longlong(_row_stride(out, "out")),
        _ptr(cache), _ptr(tiles), n_tiles, _ptr(q_start), _ptr(n_new), _ptr(cached_len), _ptr(block_table),
        block_table.size(1), n_q_heads, n_kv_heads, head_dim, page_size, window, ctypes.c_float(scale),
        dtype_code(q.dtype), q.size(0), cache.size(0), 1 if prefer_tc else 0, _ptr(tc_error_flag(q.device)),
        _stream()), "attn_prefill")


def attn_decode_scratch_floats(n_dec: int, n_q_heads: int, head_dim: int, max_splits: int) -> int:
    return int(_lib_ll("llmrs_attn_decode_scratch_floats")(n_dec, n_q_heads, head_dim, max_splits))


_decode_capacity = {}


def attn_decode_capacity(head_dim: int, cluster: int, heads: int = 4, device=None, light: bool = False) -> int:
    """Blocks of the tensor-core decode attention kernel that the device holds at a time when they come in
    thread-block clusters of ``cluster`` (1 to 16) and serve ``heads`` query heads per key head (at most 16).
    ``light``: of the kernel with the ring of two tiles (``attn_decode(ring=2)``); 0 where it does not exist."""
    key = (head_dim, cluster, heads, device, light)
    if key not in _decode_capacity:
        blocks = ctypes.c_int()
        fn = _lib().llmrs_attn_decode_capacity_light if light else _lib().llmrs_attn_decode_capacity
        _check(fn(head_dim, cluster, heads, ctypes.byref(blocks)), "attn_decode_capacity", launches=0)
        _decode_capacity[key] = blocks.value
    return _decode_capacity[key]


def _lib_ll(name: str):
    fn = getattr(_lib(), name)
    fn.restype = ctypes.c_longlong
    return fn


def attn_decode(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, dec_reqs: torch.Tensor, n_dec: int,
                q_start: torch.Tensor, cached_len: torch.Tensor, block_table: torch.Tensor, scratch: torch.Tensor,
                max_splits: int, split_keys: int, n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int,
                window: int, scale: float, counters: Optional[torch.Tensor] = None,
                then: Optional[torch.Tensor] = None, ring: int = 0) -> None:
    """Attention of single new tokens (``dec_reqs``: int32 request rows) over the paged cache,
    the keys cut into splits of ``split_keys`` and merged; ``scratch`` is float32 workspace of
    ``attn_decode_scratch_floats`` elements. (bfloat16 with head_dim <= 128 and at most 16 splits: the splits
    of a request and key head run as one thread-block cluster and merge through distributed shared memory,
    one kernel; else a second kernel merges them.) With ``counters`` (int32, at least n_dec * n_q_heads,
    all zero; the call leaves them zero) the tensor-core kernel merges the splits itself instead
    of a second kernel doing it. ``ring`` = 2 asks for the tensor-core kernel with a ring of two tiles per warp, of
    which three blocks fit an SM instead of two (head_dim 128, at most 8 query heads per key head; elsewhere it
    changes nothing): for steps whose blocks then fit one wave and otherwise do not."""
    if then is not None:
        hint_next_weights(then, PREFETCH_BYTES_AFTER_ATTENTION)   # the weights of the product after attention
    _need(q, "q", contiguous=False)
    _need(out, "out", q.dtype, contiguous=False)
    _need(cache, "cache", q.dtype)
    _need(scratch, "scratch", torch.float32)
    for name, t in (("dec_reqs", dec_reqs), ("q_start", q_start), ("cached_len", cached_len),
                    ("block_table", block_table)):
        _need(t, name, torch.int32)
    need = attn_decode_scratch_floats(n_dec, n_q_heads, head_dim, max_splits)
    if scratch.numel() < need:
        raise KernelError(f"attn_decode scratch holds {scratch.numel()} floats, {need} needed")
    if counters is not None:
        _need(counters, "counters", torch.int32)
        if counters.numel() < n_dec * n_q_heads:
            raise KernelError(f"attn_decode counters hold {counters.numel()} ints, {n_dec * n_q_heads} needed")
    if ring:
        fn = _lib().llmrs_attn_decode_next_ring
        fn.restype = None
        fn(int(ring))
    _check(_lib().llmrs_attn_decode(
        _ptr(q), ctypes.c_longlong(_row_stride(q, "q")), _ptr(out), ctypes.c_longlong(_row_stride(out, "out")),
        _ptr(cache), _ptr(dec_reqs), n_dec, _ptr(q_start), _ptr(cached_len), _ptr(block_table), block_table.size(1),
        _ptr(scratch), _ptr(counters), max_splits, split_keys, n_q_heads, n_kv_heads, head_dim, page_size, window,
        ctypes.c_float(scale), dtype_code(q.dtype), _stream()), "attn_decode",
        launches=1 if counters is not None or (q.dtype == torch.bfloat16 and head_dim <= 128 and max_splits <= 16
                                               and not _generic_only) else 2)


def scatter_tokens(dst: torch.Tensor, dst_idx: torch.Tensor, src: torch.Tensor, src_idx: torch.Tensor) -> None:
    """``dst[dst_idx[i]] = src[src_idx[i]]`` where ``dst_idx[i] >= 0`` (all int32, on the device)."""
    for name, t in (("dst", dst), ("dst_idx", dst_idx), ("src", src), ("src_idx", src_idx)):
        _need(t, name, torch.int32)
    _check(_lib().llmrs_scatter_tokens(_ptr(dst), _ptr(dst_idx), _ptr(src), _ptr(src_idx), dst_idx.numel(),
                                       _stream()), "scatter_tokens")


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the first maximum of each row of float32 ``logits``."""
    _need(logits, "logits", torch.float32)
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32)
    _check(_lib().llmrs_argmax(_ptr(logits), n, vocab, _ptr(out), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], penalty: Optional[torch.Tensor], hist_tokens: Optional[torch.Tensor],
           hist_offsets: Optional[torch.Tensor], seeds: torch.Tensor, request_ids: torch.Tensor,
           gen_index: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Choose one token per row; ``logits`` (float32) are overwritten. See csrc/sampling.cu."""
    _need(logits, "logits", torch.float32)
    n, vocab = logits.shape
    _need(temperature, "temperature", torch.float32)
    for name, t, dt in (("top_k", top_k, torch.int32), ("top_p", top_p, torch.float32),
                        ("penalty", penalty, torch.float32), ("hist_tokens", hist_tokens, torch.int32),
                        ("hist_offsets", hist_offsets, torch.int32), ("seeds", seeds, torch.int64),
                        ("request_ids", request_ids, torch.int64), ("gen_index", gen_index, torch.int32)):
        if t is not None:
            _need(t, name, dt)
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(_lib().llmrs_sample(_ptr(logits), n, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(penalty),
                               _ptr(hist_tokens), _ptr(hist_offsets), _ptr(seeds), _ptr(request_ids),
                               _ptr(gen_index), _ptr(out), _stream()), "sample")
    return out


def philox_uniform(seed: int, request_id: int, index: int) -> float:
    """The uniform number in [0, 1) that the sampler draws for (seed, request, index); host code."""
    fn = _lib().llmrs_philox_uniform
    fn.restype = ctypes.c_float
    return float(fn(ctypes.c_ulonglong(seed & (2**64 - 1)), ctypes.c_ulonglong(request_id & (2**64 - 1)),
                    ctypes.c_uint(index)))


_generic_only = False


def attention_generic_only(on: bool) -> None:
    """Make bfloat16 attention take the generic kernels too (tests compare both implementations)."""
    global _generic_only
    _generic_only = bool(on)
    fn = _lib().llmrs_attention_generic_only
    fn.restype = None
    fn(1 if on else 0)


# -- bfloat16 products on tcgen05 ------------------------------------------------------------
EPILOGUE = {"store": 0, "residual": 1, "silu_mul": 2}
_tc_flags = {}


def tc_error_flag(device) -> torch.Tensor:
    """The int32 word the tcgen05 kernels write when one of their bounded waits ran out."""
    dev = torch.device(device)
    if dev not in _tc_flags:
        _tc_flags[dev] = torch.zeros((1,), dtype=torch.int32, device=dev)
    return _tc_flags[dev]


TC_ERROR_CODES = {1: "a tcgen05 product kernel gave up waiting on a barrier",
                  2: "the tcgen05 attention kernel gave up waiting on a barrier",
                  3: "the tcgen05 attention kernel found its shared memory misaligned"}


def tc_error_message(code: int) -> str:
    return f"{TC_ERROR_CODES.get(code, 'a tcgen05 kernel failed')} (code {code}); the step's output is invalid"


def check_tc_error(device) -> None:
    """Raise if a tcgen05 kernel (product or attention) gave up on a wait since the last check (synchronises)."""
    flag = tc_error_flag(device)
    code = int(flag.item())
    if code:
        flag.zero_()
        raise KernelError(tc_error_message(code))


def set_tc_wait_limit(polls: int = 0) -> None:
    """Polls of a barrier before a wait of the tcgen05 kernels gives up; 0 restores the default (2^22)."""
    lib = _lib()
    for name in ("llmrs_tc_set_wait_limit", "llmrs_attention_tc_set_wait_limit"):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = None, [ctypes.c_uint]
        fn(int(polls))


def test_skip_copy(gemm_k_block: int = -1, attention_tile: int = -1) -> None:
    """For the test of the bounded waits only: the next launches of the tcgen05 product kernels leave out the
    copy of their k block ``gemm_k_block``, those of the attention kernel the keys of tile ``attention_tile``
    (-1: every copy is made, the default)."""
    lib = _lib()
    for name, v in (("llmrs_tc_test_skip_copy", gemm_k_block), ("llmrs_attention_tc_test_skip_copy", attention_tile)):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = None, [ctypes.c_int]
        fn(int(v))


test_skip_copy.__test__ = False     # not a test, whatever a collector makes of the name


# Bytes of the next kernel's weights that a decode kernel asks into the L2 when its own stream ends
# (LLMRS_PREFETCH_MB, 0 switches it off).
PREFETCH_BYTES = int(float(os.environ.get("LLMRS_PREFETCH_MB", "12")) * (1 << 20))
PREFETCH_BYTES_AFTER_ATTENTION = int(float(os.environ.get("LLMRS_PREFETCH_ATTN_MB", "12")) * (1 << 20))


def hint_next_weights(w: Optional[torch.Tensor], limit: Optional[int] = None) -> None:
    """Tell the next launch of a few-token product or of decode attention which weights the kernel AFTER it
    will stream: their first ``PREFETCH_BYTES`` are asked into the L2 when that launch's own loads are out.
    The hint is taken by the next such launch, whichever it is; ``None`` clears it."""
    fn = _lib().llmrs_set_next_prefetch
    limit = PREFETCH_BYTES if limit is None else limit
    if w is None or limit <= 0:
        fn(ctypes.c_void_p(0), ctypes.c_longlong(0))
        return
    n = min(w.numel() * w.element_size(), limit) // 16 * 16
    _check(fn(ctypes.c_void_p(w.data_ptr()), ctypes.c_longlong(n)), "set_next_prefetch", launches=0)


def debug_take():
    """The debug build's record (``LLMRS_DEBUG_KERNELS=1``): ``(code, value, where, count)`` of the index checks
    that failed since the last call, or None when nothing failed. Raises in a normal build, which checks nothing.
    Synchronises."""
    out = (ctypes.c_int * 4)()
    torch.cuda.synchronize()
    rc = _lib().llmrs_debug_take(out)
    if rc == 0:
        raise KernelError("this is not the debug build of the kernel library (set LLMRS_DEBUG_KERNELS=1 before import)")
    if rc < 0:
        raise KernelError("reading the debug record failed")
    return tuple(out) if out[3] else None


_SM_COUNT = {}


def sm_count(device) -> int:
    """SMs of the device (looked up once: the properties call costs microseconds, and products ask every time)."""
    n = _SM_COUNT.get(device)
    if n is None:
        n = _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def tc_splits(tokens: int, features: int, K: int, sms: int = 148) -> int:
    """Blocks of a cluster that share the k range of a skinny product: enough blocks to
    fill the GPU about twice, at least four 64-wide k blocks each."""
    if tokens > 64:
        return 1
    tiles = -(-features // 128)
    k_blocks = -(-K // 64)
    for s in (8, 4, 2):
        if tiles * s <= 2.2 * sms and k_blocks // s >= 4:
            return s
    return 1


def norm_parts(features: int, splits: int = 1, tokens: int = 1) -> int:
    """Rows of the sums of squares that a residual epilogue with ``emit`` writes: one per tile of features, 128
    wide for at most 64 tokens (the block of the cluster that owns a token writes the token's sum), 256 wide for
    more."""
    return -(-features // (128 if tokens <= 64 else 256))


def gemm_bf16_pairs(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, epilogue: str = "store",
                    out_dtype: torch.dtype = torch.bfloat16, acc_buffers: int = 2,
                    tmem_seen: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``gemm_bf16`` for many tokens through the kernel that runs a tile of 256 x 256 on a pair of SMs
    (tcgen05.mma.cta_group::2; ``gemm_tc_pair_kernel`` in csrc/gemm_tcgen05.cu), called by itself. ``gemm_bf16``
    takes the same kernel from 129 tokens on (``use_tc_pairs``). ``acc_buffers``: accumulator tiles a block holds in
    tensor memory; ``tmem_seen`` (int32, one entry per block) receives the address each block was given."""
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    tokens, K = x.shape
    features = w.size(0)
    if w.size(1) != K:
        raise KernelError(f"x has {K} columns, w has {w.size(1)}")
    epi = EPILOGUE[epilogue]
    if epilogue == "residual":
        _need(out, "out", torch.float32)
        if out.shape != (tokens, features):
            raise KernelError(f"residual stream is {tuple(out.shape)}, product is {(tokens, features)}")
        odt = torch.float32
    else:
        width = features // 2 if epilogue == "silu_mul" else features
        odt = torch.bfloat16 if epilogue == "silu_mul" else out_dtype
        if out is None:
            out = torch.empty((tokens, width), dtype=odt, device=x.device)
        _need(out, "out", odt)
    if tmem_seen is not None:
        _need(tmem_seen, "tmem_seen", torch.int32)
        if tmem_seen.numel() < 2 * sm_count(x.device):
            raise KernelError("tmem_seen needs an entry per block (two per SM)")
    _check(_lib().llmrs_gemm_bf16_pairs(_ptr(x), ctypes.c_longlong(_row_stride(x, "x")), _ptr(w), _ptr(out),
                                        ctypes.c_longlong(out.stride(0)), tokens, features, K, epi, dtype_code(odt),
                                        acc_buffers, _ptr(tmem_seen), _ptr(tc_error_flag(x.device)), _stream()),
           "gemm_bf16_pairs")
    return out


def use_tc_pairs(on: bool) -> None:
    """Whether ``gemm_bf16`` sends steps of more than 128 tokens to the kernel on pairs of SMs (the default) or keeps
    them on the one-block persistent kernel."""
    fn = _lib().llmrs_tc_use_pairs
    fn.restype, fn.argtypes = None, [ctypes.c_int]
    fn(1 if on else 0)


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, epilogue: str = "store",
              out_dtype: torch.dtype = torch.bfloat16, splits: Optional[int] = None, emit=None, scale=None,
              then: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T`` for bfloat16 ``x`` [tokens, K] and ``w`` [features, K] on tcgen05 (see csrc/gemm_tcgen05.cu).

    epilogue "store": returns [tokens, features] in ``out_dtype``. "residual": ``out`` is the
    float32 residual stream and gets the product added. "silu_mul": ``w`` alternates 64
    gate rows and 64 up rows; returns silu(gate) * up, [tokens, features / 2] bfloat16.

    A norm spread over two products: ``emit`` = (norm weight float32 [features], xw bfloat16 [tokens, features],
    parts float32 [norm_parts(features, splits, tokens), stride >= tokens]) makes a "residual" epilogue also write
    xw = (out + product) * weight and the sums of squares of each piece of the features;
    ``scale`` = (parts, n_parts, dim, eps) multiplies the product's rows by
    1 / sqrt(sum(parts[:n_parts, token]) / dim + eps).

    ``then`` (at most 64 tokens): the weights that the kernel after this one streams; their start is asked into
    the L2 when this product's own loads are out (``hint_next_weights``).
    """
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    tokens, K = x.shape
    if then is not None and tokens <= 64:
        hint_next_weights(then)
    features = w.size(0)
    if w.size(1) != K:
        raise KernelError(f"x has {K} columns, w has {w.size(1)}")
    epi = EPILOGUE[epilogue]
    if epilogue == "residual":
        _need(out, "out", torch.float32)
        if out.shape != (tokens, features):
            raise KernelError(f"residual stream is {tuple(out.shape)}, product is {(tokens, features)}")
        odt = torch.float32
    else:
        width = features // 2 if epilogue == "silu_mul" else features
        odt = torch.bfloat16 if epilogue == "silu_mul" else out_dtype
        if out is None:
            out = torch.empty((tokens, width), dtype=odt, device=x.device)
        _need(out, "out", odt)
    if splits is None:
        splits = tc_splits(tokens, features, K, sm_count(x.device))
    if emit is None and scale is None:
        _check(_lib().llmrs_gemm_bf16(_ptr(x), ctypes.c_longlong(_row_stride(x, "x")), _ptr(w), _ptr(out),
                                      ctypes.c_longlong(out.stride(0)), tokens, features, K, epi, dtype_code(odt),
                                      splits, _ptr(tc_error_flag(x.device)), _stream()), "gemm_bf16")
        return out
    e_w = e_xw = e_part = s_part = None
    stride = n_parts = dim = 0
    eps = 0.0
    if emit is not None:
        e_w, e_xw, e_part = emit
        _need(e_w, "emit weight", torch.float32)
        _need(e_xw, "emit xw", torch.bfloat16)
        _need(e_part, "emit parts", torch.float32)
        if e_w.numel() != features or e_xw.shape != (tokens, features) or e_part.size(0) < norm_parts(features, splits, tokens):
            raise KernelError("emit: weight, xw or parts do not fit the product")
        stride = e_part.size(1)
    if scale is not None:
        s_part, n_parts, dim, eps = scale
        _need(s_part, "scale parts", torch.float32)
        if emit is not None and s_part.size(1) != stride:
            raise KernelError("emit and scale parts must have rows of the same length")
        stride = s_part.size(1)
    _check(_lib().llmrs_gemm_bf16_norm(
        _ptr(x), ctypes.c_longlong(_row_stride(x, "x")), _ptr(w), _ptr(out), ctypes.c_longlong(out.stride(0)), tokens,
        features, K, epi, dtype_code(odt), splits, _ptr(e_w), _ptr(e_xw),
        ctypes.c_longlong(e_xw.stride(0) if e_xw is not None else 0), _ptr(e_part), _ptr(s_part), stride, n_parts, dim,
        ctypes.c_float(eps), _ptr(tc_error_flag(x.device)), _stream()), "gemm_bf16")
    return out


def gemm_qkv_rope(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor,
                  q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor],
                  positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor, n_q_heads: int,
                  n_kv_heads: int, page_size: int, eps: float, splits: Optional[int] = None, scale=None) -> torch.Tensor:
    """q | k | v = ``x @ w.T`` for at most 64 tokens and heads of 128 features, with the per-head norms,
    the rotation and the cache write in the product's epilogue: q lands in ``q_out`` (bfloat16
    [tokens, n_q_heads * 128]), k and v in the pages of ``cache`` that ``block_table`` names. The same
    arithmetic as ``gemm_bf16`` followed by ``qk_norm_rope_kvwrite``, one kernel and one rounding less.
    ``scale``: as in ``gemm_bf16`` (the rows of the product are scaled before the head norms)."""
    _need(x, "x", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(q_out, "q_out", torch.bfloat16)
    _need(cache, "cache", torch.bfloat16)
    tokens, K = x.shape
    features = (n_q_heads + 2 * n_kv_heads) * 128
    if w.shape != (features, K):
        raise KernelError(f"w is {tuple(w.shape)}, expected {(features, K)}")
    if q_out.shape != (tokens, n_q_heads * 128):
        raise KernelError(f"q_out is {tuple(q_out.shape)}, expected {(tokens, n_q_heads * 128)}")
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("cos_sin", cos_sin)):
        if t is not None:
            _need(t, name, torch.float32)
    if cos_sin is not None and cos_sin.size(1) != 64:
        raise KernelError(f"cos_sin table is for rotary_dim {cos_sin.size(1) * 2}, this kernel rotates 128")
    for name, t in (("positions", positions), ("token_req", token_req), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if splits is None:
        splits = tc_splits(tokens, features, K, sm_count(x.device))
    _check(_lib().llmrs_gemm_qkv_rope(
        _ptr(x), ctypes.c_longlong(_row_stride(x, "x")), _ptr(w), tokens, K, splits, _ptr(q_out),
        ctypes.c_longlong(q_out.stride(0)), _ptr(cache), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos_sin),
        _ptr(positions), _ptr(token_req), _ptr(block_table), block_table.size(1), n_q_heads, n_kv_heads, page_size,
        ctypes.c_float(eps), _ptr(scale[0] if scale else None), scale[0].size(1) if scale else 0,
        scale[1] if scale else 0, scale[2] if scale else 0, ctypes.c_float(scale[3] if scale else 0.0),
        _ptr(tc_error_flag(x.device)), _stream()), "gemm_qkv_rope")
    return q_out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2I, K]: 64 rows of gate, the 64 matching rows of up, and so on (I a multiple of 64)."""
    I, K = gate.shape
    return torch.stack([gate.reshape(I // 64, 64, K), up.reshape(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous()


def check_attention_error() -> None:
    """Raise if an attention kernel gave up on one of its bounded waits since the last check (synchronises).
    Launches through ``attn_prefill`` report into the word that ``check_tc_error`` reads; this also looks at
    the word inside the library, which launches without a word of the caller's use."""
    for dev in list(_tc_flags):
        check_tc_error(dev)
    lib = _lib()
    for name in ("llmrs_attention_tc_error",):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        if fn() > 0:
            raise KernelError(f"an attention kernel gave up waiting on a barrier ({name}); its output is invalid")
