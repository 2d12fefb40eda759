"""The allocation-free decode attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they call it: a
serving loop that has sworn off cudaMalloc after start-up because an allocation can stall
every stream, or a plug-in that is handed fixed buffers by its host. For them the library
has ``llmrs_attn_decode_static_scratch``, which keeps the partial results of its key
splits in a fixed 8 MiB array of its own instead of a caller's buffer. This test checks
that it gives what the regular entry point gives, and what a plain attention over the
gathered keys gives, on calls in a row that share the array (each with other sizes, so
that what the last one left behind is in the way), and that it refuses a request that does
not fit. In bfloat16 up to 16 splits merge inside the kernel and never touch the array,
so some cases cut the keys into more splits than that.

Collected last (the file's name, and the sort in conftest.py), so that a run that stops
at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, n_req, n_heads, n_kv, d, page, lens, dtype):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dev = "cuda:0"
    pages_per = [-(-(n + 1) // page) for n in lens]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max(pages_per)
    table = torch.full((n_req, width), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    cache = torch.randn((n_pages, n_kv, 2, page, d), generator=g, device=dev, dtype=torch.float32).to(dtype)
    q = torch.randn((n_req, n_heads * d), generator=g, device=dev, dtype=torch.float32).to(dtype)
    return dict(q=q, cache=cache, table=table.to(dev),
                dec_reqs=torch.arange(n_req, dtype=torch.int32, device=dev),
                q_start=torch.arange(n_req, dtype=torch.int32, device=dev),
                cached_len=torch.tensor(lens, dtype=torch.int32, device=dev))


def _library():
    from llm_rs_b200.csrc import build
    lib = build.library()
    lib.llmrs_attn_decode_static_scratch.restype = ctypes.c_int
    lib.llmrs_last_error.restype = ctypes.c_char_p
    return lib


def _plain(case, n_heads, n_kv, d, page, window, scale):
    """softmax(q k^T * scale) v per request over its gathered keys, float64: [requests, heads * d]."""
    q, cache, table, lens = case["q"].double().cpu(), case["cache"].double().cpu(), case["table"].cpu(), case["cached_len"].tolist()
    outs = []
    for r, n in enumerate(lens):
        total = n + 1                   # the new token's key is in the cache already
        pages = [int(table[r, i // page]) for i in range(0, total, page)]
        kv = torch.cat([cache[p] for p in pages], dim=2)[:, :, :total]        # [n_kv, 2, total, d]
        k, v = kv[:, 0].repeat_interleave(n_heads // n_kv, 0), kv[:, 1].repeat_interleave(n_heads // n_kv, 0)
        s = torch.einsum("hd,hkd->hk", q[r].reshape(n_heads, d), k) * scale
        if window > 0:
            s[:, :max(0, total - window)] = float("-inf")
        outs.append(torch.einsum("hk,hkd->hd", torch.softmax(s, -1), v).reshape(-1))
    return torch.stack(outs)


def _run_both(case, n_heads, n_kv, d, page, split_keys, window):
    from llm_rs_b200 import ops
    lib = _library()
    fn = lib.llmrs_attn_decode_static_scratch   # the exported C symbol
    q, cache, table = case["q"], case["cache"], case["table"]
    n = q.size(0)
    max_splits = -(-(int(case["cached_len"].max()) + 1) // split_keys)
    scale = d ** -0.5
    ref = torch.empty_like(q)
    scratch = torch.empty(ops.attn_decode_scratch_floats(n, n_heads, d, max_splits), dtype=torch.float32, device=q.device)
    ops.attn_decode(q, ref, cache, case["dec_reqs"], n, case["q_start"], case["cached_len"], table, scratch,
                    max_splits, split_keys, n_heads, n_kv, d, page, window, scale)
    out = torch.zeros_like(q)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = fn(p(q), ctypes.c_longlong(q.stride(0)), p(out), ctypes.c_longlong(out.stride(0)), p(cache),
            p(case["dec_reqs"]), n, p(case["q_start"]), p(case["cached_len"]), p(table), table.size(1),
            max_splits, split_keys, n_heads, n_kv, d, page, window, ctypes.c_float(scale),
            ops.dtype_code(q.dtype), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, out, ref, _plain(case, n_heads, n_kv, d, page, window, scale), lib


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_static_scratch_matches_regular_entry_point(dtype, tol):
    # Calls in a row on the same array: few splits, then 18 and 22 splits (more than the bfloat16 kernel
    # merges by itself, so the partial results go through the array), then other sizes again.
    for seed, (n_req, n_heads, n_kv, d, page, lens, split, window) in enumerate([
            (3, 8, 2, 64, 16, [700, 33, 255], 128, 0),
            (2, 8, 2, 128, 16, [1100, 40], 64, 0),
            (3, 4, 4, 32, 16, [700, 699, 5], 32, 0),
            (5, 6, 3, 48, 8, [10, 90, 300, 17, 64], 64, 40),
            (2, 16, 8, 128, 16, [1500, 1501], 64, 300)]):
        case = _case(seed, n_req, n_heads, n_kv, d, page, lens, dtype)
        rc, out, ref, plain, lib = _run_both(case, n_heads, n_kv, d, page, split, window)
        assert rc == 0, lib.llmrs_last_error().decode()
        assert torch.isfinite(out.float()).all()
        diff = (out.float() - ref.float()).abs().max().item()
        assert diff <= tol, f"call {seed}: differs from llmrs_attn_decode by {diff}"
        diff = (out.double().cpu() - plain).abs().max().item()
        assert diff <= tol, f"call {seed}: differs from the plain attention by {diff}"


def test_start_up_call_with_no_requests():
    """The call a caller makes once per device at start-up: nothing to attend to, no pointers, returns 0."""
    lib = _library()
    null = ctypes.c_void_p(0)
    rc = lib.llmrs_attn_decode_static_scratch(null, ctypes.c_longlong(0), null, ctypes.c_longlong(0), null, null, 0,
                                              null, null, null, 0, 1, 64, 8, 2, 64, 16, 0, ctypes.c_float(1.0), 1, null)
    assert rc == 0, lib.llmrs_last_error().decode()


def test_static_scratch_refuses_what_does_not_fit():
    lib = _library()
    fn = lib.llmrs_attn_decode_static_scratch
    null = ctypes.c_void_p(0)
    # 64 requests x 64 heads x 64 splits x 130 floats = 136 MB: far beyond 8 MiB. Refused before any pointer is read.
    rc = fn(null, ctypes.c_longlong(0), null, ctypes.c_longlong(0), null, null, 64, null, null, null, 0,
            64, 256, 64, 8, 128, 16, 0, ctypes.c_float(1.0), 1, null)
    assert rc != 0
    assert b"do not fit" in lib.llmrs_last_error()
