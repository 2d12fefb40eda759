"""The allocation-free decode attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they call it: a
serving loop that has sworn off cudaMalloc after start-up because an allocation can stall
every stream, or a plug-in that is handed fixed buffers by its host. For them the library
has ``llmrs_attn_decode_static_scratch``, which keeps the partial results of its key
splits in a fixed 8 MiB array of its own instead of a caller's buffer. This test checks
that it gives what the regular entry point gives, on two calls in a row that share the
array (the second with other sizes, so that what the first left behind is in the way),
and that it refuses a request that does not fit.

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


def _run_both(case, n_heads, n_kv, d, page, split_keys, window):
    from llm_rs_b200 import ops
    from llm_rs_b200.csrc import build
    lib = build.library()
    fn = lib.llmrs_attn_decode_static_scratch   # the exported C symbol
    fn.restype = ctypes.c_int
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
    return rc, out, ref, lib


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_static_scratch_matches_regular_entry_point(dtype, tol):
    # First call: long contexts, many splits. Second call: other sizes on the same array.
    for seed, (n_req, n_heads, n_kv, d, page, lens, split, window) in enumerate([
            (3, 8, 2, 64, 16, [700, 33, 255], 128, 0),
            (5, 6, 3, 48, 8, [10, 90, 300, 17, 64], 64, 40)]):
        case = _case(seed, n_req, n_heads, n_kv, d, page, lens, dtype)
        rc, out, ref, lib = _run_both(case, n_heads, n_kv, d, page, split, window)
        assert rc == 0, lib.llmrs_last_error().decode()
        assert torch.isfinite(out.float()).all()
        diff = (out.float() - ref.float()).abs().max().item()
        assert diff <= tol, f"call {seed}: differs from llmrs_attn_decode by {diff}"


def test_static_scratch_refuses_what_does_not_fit():
    from llm_rs_b200.csrc import build
    lib = build.library()
    fn = lib.llmrs_attn_decode_static_scratch
    fn.restype = ctypes.c_int
    null = ctypes.c_void_p(0)
    # 64 requests x 64 heads x 64 splits x 130 floats = 136 MB: far beyond 8 MiB. Refused before any pointer is read.
    rc = fn(null, ctypes.c_longlong(0), null, ctypes.c_longlong(0), null, null, 64, null, null, null, 0,
            64, 256, 64, 8, 128, 16, 0, ctypes.c_float(1.0), 1, null)
    assert rc != 0
    lib.llmrs_last_error.restype = ctypes.c_char_p
    assert b"do not fit" in lib.llmrs_last_error()
