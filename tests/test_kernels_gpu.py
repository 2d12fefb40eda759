"""Each CUDA kernel alone against a plain float32/float64 PyTorch restatement of the same
operation, at sizes other than the engine's test models (head sizes in steps of 16, odd
head counts and groups, widths and vocabularies that are no power of two)."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from llm_rs_b200 import ops
    return ops


def _tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


# -- element-wise --------------------------------------------------------------------------
@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embedding(table_dtype):
    ops = _ops()
    table = torch.randn(301, 72, device=DEV).to(table_dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = ops.embedding(table, ids)
    assert out.dtype == torch.float32 and torch.equal(out, table.float()[ids.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [48, 1000, 4096, 5120])
def test_add_rmsnorm(dtype, hidden):
    ops = _ops()
    torch.manual_seed(hidden)
    h = torch.randn(7, hidden, device=DEV) * 3
    delta = torch.randn(7, hidden, device=DEV).to(dtype)
    w = 1 + 0.1 * torch.randn(hidden, device=DEV)
    eps = 3e-6
    want_h = h.double() + delta.double()
    want_y = P.rms_norm(want_h, w.double(), eps)
    h2 = h.clone()
    y = ops.add_rmsnorm(h2, delta, w, eps, dtype)
    assert torch.allclose(h2.double(), want_h, atol=1e-6)
    assert torch.allclose(y.double(), want_y, **_tol(dtype))
    # without a delta, and with a row gather that leaves h alone
    h3 = h.clone()
    y0 = ops.add_rmsnorm(h3, None, w, eps, dtype)
    assert torch.equal(h3, h) and torch.allclose(y0.double(), P.rms_norm(h.double(), w.double(), eps), **_tol(dtype))
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    h4 = h.clone()
    yr = ops.add_rmsnorm(h4, delta, w, eps, dtype, rows=rows)
    assert torch.equal(h4, h) and torch.allclose(yr.double(), want_y[rows.long()], **_tol(dtype))


def test_rmsnorm_eps_matters():
    ops = _ops()
    h = torch.full((1, 64), 1e-3, device=DEV)
    w = torch.ones(64, device=DEV)
    a = ops.add_rmsnorm(h.clone(), None, w, 1e-6, torch.float32)
    b = ops.add_rmsnorm(h.clone(), None, w, 1e-5, torch.float32)
    assert abs(float(a[0, 0]) - 1e-3 / math.sqrt(1e-6 + 1e-6)) < 1e-4
    assert abs(float(b[0, 0]) - 1e-3 / math.sqrt(1e-6 + 1e-5)) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul_and_residual_add(dtype):
    ops = _ops()
    gu = (torch.randn(5, 2 * 176, device=DEV) * 4).to(dtype)
    g, u = gu[:, :176].double(), gu[:, 176:].double()
    assert torch.allclose(ops.silu_mul(gu).double(), g * torch.sigmoid(g) * u, **_tol(dtype))
    h = torch.randn(5, 88, device=DEV)
    d = torch.randn(5, 88, device=DEV).to(dtype)
    want = h.double() + d.double()
    assert torch.allclose(ops.residual_add(h, d).double(), want, atol=1e-6)


@pytest.mark.parametrize("M,N,K", [(1, 96, 80), (5, 333, 176), (70, 130, 17), (129, 64, 257)])
def test_gemm_f32_is_true_float32(M, N, K):
    ops = _ops()
    torch.manual_seed(M)
    x, w, b = torch.randn(M, K, device=DEV), torch.randn(N, K, device=DEV), torch.randn(N, device=DEV)
    want = x.double() @ w.double().t() + b.double()
    got = ops.gemm_f32(x, w, b)
    # TF32 (10 bits of mantissa) would miss this by a factor of a thousand.
    assert float((got.double() - want).abs().max()) < 1e-4 * math.sqrt(K)
    assert float((got.double() - want).abs().max() / want.abs().max()) < 1e-5
    # One row alone gives the same bits as the row inside the batch.
    if M > 1:
        assert torch.equal(ops.gemm_f32(x[3:4].contiguous(), w, b)[0], got[3])


# -- norm + rotation + cache write ---------------------------------------------------------
def _paged_setup(lens, new, n_kv, d, page, dtype, seed=0):
    """Random cache with scattered pages; returns tensors for kernels and dense copies for the reference."""
    g = torch.Generator().manual_seed(seed)
    n_req = len(lens)
    pages_per = [-(-(l + n) // page) for l, n in zip(lens, new)]
    n_pages = sum(pages_per) + 5
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n_req, max(pages_per) + 1), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    cache = torch.randn((n_pages, n_kv, 2, page, d), generator=g).to(dtype)
    return table, cache


def _dense_kv(cache, table, r, length, page):
    """[length, n_kv, d] keys and values of request r gathered from its pages."""
    ks, vs = [], []
    for pos in range(length):
        pg = int(table[r, pos // page])
        ks.append(cache[pg, :, 0, pos % page])
        vs.append(cache[pg, :, 1, pos % page])
    return torch.stack(ks).double(), torch.stack(vs).double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,rot,page", [(6, 3, 48, 48, 8), (5, 1, 16, 8, 16), (8, 2, 128, 128, 16), (2, 2, 80, 0, 4)])
def test_qk_norm_rope_kvwrite(dtype, nq, nkv, d, rot, page):
    ops = _ops()
    torch.manual_seed(d)
    lens, new = [5, 0, 37], [3, 9, 1]
    table, cache = _paged_setup(lens, new, nkv, d, page, dtype)
    T = sum(new)
    qkv = torch.randn(T, (nq + 2 * nkv) * d).to(dtype)
    qn, kn = 1 + 0.2 * torch.randn(d), 1 + 0.2 * torch.randn(d)
    eps, theta = 1e-5, 12345.0
    positions = torch.tensor([l + i for l, n in zip(lens, new) for i in range(n)], dtype=torch.int32)
    token_req = torch.tensor([r for r, n in enumerate(new) for _ in range(n)], dtype=torch.int32)
    cos_sin = None
    if rot:
        ang = P.rope_angles(range(64), rot, theta, torch.float64)
        cos_sin = torch.stack([ang.cos(), ang.sin()], -1).float().contiguous().to(DEV)
    # reference
    q = qkv[:, :nq * d].double().reshape(T, nq, d)
    k = qkv[:, nq * d:(nq + nkv) * d].double().reshape(T, nkv, d)
    v = qkv[:, (nq + nkv) * d:].double().reshape(T, nkv, d)
    q, k = P.rms_norm(q, qn.double(), eps), P.rms_norm(k, kn.double(), eps)
    if rot:
        a = P.rope_angles(positions.tolist(), rot, theta, torch.float64)
        q = torch.cat([P.rotate_half(q[..., :rot], a), q[..., rot:]], -1)
        k = torch.cat([P.rotate_half(k[..., :rot], a), k[..., rot:]], -1)
    dq, dc = qkv.to(DEV), cache.to(DEV)
    before = dc.clone()
    ops.qk_norm_rope_kvwrite(dq[:, :nq * d], dq[:, nq * d:(nq + nkv) * d], dq[:, (nq + nkv) * d:], qn.to(DEV),
                             kn.to(DEV), cos_sin, positions.to(DEV), token_req.to(DEV), table.to(DEV), dc, nq, nkv,
                             d, rot, page, eps)
    tol = _tol(dtype)
    assert torch.allclose(dq[:, :nq * d].double().cpu().reshape(T, nq, d), q, **tol)
    written = torch.zeros(dc.shape, dtype=torch.bool)
    for t in range(T):
        pos, r = int(positions[t]), int(token_req[t])
        pg = int(table[r, pos // page])
        assert torch.allclose(dc[pg, :, 0, pos % page].double().cpu(), k[t], **tol)
        assert torch.allclose(dc[pg, :, 1, pos % page].double().cpu(), v[t], **tol)
        written[pg, :, :, pos % page] = True
    assert torch.equal(dc.cpu()[~written], before.cpu()[~written]), "a slot of another token was touched"


# -- attention ------------------------------------------------------------------------------
def _attention_reference(q, cache, table, lens, new, nq, nkv, d, page, window, scale):
    """Plain attention per request over the gathered keys: [T, nq*d] float64."""
    outs, at = [], 0
    for r, (l, n) in enumerate(zip(lens, new)):
        K, V = _dense_kv(cache, table, r, l + n, page)
        qq = q[at:at + n].double().reshape(n, nq, d)
        G = nq // nkv
        kk, vv = K.repeat_interleave(G, 1), V.repeat_interleave(G, 1)
        s = torch.einsum("qhd,khd->hqk", qq, kk) * scale
        qi = torch.arange(l, l + n)[:, None]
        ki = torch.arange(l + n)[None, :]
        hidden = ki > qi
        if window > 0:
            hidden = hidden | (ki <= qi - window)
        p = torch.softmax(s.masked_fill(hidden[None], float("-inf")), -1)
        outs.append(torch.einsum("hqk,khd->qhd", p, vv).reshape(n, nq * d))
        at += n
    return torch.cat(outs)


def _run_attention(q, cache, table, lens, new, nq, nkv, d, page, window, scale, split_keys=64, fused_merge=True):
    ops = _ops()
    T = sum(new)
    dq, dc, dt = q.to(DEV), cache.to(DEV), table.to(DEV)
    out = torch.zeros(T, nq * d, dtype=q.dtype, device=DEV)
    q_start = torch.tensor(np.cumsum([0] + new[:-1]), dtype=torch.int32, device=DEV)
    n_new = torch.tensor(new, dtype=torch.int32, device=DEV)
    cached = torch.tensor(lens, dtype=torch.int32, device=DEV)
    tiles = [(r, off) for r, n in enumerate(new) if n > 1 for off in range(0, n, 64)]
    dec = [r for r, n in enumerate(new) if n == 1]
    if tiles:
        tt = torch.tensor(tiles, dtype=torch.int32, device=DEV)
        ops.attn_prefill(dq, out, dc, tt, len(tiles), q_start, n_new, cached, dt, nq, nkv, d, page, window, scale)
    if dec:
        max_splits = -(-max(lens[r] + 1 for r in dec) // split_keys)
        # Records start as NaN: every one that is read must have been written.
        scratch = torch.full((ops.attn_decode_scratch_floats(len(dec), nq, d, max_splits),), float("nan"), device=DEV)
        counters = torch.zeros(len(dec) * nq, dtype=torch.int32, device=DEV) if fused_merge else None
        ops.attn_decode(dq, out, dc, torch.tensor(dec, dtype=torch.int32, device=DEV), len(dec), q_start, cached, dt,
                        scratch, max_splits, split_keys, nq, nkv, d, page, window, scale, counters=counters)
        if counters is not None:
            assert int(counters.abs().sum()) == 0, "the kernel must leave its counters at zero"
    torch.cuda.synchronize()
    return out.double().cpu()


SHAPES = [  # nq, nkv, d, page
    (4, 2, 16, 16), (6, 3, 48, 8), (8, 1, 64, 16), (5, 5, 80, 4), (32, 8, 128, 16), (3, 1, 96, 32), (40, 2, 32, 16),
    (2, 1, 160, 16), (4, 2, 256, 16), (7, 1, 32, 8), (18, 2, 64, 16)]


@pytest.mark.parametrize("impl", ["auto", "generic", "auto-two-kernels"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("nq,nkv,d,page", SHAPES)
def test_attention_prefill_and_decode(nq, nkv, d, page, window, dtype, impl):
    """A mixed step: long portions, a two-token portion, single decode tokens, with and without earlier context."""
    if impl != "auto" and dtype == torch.float32:
        pytest.skip("float32 always takes the generic kernels")
    ops = _ops()
    lens = [0, 70, 129, 300, 3, 0, 64]
    new = [150, 65, 2, 1, 1, 1, 16]
    torch.manual_seed(nq * d + window)
    table, cache = _paged_setup(lens, new, nkv, d, page, dtype, seed=d)
    q = (torch.randn(sum(new), nq * d) * 1.5).to(dtype)
    scale = 0.7 / math.sqrt(d)
    want = _attention_reference(q, cache, table, lens, new, nq, nkv, d, page, window, scale)
    ops.attention_generic_only(impl == "generic")
    try:
        got = _run_attention(q, cache, table, lens, new, nq, nkv, d, page, window, scale,
                             fused_merge=impl != "auto-two-kernels")
    finally:
        ops.attention_generic_only(False)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2.5e-2, rtol=2e-2)
    bad = ~torch.isclose(got, want, **tol)
    assert not bad.any(), f"{int(bad.sum())} elements differ; worst {float((got - want).abs().max()):.3e} " \
                          f"first at {bad.nonzero()[0].tolist()}"


@pytest.mark.parametrize("nq,nkv,d,split_keys,lens", [
    (16, 1, 128, 64, [1000, 517, 30, 0]),      # 16 heads per key head, 16 splits: the largest merge in shared memory
    (32, 8, 128, 128, [2000, 1, 640]),        # 16 splits of 128 keys
    (12, 4, 64, 64, [575, 300]),              # 9 splits, three heads per key head
    (40, 2, 32, 64, [830, 831, 832])])        # 13 splits, two groups of heads per key head (16 and 4)
def test_decode_attention_merged_by_large_clusters(nq, nkv, d, split_keys, lens):
    """Single new tokens whose keys are cut into 9 to 16 splits that merge inside the kernel (clusters beyond
    the portable 8 blocks), some of them empty for the shorter requests."""
    new = [1] * len(lens)
    torch.manual_seed(nq + d)
    table, cache = _paged_setup(lens, new, nkv, d, 16, torch.bfloat16, seed=3)
    q = (torch.randn(len(lens), nq * d) * 1.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    assert 8 < -(-(max(lens) + 1) // split_keys) <= 16
    want = _attention_reference(q, cache, table, lens, new, nq, nkv, d, 16, 0, scale)
    got = _run_attention(q, cache, table, lens, new, nq, nkv, d, 16, 0, scale, split_keys=split_keys, fused_merge=False)
    assert torch.allclose(got, want, atol=2.5e-2, rtol=2e-2), float((got - want).abs().max())


@pytest.mark.parametrize("nq,nkv,lens,split_keys", [
    (32, 8, [511, 300, 17, 0, 512], 512), (8, 2, [1000, 999], 256), (5, 1, [70], 128), (16, 1, [200, 90], 128)])
def test_decode_attention_with_the_ring_of_two_tiles(nq, nkv, lens, split_keys):
    """The kernel of which three blocks fit an SM (one tile on its way per warp instead of two), asked for per launch:
    same results, and the request is used up by one launch. With 16 query heads per key head there is no such kernel
    and the usual one runs."""
    ops = _ops()
    d, page = 128, 16
    new = [1] * len(lens)
    torch.manual_seed(nq + len(lens))
    table, cache = _paged_setup(lens, new, nkv, d, page, torch.bfloat16, seed=5)
    q = (torch.randn(len(lens), nq * d) * 1.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    want = _attention_reference(q, cache, table, lens, new, nq, nkv, d, page, 0, scale)
    assert (ops.attn_decode_capacity(d, 1, nq // nkv, DEV, light=True) > ops.attn_decode_capacity(d, 1, nq // nkv, DEV)) == (nq // nkv <= 8)
    dq, dc, dt = q.to(DEV), cache.to(DEV), table.to(DEV)
    q_start = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    cached = torch.tensor(lens, dtype=torch.int32, device=DEV)
    dec = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    max_splits = -(-(max(lens) + 1) // split_keys)
    for ring in (2, 0):
        out = torch.full((len(lens), nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        scratch = torch.full((ops.attn_decode_scratch_floats(len(lens), nq, d, max_splits),), float("nan"), device=DEV)
        ops.attn_decode(dq, out, dc, dec, len(lens), q_start, cached, dt, scratch, max_splits, split_keys, nq, nkv, d, page,
                        0, scale, ring=ring)
        torch.cuda.synchronize()
        assert torch.allclose(out.double().cpu(), want, atol=2.5e-2, rtol=2e-2), (ring, float((out.double().cpu() - want).abs().max()))


def test_capacity_query_between_two_large_cluster_launches():
    """The capacity query (how many blocks the device holds in clusters of a size) sets the same kernel's
    shared-memory limit as the launcher: asked about small clusters between two launches with clusters of 16
    it must not lower the limit that the second launch needs."""
    ops = _ops()
    nq, nkv, d, lens = 16, 1, 128, [1000, 517]
    new = [1, 1]
    table, cache = _paged_setup(lens, new, nkv, d, 16, torch.bfloat16, seed=9)
    q = torch.randn(2, nq * d).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    want = _attention_reference(q, cache, table, lens, new, nq, nkv, d, 16, 0, scale)
    for _ in range(2):
        got = _run_attention(q, cache, table, lens, new, nq, nkv, d, 16, 0, scale, split_keys=64, fused_merge=False)
        assert torch.allclose(got, want, atol=2.5e-2, rtol=2e-2)
        ops._decode_capacity.clear()        # ask the library, not the cache of its answers
        assert ops.attn_decode_capacity(128, 1, 1, DEV) >= ops.attn_decode_capacity(128, 2, 2, DEV) > 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far", [0, 15, 16, 255, 256, 257, 1000, 1999])
def test_one_far_key_among_thousands(dtype, far):
    """Random scores would hide a key that is skipped or read from the wrong page: here one
    key far back carries nearly all the weight, so the output must be that key's value."""
    nq, nkv, d, page = 8, 2, 64, 16
    n_ctx = 2000
    lens, new = [n_ctx, n_ctx - 40], [1, 40]          # a decode token and a portion, same context
    torch.manual_seed(far)
    table, cache = _paged_setup(lens, new, nkv, d, page, dtype, seed=far)
    cache = cache * 0.05
    q = torch.randn(sum(new), nq * d) * 0.05
    # Request 0 / 1: the key at position `far` matches the queries strongly.
    spike = torch.randn(nkv, d)
    spike = spike / spike.norm(dim=-1, keepdim=True) * 6
    for r in range(2):
        cache[int(table[r, far // page]), :, 0, far % page] = spike.to(dtype)
    q = q.reshape(-1, nq, d)
    q += spike.repeat_interleave(nq // nkv, 0)[None] * 1.0
    q = q.reshape(-1, nq * d).to(dtype)
    scale = 1.0
    want = _attention_reference(q, cache, table, lens, new, nq, nkv, d, page, 0, scale)
    got = _run_attention(q, cache, table, lens, new, nq, nkv, d, page, 0, scale, split_keys=256)
    # The far key's value dominates: check against it and against the full reference.
    K, V = _dense_kv(cache, table, 0, n_ctx + 1, page)
    dom = V[far].repeat_interleave(nq // nkv, 0).reshape(-1)
    assert float((want[0] - dom).abs().max()) < 0.05
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert float((got - want).abs().max()) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_window_edge(dtype):
    """Two keys carry the weight: the last one inside the window and the first one outside it."""
    nq, nkv, d, page, window = 4, 2, 32, 8, 24
    lens, new = [100, 60], [1, 41]
    torch.manual_seed(1)
    table, cache = _paged_setup(lens, new, nkv, d, page, dtype, seed=3)
    cache = cache * 0.05
    spike = torch.randn(nkv, d)
    spike = spike / spike.norm(dim=-1, keepdim=True) * 6
    q = (torch.randn(sum(new), nq, d) * 0.05 + spike.repeat_interleave(2, 0)[None]).reshape(-1, nq * d).to(dtype)
    # For the decode token at position 100 the window holds keys 77..100: spike both 77 and 76.
    for pos in (76, 77):
        cache[int(table[0, pos // page]), :, 0, pos % page] = spike.to(dtype)
        cache[int(table[0, pos // page]), :, 1, pos % page] = (1.0 if pos == 77 else -1.0)
    # For the portion (positions 60..100) spike keys 50 and 51: query 73 sees 50 (73-24+1), query 74 does not.
    for pos in (50, 51):
        cache[int(table[1, pos // page]), :, 0, pos % page] = spike.to(dtype)
        cache[int(table[1, pos // page]), :, 1, pos % page] = (1.0 if pos == 51 else -1.0)
    want = _attention_reference(q, cache, table, lens, new, nq, nkv, d, page, window, 1.0)
    got = _run_attention(q, cache, table, lens, new, nq, nkv, d, page, window, 1.0, split_keys=32)
    assert float(want[0].mean()) > 0.9              # only key 77 (value +1) is inside
    assert abs(float(want[1 + 13].mean())) < 0.2    # query at 73: keys 50 (-1) and 51 (+1) both inside
    assert float(want[1 + 14].mean()) > 0.9         # query at 74: only key 51
    assert float((got - want).abs().max()) < (1e-4 if dtype == torch.float32 else 2e-2)


# -- sampling -------------------------------------------------------------------------------
def test_argmax_first_maximum_wins():
    ops = _ops()
    x = torch.randn(6, 1531, device=DEV)
    x[2, 77] = x[2, 900] = 50.0
    x[4, 1530] = 60.0
    got = ops.argmax(x).cpu().tolist()
    want = [int(np.argmax(r)) for r in x.cpu().numpy()]
    assert got == want and got[2] == 77 and got[4] == 1530


def test_philox_matches_the_plain_implementation():
    ops = _ops()
    for seed, rid, idx in [(0, 0, 0), (7, 3, 11), (2**40 + 5, 2**33 + 1, 4000), (2**63 + 9, 1, 2)]:
        assert ops.philox_uniform(seed, rid, idx) == pytest.approx(P.uniform(seed, rid, idx), abs=0)


def _sample(logits, rows):
    from llm_rs_b200.sampling import Sampler
    return Sampler(DEV).sample(logits.clone(), rows).cpu().tolist()


def test_sampler_greedy_temperature_and_penalty():
    from llm_rs_b200.sampling import SamplingParams
    torch.manual_seed(0)
    V = 1531
    logits = torch.randn(5, V, device=DEV) * 2
    host = logits.cpu().numpy()
    hist = [int(np.argmax(host[1])), 3, 3]
    rows = [(SamplingParams(temperature=0.0), 1, 0, []),
            (SamplingParams(temperature=0.0, repetition_penalty=3.0), 2, 0, hist),
            (SamplingParams(temperature=0.8, seed=5), 3, 0, []),
            (SamplingParams(temperature=0.8, seed=5), 3, 1, []),
            (SamplingParams(temperature=1.3, seed=6, repetition_penalty=1.5), 4, 2, [1, 2, 3])]
    got = _sample(logits, rows)
    for r, (p, rid, idx, h) in enumerate(rows):
        want = P.sample(host[r], p.temperature, p.top_k, p.top_p, p.repetition_penalty, h, p.seed, rid, idx)
        if p.temperature <= 1e-5:
            assert got[r] == want
        else:
            _assert_draw(host[r], p, h, rid, idx, got[r])
    assert got[1] != hist[0]                  # the penalised maximum lost
    # A row's token does not depend on what else is in the batch.
    assert _sample(logits[2:4], rows[2:4]) == got[2:4]
    assert _sample(logits[3:4], rows[3:4]) == got[3:4]


def _assert_draw(row, p, history, rid, idx, token):
    """The token's slice of the cumulative distribution holds the Philox draw (up to float32 rounding)."""
    probs = P.kept_probabilities(row, p.temperature, p.top_k, p.top_p, p.repetition_penalty, history)
    assert probs[token] > 0, "a token that was cut off was drawn"
    cum = np.cumsum(probs)
    u = P.uniform(p.seed, rid, idx)
    lo, hi = (cum[token - 1] if token else 0.0), cum[token]
    assert lo - 1e-4 <= u <= hi + 1e-4, (lo, u, hi)


@pytest.mark.parametrize("top_k,top_p", [(5, 1.0), (0, 0.6), (40, 0.9), (1, 1.0), (0, 0.05)])
def test_sampler_top_k_top_p(top_k, top_p):
    from llm_rs_b200.sampling import SamplingParams
    torch.manual_seed(1)
    V = 3001
    logits = torch.randn(1, V, device=DEV) * 3
    host = logits.cpu().numpy()[0]
    p = SamplingParams(temperature=0.9, top_k=top_k, top_p=top_p, seed=11)
    probs = P.kept_probabilities(host, 0.9, top_k, top_p)
    seen = set()
    for idx in range(200):
        tok = _sample(logits, [(p, 9, idx, [])])[0]
        _assert_draw(host, p, [], 9, idx, tok)
        seen.add(tok)
    kept = set(np.nonzero(probs)[0].tolist())
    assert seen <= kept
    if len(kept) <= 5:
        assert seen == kept                    # every kept token shows up in 200 draws


def test_sampler_follows_the_distribution():
    from llm_rs_b200.sampling import SamplingParams
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0] + [-30.0] * 200], device=DEV)
    p = SamplingParams(temperature=1.0, seed=3)
    n = 2000
    rows = [(p, 1, i, []) for i in range(n)]
    toks = _sample(logits.repeat(n, 1), rows)
    want = torch.softmax(logits[0].double().cpu(), 0).numpy()
    for t in range(4):
        assert abs(toks.count(t) / n - want[t]) < 0.04


# -- tcgen05 matrix product ---------------------------------------------------------------------
def _tc_case(tokens, features, K, epilogue, out_dtype, splits, ldx=None):
    ops = _ops()
    torch.manual_seed(tokens * 7 + features + K)
    x = (torch.randn(tokens, ldx or K, device=DEV) * 0.5).to(torch.bfloat16)[:, :K]
    w = (torch.randn(features, K, device=DEV) * 0.5).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    if epilogue == "residual":
        h = torch.randn(tokens, features, device=DEV)
        want = h.double() + ref
        got = ops.gemm_bf16(x, w, out=h, epilogue="residual", splits=splits).double()
        tol = 1e-5 * math.sqrt(K) * float(want.abs().max())
    elif epilogue == "silu_mul":
        half = features // 2
        g, u = w[:half], w[half:]
        gg, uu = x.double() @ g.double().t(), x.double() @ u.double().t()
        want = gg * torch.sigmoid(gg) * uu
        got = ops.gemm_bf16(x, ops.interleave_gate_up(g, u), epilogue="silu_mul", splits=splits).double()
        tol = 1e-2 * float(want.abs().max())
    else:
        want = ref
        got = ops.gemm_bf16(x, w, out_dtype=out_dtype, splits=splits).double()
        tol = (1e-2 if out_dtype == torch.bfloat16 else 1e-5 * math.sqrt(K)) * float(want.abs().max())
    ops.check_tc_error(DEV)
    err = float((got - want).abs().max())
    assert err <= tol, f"max |diff| {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("tokens,features,K,epilogue,out_dtype,splits", [
    (8, 128, 64, "store", torch.float32, 1), (8, 128, 512, "store", torch.float32, 2),
    (16, 256, 1024, "store", torch.bfloat16, 4), (1, 384, 4096, "store", torch.float32, 8),
    (17, 136, 192, "store", torch.float32, 1), (33, 512, 1000, "store", torch.bfloat16, 2),
    (64, 1024, 2048, "residual", torch.float32, 8), (5, 264, 328, "residual", torch.float32, 4),
    (8, 512, 256, "silu_mul", torch.bfloat16, 1), (40, 1280, 4096, "silu_mul", torch.bfloat16, 4),
    (3, 1000, 96, "store", torch.float32, 1), (2, 151936, 128, "store", torch.float32, None)])
def test_gemm_tcgen05_few_tokens(tokens, features, K, epilogue, out_dtype, splits):
    """Weights on the 128 rows of the MMA, tokens on the narrow side, k shared by a cluster."""
    _tc_case(tokens, features, K, epilogue, out_dtype, splits)


def test_gemm_tcgen05_few_tokens_random_shapes():
    """Random token counts, widths (multiples of 8, ragged against the tiles of 128 features and 64 of k), cluster
    sizes and epilogues: every item of the epilogue's division by tokens and quads, with and without a partner
    feature 64 further on, must land where the plain product says."""
    rng = np.random.default_rng(11)
    for _ in range(48):
        tokens = int(rng.integers(1, 65))
        K = int(rng.integers(1, 40)) * 8
        epilogue = ["store", "store", "residual", "silu_mul"][int(rng.integers(0, 4))]
        features = int(rng.integers(1, 6)) * 128 if epilogue == "silu_mul" else int(rng.integers(1, 80)) * 8
        k_blocks = -(-K // 64)
        splits = int(rng.choice([s for s in (1, 2, 4, 8) if s <= max(1, k_blocks)]))
        out_dtype = torch.float32 if rng.integers(0, 2) else torch.bfloat16
        try:
            _tc_case(tokens, features, K, epilogue, out_dtype, splits)
        except AssertionError as e:
            raise AssertionError(f"tokens {tokens} features {features} K {K} {epilogue} {out_dtype} splits {splits}: {e}")


@pytest.mark.parametrize("tokens,features,K,epilogue,out_dtype", [
    (65, 128, 64, "store", torch.float32), (128, 256, 512, "store", torch.bfloat16),
    (300, 392, 1000, "store", torch.float32), (200, 512, 4096, "residual", torch.float32),
    (130, 1024, 512, "silu_mul", torch.bfloat16), (515, 768, 320, "store", torch.bfloat16),
    (1100, 10496, 192, "store", torch.bfloat16), (2048, 12288, 128, "silu_mul", torch.bfloat16),
    (1500, 8200, 72, "residual", torch.float32)])
@pytest.mark.parametrize("pairs", [True, False])
def test_gemm_tcgen05_many_tokens(tokens, features, K, epilogue, out_dtype, pairs):
    """Tokens on the rows of the MMA; with 256 features or more a persistent kernel, whose blocks walk several
    tiles each (the last three cases give every block two to four tiles, so that both accumulator buffers and the
    ring of stages wrap, with a ragged edge in tokens, features and k): from 129 tokens tiles of 256 x 256 on pairs
    of SMs (``pairs``), else tiles of 128 x 256 on one."""
    ops = _ops()
    ops.use_tc_pairs(pairs)
    try:
        _tc_case(tokens, features, K, epilogue, out_dtype, None)
    finally:
        ops.use_tc_pairs(True)


def test_gemm_on_pairs_of_sms_alone():
    """The kernel on pairs of SMs called by itself, with one and with two accumulator buffers; both blocks of
    every pair are given the same columns of tensor memory (the pair's MMA writes one address in both)."""
    ops = _ops()
    torch.manual_seed(5)
    for tokens, features, K, bufs in [(256, 256, 64, 1), (300, 520, 200, 1), (1000, 1288, 1032, 2), (2048, 4096, 512, 2)]:
        x = (torch.randn(tokens, K, device=DEV) * 0.5).to(torch.bfloat16)
        w = (torch.randn(features, K, device=DEV) * 0.5).to(torch.bfloat16)
        seen = torch.full((2 * torch.cuda.get_device_properties(DEV).multi_processor_count,), -1, dtype=torch.int32, device=DEV)
        got = ops.gemm_bf16_pairs(x, w, out_dtype=torch.float32, acc_buffers=bufs, tmem_seen=seen).double()
        ops.check_tc_error(DEV)
        want = x.double() @ w.double().t()
        assert float((got - want).abs().max()) <= 1e-5 * math.sqrt(K) * float(want.abs().max())
        used = seen[seen >= 0].cpu().tolist()
        n_tiles = -(-tokens // 256) * -(-features // 256)
        assert len(used) == 2 * min(n_tiles, len(used) // 2) and len(used) % 2 == 0
        assert all(a == b for a, b in zip(used[0::2], used[1::2])), "the blocks of a pair were given different columns"


@pytest.mark.parametrize("pairs", [True, False])
@pytest.mark.parametrize("tokens,features,K,consumer", [
    (300, 512, 256, "store"), (1000, 1288, 520, "silu_mul"), (257, 4096, 128, "store"), (129, 256, 64, "silu_mul")])
def test_gemm_norm_spread_over_two_products_many_tokens(tokens, features, K, consumer, pairs):
    """The same for many tokens: the residual epilogue of the persistent kernels turns its 32 x 32 pieces round in
    shared memory, writes h, h * weight and the rows' sums of squares per tile of 256 features; the products after
    it scale their rows. Against rmsnorm(h + x W^T) W2^T in float64."""
    ops = _ops()
    ops.use_tc_pairs(pairs)
    try:
        torch.manual_seed(tokens + features)
        x = (torch.randn(tokens, K) * 0.5).to(torch.bfloat16)
        w = (torch.randn(features, K) * 0.05).to(torch.bfloat16)
        h0 = torch.randn(tokens, features) * torch.linspace(0.2, 3.0, tokens)[:, None]   # rows of different size
        nw = 1 + 0.2 * torch.randn(features)
        eps = 3e-5
        h = h0.to(DEV).clone()
        xw = torch.full((tokens, features), float("nan"), dtype=torch.bfloat16, device=DEV)
        n_parts = ops.norm_parts(features, 1, tokens)
        assert n_parts == -(-features // 256)
        parts = torch.full((n_parts, tokens + 3), float("nan"), dtype=torch.float32, device=DEV)
        ops.gemm_bf16(x.to(DEV), w.to(DEV), out=h, epilogue="residual", emit=(nw.to(DEV), xw, parts))
        torch.cuda.synchronize()
        ops.check_tc_error(DEV)
        want_h = h0.double() + x.double() @ w.double().t()
        assert float((h.double().cpu() - want_h).abs().max()) < 1e-3
        assert bool(torch.isnan(parts[:, tokens:]).all()), "a sum was written beyond the tokens"
        ss = parts[:, :tokens].double().cpu().sum(0)
        assert float(((ss - (want_h ** 2).sum(-1)) / (want_h ** 2).sum(-1)).abs().max()) < 1e-4
        assert float((xw.double().cpu() - want_h * nw.double()).abs().max()) < 2e-2 * float((want_h * nw.double()).abs().max())
        normed = want_h / torch.sqrt((want_h ** 2).mean(-1, keepdim=True) + eps) * nw.double()
        scale = (parts, n_parts, features, eps)
        if consumer == "store":
            w2 = (torch.randn(264, features) * 0.05).to(torch.bfloat16)
            got = ops.gemm_bf16(xw, w2.to(DEV), out_dtype=torch.float32, scale=scale)
            want = normed @ w2.double().t()
        else:
            g, u = (torch.randn(256, features) * 0.05).to(torch.bfloat16), (torch.randn(256, features) * 0.05).to(torch.bfloat16)
            got = ops.gemm_bf16(xw, ops.interleave_gate_up(g, u).to(DEV), epilogue="silu_mul", scale=scale)
            a, b = normed @ g.double().t(), normed @ u.double().t()
            want = a * torch.sigmoid(a) * b
        torch.cuda.synchronize()
        ops.check_tc_error(DEV)
        assert float((got.double().cpu() - want).abs().max()) < 2e-2 * float(want.abs().max())
    finally:
        ops.use_tc_pairs(True)


def test_gemm_tcgen05_strided_input_and_refusals():
    ops = _ops()
    _tc_case(8, 256, 256, "store", torch.float32, 1, ldx=1024)
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, 100, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.gemm_bf16(x, w)
    with pytest.raises(ops.KernelError, match="splits"):
        ops.gemm_bf16(torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV),
                      torch.zeros(64, 64, dtype=torch.bfloat16, device=DEV), splits=3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul_interleaved_layout(dtype):
    ops = _ops()
    gate, up = torch.randn(5, 256, device=DEV).to(dtype), torch.randn(5, 256, device=DEV).to(dtype)
    inter = torch.stack([gate.reshape(5, 4, 64), up.reshape(5, 4, 64)], 2).reshape(5, 512).contiguous()
    want = gate.double() * torch.sigmoid(gate.double()) * up.double()
    assert torch.allclose(ops.silu_mul(inter, block=64).double(), want, **_tol(dtype))


# -- tcgen05 prefill attention (head_dim 128) ------------------------------------------------------
@pytest.mark.parametrize("lens,new,nq,nkv,page,window", [
    ([0], [128], 1, 1, 16, 0), ([0], [64], 2, 1, 16, 0), ([0], [300], 4, 2, 16, 0),
    ([70, 0, 129, 300], [150, 65, 2, 130], 8, 2, 16, 0), ([70, 0, 129, 300], [150, 65, 2, 130], 8, 2, 32, 37),
    ([1000], [1000], 4, 1, 16, 0), ([0, 500], [1100, 700], 8, 8, 16, 200), ([5], [257], 6, 3, 48, 129),
    ([70, 0, 129, 300], [150, 65, 2, 130], 8, 2, 64, 0), ([0, 500], [1100, 700], 8, 8, 64, 200),
    ([5], [257], 6, 3, 128, 129), ([1000], [1000], 4, 1, 64, 0), ([0], [1], 2, 1, 64, 0),
    ([100, 0, 900, 5], [1500, 700, 129, 3], 16, 4, 16, 0), ([100, 0, 900, 5], [1500, 700, 129, 3], 16, 2, 64, 300),
    ([0], [2048], 12, 4, 16, 0)])
def test_attention_prefill_tcgen05(lens, new, nq, nkv, page, window):
    """Blocks of 128 queries on tcgen05 against the plain attention: partial blocks, several requests,
    earlier context, windows that start inside a tile, pages larger than a 16-key box, and pages of a
    multiple of 64 keys (which are copied 64 keys at a time). The last three cases have more 128-row items than
    the device has SMs: one block per SM then walks several items, of different requests and lengths, and
    carries barriers' phases, stages and tensor memory from one to the next."""
    ops = _ops()
    d = 128
    torch.manual_seed(len(lens) * 31 + window)
    table, cache = _paged_setup(lens, new, nkv, d, page, torch.bfloat16, seed=page + window)
    q = torch.randn(sum(new), nq * d).to(torch.bfloat16)
    scale = 1 / math.sqrt(d)
    want = _attention_reference(q, cache, table, lens, new, nq, nkv, d, page, window, scale)
    dq, dc, dt = q.to(DEV), cache.to(DEV), table.to(DEV)
    q_start = torch.tensor(np.cumsum([0] + new[:-1]), dtype=torch.int32, device=DEV)
    tiles = torch.tensor([(r, off) for r, n in enumerate(new) for off in range(0, n, 64)], dtype=torch.int32, device=DEV)
    out = torch.full((sum(new), nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attn_prefill(dq, out, dc, tiles, tiles.size(0), q_start, torch.tensor(new, dtype=torch.int32, device=DEV),
                     torch.tensor(lens, dtype=torch.int32, device=DEV), dt, nq, nkv, d, page, window, scale,
                     prefer_tc=True)
    torch.cuda.synchronize()
    ops.check_attention_error()
    got = out.double().cpu()
    assert torch.isfinite(got).all(), "a row was not written"
    assert float((got - want).abs().max()) < 2.5e-2


@pytest.mark.parametrize("page", [16, 64])
def test_attention_prefill_tcgen05_growing_scores(page):
    """Keys grow along the sequence, so the reference maximum of every row moves again and again:
    each move rescales O in tensor memory between two tiles."""
    ops = _ops()
    nq, nkv, d = 4, 2, 128
    lens, new = [900], [400]
    torch.manual_seed(page)
    table, cache = _paged_setup(lens, new, nkv, d, page, torch.bfloat16, seed=page)
    direction = torch.randn(nkv, d)
    direction = direction / direction.norm(dim=-1, keepdim=True)
    for pos in range(lens[0] + new[0]):
        k = cache[int(table[0, pos // page]), :, 0, pos % page].float() * 0.05 + direction * (pos / 20.0)
        cache[int(table[0, pos // page]), :, 0, pos % page] = k.to(torch.bfloat16)
    q = (torch.randn(sum(new), nq, d) * 0.05 + direction.repeat_interleave(2, 0)[None]).reshape(-1, nq * d).to(torch.bfloat16)
    want = _attention_reference(q, cache, table, lens, new, nq, nkv, d, page, 0, 1.0)
    dq, dc, dt = q.to(DEV), cache.to(DEV), table.to(DEV)
    tiles = torch.tensor([(0, off) for off in range(0, new[0], 64)], dtype=torch.int32, device=DEV)
    out = torch.zeros(new[0], nq * d, dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.attn_prefill(dq, out, dc, tiles, tiles.size(0), z, torch.tensor(new, dtype=torch.int32, device=DEV),
                     torch.tensor(lens, dtype=torch.int32, device=DEV), dt, nq, nkv, d, page, 0, 1.0, prefer_tc=True)
    torch.cuda.synchronize()
    ops.check_attention_error()
    assert float((out.double().cpu() - want).abs().max()) < 2e-2


def test_attention_prefill_tcgen05_far_key():
    """One key 1,900 positions back carries the weight: the lazily rescaled maximum and the page boxes must find it."""
    ops = _ops()
    nq, nkv, d, page = 4, 2, 128, 16
    lens, new = [1800], [200]
    for far in (0, 63, 64, 1000, 1799, 1800, 1927):
        torch.manual_seed(far)
        table, cache = _paged_setup(lens, new, nkv, d, page, torch.bfloat16, seed=far)
        cache = cache * 0.05
        spike = torch.randn(nkv, d)
        spike = spike / spike.norm(dim=-1, keepdim=True) * 6
        cache[int(table[0, far // page]), :, 0, far % page] = spike.to(torch.bfloat16)
        q = (torch.randn(sum(new), nq, d) * 0.05 + spike.repeat_interleave(2, 0)[None]).reshape(-1, nq * d).to(torch.bfloat16)
        want = _attention_reference(q, cache, table, lens, new, nq, nkv, d, page, 0, 1.0)
        dq, dc, dt = q.to(DEV), cache.to(DEV), table.to(DEV)
        tiles = torch.tensor([(0, off) for off in range(0, 200, 64)], dtype=torch.int32, device=DEV)
        out = torch.zeros(200, nq * d, dtype=torch.bfloat16, device=DEV)
        z = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops.attn_prefill(dq, out, dc, tiles, 4, z, torch.tensor(new, dtype=torch.int32, device=DEV),
                         torch.tensor(lens, dtype=torch.int32, device=DEV), dt, nq, nkv, d, page, 0, 1.0, prefer_tc=True)
        torch.cuda.synchronize()
        assert float((out.double().cpu() - want).abs().max()) < 2e-2, far


@pytest.mark.parametrize("tokens,nq,nkv,K,page,rope,norm", [
    (8, 4, 2, 256, 16, True, True), (1, 2, 1, 128, 16, True, True), (13, 8, 2, 512, 32, True, False),
    (33, 4, 4, 192, 16, False, True), (64, 6, 3, 320, 64, True, True)])
def test_gemm_qkv_rope_epilogue(tokens, nq, nkv, K, page, rope, norm):
    """The q|k|v product with norms, rotation and cache write in its epilogue against the product
    followed by the separate kernel's arithmetic in float64."""
    ops = _ops()
    d = 128
    torch.manual_seed(tokens + nq)
    x = (torch.randn(tokens, K) * 0.5).to(torch.bfloat16)
    w = (torch.randn((nq + 2 * nkv) * d, K) * 0.05).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(d)) if norm else None
    kw = (1 + 0.1 * torch.randn(d)) if norm else None
    n_req = 3
    req_of = torch.tensor([i % n_req for i in range(tokens)], dtype=torch.int32)
    pos = torch.tensor([5 + 7 * (i // n_req) + (i % n_req) * 40 for i in range(tokens)], dtype=torch.int32)
    max_pos = int(pos.max()) + 1
    pages_per = -(-max_pos // page)
    table = torch.randperm(n_req * pages_per).to(torch.int32).view(n_req, pages_per)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * (1e4 ** (-torch.arange(64, dtype=torch.float64) / 64))[None, :]
    cos_sin = torch.stack([ang.cos(), ang.sin()], -1).float() if rope else None
    eps = 1e-5
    # reference in float64
    y = x.double() @ w.double().t()
    q = y[:, : nq * d].reshape(tokens, nq, d)
    k = y[:, nq * d: (nq + nkv) * d].reshape(tokens, nkv, d)
    v = y[:, (nq + nkv) * d:].reshape(tokens, nkv, d)
    if norm:
        q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * qw.double()
        k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * kw.double()
    if rope:
        a = ang[pos.long()][:, None, :]
        rot = lambda z: torch.cat([z[..., :64] * a.cos() - z[..., 64:] * a.sin(), z[..., 64:] * a.cos() + z[..., :64] * a.sin()], -1)
        q, k = rot(q), rot(k)
    cache = torch.zeros(n_req * pages_per, nkv, 2, page, d, dtype=torch.bfloat16, device=DEV)
    q_out = torch.full((tokens, nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    dev = lambda t: None if t is None else t.to(DEV)
    ops.gemm_qkv_rope(x.to(DEV), w.to(DEV), q_out, cache, dev(qw), dev(kw), dev(cos_sin), pos.to(DEV), req_of.to(DEV),
                      table.to(DEV), nq, nkv, page, eps)
    torch.cuda.synchronize()
    ops.check_tc_error(DEV)
    tol = 2e-2 * float(max(q.abs().max(), k.abs().max(), v.abs().max()))
    assert float((q_out.double().cpu().reshape(tokens, nq, d) - q).abs().max()) < tol
    host = cache.double().cpu()
    touched = torch.zeros(cache.shape[0], page, dtype=torch.bool)
    for t in range(tokens):
        pg, slot = int(table[int(req_of[t]), int(pos[t]) // page]), int(pos[t]) % page
        touched[pg, slot] = True
        assert float((host[pg, :, 0, slot] - k[t]).abs().max()) < tol
        assert float((host[pg, :, 1, slot] - v[t]).abs().max()) < tol
    assert float(host[~touched[:, None, None, :, None].expand_as(host)].abs().max()) == 0.0   # nothing else was written


@pytest.mark.parametrize("tokens,features,K,splits,consumer", [
    (8, 256, 512, 2, "store"), (1, 384, 256, 4, "silu_mul"), (19, 200, 1024, 8, "store"), (32, 512, 512, 2, "qkv_rope"),
    (64, 136, 256, 2, "silu_mul"), (5, 264, 128, 1, "store"), (33, 128, 512, 4, "qkv_rope")])
def test_gemm_norm_spread_over_two_products(tokens, features, K, splits, consumer):
    """A residual epilogue that also writes the next norm's input (h * weight and sums of squares in
    pieces), and the products that take it and scale their rows, against
    rmsnorm(h + x W^T) W2^T in float64."""
    ops = _ops()
    torch.manual_seed(tokens * 7 + features)
    x = (torch.randn(tokens, K) * 0.5).to(torch.bfloat16)
    w = (torch.randn(features, K) * 0.05).to(torch.bfloat16)
    h0 = torch.randn(tokens, features) * torch.linspace(0.2, 3.0, tokens)[:, None]   # rows of different size
    nw = 1 + 0.2 * torch.randn(features)
    eps = 3e-5
    h = h0.to(DEV).clone()
    xw = torch.full((tokens, features), float("nan"), dtype=torch.bfloat16, device=DEV)
    n_parts = ops.norm_parts(features, splits)
    parts = torch.full((n_parts, 64), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_bf16(x.to(DEV), w.to(DEV), out=h, epilogue="residual", splits=splits, emit=(nw.to(DEV), xw, parts))
    torch.cuda.synchronize()
    ops.check_tc_error(DEV)
    want_h = h0.double() + x.double() @ w.double().t()
    assert float((h.double().cpu() - want_h).abs().max()) < 1e-3
    ss = parts[:, :tokens].double().cpu().sum(0)
    assert float(((ss - (want_h ** 2).sum(-1)) / (want_h ** 2).sum(-1)).abs().max()) < 1e-4
    assert float((xw.double().cpu() - want_h * nw.double()).abs().max()) < 2e-2 * float((want_h * nw.double()).abs().max())
    normed = want_h / torch.sqrt((want_h ** 2).mean(-1, keepdim=True) + eps) * nw.double()
    scale = (parts, n_parts, features, eps)
    if consumer == "store":
        w2 = (torch.randn(264, features) * 0.05).to(torch.bfloat16)
        got = ops.gemm_bf16(xw, w2.to(DEV), out_dtype=torch.float32, scale=scale)
        want = normed @ w2.double().t()
    elif consumer == "silu_mul":
        g, u = (torch.randn(128, features) * 0.05).to(torch.bfloat16), (torch.randn(128, features) * 0.05).to(torch.bfloat16)
        got = ops.gemm_bf16(xw, ops.interleave_gate_up(g, u).to(DEV), epilogue="silu_mul", scale=scale)
        a, b = normed @ g.double().t(), normed @ u.double().t()
        want = a * torch.sigmoid(a) * b
    else:
        nq, nkv, d, page = 2, 1, 128, 16
        w2 = (torch.randn((nq + 2 * nkv) * d, features) * 0.05).to(torch.bfloat16)
        pos = torch.arange(tokens, dtype=torch.int32)
        table = torch.arange(-(-tokens // page), dtype=torch.int32).view(1, -1)
        cache = torch.zeros(table.numel(), nkv, 2, page, d, dtype=torch.bfloat16, device=DEV)
        got = torch.empty(tokens, nq * d, dtype=torch.bfloat16, device=DEV)
        ops.gemm_qkv_rope(xw, w2.to(DEV), got, cache, None, None, None, pos.to(DEV), torch.zeros(tokens, dtype=torch.int32, device=DEV),
                          table.to(DEV), nq, nkv, page, 1e-6, scale=scale)
        y = normed @ w2.double().t()
        want = y[:, : nq * d]
        k_got = torch.stack([cache[t // page, :, 0, t % page] for t in range(tokens)]).double().cpu().reshape(tokens, -1)
        assert float((k_got - y[:, nq * d: (nq + nkv) * d]).abs().max()) < 2e-2 * float(y.abs().max())
    torch.cuda.synchronize()
    ops.check_tc_error(DEV)
    assert float((got.double().cpu() - want).abs().max()) < 2e-2 * float(want.abs().max())


def test_gemm_norm_emission_refusals():
    ops = _ops()
    x = torch.zeros(8, 256, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(256, 256, dtype=torch.bfloat16, device=DEV)
    h = torch.zeros(8, 256, device=DEV)
    nw, xw, parts = torch.ones(256, device=DEV), torch.empty(8, 256, dtype=torch.bfloat16, device=DEV), torch.empty(8, 64, device=DEV)
    with pytest.raises(ops.KernelError):      # a row stride of the norm's input that is no multiple of 8
        ops.gemm_bf16(x, w, out=h, epilogue="residual", splits=2,
                      emit=(nw, torch.empty(8, 260, dtype=torch.bfloat16, device=DEV)[:, :256], parts))
    with pytest.raises(ops.KernelError):      # too few rows for the pieces
        ops.gemm_bf16(x, w, out=h, epilogue="residual", splits=4, emit=(nw, xw, parts[:1]))


# -- bounded waits ------------------------------------------------------------------------------------
@pytest.mark.parametrize("tokens,features,K,splits,skip", [
    (8, 256, 256, 1, 1),        # few tokens, one block per tile; every stage is requested before the first wait
    (8, 256, 1024, 2, 3),       # a cluster of two blocks shares the k range: both give up, both reach the cluster's barriers
    (16, 128, 1024, 1, 9),      # the ring of six stages has wrapped: the producer is waiting for a free stage
    (100, 128, 256, None, 2),   # tokens on the rows, one tile per block
    (300, 512, 512, None, 5),   # the kernel on pairs of SMs: both blocks' copying, MMA and epilogue warps leave their loops
    (300, 512, 1024, None, 13), # the same after the ring of six stages has wrapped
    (100, 512, 512, None, 5)])  # the persistent kernel on single SMs (at most 128 tokens)
def test_gemm_tcgen05_wait_runs_out_and_the_kernel_returns(tokens, features, K, splits, skip):
    """A copy that never arrives (the producer leaves it out on request) with a wait limit of 1,024 polls: the
    kernel returns by itself, the error word is set, nothing is stored where the block gave up; and the next,
    normal launch gives the right product, so tensor memory was freed and no barrier is left waiting."""
    ops = _ops()
    torch.manual_seed(skip)
    x = (torch.randn(tokens, K, device=DEV) * 0.5).to(torch.bfloat16)
    w = (torch.randn(features, K, device=DEV) * 0.5).to(torch.bfloat16)
    want = x.double() @ w.double().t()
    ops.check_tc_error(DEV)
    ops.set_tc_wait_limit(1 << 10)
    ops.test_skip_copy(gemm_k_block=skip)
    try:
        ops.gemm_bf16(x, w, out_dtype=torch.float32, splits=splits)
        torch.cuda.synchronize()            # the kernel has returned
        with pytest.raises(ops.KernelError, match="gave up waiting"):
            ops.check_tc_error(DEV)
        ops.check_tc_error(DEV)             # reading the word clears it
    finally:
        ops.test_skip_copy()
        ops.set_tc_wait_limit(0)
    for _ in range(3):                      # enough launches to come by every SM again
        got = ops.gemm_bf16(x, w, out_dtype=torch.float32, splits=splits).double()
        assert float((got - want).abs().max()) <= 1e-5 * math.sqrt(K) * float(want.abs().max())
    ops.check_tc_error(DEV)


@pytest.mark.parametrize("skip,nq", [(0, 4), (2, 4), (4, 4), (3, 32), (9, 32)])
def test_attention_tcgen05_wait_runs_out_and_the_kernel_returns(skip, nq):
    """The same for the tcgen05 prefill attention: the keys of one tile never arrive; the blocks that wait for
    them give up after 1,024 polls, store nothing, and the error word is set. The next launch is right. With 32
    heads there are more items than SMs and a block walks several: the tile that never arrives is then counted
    over a block's items, so some blocks give up in their first item and some in a later one."""
    ops = _ops()
    d, nkv, page, lens, new = 128, 2, 16, [0, 200], [700, 520]
    torch.manual_seed(skip)
    table, cache = _paged_setup(lens, new, nkv, d, page, torch.bfloat16, seed=skip)
    q = torch.randn(sum(new), nq * d).to(torch.bfloat16)
    scale = 1 / math.sqrt(d)
    want = _attention_reference(q, cache, table, lens, new, nq, nkv, d, page, 0, scale)
    dq, dc, dt = q.to(DEV), cache.to(DEV), table.to(DEV)
    q_start = torch.tensor(np.cumsum([0] + new[:-1]), dtype=torch.int32, device=DEV)
    tiles = torch.tensor([(r, off) for r, n in enumerate(new) for off in range(0, n, 64)], dtype=torch.int32, device=DEV)
    args = (dc, tiles, tiles.size(0), q_start, torch.tensor(new, dtype=torch.int32, device=DEV),
            torch.tensor(lens, dtype=torch.int32, device=DEV), dt, nq, nkv, d, page, 0, scale)
    ops.check_tc_error(DEV)
    ops.set_tc_wait_limit(1 << 10)
    ops.test_skip_copy(attention_tile=skip)
    try:
        out = torch.full((sum(new), nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attn_prefill(dq, out, *args, prefer_tc=True)
        torch.cuda.synchronize()
        with pytest.raises(ops.KernelError, match="attention kernel gave up"):
            ops.check_tc_error(DEV)
        # Blocks with more than `skip` tiles of keys gave up and stored nothing; the others are right.
        got = out.double().cpu()
        written = torch.isfinite(got).all(dim=1)
        assert not written.all()
        assert float((got[written] - want[written]).abs().max()) < 2.5e-2 if written.any() else True
    finally:
        ops.test_skip_copy()
        ops.set_tc_wait_limit(0)
    for _ in range(3):
        out = torch.full((sum(new), nq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attn_prefill(dq, out, *args, prefer_tc=True)
        got = out.double().cpu()
        assert torch.isfinite(got).all() and float((got - want).abs().max()) < 2.5e-2
    ops.check_attention_error()
