"""The host library's packing of a step (CPU): every index array against a restatement in
numpy, for ragged batches with portions, decoded tokens, tokens still on the device,
window groups with released pages and padded block tables."""
import ctypes
import random

import numpy as np
import pytest

from llm_rs_b200 import host
from llm_rs_b200.cache import CacheManager, GroupSpec, RELEASED
from llm_rs_b200.parts import CacheNeed


def pack(manager, entries, table_round, capacity=1 << 16):
    """entries: (request id, tokens, want, device_token). Returns (arrays by index, shape, widths) or the size needed."""
    R, G = len(entries), len(manager.groups)
    numbers = np.array([manager.record(e[0]).number for e in entries], np.int64)
    n_tokens = np.array([len(e[1]) for e in entries], np.int32)
    tokens = np.array([t for e in entries for t in e[1]], np.int32)
    n_want = np.array([len(e[2]) for e in entries], np.int32)
    want = np.array([w for e in entries for w in e[2]], np.int32)
    dev_tok = np.array([e[3] for e in entries], np.int32)
    out = np.full(capacity, 12345, np.int32)
    offsets, sizes = np.zeros(host.FIRST_TABLE + G, np.int64), np.zeros(host.FIRST_TABLE + G, np.int64)
    widths, shape = np.zeros(max(G, 1), np.int32), np.zeros(4, np.int32)
    total, written = ctypes.c_int64(), ctypes.c_int()
    rc = host.lib().llmrs_pack_step(manager._handle, R, numbers.ctypes.data, n_tokens.ctypes.data, tokens.ctypes.data,
                                    n_want.ctypes.data, want.ctypes.data, dev_tok.ctypes.data, table_round,
                                    out.ctypes.data, capacity, offsets.ctypes.data, sizes.ctypes.data,
                                    widths.ctypes.data, shape.ctypes.data, ctypes.byref(total), ctypes.byref(written))
    if rc != 0:
        raise ValueError(host.last_error())
    if not written.value:
        assert (out == 12345).all(), "a refused packing wrote into the buffer"
        return total.value
    assert all(o % 4 == 0 for o in offsets), "every array starts at a multiple of four elements"
    assert total.value <= capacity and (out[total.value:] == 12345).all()
    arrays = [out[o:o + n].copy() for o, n in zip(offsets, sizes)]
    return arrays, shape.tolist(), widths[:G].tolist()


def expected(manager, entries, table_round):
    tok, pos, treq, qs, nn, cl, sl, wr, pd, ps = ([] for _ in range(10))
    at = 0
    for r, (rid, tokens, want, dev) in enumerate(entries):
        rec = manager.record(rid)
        n = len(tokens)
        tok += [0] + list(tokens[1:]) if dev >= 0 else list(tokens)
        pos += list(range(rec.cached_len, rec.cached_len + n))
        treq += [r] * n
        qs.append(at), nn.append(n), cl.append(rec.cached_len), sl.append(rec.slot)
        wr += [at + w for w in want]
        pd.append(at if dev >= 0 else -1), ps.append(dev if dev >= 0 else 0)
        at += n
    tables = []
    for g in range(len(manager.groups)):
        rows = [manager.table(e[0], g) for e in entries]
        width = -(-max(len(t) for t in rows) // table_round) * table_round
        tables.append([p for t in rows for p in t + [RELEASED] * (width - len(t))])
    return [tok, pos, treq, qs, nn, cl, sl, wr, pd, ps, *tables]


def expected_attention_plan(n_new, cached, tile):
    tiles, dec = [], []
    for r, n in enumerate(n_new):
        if n == 1:
            dec.append(r)
        else:
            tiles += [[r, off] for off in range(0, n, tile)]
    portions = [n for n in n_new if n > 1]
    blocks = sum(-(-n // 128) for n in portions)
    return tiles, dec, max([c + 1 for n, c in zip(n_new, cached) if n == 1], default=0), \
        bool(blocks and sum(portions) >= 64 * blocks)


def _manager(window=0):
    groups = [GroupSpec(CacheNeed("full", 2, 16), [0], 400)]
    if window:
        groups.append(GroupSpec(CacheNeed("window", 2, 16, window), [1], 400))
    return CacheManager(groups, 4, 6)


@pytest.mark.parametrize("window", [0, 9])
def test_packing_matches_restatement(window):
    rng = random.Random(3 + window)
    m = _manager(window)
    for rid, cached in (("a", 0), ("b", 37), ("c", 5), ("d", 18)):
        m.admit(rid)
        if cached:
            m.reserve(rid, cached)
            m.commit(rid, cached)
    for trial in range(20):
        entries = []
        for rid in rng.sample(["a", "b", "c", "d"], rng.randint(1, 4)):
            n = rng.choice([1, 1, 2, 3, 7, 13])
            toks = [rng.randrange(1, 100) for _ in range(n)]
            want = sorted(rng.sample(range(n), rng.randint(0, min(n, 2))))
            dev = rng.randrange(8) if n == 1 and rng.random() < 0.4 else -1
            entries.append((rid, toks, want, dev))
        for e in entries:
            m.reserve(e[0], len(e[1]))
        tile, table_round = rng.choice([2, 4, 64]), rng.choice([1, 8])
        arrays, shape, widths = pack(m, entries, table_round)
        want_arrays = expected(m, entries, table_round)
        assert len(arrays) == len(want_arrays)
        for i, (got, exp) in enumerate(zip(arrays, want_arrays)):
            assert got.tolist() == exp, f"array {i} differs in trial {trial}"
        T = sum(len(e[1]) for e in entries)
        assert shape[:3] == [T, len(entries), sum(len(e[2]) for e in entries)]
        # The plan of paged attention comes from the per-request numbers that the packing wrote.
        n_new, cached = arrays[host.N_NEW], arrays[host.CACHED_LEN]
        tiles, dec, max_kv, long_portions = host.plan_paged_attention(n_new, cached, tile)
        exp = expected_attention_plan(n_new.tolist(), cached.tolist(), tile)
        assert (tiles.tolist(), dec.tolist(), max_kv, long_portions) == exp
        for e in entries:
            m.commit(e[0], len(e[1]))
        m.check_invariants()


def test_long_portions_flag_and_small_buffer():
    plan = lambda n_new: host.plan_paged_attention(np.array(n_new, np.int32), np.zeros(len(n_new), np.int32), 64)
    assert plan([200])[3] is True                 # two blocks of 128, 200 >= 128 tokens
    assert plan([200, 3])[3] is True              # 203 tokens over three blocks
    assert plan([3])[3] is False
    assert plan([1, 1])[0].shape == (0, 2) and plan([1, 1])[1].tolist() == [0, 1]
    m = _manager()
    m.admit("a")
    m.reserve("a", 200)
    big = [("a", list(range(200)), [199], -1)]
    need = pack(m, big, 8, capacity=16)               # too small: only the size comes back
    assert isinstance(need, int) and need > 400
    arrays, _, _ = pack(m, big, 8, capacity=need)
    assert arrays[0].tolist() == list(range(200))


def test_refusals():
    m = _manager()
    m.admit("a")
    m.reserve("a", 2)
    with pytest.raises(ValueError, match="wanted place"):
        pack(m, [("a", [1, 2], [2], -1)], 8)
    with pytest.raises(ValueError, match="at least one entry"):
        pack(m, [], 8)
    with pytest.raises(ValueError, match="not live"):
        m.requests["ghost"] = type(m.record("a"))(m, "ghost", 99, 0)   # a record the library does not know
        try:
            pack(m, [("ghost", [1], [], -1)], 8)
        finally:
            del m.requests["ghost"]
