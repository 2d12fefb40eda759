"""The scheduler's decisions against a fake step function (CPU): admission, token budget,
portions, finishing, what happens when pages run out."""
import pytest

from llm_rs_b200.cache import CacheManager, GroupSpec
from llm_rs_b200.engine import Request, Scheduler
from llm_rs_b200.parts import CacheNeed
from llm_rs_b200.sampling import SamplingParams


def make(n_pages=16, page=4, slots=4, budget=16, chunk=8, eos=(99,), max_positions=64):
    m = CacheManager([GroupSpec(CacheNeed("full", 1, 16), [0], n_pages)], page, slots)
    return m, Scheduler(m, max_positions, eos, max_tokens_per_step=budget, prefill_chunk=chunk,
                        max_requests_per_step=slots)


def run_step(m, s, token_of=lambda req: 7):
    """What the engine does around the real step function, with a fake one."""
    batch = s.schedule()
    for b in batch:
        if b.request.request_id not in m.requests:
            m.admit(b.request.request_id)
        m.reserve(b.request.request_id, len(b.tokens))
    for b in batch:
        m.commit(b.request.request_id, len(b.tokens))
    sampled = {b.request.request_id: token_of(b.request) for b in batch if b.sample}
    outs = s.update(batch, sampled)
    m.check_invariants()
    return batch, outs


def req(i, n, max_new=4, **kw):
    return Request(i, list(range(1, n + 1)), SamplingParams(temperature=0.0, max_new_tokens=max_new, **kw))


def test_prompt_is_cut_into_portions_under_the_budget():
    m, s = make(budget=16, chunk=8)
    s.add_request(req(1, 20))
    sizes = []
    while s.has_work():
        batch, outs = run_step(m, s)
        sizes.append([len(b.tokens) for b in batch])
    assert sizes[:3] == [[8], [8], [4]]          # chunks of at most prefill_chunk
    assert sizes[3:] == [[1], [1], [1]]          # then one token a step until max_new_tokens
    assert not m.requests and m.free_pages() == 16


def test_decode_first_then_portions_in_arrival_order():
    m, s = make(budget=10, chunk=8, n_pages=32)
    s.add_request(req(1, 3))
    run_step(m, s)                                # request 1 is now decoding
    s.add_request(req(2, 12))
    s.add_request(req(3, 5))
    batch, _ = run_step(m, s)
    assert [(b.request.request_id, len(b.tokens), b.sample) for b in batch] == [(1, 1, True), (2, 8, False), (3, 1, False)]
    batch, _ = run_step(m, s)
    assert [(b.request.request_id, len(b.tokens), b.sample) for b in batch] == [(1, 1, True), (2, 4, True), (3, 4, True)]


def test_sample_only_when_the_prompt_is_complete_and_outputs():
    m, s = make()
    s.add_request(req(1, 10, max_new=2))
    batch, outs = run_step(m, s)
    assert [b.sample for b in batch] == [False] and outs == []
    batch, outs = run_step(m, s)
    assert [b.sample for b in batch] == [True]
    assert [(o.request_id, o.token, o.finished) for o in outs] == [(1, 7, False)]
    batch, outs = run_step(m, s)
    assert [(o.token, o.finished, o.reason) for o in outs] == [(7, True, "length")]


def test_eos_finishes_and_is_emitted_unless_ignored():
    m, s = make()
    s.add_request(req(1, 3, max_new=10))
    s.add_request(req(2, 3, max_new=3, ignore_eos=True))
    outs = []
    while s.has_work():
        outs += run_step(m, s, token_of=lambda r: 99)[1]
    one = [(o.token, o.finished, o.reason) for o in outs if o.request_id == 1]
    two = [(o.token, o.finished, o.reason) for o in outs if o.request_id == 2]
    assert one == [(99, True, "stop")]
    assert two == [(99, False, None), (99, False, None), (99, True, "length")]


def test_context_limit_finishes():
    m, s = make(max_positions=8, n_pages=8)
    s.add_request(req(1, 6, max_new=50))
    outs = []
    while s.has_work():
        outs += run_step(m, s)[1]
    assert len(outs) == 2 and outs[-1].reason == "length"      # 6 + 2 = 8 positions
    with pytest.raises(ValueError, match="no room"):
        s.add_request(req(2, 8))
    with pytest.raises(ValueError, match="at least one"):
        s.add_request(Request(3, [], SamplingParams()))


def test_admission_waits_behind_the_head_of_the_queue():
    m, s = make(n_pages=4, page=4, budget=64, chunk=64)        # 16 tokens of cache
    s.add_request(req(1, 10, max_new=3))
    s.add_request(req(2, 9, max_new=2))                          # does not fit beside request 1
    s.add_request(req(3, 2, max_new=2))                          # would fit, but waits behind 2
    batch, _ = run_step(m, s)
    assert [b.request.request_id for b in batch] == [1]
    assert [r.request_id for r in s.waiting] == [2, 3]
    done = []
    while s.has_work():
        done += [o.request_id for o in run_step(m, s)[1] if o.finished]
    assert done == [1, 2, 3]
    assert s.stats["preemptions"] == 0


def test_out_of_pages_preempts_the_last_admitted_and_recomputes():
    m, s = make(n_pages=4, page=4, budget=64, chunk=64, slots=3)
    s.add_request(req(1, 7, max_new=6))
    s.add_request(req(2, 7, max_new=6))
    outs = []
    steps = 0
    while s.has_work():
        batch, o = run_step(m, s)
        outs += o
        steps += 1
        assert steps < 100
    # 16 tokens of cache cannot hold 2 x (7 + 6): request 2 was sent back and came again.
    assert s.stats["preemptions"] >= 1
    by = {1: [], 2: []}
    for o in outs:
        by[o.request_id].append(o)
    assert [len(v) for v in by.values()] == [6, 6]              # nothing dropped, nothing emitted twice
    assert by[1][-1].reason == by[2][-1].reason == "length"
    assert not m.requests and m.free_pages() == 4


def test_preempted_request_recomputes_prompt_plus_generated():
    m, s = make(n_pages=3, page=4, budget=64, chunk=64)
    s.add_request(req(1, 4, max_new=8))
    s.add_request(req(2, 4, max_new=8))
    seen = []
    while s.has_work():
        batch, _ = run_step(m, s)
        seen += [(b.request.request_id, len(b.tokens), b.request.preemptions) for b in batch]
    again = [n for rid, n, p in seen if rid == 2 and p >= 1 and n > 1]
    assert again and again[0] > 4            # came back with its prompt AND what it had generated


def test_request_that_can_never_fit_ends_with_an_error():
    m, s = make(n_pages=2, page=4, budget=64, chunk=64)        # 8 tokens of cache
    s.add_request(req(1, 12))
    s.add_request(req(2, 3, max_new=2))
    outs = []
    while s.has_work():
        outs += run_step(m, s)[1]
    assert [(o.request_id, o.reason) for o in outs if o.finished] == [(1, "error_too_long"), (2, "length")]


def test_lone_request_that_outgrows_the_pool_ends_with_an_error():
    m, s = make(n_pages=2, page=4, budget=64, chunk=64)
    s.add_request(req(1, 6, max_new=10))
    outs = []
    while s.has_work():
        outs += run_step(m, s)[1]
    assert outs[-1].reason == "error_too_long" and outs[-1].token is None
    assert [o.token for o in outs[:-1]] == [7, 7, 7]             # tokens 7, 8 and the one at position 8 fails
    assert not m.requests and m.free_pages() == 2


def test_abort_frees_everything():
    m, s = make()
    s.add_request(req(1, 5))
    s.add_request(req(2, 5))
    run_step(m, s)
    outs = s.abort_all()
    assert sorted(o.request_id for o in outs) == [1, 2] and all(o.finished for o in outs)
    assert not m.requests and m.free_pages() == 16


def test_abort_with_a_step_in_flight_leaves_nothing_behind():
    """A step is queued (its samples in flight), the next one is scheduled, and then the step function
    fails: after ``abort_all`` the scheduler knows no request and no batch, in the library or here."""
    m, s = make()
    s.add_request(req(1, 5, max_new=8))
    s.add_request(req(2, 5, max_new=8))
    first = s.schedule()
    for b in first:
        m.admit(b.request.request_id)
        m.reserve(b.request.request_id, len(b.tokens))
        m.commit(b.request.request_id, len(b.tokens))
    s.on_launched(first)
    assert all(b.request.n_inflight == 1 for b in first)
    second = s.schedule()                       # scheduled with the tokens still on the device ...
    assert second and all(b.pending for b in second)
    outs = s.abort_all()                        # ... and never launched: the step function raised
    assert sorted(o.request_id for o in outs) == [1, 2]
    assert not s._requests and not s.has_work()
    assert not m.requests and m.free_pages() == 16
    m.check_invariants()
    # The scheduler is usable afterwards.
    s.add_request(req(3, 4, max_new=2))
    done = []
    while s.has_work():
        done += run_step(m, s)[1]
    assert [o.token for o in done] == [7, 7] and not s._requests


def run_async(m, s, token_of, max_steps=200):
    """The engine's pipelined loop with a fake step function: a step's tokens are handed to
    the scheduler only after the NEXT step has been scheduled and 'launched'."""
    outs, flight, steps = [], None, 0
    while s.has_work() or flight is not None:
        batch = s.schedule()
        for b in batch:
            if b.request.request_id not in m.requests:
                m.admit(b.request.request_id)
            m.reserve(b.request.request_id, len(b.tokens))
            m.commit(b.request.request_id, len(b.tokens))
            if b.pending:
                assert b.request.n_inflight == 1 and len(b.tokens) == 1
        s.on_launched(batch)
        m.check_invariants()
        launched = (batch, {b.request.request_id: token_of(b.request) for b in batch if b.sample}) if batch else None
        if flight is not None:
            outs += s.on_result(*flight)
        flight = launched
        if launched is None and flight is None:
            outs += s.on_result([], {})
        steps += 1
        assert steps < max_steps
    return outs


def test_pipelined_results_one_step_late():
    m, s = make(n_pages=32)
    s.add_request(req(1, 5, max_new=4))
    s.add_request(req(2, 3, max_new=6))
    outs = run_async(m, s, lambda r: 7)
    by = {1: [o for o in outs if o.request_id == 1], 2: [o for o in outs if o.request_id == 2]}
    assert [len(v) for v in by.values()] == [4, 6]           # exactly max_new_tokens each: no step wasted on length
    assert by[1][-1].reason == by[2][-1].reason == "length"
    assert s.stats["tokens"] == 5 + 3 + 3 + 5                 # prompts + one decode token per generated token but the last
    assert not m.requests and m.free_pages() == 32


def test_pipelined_eos_drops_the_token_that_was_one_too_many():
    m, s = make(n_pages=32)
    s.add_request(req(1, 4, max_new=20))
    n = {"calls": 0}

    def token_of(r):
        n["calls"] += 1
        return 99 if n["calls"] == 3 else 7                   # the third sampled token is EOS
    outs = run_async(m, s, token_of)
    assert [(o.token, o.finished, o.reason) for o in outs] == [(7, False, None), (7, False, None), (99, True, "stop")]
    assert n["calls"] == 4                                    # one more step had been queued before EOS was seen
    assert not m.requests and m.free_pages() == 32


def test_pipelined_preemption_keeps_every_token():
    m, s = make(n_pages=4, page=4, budget=64, chunk=64, slots=3)
    s.add_request(req(1, 7, max_new=6))
    s.add_request(req(2, 7, max_new=6))
    outs = run_async(m, s, lambda r: 7)
    assert s.stats["preemptions"] >= 1
    assert sorted(o.request_id for o in outs if o.token is not None) == [1] * 6 + [2] * 6
    assert not m.requests and m.free_pages() == 4


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_finish_every_request_and_lose_no_page(seed):
    """Requests of random lengths arrive at random times into a pool that is too small for all of
    them; results come back one step late. Every request ends with exactly the tokens it asked for
    (or at EOS), nothing is scheduled twice in a step, no step exceeds its budget, and all pages
    are back at the end."""
    import random
    rng = random.Random(seed)
    page, n_pages, slots, budget, chunk = 4, rng.choice([12, 20, 40]), rng.choice([3, 5]), rng.choice([8, 16]), rng.choice([4, 8])
    m, s = make(n_pages=n_pages, page=page, slots=slots, budget=budget, chunk=chunk, eos=(99,), max_positions=n_pages * page)
    todo = [(rng.randint(1, 3 * page * 2), rng.randint(1, 9)) for _ in range(rng.randint(6, 14))]
    want, got, flight, next_id, steps = {}, {}, None, 1, 0
    while todo or s.has_work() or flight is not None:
        while todo and rng.random() < 0.5:
            n, max_new = todo.pop()
            n = min(n, n_pages * page - max_new - 1)
            s.add_request(req(next_id, n, max_new=max_new))
            want[next_id], got[next_id] = max_new, []
            next_id += 1
        batch = s.schedule()
        ids = [b.request.request_id for b in batch]
        assert len(ids) == len(set(ids)) and sum(len(b.tokens) for b in batch) <= budget and len(batch) <= slots
        for b in batch:
            if b.request.request_id not in m.requests:
                m.admit(b.request.request_id)
            m.reserve(b.request.request_id, len(b.tokens))       # must fit: the scheduler counted the pages
            m.commit(b.request.request_id, len(b.tokens))
        s.on_launched(batch)
        m.check_invariants()
        launched = (batch, {b.request.request_id: (99 if rng.random() < 0.03 else 7) for b in batch if b.sample}) if batch else None
        outs = s.on_result(*flight) if flight is not None else []
        flight = launched
        if launched is None and flight is None:
            outs += s.on_result([], {})
        for o in outs:
            if o.token is not None:
                got[o.request_id].append(o.token)
            if o.finished:
                assert o.reason in ("stop", "length", "error_too_long")
                if o.reason == "length":
                    assert len(got[o.request_id]) == want[o.request_id]
                elif o.reason == "stop":
                    assert got[o.request_id][-1] == 99 and len(got[o.request_id]) <= want[o.request_id]
                want.pop(o.request_id)
        steps += 1
        assert steps < 3000, "the scheduler does not come to an end"
    assert not want, f"requests {sorted(want)} never finished"
    assert not m.requests and m.free_pages() == n_pages
