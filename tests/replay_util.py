"""Traces for the replay tests and a driver that runs them through the engine's step function."""
import random
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch


def whole(reqs: Dict[str, List[int]]):
    """Each request alone and whole: one step per request, all logits wanted."""
    return [{"entries": [{"id": r, "tokens": toks, "want": list(range(len(toks)))}], "end": [r]}
            for r, toks in reqs.items()]


def tail_one_by_one(reqs: Dict[str, List[int]], tail: int = 32):
    """All but the last ``tail`` tokens in one step, the rest one by one."""
    steps = []
    for r, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"entries": [{"id": r, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"entries": [{"id": r, "tokens": [toks[i]], "want": [0]}], "end": []})
        steps[-1]["end"] = [r]
    return steps


def portions(reqs: Dict[str, List[int]], sizes=(7, 2, 13, 5, 2, 31, 3, 17, 2, 64)):
    """Portions of changing size, down to two tokens."""
    steps = []
    for r, toks in reqs.items():
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            steps.append({"entries": [{"id": r, "tokens": toks[at:at + n], "want": list(range(n))}], "end": []})
            at += n
            k += 1
        steps[-1]["end"] = [r]
    return steps


def mixed(reqs: Dict[str, List[int]], seed: int = 0, max_live: int = 4, decode_tail: int = 12,
          sizes=(2, 3, 5, 8, 16, 17, 29, 40)):
    """Up to ``max_live`` live requests: portions of some beside single tokens of others.
    Each request is fed in random portions (of the given ``sizes``), its last ``decode_tail`` tokens
    one by one; a request may sit out a step. A finished request is ended and the next one admitted."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: Dict[str, int] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            r, _ = waiting.pop(0)
            live[r] = 0
        entries, end = [], []
        for r in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            toks, at = reqs[r], live[r]
            left = len(toks) - at
            if left <= decode_tail:
                n = 1
            else:
                n = min(left - decode_tail, rng.choice(list(sizes)))
            entries.append({"id": r, "tokens": toks[at:at + n], "want": list(range(n))})
            live[r] = at + n
            if live[r] == len(toks):
                end.append(r)
                del live[r]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def want_only(steps, wanted: Dict[str, set]):
    """The same trace asking for logits at the absolute positions in ``wanted[request]`` only."""
    at: Dict[str, int] = {}
    out = []
    for st in steps:
        entries = []
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            entries.append({"id": e["id"], "tokens": e["tokens"],
                            "want": [i for i in range(len(e["tokens"])) if base + i in wanted[e["id"]]]})
            at[e["id"]] = base + len(e["tokens"])
        for r in st["end"]:
            at.pop(r, None)
        out.append({"entries": entries, "end": st["end"]})
    return out


def live_token_peak(steps) -> int:
    """Most tokens that live requests hold at any time, each rounded up to 64."""
    held: Dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // 64) * 64 for n in held.values()))
        for r in st["end"]:
            held.pop(r, None)
    return peak


def run_steps(runner, steps) -> Dict[Tuple[str, int], np.ndarray]:
    """Drive ``ModelRunner.step`` with a trace; logits by (request, absolute position)."""
    from llm_rs_b200.engine import StepEntry
    out: Dict[Tuple[str, int], np.ndarray] = {}
    at: Dict[str, int] = {}
    for st in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]
        logits = runner.step(entries)
        rows = None if logits is None else logits.float().cpu().numpy()
        k = 0
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = rows[k]
                k += 1
            at[e["id"]] = base + len(e["tokens"])
        for r in st["end"]:
            runner.release(r)
            at.pop(r, None)
        runner.manager.check_invariants()
    return out


def max_diff(got: Dict[Tuple[str, int], np.ndarray], ref: Dict[str, np.ndarray]):
    """Largest absolute difference and where it is; every wanted position must be there."""
    worst, where = 0.0, None
    n = 0
    for (r, pos), row in got.items():
        d = float(np.abs(row.astype(np.float64) - ref[r][pos]).max())
        n += 1
        if d > worst or not np.isfinite(d):
            worst, where = d, (r, pos)
            if not np.isfinite(d):
                break
    return worst, where, n
