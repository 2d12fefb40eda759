"""Chooses the next token of each request from its row of logits, on the device."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams


class Sampler:
    """``sample(logits, rows)``: ``logits`` is float32 [n, vocab] on the device, ``rows`` gives per
    row ``(params, request_id, index of the token to generate, token history)``. Returns
    int32 tokens on the device. Rows that are plainly greedy take the argmax kernel; any
    other row sends the batch through the sampling kernel, whose result for a row
    depends on that row's logits, parameters, request id and index only."""

    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, rows: Sequence[tuple]) -> torch.Tensor:
        n = logits.size(0)
        if n != len(rows):
            raise ValueError(f"{n} rows of logits for {len(rows)} requests")
        if all(p.plain for p, _, _, _ in rows):
            return ops.argmax(logits)
        need_hist = any(p.repetition_penalty != 1.0 for p, _, _, _ in rows)
        f = np.zeros((3, n), np.float32)      # temperature, top_p, penalty
        i = np.zeros((2, n), np.int32)        # top_k, index
        l = np.zeros((2, n), np.int64)        # seed, request id
        hist: List[int] = []
        offsets = [0]
        for r, (p, rid, index, history) in enumerate(rows):
            f[0, r], f[1, r], f[2, r] = p.temperature, p.top_p, p.repetition_penalty
            i[0, r], i[1, r] = p.top_k, index
            l[0, r], l[1, r] = np.int64(np.uint64(p.seed & (2**64 - 1)).astype(np.int64)), \
                np.int64(np.uint64(rid & (2**64 - 1)).astype(np.int64))
            if need_hist and p.repetition_penalty != 1.0:
                hist.extend(sorted(set(int(t) for t in history)))
            offsets.append(len(hist))
        dev = self.device
        fd = torch.from_numpy(f).to(dev, non_blocking=True)
        idv = torch.from_numpy(i).to(dev, non_blocking=True)
        ld = torch.from_numpy(l).to(dev, non_blocking=True)
        hist_t = off_t = None
        if need_hist:
            hist_t = torch.tensor(hist if hist else [0], dtype=torch.int32, device=dev)
            off_t = torch.tensor(offsets, dtype=torch.int32, device=dev)
        return ops.sample(logits, fd[0], idv[0], fd[1], fd[2] if need_hist else None, hist_t, off_t,
                          ld[0], ld[1], idv[1])
