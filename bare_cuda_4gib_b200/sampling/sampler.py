"""Choosing the next token from logits.

Greedy rows and plain temperature rows are drawn on the device (argmax with the lowest index on
ties; softmax(l / T) walked as an inverse CDF in id order with one uniform number per row).
Rows whose distribution is cut by top-k or top-p are drawn on the host from the downloaded
row with the reference's algorithm: weights exp((l - max) / T); sort by weight descending, id
ascending; keep k; top-p measured on the kept set renormalised; inverse-CDF walk
(cuongvng/bare-cuda-4gib engine/src/sampler.cpp:35-104).  The uniform number of every draw comes
from the request's own generator.
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .params import SamplingParams


def host_sample(logits: np.ndarray, p: SamplingParams, u: float) -> int:
    """Draws from one float32 logits row on the CPU (every option supported)."""
    if p.greedy():
        return int(np.argmax(logits))
    w = np.exp((logits.astype(np.float32) - np.float32(logits.max())) * np.float32(1.0 / p.temperature))
    vocab = w.shape[0]
    k = min(p.top_k, vocab) if p.top_k > 0 else vocab
    if k == vocab and p.top_p >= 1.0:
        target = u * float(w.astype(np.float64).sum())
        cum = np.cumsum(w.astype(np.float64))
        i = int(np.searchsorted(cum, target, side="right"))
        return i if i < vocab else int(np.argmax(logits))
    order = np.lexsort((np.arange(vocab), -w.astype(np.float64)))[:k]   # weight desc, id asc
    kept_w = w[order].astype(np.float64)
    keep = k
    if p.top_p < 1.0:
        cum = np.cumsum(kept_w)
        reach = np.nonzero(cum >= p.top_p * kept_w.sum())[0]
        keep = int(reach[0]) + 1 if reach.size else k
    kept_w, order = kept_w[:keep], order[:keep]
    target = u * float(kept_w.sum())
    cum = np.cumsum(kept_w)
    i = int(np.searchsorted(cum, target, side="right"))
    return int(order[min(i, keep - 1)])


class DeviceSampler:
    """Samples all wanted rows of a step: one device pass, one small download."""

    def __init__(self, device, max_rows: int):
        self.device = device
        self.max_rows = max_rows
        self._host = torch.empty(2 * max_rows, dtype=torch.float32).pin_memory()
        self._dev = torch.empty(2 * max_rows, dtype=torch.float32, device=device)
        self._out = torch.empty(max_rows, dtype=torch.int32, device=device)
        self._out_host = torch.empty(max_rows, dtype=torch.int32).pin_memory()

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence,
               argmax: Optional[torch.Tensor] = None) -> List[int]:
        """`argmax` (optional): the rows' argmax already computed on the device; a batch of greedy
        requests then needs one small download and nothing else."""
        from ..kernels import lib as K

        rows = len(params)
        if argmax is not None and all(p.greedy() for p in params):
            self._out_host[:rows].copy_(argmax[:rows], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return self._out_host[:rows].tolist()
        temps, uniforms = self._host[:rows].numpy(), self._host[self.max_rows: self.max_rows + rows].numpy()
        host_rows = []
        for r, (p, rng) in enumerate(zip(params, rngs)):
            if p.greedy():
                temps[r], uniforms[r] = 0.0, 0.0
            else:
                uniforms[r] = rng.random()
                if p.filtered():
                    host_rows.append(r)
                    temps[r] = 0.0
                else:
                    temps[r] = p.temperature
        self._dev[:rows].copy_(self._host[:rows], non_blocking=True)
        self._dev[self.max_rows: self.max_rows + rows].copy_(self._host[self.max_rows: self.max_rows + rows],
                                                             non_blocking=True)
        K.sample_rows(logits, self._dev[:rows], self._dev[self.max_rows: self.max_rows + rows], self._out, rows)
        self._out_host[:rows].copy_(self._out[:rows], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        tokens = self._out_host[:rows].tolist()
        for r in host_rows:
            row = logits[r].float().cpu().numpy()
            tokens[r] = host_sample(row, params[r], float(uniforms[r]))
        return tokens
