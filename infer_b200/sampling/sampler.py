"""Sampling on the device.

Greedy (temperature 0): first index of the maximum.  Temperature: argmax of logit/T + Gumbel noise,
the noise a hash of (seed, position of the token fed, vocabulary index); this is an exact sample of
softmax(logits/T), needs no state, and gives the same stream however the request is batched or cut
(kernels/ops/batch.cu:450-478; kernels/batch_gpu.cu:245).  top-k / top-p (src/sampler.cpp:8-63):
keep the k highest logits, then the smallest set of highest probabilities whose mass reaches p,
and sample among those the same way.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .. import ops


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._pinned, self._flip = {}, 0

    def sample(self, logits: torch.Tensor, params: Sequence, positions: Sequence[int],
               feedback: torch.Tensor = None, slots: Sequence[int] = None) -> torch.Tensor:
        """logits float32 [B, vocab] on the device; params: objects with temperature, seed, top_k, top_p;
        positions: the sampler's step key per row. Returns int32 [B] on the device. With ``feedback`` (int32 per
        request slot) and ``slots`` (one per row) each token is also left at feedback[slot] for the next step."""
        B = logits.shape[0]
        if B != len(params) or B != len(positions):
            raise ValueError("one SampleParams and one position per row of logits")
        host = np.zeros((B, 4), dtype=np.int64)
        temp = np.zeros(B, dtype=np.float32)
        top_p = np.ones(B, dtype=np.float32)
        filtered = False
        for i, (p, pos) in enumerate(zip(params, positions)):
            temp[i] = max(0.0, float(p.temperature))
            host[i, 0] = int(p.seed) & 0x7FFFFFFFFFFFFFFF
            host[i, 1] = int(pos)
            host[i, 2] = int(getattr(p, "top_k", 0) or 0)
            host[i, 3] = int(slots[i]) if slots is not None else 0
            top_p[i] = float(getattr(p, "top_p", 1.0))
            if temp[i] > 0 and (host[i, 2] > 0 or top_p[i] < 1.0):
                filtered = True
        # two pinned staging buffers per batch size take turns; the event says when the copies out of one have run,
        # and is waited for before the buffer is written again
        self._flip ^= 1
        key = (B, self._flip)
        stage = self._pinned.get(key)
        if stage is None:
            stage = self._pinned[key] = (torch.empty((B, 4), dtype=torch.int64).pin_memory(),
                                         torch.empty(B, dtype=torch.float32).pin_memory(), torch.cuda.Event())
        stage[2].synchronize()
        stage[0].numpy()[:] = host
        stage[1].numpy()[:] = temp
        ints = stage[0].to(self.device, non_blocking=True)
        t = stage[1].to(self.device, non_blocking=True)
        stage[2].record()
        self.last_h2d_bytes = host.nbytes + temp.nbytes
        seed, step = ints[:, 0].contiguous(), ints[:, 1].contiguous()
        fb = feedback if slots is not None else None
        sl = ints[:, 3].contiguous() if fb is not None else None
        if not filtered:
            return ops.sample(logits, t, seed, step, fb, sl)
        tp = torch.from_numpy(top_p).pin_memory().to(self.device, non_blocking=True)
        return ops.sample_filtered(logits, t, seed, step, ints[:, 2].contiguous(), tp, fb, sl)
