"""Sampling on the device: one kernel launch for all rows of a step, per-row parameters.

Reference: inference/sampler.py:5-56 (greedy, temperature, top-k) and
inference/model_worker.py:32-41 (greedy when temperature <= 0, top-k when both are set).
Every draw is fixed by (seed, request key, position of the new token), so a request samples
the same tokens alone, in a batch, or after being preempted and recomputed.
"""

from __future__ import annotations

from typing import Sequence

import torch

from ..kernels import ops


class Sampler:
    def __init__(self, device, status: torch.Tensor):
        self.device = torch.device(device)
        self.status = status

    def sample(self, logits: torch.Tensor, temperature: Sequence[float], top_k: Sequence[int],
               request_key: Sequence[int], position: Sequence[int], seed: Sequence[int],
               out: torch.Tensor = None) -> torch.Tensor:
        """logits: float32 [R, V] on the device; the sequences have R entries each (``position``
        = index the new token will have in its request).  Returns int32 [R] on the device
        (``out`` if given)."""
        R = logits.shape[0]
        if out is None:
            out = torch.empty(R, dtype=torch.int32, device=self.device)
        if R == 0:
            return out
        if all(t <= 0 for t in temperature):
            ops.sample(logits, out, self.status)
            return out
        seeds = set(int(s) for s, t in zip(seed, temperature) if t > 0)
        if len(seeds) > 1:
            # rows with different seeds go in groups; the common case is one seed per engine
            for s in seeds:
                rows = [i for i in range(R) if temperature[i] > 0 and int(seed[i]) == s]
                idx = torch.tensor(rows, device=self.device)
                sub = self.sample(logits[idx].contiguous(), [temperature[i] for i in rows],
                                  [top_k[i] for i in rows], [request_key[i] for i in rows],
                                  [position[i] for i in rows], [s] * len(rows))
                out[idx] = sub
            greedy = [i for i in range(R) if temperature[i] <= 0]
            if greedy:
                idx = torch.tensor(greedy, device=self.device)
                sub = torch.empty(len(greedy), dtype=torch.int32, device=self.device)
                ops.sample(logits[idx].contiguous(), sub, self.status)
                out[idx] = sub
            return out
        host = torch.tensor([list(map(float, temperature))], dtype=torch.float32)
        ints = torch.tensor([list(map(int, top_k)), list(map(int, position))], dtype=torch.int32)
        keys = torch.tensor(list(map(int, request_key)), dtype=torch.int64)
        temp_d = host.to(self.device, non_blocking=True)[0]
        ints_d = ints.to(self.device, non_blocking=True)
        keys_d = keys.to(self.device, non_blocking=True)
        ops.sample(logits, out, self.status, temperature=temp_d, top_k=ints_d[0].contiguous(),
                   request_key=keys_d, position=ints_d[1].contiguous(), seed=seeds.pop())
        return out
