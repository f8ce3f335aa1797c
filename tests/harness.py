"""Helpers of the GPU tests: replaying requests through a Session in different cuts and
collecting the logits per (request, position)."""

from __future__ import annotations

from typing import Dict, Hashable, List, Sequence, Tuple

import torch

import plain_qwen3 as plain

# Bounds on |engine - plain| relative to the largest |logit| of the plain result.
# float32: both sides are float32 with different summation orders; sums of a few hundred terms
# over a handful of layers stay within ~1e-6 relative, 1e-5 leaves room without hiding a fault.
# bfloat16: activations are rounded to 8 significant bits (relative 2^-9 ~ 2e-3) at every
# projection input and output; over the 2-3 layers of the tiny models that compounds to
# well under 1e-2 of the logits' scale, 2e-2 is the bound.
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def plain_logits(folder: str, sequences: Dict[Hashable, Sequence[int]]) -> Dict[Hashable, torch.Tensor]:
    cfg, w = plain.read_model_folder(folder)
    return {req: plain.forward_logits(cfg, w, ids) for req, ids in sequences.items()}


class Replayer:
    """Feeds each request's tokens in the portions a schedule names; wants every position."""

    def __init__(self, session, sequences: Dict[Hashable, Sequence[int]]):
        from qwen3_from_scratch_b200.engine.batch import Entry
        self._Entry = Entry
        self.session = session
        self.sequences = {r: list(s) for r, s in sequences.items()}
        self.fed = {r: 0 for r in sequences}
        self.rows: Dict[Hashable, List[torch.Tensor]] = {r: [] for r in sequences}

    def step(self, portions: Sequence[Tuple[Hashable, int]], end_finished: bool = True) -> None:
        entries, counts = [], []
        for req, n in portions:
            start = self.fed[req]
            n = min(n, len(self.sequences[req]) - start)
            assert n > 0, f"request {req} has no tokens left"
            entries.append(self._Entry(req, self.sequences[req][start:start + n], list(range(n))))
            counts.append((req, n))
        logits = self.session.step(entries).float().cpu()
        self.session.check_status()
        at = 0
        for req, n in counts:
            self.rows[req].append(logits[at:at + n])
            at += n
            self.fed[req] += n
            if end_finished and self.fed[req] == len(self.sequences[req]):
                self.session.end(req)
        assert at == logits.shape[0]

    def remaining(self, req) -> int:
        return len(self.sequences[req]) - self.fed[req]

    def result(self) -> Dict[Hashable, torch.Tensor]:
        return {r: torch.cat(rows) if rows else torch.empty(0) for r, rows in self.rows.items()}


def assert_close(got: Dict[Hashable, torch.Tensor], want: Dict[Hashable, torch.Tensor], dtype: str, what: str):
    for req, w in want.items():
        g = got[req]
        assert g.shape == w.shape, f"{what}: request {req}: {tuple(g.shape)} vs {tuple(w.shape)}"
        assert torch.isfinite(g).all(), f"{what}: request {req} has non-finite logits"
        scale = max(float(w.abs().max()), 1e-6)
        err = (g - w).abs().max(dim=-1).values / scale
        worst = int(err.argmax())
        assert float(err[worst]) <= TOL[dtype], (
            f"{what}: request {req}: first position beyond {TOL[dtype]:g} is "
            f"{int((err > TOL[dtype]).nonzero()[0])}, worst {float(err[worst]):.3g} at position {worst}")
