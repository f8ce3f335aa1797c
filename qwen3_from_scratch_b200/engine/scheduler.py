"""Continuous batching: who runs in the next step, with how many tokens.

Policy, after the reference's scheduler (inference/scheduler.py:48-153):
  1. requests that are decoding get one token each, first come first served;
  2. then requests already running whose prompt is not finished get their next portion;
  3. then waiting requests are admitted, in arrival order;
under two budgets per step, ``max_num_seqs`` requests and ``max_num_tokens`` tokens, with a
portion never longer than ``chunked_prefill_size``.  The last portion of a prompt, and every
decoded token, asks for logits.

When pages run out:
  * a decoding request that cannot get its next page preempts the most recently admitted
    other decoding request, or itself if there is none (inference/scheduler.py:69-79);
  * a portion that cannot get its pages waits for a later step (:113-115), and no new request
    is admitted in that step;
  * if nothing at all can run although requests are running, the most recently admitted
    running request is preempted until something can.
A preempted request gives back its pages and slot and goes to the *front* of the waiting
queue; it keeps the tokens it has generated and is recomputed from position 0 over prompt +
generated (the reference drops the generated tokens and queues it last: :155-162).
A request that could never fit (prompt + max_new_tokens beyond the pool or the model's
positions) is refused at ``add_request`` (:39-46).
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Callable, Deque, List, Optional

from ..cache.manager import CacheManager
from .request import Request, RequestStatus


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 32
    max_num_tokens: int = 3000
    chunked_prefill_size: int = 512
    max_positions: int = 1 << 30


@dataclass
class ScheduledRequest:
    request: Request
    num_tokens: int
    wants_logits: bool  # the step reaches the end of prompt + output, so a token is sampled after it


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager,
                 is_finished: Optional[Callable[[Request], Optional[str]]] = None):
        """``is_finished(request)`` returns a finish reason after a token was appended, or None."""
        self.config = config
        self.cache = cache
        self.is_finished = is_finished or self._length_only
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []  # in admission order
        self.num_preemptions = 0

    @staticmethod
    def _length_only(req: Request) -> Optional[str]:
        return "length" if len(req.output) >= req.params.max_new_tokens else None

    # ------------------------------------------------------------------ admission
    def add_request(self, req: Request) -> bool:
        total = len(req.prompt) + req.params.max_new_tokens
        if total > self.cache.capacity_tokens() or total > self.config.max_positions:
            return False
        req.status = RequestStatus.WAITING
        self.waiting.append(req)
        return True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ one step's plan
    def schedule(self) -> List[ScheduledRequest]:
        while True:
            plan = self._schedule_once()
            if plan or not self.running:
                return plan
            # nothing can run although requests hold pages: free the newest one's and try again
            self._preempt(self.running[-1])

    def _schedule_once(self) -> List[ScheduledRequest]:
        cfg = self.config
        plan: List[ScheduledRequest] = []
        tokens_left = cfg.max_num_tokens
        seqs_left = cfg.max_num_seqs

        # 1. decoding requests, oldest first
        decoding = [r for r in self.running if r.is_decoding]
        i = 0
        while i < len(decoding) and seqs_left > 0 and tokens_left > 0:
            req = decoding[i]
            preempted_self = False
            while not self.cache.can_reserve(req, len(req)):
                victim = decoding[-1]
                if victim is req:
                    preempted_self = True
                decoding.pop()
                self._preempt(victim)
                if preempted_self:
                    break
            if preempted_self:
                break
            self.cache.reserve(req, len(req))
            plan.append(ScheduledRequest(req, 1, True))
            seqs_left -= 1
            tokens_left -= 1
            i += 1

        # 2. running requests that still have a prompt (or a recomputation) to finish
        blocked = False
        for req in [r for r in self.running if not r.is_decoding]:
            if seqs_left <= 0 or tokens_left <= 0:
                break
            n = min(req.remaining, cfg.chunked_prefill_size, tokens_left)
            if not self.cache.can_reserve(req, req.num_computed + n):
                blocked = True
                continue
            self.cache.reserve(req, req.num_computed + n)
            plan.append(ScheduledRequest(req, n, n == req.remaining))
            seqs_left -= 1
            tokens_left -= n

        # 3. waiting requests, in order, while the first one fits
        while self.waiting and not blocked and seqs_left > 0 and tokens_left > 0:
            req = self.waiting[0]
            if self.cache.free_slots() == 0:
                break
            n = min(req.remaining, cfg.chunked_prefill_size, tokens_left)
            self.cache.open(req)
            if not self.cache.can_reserve(req, n):
                self.cache.close(req)
                break
            self.cache.reserve(req, n)
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            plan.append(ScheduledRequest(req, n, n == req.remaining))
            seqs_left -= 1
            tokens_left -= n

        for s in plan:
            s.request.num_scheduled = s.num_tokens
        return plan

    def _preempt(self, req: Request) -> None:
        self.cache.close(req)
        self.running.remove(req)
        req.num_computed = 0
        req.num_scheduled = 0
        req.status = RequestStatus.WAITING
        req.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)

    def abort(self, req: Request) -> None:
        """Takes a request out wherever it is and gives back what it holds."""
        if req in self.running:
            self.running.remove(req)
            self.cache.close(req)
        elif req in self.waiting:
            self.waiting.remove(req)
        req.status = RequestStatus.FINISHED
        req.finish_reason = req.finish_reason or "abort"

    # ------------------------------------------------------------------ after the step
    def post_process(self, plan: List[ScheduledRequest], sampled: List[Optional[int]]) -> List[Request]:
        """``sampled[i]``: the token drawn for plan[i] (ignored unless it wanted logits).
        Records progress, appends tokens, finishes and frees.  Returns the finished requests."""
        finished = []
        for s, token in zip(plan, sampled):
            req = s.request
            req.num_computed += s.num_tokens
            req.num_scheduled = 0
            self.cache.advance(req, req.num_computed)
            if not s.wants_logits:
                continue
            if token is None:
                raise ValueError(f"request {req.request_id} wanted a token and got none")
            req.output.append(int(token))
            reason = self.is_finished(req)
            if reason is not None:
                req.status = RequestStatus.FINISHED
                req.finish_reason = reason
                self.running.remove(req)
                self.cache.close(req)
                finished.append(req)
        return finished
