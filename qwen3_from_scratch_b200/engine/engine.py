"""The Python entry point: an in-process engine with continuous batching.

It follows the reference's ``SyncEngine`` (inference/sync_engine.py:28-182): ``warmup``,
``generate_stream``, ``generate``, ``batch_generate``, with the scheduler options of its YAML
(``max_num_seqs``, ``max_num_tokens``, ``block_size``, ``gpu_utilization``,
``chunked_prefill_size``: factory/batch_config.py:141-148) and its generation options
(``temperature``, ``top_k``, ``max_new_tokens``: :83-91).  Prompts are lists of token ids;
text works when the model folder has a ``tokenizer.json``.  ``SyncEngine.from_config`` reads
a YAML file of the reference's layout.
"""

from __future__ import annotations

import json
import logging
import os
import time
from dataclasses import dataclass
from typing import Iterator, List, Optional, Sequence, Tuple, Union

import torch

from ..sampling.sampler import Sampler
from .batch import Entry
from .request import Request, RequestStatus, SamplingParams
from .scheduler import ScheduledRequest, Scheduler, SchedulerConfig
from .session import Session

logger = logging.getLogger("qwen3_from_scratch_b200")

Prompt = Union[str, Sequence[int], Sequence[dict]]


@dataclass
class PerfMetrics:
    """Wall-clock figures of one request, as in the reference (inference/llm_engine.py:48-58)."""

    ttft: float
    token_count: int
    tps: float
    total_elapsed: float


@dataclass
class StreamChunk:
    delta: str
    token_id: int
    metrics: PerfMetrics


@dataclass
class BatchPerfMetrics:
    per_request: List[PerfMetrics]
    num_requests: int
    total_tokens: int
    total_elapsed: float
    aggregate_tps: float


@dataclass
class GenerationResult:
    token_ids: List[int]
    text: Optional[str]
    finish_reason: str
    metrics: PerfMetrics


@dataclass
class _InFlight:
    """A step that has been put on the device and whose results have not been read yet."""
    plan: List[ScheduledRequest]
    wanting: List[ScheduledRequest]
    box: torch.Tensor          # device: [0] unused here, then the sampled tokens
    host_box: torch.Tensor     # pinned copy of it
    host_status: torch.Tensor  # pinned copy of the status word
    done: torch.cuda.Event
    ahead: bool                # launched before the step before it had been read


class SyncEngine:
    def __init__(self, model_path: str, *, dtype: str = "bfloat16", device: str = "cuda:0",
                 max_num_seqs: int = 32, max_num_tokens: int = 3000, block_size: int = 16,
                 gpu_utilization: float = 0.5, num_pages: Optional[int] = None,
                 chunked_prefill_size: int = 512, enable_prefix_cache: bool = False,
                 temperature: float = 0.0, top_k: int = 0, max_new_tokens: int = 100, seed: int = 0,
                 eos_token_id: Optional[int] = None, log_interval: int = 0, cuda_graphs: bool = True,
                 lookahead: bool = True, random_weights: Optional[int] = None):
        """``random_weights``: a seed; ``model_path`` then needs only config.json and the weights are drawn on
        the device.  ``num_pages`` fixes the size of the cache pool; otherwise ``gpu_utilization`` of the
        memory that is free after the weights are loaded is given to it.  ``lookahead``: while a plain
        decode step runs, the step after it is already put on the device (see ``step``)."""
        if enable_prefix_cache:
            # The reference's own configurations set this (its default is true: factory/batch_config.py:147).
            # Sharing pages between requests with a common prefix saves work and changes no output, so the
            # option is taken and the engine runs without sharing.
            logger.warning("enable_prefix_cache: prefix sharing between requests is not built; running without it "
                           "(outputs are the same)")
        self.model_path = model_path
        self.log_interval = log_interval
        self.defaults = SamplingParams(temperature=temperature, top_k=top_k, max_new_tokens=max_new_tokens,
                                       seed=seed)
        cache_pages = num_pages
        if cache_pages is None:
            cache_pages = self._pages_from_memory(model_path, dtype, device, block_size, gpu_utilization,
                                                  max_num_seqs)
        self.session = Session(model_path, dtype=dtype, device=device, page_size=block_size,
                               num_pages=cache_pages, max_seqs=max_num_seqs, max_step_tokens=max_num_tokens,
                               cuda_graphs=cuda_graphs, random_weights=random_weights)
        self.config = self.session.config
        spec = self.session.model.spec
        self.eos_token_id = eos_token_id if eos_token_id is not None else spec.eos_token_id
        self.scheduler = Scheduler(
            SchedulerConfig(max_num_seqs=max_num_seqs, max_num_tokens=max_num_tokens,
                            chunked_prefill_size=chunked_prefill_size, max_positions=spec.max_positions),
            self.session.manager, is_finished=self._finish_reason)
        self.sampler = Sampler(self.session.rt.device, self.session.rt.status)
        self.tokenizer = self._load_tokenizer(model_path)
        self.num_steps = 0
        # Two places for a step's sampled tokens (a step and the one launched ahead of its results use one
        # each), and pinned host copies of them with the status word.
        rt = self.session.rt
        self.lookahead = bool(lookahead)
        self._boxes = [rt.mailbox, torch.zeros_like(rt.mailbox)]
        self._host_boxes = [torch.zeros(rt.mailbox.numel(), dtype=torch.int32).pin_memory() for _ in range(2)]
        self._host_status = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._launches = 0
        self.num_ahead = 0  # steps launched before the step before them had been read
        self._inflight: Optional[_InFlight] = None

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def from_config(cls, config_path: str, model_name: str, log_interval: int = 0) -> "SyncEngine":
        """Reads a YAML file laid out like the reference's batch configuration
        (``generation``, ``scheduler``, ``models[]`` with ``name``, ``path``, ``dtype``)."""
        import yaml
        with open(config_path) as f:
            data = yaml.safe_load(f) or {}
        entry = next((m for m in data.get("models", []) if m.get("name") == model_name), None)
        if entry is None:
            names = [m.get("name") for m in data.get("models", [])]
            raise KeyError(f"model '{model_name}' is not in {config_path} (it lists {names})")
        gen = dict(data.get("generation", {}))
        gen.update(entry.get("generation") or {})
        sched = data.get("scheduler", {})
        known = {"max_num_seqs", "max_num_tokens", "block_size", "gpu_utilization", "chunked_prefill_size",
                 "enable_prefix_cache"}
        unknown = set(sched) - known
        if unknown:
            raise ValueError(f"{config_path}: unknown scheduler keys {sorted(unknown)}")
        kwargs = {k: sched[k] for k in known & set(sched)}
        kwargs["enable_prefix_cache"] = bool(sched.get("enable_prefix_cache", False))
        dtype = str(entry.get("dtype", "bfloat16")).replace("torch.", "")
        dtype = {"bf16": "bfloat16", "fp32": "float32", "float": "float32"}.get(dtype, dtype)
        return cls(entry["path"], dtype=dtype,
                   temperature=float(gen.get("temperature", 0.0)) if gen.get("do_sample", True) else 0.0,
                   top_k=int(gen.get("top_k", 0)), max_new_tokens=int(gen.get("max_new_tokens", 100)),
                   log_interval=log_interval, **kwargs)

    @staticmethod
    def _pages_from_memory(model_path, dtype, device, block_size, gpu_utilization, max_num_seqs) -> int:
        """Pages that fit in ``gpu_utilization`` of what will be free once the weights are loaded
        (the reference sizes its pool from free memory the same way: inference/model_worker.py:49-59)."""
        from ..cache.manager import CacheManager  # noqa: F401
        from ..registry import build_model_spec, load_config
        from .model import Model, resolve_dtype
        model = Model(build_model_spec(load_config(model_path)))
        item = 2 if resolve_dtype(dtype) == torch.bfloat16 else 4
        weight_bytes = 0
        for s in model.weight_specs():
            n = 1
            for d in s.shape:
                n *= d
            weight_bytes += n * (4 if s.kind == "vector" else item)
        layout = model.cache_layout()
        per_page = sum(len(g.cache_ids) * g.spec.bytes_per_token(item) * block_size for g in layout.groups)
        state_bytes = 0  # the slots of fixed-size state are there for max_num_seqs requests whatever runs
        for spec in layout.states.values():
            n = 4 if spec.dtype == "float32" else item
            for d in spec.shape:
                n *= d
            state_bytes += n * max_num_seqs
        free, _total = torch.cuda.mem_get_info(torch.device(device))
        budget = int((free - weight_bytes - state_bytes) * gpu_utilization)
        pages = budget // max(per_page, 1) if per_page else 1
        if pages < 1:
            raise RuntimeError(f"no memory left for the cache: {free} bytes free, weights need {weight_bytes}")
        return int(pages)

    @staticmethod
    def _load_tokenizer(model_path: str):
        path = os.path.join(model_path, "tokenizer.json")
        if not os.path.isfile(path):
            return None
        from tokenizers import Tokenizer
        return Tokenizer.from_file(path)

    # ------------------------------------------------------------------ prompts and text
    def _encode(self, prompt: Prompt) -> List[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("text prompts need a tokenizer.json in the model folder; pass token ids instead")
            return self.tokenizer.encode(prompt).ids
        prompt = list(prompt)
        if prompt and isinstance(prompt[0], dict):
            return self._encode(self._render_chat(prompt))
        return [int(t) for t in prompt]

    def _render_chat(self, messages: List[dict]) -> str:
        """Chat messages -> text with the folder's chat template (tokenizer_config.json)."""
        path = os.path.join(self.model_path, "tokenizer_config.json")
        template = None
        if os.path.isfile(path):
            with open(path) as f:
                template = json.load(f).get("chat_template")
        if template is None:
            raise ValueError("chat prompts need a chat_template in tokenizer_config.json")
        import jinja2
        env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True)
        return env.from_string(template).render(messages=messages, add_generation_prompt=True)

    def _decode(self, token_ids: Sequence[int]) -> str:
        if self.tokenizer is None:
            return ""
        return self.tokenizer.decode(list(token_ids), skip_special_tokens=True)

    # ------------------------------------------------------------------ low level
    def _finish_reason(self, req: Request) -> Optional[str]:
        if (not req.params.ignore_eos and self.eos_token_id is not None
                and req.output and req.output[-1] == self.eos_token_id):
            return "eos"
        if len(req.output) >= req.params.max_new_tokens:
            return "length"
        return None

    def add_request(self, prompt: Prompt, max_new_tokens: Optional[int] = None,
                    params: Optional[SamplingParams] = None, ignore_eos: bool = False) -> Request:
        if params is None:
            params = SamplingParams(
                temperature=self.defaults.temperature, top_k=self.defaults.top_k,
                max_new_tokens=max_new_tokens or self.defaults.max_new_tokens, ignore_eos=ignore_eos,
                seed=self.defaults.seed)
        req = Request(self._encode(prompt), params)
        req.arrival_time = time.perf_counter()
        if not self.scheduler.add_request(req):
            raise ValueError(
                f"a request of {len(req.prompt)} prompt tokens and {params.max_new_tokens} new tokens can never "
                f"fit: the cache holds {self.session.manager.capacity_tokens()} tokens and the model "
                f"{self.session.max_positions} positions")
        return req

    def abort(self, req: Request) -> None:
        self.drain()
        self.scheduler.abort(req)
        self.session.after_step()

    def step(self) -> List[ScheduledRequest]:
        """One scheduling round and one model step.  Returns what ran (with tokens appended).

        With ``lookahead``, a step in which every running request decodes one token is followed on the
        device by the next such step before its own tokens have been read: the next step's token ids
        are copied from the sampler's output on the device, and positions, lengths and pages do not
        depend on which tokens were drawn.  The host then reads a step's tokens while the next one
        runs, so the device does not wait for the host between steps.  A request that turns out to have
        finished (an end-of-sequence token) has then been run one token too far; that token is dropped.
        Anything else (prompts to compute, requests waiting, a request at its last token, pages running
        short) is planned by the scheduler with all results in hand, as without lookahead."""
        flight = self._inflight
        self._inflight = None
        if flight is None:
            plan = self.scheduler.schedule()
            if not plan:
                return []
            flight = self._launch(plan, None)
        if self.lookahead:
            self._inflight = self._launch_ahead(flight)
        self._collect(flight)
        return flight.plan

    def drain(self) -> None:
        """Waits for a step launched ahead, if there is one, and records its results."""
        if self._inflight is not None:
            flight, self._inflight = self._inflight, None
            self._collect(flight)

    def _launch(self, plan: List[ScheduledRequest], after: Optional["_InFlight"]) -> "_InFlight":
        """Puts the plan's step on the device: batch, model, sampling, and the copy of the sampled tokens
        and the status word to pinned memory.  ``after``: the step (still running) whose sampled tokens
        are this step's input."""
        ahead = 0 if after is None else 1
        if after is None:
            entries = [Entry(s.request, s.request.next_tokens(s.num_tokens),
                             (s.num_tokens - 1,) if s.wants_logits else ()) for s in plan]
            logits = self.session.step_reserved(entries)
        else:
            entries = [Entry(s.request, (0,), (0,)) for s in plan]  # the ids come from the device
            logits = self.session.step_reserved(entries, ahead=1, token_source=after.box[1:1 + len(plan)])
        wanting = [s for s in plan if s.wants_logits]
        which = self._launches % 2
        self._launches += 1
        box = self._boxes[which]
        flight = _InFlight(plan, wanting, box, self._host_boxes[which], self._host_status[which], torch.cuda.Event(),
                           ahead == 1)
        if wanting:
            reqs = [s.request for s in wanting]
            self.sampler.sample(
                logits, [r.params.temperature for r in reqs], [r.params.top_k for r in reqs],
                [r.key for r in reqs], [len(r) + ahead for r in reqs], [r.params.seed for r in reqs],
                out=box[1:1 + len(reqs)])
            flight.host_box[:1 + len(reqs)].copy_(box[:1 + len(reqs)], non_blocking=True)
        flight.host_status.copy_(self.session.rt.status, non_blocking=True)
        flight.done.record()
        return flight

    def _launch_ahead(self, flight: "_InFlight") -> Optional["_InFlight"]:
        """The step after ``flight``, if it needs no decision that depends on flight's tokens."""
        sched = self.scheduler
        plan = flight.plan
        if sched.waiting or len(plan) != len(sched.running) or not all(s.num_tokens == 1 and s.wants_logits for s in plan):
            return None
        reqs = [s.request for s in plan]
        limit = self.session.max_positions
        for r in reqs:
            # (its last token, by count or by position, is decided when the scheduler sees it finished)
            if (r.status != RequestStatus.RUNNING or len(r.output) + 2 > r.params.max_new_tokens
                    or len(r) + 1 > limit or not sched.cache.can_reserve(r, len(r) + 1)):
                return None
        need = None
        for r in reqs:
            more = sched.cache.pages_needed(r, len(r) + 1)
            need = more if need is None else [a + b for a, b in zip(need, more)]
        if any(n > sched.cache.free_pages(g) for g, n in enumerate(need)):
            return None
        for r in reqs:
            sched.cache.reserve(r, len(r) + 1)
        self.num_ahead += 1
        return self._launch([ScheduledRequest(r, 1, True) for r in reqs], flight)

    def _collect(self, flight: "_InFlight") -> None:
        """Waits for the step, reads its tokens and lets the scheduler record them."""
        flight.done.synchronize()
        self.session.raise_on_status(int(flight.host_status[0]))
        plan = flight.plan
        sampled: List[Optional[int]] = [None] * len(plan)
        if flight.wanting:
            it = iter(flight.host_box[1:1 + len(flight.wanting)].tolist())
            sampled = [next(it) if s.wants_logits else None for s in plan]
        if flight.ahead:
            # a request that finished or was taken out while this step ran has been run one token too far
            live = [i for i, s in enumerate(plan) if s.request.status == RequestStatus.RUNNING]
            plan_live, sampled = [plan[i] for i in live], [sampled[i] for i in live]
        else:
            plan_live = plan
        now = time.perf_counter()
        for s in plan_live:
            if s.wants_logits and s.request.first_token_time is None:
                s.request.first_token_time = now
        for req in self.scheduler.post_process(plan_live, sampled):
            req.finish_time = now
        self.session.after_step()
        self.num_steps += 1

    # ------------------------------------------------------------------ the reference's interface
    def warmup(self, prompt: Optional[Prompt] = None, num_tokens: int = 3) -> None:
        """One short request, so that compilation and first-use costs are not in the first answer."""
        for _ in self.generate_stream(prompt if prompt is not None else [0], num_tokens, ignore_eos=True):
            pass

    def generate_stream(self, prompt: Prompt, max_new_tokens: Optional[int] = None,
                        ignore_eos: bool = False) -> Iterator[StreamChunk]:
        req = self.add_request(prompt, max_new_tokens, ignore_eos=ignore_eos)
        emitted = 0
        while True:
            self.step()
            now = time.perf_counter()
            while emitted < len(req.output):
                token = req.output[emitted]
                emitted += 1
                yield StreamChunk(self._decode([token]), token, self._metrics(req, now, emitted))
                if self.log_interval > 0 and emitted % self.log_interval == 0:
                    m = self._metrics(req, now, emitted)
                    logger.info("[stream] step=%d TTFT=%.4fs tokens=%d TPS=%.2f elapsed=%.4fs", emitted, m.ttft,
                                m.token_count, m.tps, m.total_elapsed)
            if req.status == RequestStatus.FINISHED:
                return

    def generate(self, prompt: Prompt, max_new_tokens: Optional[int] = None, ignore_eos: bool = False):
        """Generated token ids for a token-id prompt, text for a text prompt."""
        tokens = [c.token_id for c in self.generate_stream(prompt, max_new_tokens, ignore_eos)]
        if isinstance(prompt, str) or (len(prompt) and isinstance(list(prompt)[0], dict)):
            return self._decode(tokens)
        return tokens

    def batch_generate(self, prompts: Sequence[Prompt], max_new_tokens: Optional[int] = None,
                       ignore_eos: bool = False, params: Optional[Sequence[SamplingParams]] = None
                       ) -> Tuple[List[GenerationResult], BatchPerfMetrics]:
        """All prompts enter at once and run under continuous batching until every one has finished."""
        reqs = [self.add_request(p, max_new_tokens, params=params[i] if params else None, ignore_eos=ignore_eos)
                for i, p in enumerate(prompts)]
        start = min(r.arrival_time for r in reqs) if reqs else time.perf_counter()
        steps = 0
        while any(r.status != RequestStatus.FINISHED for r in reqs):
            if not self.step():
                raise RuntimeError("the scheduler has requests but could plan nothing")
            steps += 1
            if self.log_interval > 0 and steps % self.log_interval == 0:
                done = sum(r.status == RequestStatus.FINISHED for r in reqs)
                total = sum(len(r.output) for r in reqs)
                elapsed = time.perf_counter() - start
                logger.info("[batch] step=%d pending=%d completed=%d total_tokens=%d aggregate_tps=%.2f",
                            steps, len(reqs) - done, done, total, total / elapsed if elapsed > 0 else 0.0)
        results = []
        for r in reqs:
            m = self._metrics(r, r.finish_time, len(r.output))
            results.append(GenerationResult(list(r.output), self._decode(r.output) if self.tokenizer else None,
                                            r.finish_reason, m))
        total_tokens = sum(len(r.output) for r in reqs)
        elapsed = max((r.finish_time - start for r in reqs), default=0.0)
        batch = BatchPerfMetrics([x.metrics for x in results], len(reqs), total_tokens, elapsed,
                                 total_tokens / elapsed if elapsed > 0 else 0.0)
        return results, batch

    @staticmethod
    def _metrics(req: Request, now: float, count: int) -> PerfMetrics:
        first = req.first_token_time if req.first_token_time is not None else now
        decode_elapsed = now - first
        tps = (count - 1) / decode_elapsed if decode_elapsed > 0 and count > 1 else 0.0
        return PerfMetrics(ttft=first - req.arrival_time, token_count=count, tps=tps,
                           total_elapsed=now - req.arrival_time)
