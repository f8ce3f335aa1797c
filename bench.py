"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--model 0.6b|8b|32b]

One "step" is one decode step of the whole batch.  The default run uses the layer sizes of
Qwen3-0.6B (28 layers, hidden 1024, 16/8 heads of 128, intermediate 3072, vocabulary 151936,
tied head) with seeded random weights, a batch of 8 and a context of 4096 tokens per sequence,
pages of 16 tokens.  It prints one JSON line:

  value      decoded tokens per second, timed on the device (CUDA events): K steps, repeated
             ``--repeats`` times, the median repeat
  e2e        the same through the Python entry point (``SyncEngine.step``): every step copies its
             token ids and block tables from pinned host memory and reads the sampled ids back; all K
             steps of a repeat are launched and collected inside its clock.  The repeats decode one after
             the other, so all but the last run at contexts up to ``repeats * K`` tokens shorter than the
             device-timed one
  prefill    one step over a 2,048-token prompt: tokens/s and flops / time / bf16 peak
  roofline   bytes a decode step has to read (every weight once + the keys and values of the live
             requests) / its time, against the measured copy bandwidth
  points     decode tokens/s at the other batch sizes, and (default run) the figures of the Qwen3-8B
             and Qwen3-32B layer sizes, which ``--model 8b`` / ``--model 32b`` print as lines of their own

``--model 8b`` also runs the load the 8B configuration is quoted on: 64 requests at once, prompts of
128 to 2,048 random tokens, 256 new tokens each, through ``SyncEngine.batch_generate`` (continuous
batching, prompts cut into portions beside decoding requests): ``serving`` in its line.  The 8B and 32B
models take their random weights straight on the device (no file of 16 or 65 GB is written); the 0.6B
model goes through a folder and the real loader.

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else from the fallback
figures (6.65 TB/s, 1.59 PFLOP/s).  ``--impl reference`` runs the unmodified reference from
``baseline/_ref`` through its own scheduler and worker for the same metric.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

def _qwen3(hidden, heads, kv_heads, inter, layers, tied):
    return dict(architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=hidden, hidden_act="silu",
                num_hidden_layers=layers, max_position_embeddings=40960, num_key_value_heads=kv_heads,
                num_attention_heads=heads, head_dim=128, intermediate_size=inter, rms_norm_eps=1e-6,
                rope_theta=1000000.0, tie_word_embeddings=tied)


# The layer sizes the figures are quoted on, the decode batches measured at each (the first is the one of
# ``value``), and how the random weights get onto the device.
MODELS = {
    "0.6b": dict(name="Qwen3-0.6B", config=_qwen3(1024, 16, 8, 3072, 28, True), batches=(8, 1, 64),
                 weights="folder", serving=False),
    "8b": dict(name="Qwen3-8B", config=_qwen3(4096, 32, 8, 12288, 36, False), batches=(8, 1, 64),
               weights="device", serving=True),
    "32b": dict(name="Qwen3-32B", config=_qwen3(5120, 64, 8, 25600, 64, False), batches=(8, 1, 32),
                weights="device", serving=False),
}
CONFIG = MODELS["0.6b"]["config"]  # the configuration the headline figure is quoted on
CONTEXT = 4096
PAGE = 16
PREFILL_TOKENS = 2048
SERVING = dict(requests=64, prompt_min=128, prompt_max=2048, new_tokens=256, seed=4242)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks():
    """Measured peaks of this pool's GPUs if the file is there (keys hbm_gbs, bf16_tflops,
    bf16_tflops_sustained, looked for at any depth, as numbers or as {"value": number}), else the fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")

    def find(node, key):
        if isinstance(node, dict):
            if key in node:
                v = node[key]
                if isinstance(v, dict):
                    v = v.get("value")
                if isinstance(v, (int, float)) and v > 0:
                    return float(v)
            for child in node.values():
                got = find(child, key)
                if got is not None:
                    return got
        elif isinstance(node, list):
            for child in node:
                got = find(child, key)
                if got is not None:
                    return got
        return None

    if os.path.isfile(path):
        try:
            with open(path) as f:
                data = json.load(f)
            hbm, burst = find(data, "hbm_gbs"), find(data, "bf16_tflops")
            if hbm is not None and burst is not None:
                out = {"hbm_gbs": hbm, "bf16_tflops": burst, "source": "measured"}
                sustained = find(data, "bf16_tflops_sustained")
                if sustained is not None:
                    out["bf16_tflops_sustained"] = sustained
                return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: through NVML from a thread of
    this process (a query takes tens of microseconds), or with nvidia-smi if NVML cannot be loaded.
    Reading only; no setting of the GPU is touched."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, device_index: int = 0):
        """``device_index``: the CUDA device that is measured.  NVML and nvidia-smi number GPUs without regard
        to CUDA_VISIBLE_DEVICES, so the device is looked up by its UUID."""
        self.uuid = None
        try:
            import torch
            self.uuid = "GPU-" + str(torch.cuda.get_device_properties(device_index).uuid)
        except Exception:  # an older torch without the field: the first GPU is taken, and said
            self.uuid = None
        self.samples = []  # (sm MHz, max sm MHz, [active reasons])
        self.proc = None
        self.stopping = threading.Event()
        self.thread = None
        self.source = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = (pynvml.nvmlDeviceGetHandleByUUID(self.uuid.encode()) if self.uuid
                      else pynvml.nvmlDeviceGetHandleByIndex(0))
            bits = {"hw_slowdown": pynvml.nvmlClocksThrottleReasonHwSlowdown,
                    "hw_thermal_slowdown": pynvml.nvmlClocksThrottleReasonHwThermalSlowdown,
                    "sw_thermal_slowdown": pynvml.nvmlClocksThrottleReasonSwThermalSlowdown,
                    "sw_power_cap": pynvml.nvmlClocksThrottleReasonSwPowerCap}
            top = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))

            def poll():
                while not self.stopping.is_set():
                    try:
                        mhz = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                        mask = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                        self.samples.append((mhz, top, [n for n, bit in bits.items() if mask & bit]))
                    except pynvml.NVMLError:
                        pass
                    self.stopping.wait(0.02)

            self.source = "nvml"
            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            return
        except Exception:  # no NVML binding or no library: fall back to the command line tool
            self.source = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.uuid or "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.source = "nvidia-smi"
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                try:
                    self.samples.append((float(parts[0]), float(parts[1]),
                                         [n for n, flag in zip(self.NAMES, parts[2:6]) if flag.lower().startswith("active")]))
                except ValueError:
                    continue

    def stop(self):
        if self.source is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML and no nvidia-smi"]}
        if self.source == "nvml":
            self.stopping.set()
            self.thread.join(timeout=2)
        else:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        clocks = [s[0] for s in self.samples]
        reasons = sorted({r for s in self.samples for r in s[2]})
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(s[1] for s in self.samples) if self.samples else None, "reasons": reasons,
                "samples": len(clocks), "source": self.source, "gpu": self.uuid or "index 0"}


def model_numbers(cfg, layers):
    """Bytes of weights a decode step reads, bytes of cache per token, flops of a prefill."""
    H, D = cfg["hidden_size"], cfg["head_dim"]
    hq, hkv, inter, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"]
    per_layer = (hq + 2 * hkv) * D * H + H * hq * D + 3 * H * inter
    head = V * H  # read once as the output head (tied or not); embedding rows are negligible
    weight_bytes = 2 * (layers * per_layer + head) + 4 * (layers * (2 * H + 2 * D) + H)
    kv_bytes_per_token = 2 * layers * hkv * D * 2

    def prefill_flops(T):
        linear = 2 * T * layers * per_layer + 2 * V * H  # logits at one position
        attention = layers * 4 * hq * D * T * (T + 1) // 2
        return linear + attention

    return weight_bytes, kv_bytes_per_token, prefill_flops


def time_device_steps(fn, steps, warmup, repeats):
    """Seconds of ``steps`` calls of ``fn`` between CUDA events, once per repeat."""
    import torch
    for _ in range(warmup):
        fn()
    out = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        torch.cuda.synchronize()
        out.append(start.elapsed_time(end) / 1e3)
    return out


def schedule_lead(engine, batch, prompt_len):
    """Tokens each of ``batch`` equal requests has decoded when the last one finishes its prompt."""
    from qwen3_from_scratch_b200.cache import CacheManager
    from qwen3_from_scratch_b200.engine.request import Request, SamplingParams
    from qwen3_from_scratch_b200.engine.scheduler import Scheduler
    real = engine.session.manager
    lead = [0] * batch
    for _ in range(3):  # shortening a prompt by its lead can shift the schedule; it settles at once
        cache = CacheManager(real.layout, real.page_size, real._pools[0].num_pages if real._pools else 1, real.max_seqs)
        sched = Scheduler(engine.scheduler.config, cache)
        reqs = [Request([0] * (prompt_len - lead[i]), SamplingParams(max_new_tokens=8 * batch + 64))
                for i in range(batch)]
        for r in reqs:
            if not sched.add_request(r):
                raise RuntimeError("the benchmark's requests do not fit the cache pool")
        guard = 0
        while any(not r.is_decoding for r in reqs):
            plan = sched.schedule()
            sched.post_process(plan, [0 if s.wants_logits else None for s in plan])
            guard += 1
            if not plan or guard > 100 * batch:
                raise RuntimeError("the dry run of the schedule does not settle")
        new = [len(r.output) - 1 for r in reqs]
        if new == lead:
            break
        lead = new
    return lead


def decode_bench(engine, batch, context, steps, warmup, repeats, vocab):
    """Puts ``batch`` requests in the cache through the entry point, so short that the last timed step
    brings each to ``context`` tokens, then measures ``repeats`` times (a) K engine steps end to end and
    (b) K replays of the last step's batch on the device alone.  Returns a dict of the medians."""
    import torch

    from qwen3_from_scratch_b200.engine.request import SamplingParams

    g = torch.Generator().manual_seed(1234 + batch)
    # Requests whose prompt is done decode while later prompts are still being cut into portions, so
    # request i is `ahead[i]` tokens ahead when the last one starts decoding.  The scheduler is
    # deterministic: a dry run of the same schedule on a cache manager alone tells `ahead`, and the
    # prompts are shortened by it, so that the last timed step brings every request to `context`.
    # (The step that the last warm-up call launched ahead is collected before the clock starts: + 1.)
    total_new = warmup + 1 + repeats * steps
    ahead = schedule_lead(engine, batch, context - total_new)
    reqs = []
    for i in range(batch):
        prompt = torch.randint(0, vocab, (context - total_new - ahead[i],), generator=g).tolist()
        reqs.append(engine.add_request(prompt, params=SamplingParams(max_new_tokens=total_new + ahead[i] + 8,
                                                                      ignore_eos=True)))
    while any(not r.is_decoding for r in reqs):
        engine.step()
    # (a) end to end through SyncEngine.step: host ids in (pinned copy), sampled ids out, every step.
    # Every one of a repeat's K steps is launched and collected between its two clock readings: a step
    # launched ahead is collected before the first reading, and the K-th call launches nothing beyond itself.
    for _ in range(warmup):
        engine.step()
    e2e, h2d = [], 0
    host_ms = []
    for _ in range(repeats):
        engine.drain()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(steps):
            if i == steps - 1:
                engine.lookahead = False
            plan = engine.step()
            assert len(plan) == batch and all(s.num_tokens == 1 for s in plan)
            h2d += engine.session.last_context.h2d_bytes
        torch.cuda.synchronize()
        e2e.append(time.perf_counter() - t0)
        engine.lookahead = True
    d2h = (1 + batch) * 4 + 4  # the sampled ids behind their buffer's first word, and the status word
    # (b) the same step on the device alone: replay the last batch (same lengths, same pages)
    ctx = engine.session.last_context
    # with the default sizes every request ends at exactly `context`; with many long prompts the dry run can
    # be a token off for some, which the bytes below account for
    assert all(abs(n - context) <= 2 for n in ctx.kv_lens), f"contexts {sorted(set(ctx.kv_lens))} instead of {context}"
    cached_tokens = sum(ctx.kv_lens)
    session, sampler = engine.session, engine.sampler
    zeros = [0.0] * batch

    def one_step():
        logits = session.rerun_last()
        sampler.sample(logits, zeros, [0] * batch, [0] * batch, [0] * batch, [0] * batch)

    launches = session.launches_per_decode_step(ctx) + 1  # + the sampling kernel
    device = time_device_steps(one_step, steps, warmup, repeats)
    for r in reqs:
        engine.abort(r)
    return dict(device=statistics.median(device), e2e=statistics.median(e2e), device_all=device, e2e_all=e2e,
                launches=launches, h2d=h2d // (steps * repeats), d2h=d2h, cached=cached_tokens)


def prefill_bench(engine, tokens, steps, warmup, vocab):
    import torch

    from qwen3_from_scratch_b200.engine.batch import Entry
    g = torch.Generator().manual_seed(99)
    prompt = torch.randint(0, vocab, (tokens,), generator=g).tolist()
    session = engine.session
    session.open("prefill-bench")
    session.manager.reserve("prefill-bench", tokens)
    entries = [Entry("prefill-bench", prompt, (tokens - 1,))]
    # The step as the engine runs a full-size prompt portion: the first time kernel by kernel, from
    # the third time on as a replay of the graph recorded at the second.  Every step is timed by its
    # own pair of events and the median is reported, so that one stall of the host does not show.
    for _ in range(max(warmup, 3)):
        session.step_reserved(entries)
    torch.cuda.synchronize()
    pairs = []
    for _ in range(steps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        session.step_reserved(entries)
        end.record()
        pairs.append((start, end))
    torch.cuda.synchronize()
    session.end("prefill-bench")
    times = sorted(a.elapsed_time(b) for a, b in pairs)
    return times[len(times) // 2] / 1e3


def serving_bench(engine, vocab):
    """The load the 8B configuration is quoted on: all requests at once, prompts of random length and random
    tokens, a fixed number of new tokens each, through ``SyncEngine.batch_generate``.  Run three times: the
    first run meets every batch shape for the first time (decode shapes are recorded as CUDA graphs then, the
    mixed steps run kernel by kernel), the second records the mixed steps' shapes, the third replays every
    step.  A live load lies between the first and the third; both are reported."""
    import torch

    w = SERVING
    g = torch.Generator().manual_seed(w["seed"])
    lengths = torch.randint(w["prompt_min"], w["prompt_max"] + 1, (w["requests"],), generator=g).tolist()
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
    runs = []
    for _ in range(3):
        steps0, pre0 = engine.num_steps, engine.scheduler.num_preemptions
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        results, batch = engine.batch_generate(prompts, max_new_tokens=w["new_tokens"], ignore_eos=True)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        assert all(len(r.token_ids) == w["new_tokens"] for r in results)
        ttft = [r.metrics.ttft for r in results]
        runs.append({"output_tok_s": batch.total_tokens / wall, "total_tok_s": (batch.total_tokens + sum(lengths)) / wall,
                     "seconds": wall, "ttft_mean_ms": 1e3 * statistics.mean(ttft), "ttft_max_ms": 1e3 * max(ttft),
                     "steps": engine.num_steps - steps0, "preemptions": engine.scheduler.num_preemptions - pre0})
    out = dict(runs[2])
    out.update(requests=w["requests"], prompt_tokens=sum(lengths), new_tokens_each=w["new_tokens"],
               first_run_output_tok_s=runs[0]["output_tok_s"], first_run_ttft_mean_ms=runs[0]["ttft_mean_ms"],
               second_run_output_tok_s=runs[1]["output_tok_s"])
    return out


def make_engine(spec, layers, batches, context, folder=None):
    """The engine of one model size: pool for the largest batch at ``context`` plus a prompt's worth."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model

    cfg = dict(spec["config"], num_hidden_layers=layers)
    pool_tokens = max(max(batches) * context, SERVING["requests"] * (SERVING["prompt_max"] + SERVING["new_tokens"])
                      if spec["serving"] else 0) + PREFILL_TOKENS + 64 * PAGE
    kwargs = dict(dtype="bfloat16", block_size=PAGE, num_pages=pool_tokens // PAGE,
                  max_num_seqs=max(max(batches), SERVING["requests"] if spec["serving"] else 0), max_num_tokens=4096,
                  chunked_prefill_size=2048)
    t0 = time.time()
    if spec["weights"] == "folder":
        with tempfile.TemporaryDirectory(prefix="q3b200-bench-") as tmp:
            write_random_model(tmp, config_from_dict(cfg), seed=0)
            engine = SyncEngine(tmp, **kwargs)
    else:
        with tempfile.TemporaryDirectory(prefix="q3b200-bench-") as tmp:
            config_from_dict(cfg).save(tmp)
            engine = SyncEngine(tmp, random_weights=0, **kwargs)
    print(f"[bench] {spec['name']} sizes, {layers} layers: engine with random weights ready in {time.time() - t0:.1f}s",
          file=sys.stderr, flush=True)
    return engine, cfg


def measure_model(key, args, peaks, sample_clocks):
    """All figures of one model size as a dict (see ``line_of``)."""
    import gc

    import torch

    spec = MODELS[key]
    full_layers = spec["config"]["num_hidden_layers"]
    layers = args.layers or full_layers
    batches = list(spec["batches"])
    if args.batches and key == args.model:
        batches = [int(b) for b in args.batches.split(",")]
    if args.batch and key == args.model:
        batches = [args.batch] + [b for b in batches if b != args.batch]
    engine, cfg = make_engine(spec, layers, batches, args.context)
    weight_bytes, kv_per_token, prefill_flops = model_numbers(cfg, layers)
    vocab = cfg["vocab_size"]
    results, clocks = {}, None
    for b in sorted(batches):
        sampler = ClockSampler() if (sample_clocks and b == batches[0]) else None
        if sampler:
            sampler.start()
        r = decode_bench(engine, b, args.context, args.steps, args.warmup, args.repeats, vocab)
        if sampler:
            clocks = sampler.stop()
        step_s = r["device"] / args.steps
        r["tok_s"] = b * args.steps / r["device"]
        r["e2e_tok_s"] = b * args.steps / r["e2e"]
        r["gbs"] = (weight_bytes + r["cached"] * kv_per_token) / step_s / 1e9
        r["frac"] = r["gbs"] / peaks["hbm_gbs"]
        results[b] = r
        print(f"[bench] {spec['name']} batch {b}: {r['tok_s']:.0f} tok/s on the device ({step_s * 1e3:.3f} ms/step, "
              f"{r['frac']:.2f} of the HBM roofline), {r['e2e_tok_s']:.0f} tok/s end to end "
              f"({r['e2e_tok_s'] / r['tok_s']:.3f} of it; repeats {' '.join(f'{1e3 * t / args.steps:.3f}' for t in r['e2e_all'])} "
              f"ms/step)", file=sys.stderr, flush=True)
    prefill_s = prefill_bench(engine, PREFILL_TOKENS, max(3, min(args.steps, 10)), args.warmup, vocab)
    flops = prefill_flops(PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / prefill_s, "tokens": PREFILL_TOKENS, "ms": prefill_s * 1e3,
               "frac": flops / prefill_s / (peaks["bf16_tflops"] * 1e12)}
    print(f"[bench] {spec['name']} prompt of {PREFILL_TOKENS}: {prefill_s * 1e3:.2f} ms, {prefill['value']:.0f} tok/s, "
          f"{prefill['frac']:.2f} of the bf16 peak", file=sys.stderr, flush=True)
    # the prompt step at two further lengths (the contract's figure stays the 2,048-token one)
    more = {}
    for tokens in (512, 4096):
        t = prefill_bench(engine, tokens, max(3, min(args.steps, 10)), args.warmup, vocab)
        more[tokens] = {"tok_s": tokens / t, "frac": prefill_flops(tokens) / t / (peaks["bf16_tflops"] * 1e12)}
        print(f"[bench] {spec['name']} prompt of {tokens}: {t * 1e3:.2f} ms, {tokens / t:.0f} tok/s, "
              f"{more[tokens]['frac']:.2f} of the bf16 peak", file=sys.stderr, flush=True)
    serving = None
    if spec["serving"] and not args.no_serving:
        serving = serving_bench(engine, vocab)
        print(f"[bench] {spec['name']} serving load: {json.dumps(serving)}", file=sys.stderr, flush=True)
    del engine
    gc.collect()
    torch.cuda.empty_cache()
    return dict(key=key, spec=spec, cfg=cfg, layers=layers, full_layers=full_layers, batches=batches, results=results,
                prefill=prefill, prefill_more=more, serving=serving, clocks=clocks)


def line_of(m, args, peaks):
    """The JSON line of one model size."""
    spec, cfg, results = m["spec"], m["cfg"], m["results"]
    b0 = m["batches"][0]
    main = results[b0]
    line = {
        "metric": f"decode tok/s at batch {b0} ({spec['name']} sizes, context {args.context}, bf16, random weights)",
        "value": main["tok_s"], "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": main["device"] / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded random weights and token ids)", "impl": "ours",
        "config": {
            "model": f"{spec['name']} sizes, random weights", "global_batch": b0, "seq_len": args.context,
            "parallelism": "single GPU", "layers": m["layers"], "layers_full": m["full_layers"],
            "hidden_size": cfg["hidden_size"], "num_attention_heads": cfg["num_attention_heads"],
            "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate_size": cfg["intermediate_size"], "vocab_size": cfg["vocab_size"],
            "tie_word_embeddings": cfg["tie_word_embeddings"], "page_size": PAGE, "prefill_tokens": PREFILL_TOKENS,
            "repeats": args.repeats, "l2": "inputs larger than L2 (weights + cache)", "peaks": peaks["source"],
        },
        "e2e": {"value": main["e2e_tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": main["h2d"],
                "d2h_bytes_per_step": main["d2h"]},
        "gpu_launches": main["launches"] * args.steps,
        "prefill": m["prefill"],
        "roofline": {"bound": "hbm", "achieved": main["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": main["frac"]},
        "points": {},
        "clocks": m["clocks"],
    }
    for b in m["batches"][1:]:
        line["points"][f"decode_b{b}"] = results[b]["tok_s"]
    for b in m["batches"]:
        line["points"][f"decode_b{b}_e2e"] = results[b]["e2e_tok_s"]
        line["points"][f"decode_b{b}_hbm_frac"] = results[b]["frac"]
    for tokens, r in m["prefill_more"].items():
        line["points"][f"prefill_{tokens}_tok_s"] = r["tok_s"]
        line["points"][f"prefill_{tokens}_frac"] = r["frac"]
    if m["serving"]:
        line["serving"] = m["serving"]
    return line


def ours(args):
    peaks = load_peaks()
    m = measure_model(args.model, args, peaks, sample_clocks=True)
    line = line_of(m, args, peaks)
    # Every repeat of the end-to-end loop does the device's work of the device-timed loop and more.
    main = m["results"][m["batches"][0]]
    # (the end-to-end repeats decode one after the other, so all but the last run at contexts up to
    # repeats x K tokens shorter than the device-timed step: up to about 1 % fewer bytes)
    if main["e2e_tok_s"] > 1.03 * main["tok_s"]:
        print(f"[bench] end to end ({main['e2e_tok_s']:.0f}) above the device rate ({main['tok_s']:.0f}): "
              "the clock of one of them is wrong", file=sys.stderr)
        return 1
    if args.model == "0.6b" and not args.headline_only and not args.layers:
        # the other sizes' figures ride along under `points`; a failure there must not cost the headline
        started = time.time()
        for key in ("8b", "32b"):
            if time.time() - started > 120:
                print(f"[bench] {key} left out: the run is long already", file=sys.stderr)
                continue
            try:
                other = measure_model(key, args, peaks, sample_clocks=False)
            except Exception as e:  # noqa: BLE001
                print(f"[bench] {key} failed: {type(e).__name__}: {e}", file=sys.stderr)
                line["points"][f"{key}_error"] = f"{type(e).__name__}: {str(e)[:120]}"
                continue
            for b in other["batches"]:
                r = other["results"][b]
                line["points"][f"{key}_decode_b{b}"] = r["tok_s"]
                line["points"][f"{key}_decode_b{b}_e2e"] = r["e2e_tok_s"]
                line["points"][f"{key}_decode_b{b}_hbm_frac"] = r["frac"]
            line["points"][f"{key}_prefill_tok_s"] = other["prefill"]["value"]
            line["points"][f"{key}_prefill_frac"] = other["prefill"]["frac"]
            for tokens, r in other["prefill_more"].items():
                line["points"][f"{key}_prefill_{tokens}_tok_s"] = r["tok_s"]
                line["points"][f"{key}_prefill_{tokens}_frac"] = r["frac"]
            line["points"][f"{key}_layers"] = other["layers"]
            if other["serving"]:
                line["points"][f"{key}_serving_output_tok_s"] = other["serving"]["output_tok_s"]
                line["points"][f"{key}_serving_first_run_output_tok_s"] = other["serving"]["first_run_output_tok_s"]
                line["points"][f"{key}_serving_ttft_mean_ms"] = other["serving"]["ttft_mean_ms"]
                line["points"][f"{key}_serving_steps"] = other["serving"]["steps"]
                line["points"][f"{key}_serving_preemptions"] = other["serving"]["preemptions"]
    print(json.dumps(line))
    return 0


def profile(args):
    """A short run for a profiler: builds the model (``--layers`` keeps it small), brings ``--batch``
    requests to ``--context`` tokens, then brackets two steps with cudaProfilerStart/Stop.
    ``--profile decode``: two decode steps launched kernel by kernel; ``--profile prefill``: two
    steps over a 2,048-token prompt."""
    import torch

    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    from qwen3_from_scratch_b200.engine.request import SamplingParams
    from qwen3_from_scratch_b200.registry import config_from_dict

    cfg = dict(MODELS[args.model]["config"])
    cfg["num_hidden_layers"] = args.layers or cfg["num_hidden_layers"]
    args.batch = args.batch or 8
    with tempfile.TemporaryDirectory(prefix="q3b200-prof-") as folder:
        config_from_dict(cfg).save(folder)
        pool_tokens = args.batch * args.context + PREFILL_TOKENS + 64 * PAGE
        engine = SyncEngine(folder, dtype="bfloat16", block_size=PAGE, num_pages=pool_tokens // PAGE,
                            max_num_seqs=max(args.batch, 1), max_num_tokens=4096, chunked_prefill_size=2048,
                            cuda_graphs=False, random_weights=0)
    vocab = cfg["vocab_size"]
    if args.profile == "prefill":
        from qwen3_from_scratch_b200.engine.batch import BatchContext, Entry
        session = engine.session
        g = torch.Generator().manual_seed(99)
        tokens = args.prefill_tokens
        prompt = torch.randint(0, vocab, (tokens,), generator=g).tolist()
        session.open("p")
        session.manager.reserve("p", tokens)
        ctx = BatchContext(session.manager, session.storage, session.rt).build(
            [Entry("p", prompt, (tokens - 1,))], session.vocab_size)
        run = lambda: session.model.step(ctx)  # noqa: E731
    else:
        g = torch.Generator().manual_seed(1234)
        lead = schedule_lead(engine, args.batch, args.context - 8)
        reqs = [engine.add_request(torch.randint(0, vocab, (args.context - 8 - lead[i],), generator=g).tolist(),
                                   params=SamplingParams(max_new_tokens=lead[i] + 64, ignore_eos=True))
                for i in range(args.batch)]
        while any(not r.is_decoding for r in reqs):
            engine.step()
        for _ in range(7):
            engine.step()
        run = engine.session.rerun_last
    for _ in range(2):
        run()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    for _ in range(2):
        run()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    if args.leave_out:
        # What each kind of kernel costs inside the step as it really runs: the step is recorded as a
        # CUDA graph (warm caches, programmatic dependent launch between neighbours) once whole and once
        # with every launch of one kind left out, and the replays are timed.  A profiler that runs
        # kernels one by one with flushed caches cannot show this.  The results of such a step are wrong,
        # of course; nothing reads them.
        from qwen3_from_scratch_b200.kernels import ops
        step = (lambda: engine.session.model.step(engine.session.last_context)) if args.profile == "decode" else run

        def replay_us():
            for _ in range(2):
                step()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            for _ in range(5):
                graph.replay()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(20):
                graph.replay()
            t1.record()
            torch.cuda.synchronize()
            return t0.elapsed_time(t1) * 1e3 / 20

        layers = cfg["num_hidden_layers"]
        whole = replay_us()
        print(f"  whole step {whole:9.1f} us, {whole / layers:7.2f} per layer")
        kinds = ["paged_attention", "gemm_skinny", "gemm_skinny_normed", "gemm_skinny_into_stream", "gemm_tc",
                 "gemm_tc_qkv", "add_rmsnorm", "qkv_post", "swiglu", "rope_table", "embed"]
        nothing = {"gemm_skinny_into_stream": lambda x, w, stream, sumsq, *more: ops.sumsq_parts(w.shape[0])}
        for kind in kinds:
            real = getattr(ops, kind)
            setattr(ops, kind, nothing.get(kind, lambda *a, **k: None))
            try:
                without = replay_us()
            finally:
                setattr(ops, kind, real)
            print(f"  without {kind:16s} {without:9.1f} us: it costs {whole - without:8.1f} us, "
                  f"{(whole - without) / layers:6.2f} per layer")
        real_mm = torch.mm
        torch.mm = lambda a, b, out=None, **k: out if out is not None else torch.empty(
            a.shape[0], b.shape[1], dtype=k.get("out_dtype", a.dtype), device=a.device)
        try:
            without = replay_us()
        finally:
            torch.mm = real_mm
        print(f"  without {'library products':16s} {without:9.1f} us: they cost {whole - without:8.1f} us, "
              f"{(whole - without) / layers:6.2f} per layer")
    print(f"profiled 2 {args.profile} steps, batch {args.batch}, context {args.context}, layers {cfg['num_hidden_layers']}")
    return 0


def profile_products(args):
    """``--profile products``: the engine's tcgen05 product (single CTAs and pairs of CTAs) against the
    library's, stand-alone, on the projections of a prompt portion at four reduction lengths: the plain
    product, and gate/up with SwiGLU in the epilogue against the library's product followed by the gate
    kernel.  Each way is recorded as a CUDA graph of 10 launches; the ways are replayed in turn three
    times and the best time of each counts (under the power cap a long run of one way slows the next)."""
    import torch

    from qwen3_from_scratch_b200.kernels import ops
    dev = "cuda:0"
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    reps = 10

    def recorded(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(stream):
            fn()
            graph.capture_begin()
            for _ in range(reps):
                fn()
            graph.capture_end()
        torch.cuda.synchronize()
        return graph

    def best_us(fns):
        graphs = [recorded(fn) for fn in fns]
        best = [float("inf")] * len(fns)
        for _ in range(3):
            for i, graph in enumerate(graphs):
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                graph.replay()
                t1.record()
                torch.cuda.synchronize()
                best[i] = min(best[i], t0.elapsed_time(t1) * 1e3 / reps)
        return best

    # (reduction K, 2 x intermediate, QKV width, name): the sizes of Qwen3-0.6B, 1.7B, 8B and 32B
    sizes = [(1024, 6144, 4096, "0.6B"), (2048, 12288, 4096, "1.7B"), (4096, 24576, 6144, "8B"),
             (5120, 51200, 10240, "32B")]
    if args.only_size:  # a short run for a profiler: one size, one number of rows
        sizes = [s for s in sizes if s[3].lower() == args.only_size.lower()]
    print("us: single CTAs / pairs of CTAs / library   (TFLOP/s of the pair form)")
    for K, two_i, qkv_n, name in sizes:
        for rows in ((args.only_rows,) if args.only_rows else (512, 2048, 4096)):
            x = torch.randn(rows, K, device=dev).to(torch.bfloat16)
            for what, N, swiglu in (("qkv", qkv_n, False), ("gate/up + SwiGLU", two_i, True)):
                w = (torch.randn(N, K, device=dev) * 0.1).to(torch.bfloat16)
                out = torch.empty(rows, N // 2 if swiglu else N, device=dev, dtype=torch.bfloat16)
                full = torch.empty(rows, N, device=dev, dtype=torch.bfloat16)

                def library():
                    torch.mm(x, w.t(), out=full)
                    if swiglu:
                        ops.swiglu(full, out, interleave8=True)

                single, pair, lib = best_us([
                    lambda: ops.gemm_tc(x, w, out, status, swiglu_blocks=swiglu),
                    lambda: ops.gemm_tc(x, w, out, status, swiglu_blocks=swiglu, pair=True), library])
                print(f"  {name:5s} K {K:5d} rows {rows:5d} {what:17s} N {N:6d}: {single:8.1f} / {pair:8.1f} / {lib:8.1f}"
                      f"   ({2.0 * rows * N * K / pair / 1e6:6.0f})", flush=True)
                del w, out, full
    print(f"status word {int(status.item())}")
    return 0


def main() -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=64)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--model", default="0.6b", choices=sorted(MODELS), help="layer sizes (default: the headline's)")
    p.add_argument("--batch", type=int, default=None, help="decode batch of `value` (default 8)")
    p.add_argument("--batches", default=None,
                   help="decode batch sizes to measure, comma separated, the first one is `value` (default: the model's three)")
    p.add_argument("--context", type=int, default=CONTEXT)
    p.add_argument("--repeats", type=int, default=5, help="the K-step region is timed this often; the median counts")
    p.add_argument("--headline-only", action="store_true",
                   help="default run without the 8B and 32B figures under `points`")
    p.add_argument("--no-serving", action="store_true", help="--model 8b without the 64-request load")
    p.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in the output)")
    p.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                   help="with --profile prefill: length of the prompt (at most 4,096)")
    p.add_argument("--only-size", default=None, help="with --profile products: one of 0.6B, 1.7B, 8B, 32B")
    p.add_argument("--only-rows", type=int, default=None, help="with --profile products: one number of rows")
    p.add_argument("--leave-out", action="store_true",
                   help="with --profile: time the step as a CUDA graph, whole and with each kind of kernel left out")
    p.add_argument("--profile", choices=["decode", "prefill", "products"], default=None,
                   help="short run for a profiler instead of the benchmark (see profile())")
    args = p.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.profile == "products":
        return profile_products(args)
    if args.profile:
        return profile(args)
    if args.impl == "reference":
        from baseline.reference_arm import run_reference
        args.batch = args.batch or 8
        if args.model != "0.6b":
            from baseline.reference_arm import unavailable
            return unavailable(f"the reference arm runs the headline configuration only: the reference reads its weights "
                               f"from a folder, and a random folder of {MODELS[args.model]['name']} size is not written")
        return run_reference(args, MODELS[args.model]["config"], PAGE)
    return ours(args)


if __name__ == "__main__":
    sys.exit(main())
