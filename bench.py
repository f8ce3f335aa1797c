"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step of the whole batch.  The default run uses the layer sizes of
Qwen3-0.6B (28 layers, hidden 1024, 16/8 heads of 128, intermediate 3072, vocabulary 151936,
tied head) with seeded random weights, a batch of 8 and a context of 4096 tokens per sequence,
pages of 16 tokens.  It prints one JSON line:

  value      decoded tokens per second, timed on the device (CUDA events) over exactly K steps
  e2e        the same through the Python entry point (``SyncEngine.step``): every step copies its
             token ids and block tables from pinned host memory and reads the sampled ids back
  prefill    one step over a 2,048-token prompt: tokens/s and flops / time / bf16 peak
  roofline   bytes a decode step has to read (every weight once + the keys and values of the live
             requests) / its time, against the measured copy bandwidth
  points     decode tokens/s at batch 1 and 64

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

# the configuration the headline figure is quoted on: Qwen3-0.6B layer sizes
CONFIG = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=1024, hidden_act="silu",
    num_hidden_layers=28, max_position_embeddings=40960, num_key_value_heads=8, num_attention_heads=16,
    head_dim=128, intermediate_size=3072, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=True)
FULL_LAYERS = 28
CONTEXT = 4096
PAGE = 16
PREFILL_TOKENS = 2048
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

    def __init__(self):
        self.samples = []  # (sm MHz, max sm MHz, [active reasons])
        self.proc = None
        self.stopping = threading.Event()
        self.thread = None
        self.source = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(0)
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
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
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
                "samples": len(clocks), "source": self.source}


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


def time_device_steps(fn, steps, warmup):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / 1e3


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


def decode_bench(engine, batch, context, steps, warmup, vocab):
    """Puts ``batch`` requests of ``context - steps - warmup`` tokens in the cache through the entry
    point, then measures (a) K engine steps end to end and (b) K replays of the last step's batch
    on the device alone.  Returns (device seconds, e2e seconds, launches per step, h2d, d2h bytes)."""
    import torch

    from qwen3_from_scratch_b200.engine.request import SamplingParams
    from qwen3_from_scratch_b200.kernels import ops

    g = torch.Generator().manual_seed(1234 + batch)
    # Requests whose prompt is done decode while later prompts are still being cut into portions, so
    # request i is `ahead[i]` tokens ahead when the last one starts decoding.  The scheduler is
    # deterministic: a dry run of the same schedule on a cache manager alone tells `ahead`, and the
    # prompts are shortened by it, so that the last timed step brings every request to `context`.
    total_new = steps + warmup
    ahead = schedule_lead(engine, batch, context - total_new)
    reqs = []
    for i in range(batch):
        prompt = torch.randint(0, vocab, (context - total_new - ahead[i],), generator=g).tolist()
        reqs.append(engine.add_request(prompt, params=SamplingParams(max_new_tokens=total_new + ahead[i] + 8,
                                                                      ignore_eos=True)))
    while any(not r.is_decoding for r in reqs):
        engine.step()
    # (a) end to end through SyncEngine.step: host ids in (pinned copy), sampled ids out, every step
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    h2d = 0
    for i in range(steps):
        if i == steps - 1:
            engine.lookahead = False  # the last call launches nothing beyond the K-th step
        plan = engine.step()
        assert len(plan) == batch and all(s.num_tokens == 1 for s in plan)
        h2d += engine.session.last_context.h2d_bytes
    torch.cuda.synchronize()
    e2e_seconds = time.perf_counter() - t0
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
    device_seconds = time_device_steps(one_step, steps, warmup)
    for r in reqs:
        engine.abort(r)
    return device_seconds, e2e_seconds, launches, h2d // steps, d2h, cached_tokens


def prefill_bench(engine, tokens, steps, warmup, vocab):
    import torch

    from qwen3_from_scratch_b200.engine.batch import BatchContext, Entry
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


def ours(args):
    import torch

    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model

    peaks = load_peaks()
    cfg = dict(CONFIG)
    layers = args.layers or FULL_LAYERS
    cfg["num_hidden_layers"] = layers
    weight_bytes, kv_per_token, prefill_flops = model_numbers(cfg, layers)
    batches = sorted({args.batch, 1, 64})
    with tempfile.TemporaryDirectory(prefix="q3b200-bench-") as folder:
        t0 = time.time()
        write_random_model(folder, config_from_dict(cfg), seed=0)
        print(f"[bench] wrote random {layers}-layer model in {time.time() - t0:.1f}s", file=sys.stderr, flush=True)
        pool_tokens = max(batches) * args.context + PREFILL_TOKENS + 64 * PAGE
        engine = SyncEngine(folder, dtype="bfloat16", block_size=PAGE, num_pages=pool_tokens // PAGE,
                            max_num_seqs=max(batches), max_num_tokens=4096, chunked_prefill_size=2048)
    vocab = cfg["vocab_size"]
    results = {}
    clocks = None
    for b in batches:
        sampler = ClockSampler() if b == args.batch else None
        if sampler:
            sampler.start()
        dev_s, e2e_s, launches, h2d, d2h, cached = decode_bench(engine, b, args.context, args.steps, args.warmup, vocab)
        if sampler:
            clocks = sampler.stop()
        results[b] = dict(device=dev_s, e2e=e2e_s, launches=launches, h2d=h2d, d2h=d2h, cached=cached)
        print(f"[bench] batch {b}: {b * args.steps / dev_s:.0f} tok/s on the device, "
              f"{b * args.steps / e2e_s:.0f} tok/s end to end", file=sys.stderr, flush=True)
    prefill_s = prefill_bench(engine, PREFILL_TOKENS, max(3, min(args.steps, 10)), args.warmup, vocab)
    main = results[args.batch]
    step_s = main["device"] / args.steps
    step_bytes = weight_bytes + main["cached"] * kv_per_token
    achieved = step_bytes / step_s / 1e9
    flops = prefill_flops(PREFILL_TOKENS)
    line = {
        "metric": "decode tok/s at batch 8 (Qwen3-0.6B sizes, context 4096, bf16, random weights)",
        "value": args.batch * args.steps / main["device"], "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": "Qwen3-0.6B sizes, random weights", "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "single GPU", "layers": layers, "layers_full": FULL_LAYERS,
            "hidden_size": cfg["hidden_size"], "num_attention_heads": cfg["num_attention_heads"],
            "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate_size": cfg["intermediate_size"], "vocab_size": vocab, "tie_word_embeddings": True,
            "page_size": PAGE, "prefill_tokens": PREFILL_TOKENS, "l2": "inputs larger than L2 (weights + cache)",
            "peaks": peaks["source"],
        },
        "e2e": {"value": args.batch * args.steps / main["e2e"], "unit": "tokens/s",
                "h2d_bytes_per_step": main["h2d"], "d2h_bytes_per_step": main["d2h"]},
        "gpu_launches": main["launches"] * args.steps,
        "prefill": {"value": PREFILL_TOKENS / prefill_s, "tokens": PREFILL_TOKENS, "ms": prefill_s * 1e3,
                    "frac": flops / prefill_s / (peaks["bf16_tflops"] * 1e12)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"]},
        "points": {f"decode_b{b}": b * args.steps / results[b]["device"] for b in batches if b != args.batch},
        "clocks": clocks,
    }
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
    from qwen3_from_scratch_b200.weights import write_random_model

    cfg = dict(CONFIG)
    cfg["num_hidden_layers"] = args.layers or FULL_LAYERS
    with tempfile.TemporaryDirectory(prefix="q3b200-prof-") as folder:
        write_random_model(folder, config_from_dict(cfg), seed=0)
        pool_tokens = args.batch * args.context + PREFILL_TOKENS + 64 * PAGE
        engine = SyncEngine(folder, dtype="bfloat16", block_size=PAGE, num_pages=pool_tokens // PAGE,
                            max_num_seqs=max(args.batch, 1), max_num_tokens=4096, chunked_prefill_size=2048,
                            cuda_graphs=False)
    vocab = cfg["vocab_size"]
    if args.profile == "prefill":
        from qwen3_from_scratch_b200.engine.batch import BatchContext, Entry
        session = engine.session
        g = torch.Generator().manual_seed(99)
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=g).tolist()
        session.open("p")
        session.manager.reserve("p", PREFILL_TOKENS)
        ctx = BatchContext(session.manager, session.storage, session.rt).build(
            [Entry("p", prompt, (PREFILL_TOKENS - 1,))], session.vocab_size)
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
                 "add_rmsnorm", "qkv_post", "swiglu", "rope_table", "embed"]
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


def main() -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=64)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=CONTEXT)
    p.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in the output)")
    p.add_argument("--leave-out", action="store_true",
                   help="with --profile: time the step as a CUDA graph, whole and with each kind of kernel left out")
    p.add_argument("--profile", choices=["decode", "prefill"], default=None,
                   help="short run for a profiler instead of the benchmark (see profile())")
    args = p.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.profile:
        return profile(args)
    if args.impl == "reference":
        from baseline.reference_arm import run_reference
        return run_reference(args, CONFIG, PAGE)
    return ours(args)


if __name__ == "__main__":
    sys.exit(main())
