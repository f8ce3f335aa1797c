"""Command line of the engine.

    python -m qwen3_from_scratch_b200.cli generate --model DIR --prompt-ids 1,2,3 [options]
    python -m qwen3_from_scratch_b200.cli generate --config-path batch.yaml --model-name NAME --prompt "text"
    python -m qwen3_from_scratch_b200.cli make-random-model --config config.json --out DIR --seed 0

The reference has no generation command line (its examples are scripts with fixed prompts:
examples/sync_engine_example.py, examples/llm_runner.py; argparse only in examples/server.py with
``--config_path`` and ``--model``).  The options here carry the names of its YAML configuration:
``scheduler.{max_num_seqs, max_num_tokens, block_size, gpu_utilization, chunked_prefill_size}``,
``generation.{temperature, top_k, max_new_tokens}`` (factory/batch_config.py:83-148), and
``ignore_eos`` of its engine call (inference/llm_engine.py:34-35).
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import List


def _ids(text: str) -> List[int]:
    return [int(x) for x in text.replace(",", " ").split()]


def _add_engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", help="model folder (config.json + model.safetensors)")
    p.add_argument("--config-path", "--config_path", help="YAML file in the reference's batch layout")
    p.add_argument("--model-name", "--model_name", help="name of the model entry in --config-path")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--max-num-seqs", type=int, default=32)
    p.add_argument("--max-num-tokens", type=int, default=3000)
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    p.add_argument("--gpu-utilization", type=float, default=0.5,
                   help="share of the free GPU memory given to the cache")
    p.add_argument("--num-pages", type=int, default=None, help="size of the cache pool in pages (overrides --gpu-utilization)")
    p.add_argument("--chunked-prefill-size", type=int, default=512)
    p.add_argument("--temperature", type=float, default=0.0, help="<= 0: greedy")
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--max-new-tokens", type=int, default=100)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--random-weights", action="store_true",
                   help="--model needs only config.json: weights are drawn on the device from --seed")
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--eos-token-id", type=int, default=None)
    p.add_argument("--log-interval", type=int, default=0)


def _engine(args):
    from .engine.engine import SyncEngine
    if args.config_path:
        if not args.model_name:
            raise SystemExit("--config-path needs --model-name")
        return SyncEngine.from_config(args.config_path, args.model_name, log_interval=args.log_interval)
    if not args.model:
        raise SystemExit("give --model DIR or --config-path FILE --model-name NAME")
    return SyncEngine(args.model, dtype=args.dtype, device=args.device, max_num_seqs=args.max_num_seqs,
                      max_num_tokens=args.max_num_tokens, block_size=args.block_size,
                      gpu_utilization=args.gpu_utilization, num_pages=args.num_pages,
                      chunked_prefill_size=args.chunked_prefill_size, temperature=args.temperature,
                      top_k=args.top_k, max_new_tokens=args.max_new_tokens, seed=args.seed,
                      eos_token_id=args.eos_token_id, log_interval=args.log_interval,
                      random_weights=args.seed if args.random_weights else None)


def cmd_generate(args) -> int:
    prompts = []
    for text in args.prompt_ids or []:
        prompts.append(_ids(text))
    if args.prompt_ids_file:
        with open(args.prompt_ids_file) as f:
            for line in f:
                if line.strip():
                    prompts.append(_ids(line))
    for text in args.prompt or []:
        prompts.append(text)
    if not prompts:
        raise SystemExit("no prompt: give --prompt-ids, --prompt-ids-file or --prompt")
    engine = _engine(args)
    if args.stream and len(prompts) == 1:
        ids = []
        for chunk in engine.generate_stream(prompts[0], args.max_new_tokens, ignore_eos=args.ignore_eos):
            ids.append(chunk.token_id)
            sys.stdout.write(chunk.delta if chunk.delta else f"{chunk.token_id} ")
            sys.stdout.flush()
        m = chunk.metrics
        print(f"\nTTFT: {m.ttft:.4f}s | tokens: {m.token_count} | TPS: {m.tps:.2f} | total: {m.total_elapsed:.4f}s")
        return 0
    results, batch = engine.batch_generate(prompts, args.max_new_tokens, ignore_eos=args.ignore_eos)
    for i, r in enumerate(results):
        print(json.dumps({"index": i, "token_ids": r.token_ids, "text": r.text, "finish_reason": r.finish_reason,
                          "ttft": round(r.metrics.ttft, 6), "tps": round(r.metrics.tps, 3)}))
    print(f"requests: {batch.num_requests} | total tokens: {batch.total_tokens} | "
          f"elapsed: {batch.total_elapsed:.4f}s | throughput: {batch.aggregate_tps:.2f} tokens/s", file=sys.stderr)
    return 0


def cmd_make_random_model(args) -> int:
    from .registry import load_config
    from .weights import write_random_model
    config = load_config(args.config)
    write_random_model(args.out, config, args.seed, dtype=args.store_dtype)
    print(args.out)
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="qwen3_from_scratch_b200", description=__doc__.split("\n\n")[0])
    sub = parser.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate tokens for one or more prompts")
    _add_engine_options(g)
    g.add_argument("--prompt-ids", action="append", help="token ids, comma or space separated (repeatable)")
    g.add_argument("--prompt-ids-file", help="one prompt of token ids per line")
    g.add_argument("--prompt", action="append", help="text (needs tokenizer.json in the model folder; repeatable)")
    g.add_argument("--stream", action="store_true", help="print tokens as they come (one prompt)")
    g.set_defaults(fn=cmd_generate)
    r = sub.add_parser("make-random-model", help="write a model folder with seeded random weights")
    r.add_argument("--config", required=True, help="config.json (or a folder that has one)")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.set_defaults(fn=cmd_make_random_model)
    args = parser.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
