"""
Command line of the engine, in the manner of tinyserve-llm's runners (benchmarks/run_ours.py:59-72:
argparse, progress lines on standard output, one JSON record written to --out).

    python -m tinyserve_llm_b200.cli.generate --model DIR --prompt-ids 1,2,3 --prompt-ids 4,5 \
        --max-tokens 16 --temperature 0 --out result.json

Prompts are token ids (--prompt-ids, repeatable; or --prompt-file with one comma- or space-separated
list per line) or text (--prompt, needs tokenizer files in the model folder).  Options shared with
tinyserve-llm keep its names and meanings: --model, --temperature, --seed, --gpu-memory-utilization,
--device, --caching on|off, --out.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from dataclasses import asdict


def _ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="tinyserve_llm_b200.cli.generate", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model*.safetensors")
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="draw the weights from this seed instead of reading them (the folder needs only config.json)")
    p.add_argument("--prompt-ids", action="append", default=[], help="a prompt as token ids, e.g. 1,2,3 (repeatable)")
    p.add_argument("--prompt-file", help="file with one prompt of token ids per line")
    p.add_argument("--prompt", action="append", default=[], help="a text prompt (needs a tokenizer; repeatable)")
    p.add_argument("--max-tokens", type=int, default=256)
    p.add_argument("--temperature", type=float, default=0.6)
    p.add_argument("--n", type=int, default=1, help="parallel samples per prompt")
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--block-size", type=int, default=256, help="tokens per cache page")
    p.add_argument("--num-blocks", type=int, default=None, help="cache pages; default: sized from free memory")
    p.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    p.add_argument("--max-model-len", type=int, default=4096)
    p.add_argument("--max-num-seqs", type=int, default=512)
    p.add_argument("--max-num-batched-tokens", type=int, default=16384)
    p.add_argument("--chunk", type=int, default=2048, help="most prompt tokens of one request per step; 0: no limit")
    p.add_argument("--caching", choices=["on", "off"], default="on")
    p.add_argument("--device", default="cuda")
    p.add_argument("--out", help="write one JSON record here")
    return p


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    prompts: list = [_ids(t) for t in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    prompts += args.prompt
    if not prompts:
        print("no prompt given: use --prompt-ids, --prompt-file or --prompt", file=sys.stderr)
        return 2

    from tinyserve_llm_b200 import LLM, CacheConfig, SamplingParams, SchedulerConfig
    from tinyserve_llm_b200.config import read_config_json

    max_pos = read_config_json(args.model).get("max_position_embeddings", args.max_model_len)
    scheduler_config = SchedulerConfig(
        max_model_len=min(args.max_model_len, max_pos), max_num_seqs=args.max_num_seqs,
        max_num_batched_tokens=args.max_num_batched_tokens, prefill_chunk=args.chunk)
    cache_config = CacheConfig(block_size=args.block_size, caching=args.caching == "on", device=args.device)
    started = time.time()
    llm = LLM(args.model, scheduler_config, cache_config, dtype=args.dtype, num_blocks=args.num_blocks,
              gpu_memory_utilization=args.gpu_memory_utilization, seed=args.seed,
              random_weights_seed=args.random_weights)
    print(f"model {args.model} ({args.dtype}); cache {llm.cache.num_pages} pages of {args.block_size} tokens; "
          f"{len(prompts)} prompts", flush=True)
    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, n=args.n,
                            ignore_eos=args.ignore_eos)
    t0 = time.perf_counter()
    completions = llm.generate(prompts, params)
    seconds = time.perf_counter() - t0
    produced = sum(len(t) for c in completions for t in c.token_ids)
    for c in completions:
        for i, tokens in enumerate(c.token_ids):
            shown = c.texts[i] if c.texts else " ".join(map(str, tokens))
            print(f"request {c.request_id} sample {i} [{c.finish_reasons[i]}]: {shown}", flush=True)
    print(f"{produced} tokens in {seconds:.3f} s ({produced / seconds:,.0f} output tok/s), {len(llm.steps)} steps",
          flush=True)
    if args.out:
        record = {
            "engine": "tinyserve_llm_b200",
            "model": args.model,
            "dtype": args.dtype,
            "caching": args.caching,
            "temperature": args.temperature,
            "seed": args.seed,
            "num_blocks": llm.cache.num_pages,
            "block_size": args.block_size,
            "started": started,
            "seconds": seconds,
            "output_tokens": produced,
            "output_tokens_per_second": produced / seconds,
            "steps": len(llm.steps),
            "scheduler_stats": asdict(llm.scheduler.stats()),
            "cache_stats": asdict(llm.cache.stats()),
            "completions": [{"request_id": c.request_id, "prompt_token_ids": c.prompt_token_ids,
                             "token_ids": c.token_ids, "texts": c.texts, "finish_reasons": c.finish_reasons}
                            for c in completions],
        }
        with open(args.out, "w") as f:
            json.dump(record, f)
        print(f"wrote {args.out}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
