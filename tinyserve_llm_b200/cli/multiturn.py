"""
Multi-turn chat replay under cache pressure: the workload tinyserve-llm measures its cache policy with
(benchmarks/multiturn.py:1-17, benchmarks/run_ours.py:59-72), here with seeded synthetic conversations
(no dataset, no tokenizer) or a trace file in tinyserve-llm's JSON layout.

    python -m tinyserve_llm_b200.cli.multiturn --model DIR --conversations 64 --rho 1 --out result.json

Each turn's prompt is the conversation so far as token ids: the previous prompt, the engine's own reply,
then the next user message.  Every reply is generated with ignore_eos to the length the trace gives, so a
turn's prompt has the same length whatever the engine answered.  Turns run in waves: wave k sends turn k
of every conversation that has one, in one generate() call; between waves nothing runs, so how much of
each history is still in the cache at its next turn is what the cache policy decides.  --rho sets the
cache's capacity to (peak demand / rho) tokens, where peak demand is the most tokens the live histories
hold between two waves (benchmarks/multiturn.py:158-181); "full" sizes the cache from free memory.

Options shared with tinyserve-llm's runner keep its names and meanings: --model, --trace, --conversations,
--rho, --caching on|off, --max-waves, --temperature, --seed, --gpu-memory-utilization, --device, --out.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import math
import random
import statistics
import sys
import time
from dataclasses import asdict, dataclass


@dataclass
class Turn:
    user_ids: list[int]      # fed before this turn's reply: the first prompt, or the next user message
    reply_len: int           # tokens to generate


@dataclass
class Conversation:
    id: str
    turns: list[Turn]

    def history_len(self, k: int) -> int:
        """Tokens in the conversation after turn k's reply (k counts from 1)."""
        return sum(len(t.user_ids) + t.reply_len for t in self.turns[:k])


def synthetic_trace(n: int, vocab: int, max_model_len: int, seed: int, turns: tuple[int, int],
                    user_tokens: tuple[int, int], reply_tokens: tuple[int, int]) -> list[Conversation]:
    """n conversations of seeded random token ids; a conversation is cut at the last turn that still fits."""
    rng = random.Random(seed)
    trace = []
    for c in range(n):
        made, total = [], 0
        for _ in range(rng.randint(*turns)):
            user, reply = rng.randint(*user_tokens), rng.randint(*reply_tokens)
            if total + user + reply > max_model_len:
                break
            made.append(Turn([rng.randrange(vocab) for _ in range(user)], reply))
            total += user + reply
        if made:
            trace.append(Conversation(f"synthetic-{c}", made))
    return trace


def load_trace(path: str) -> tuple[dict, list[Conversation]]:
    """{"meta": {...}, "conversations": [{"id", "turns": [{"user_ids", "reply_len"}]}]} (benchmarks/multiturn.py:150-155)."""
    with open(path) as f:
        raw = json.load(f)
    return raw.get("meta", {}), [Conversation(c["id"], [Turn(t["user_ids"], t["reply_len"]) for t in c["turns"]])
                                 for c in raw["conversations"]]


def peak_demand(trace: list[Conversation]) -> tuple[int, int]:
    """(tokens, wave): after which wave the histories that still have a next turn hold the most tokens."""
    best, best_k = 0, 0
    for k in range(1, max(len(c.turns) for c in trace)):
        tokens = sum(c.history_len(k) for c in trace if len(c.turns) > k)
        if tokens > best:
            best, best_k = tokens, k
    return best, best_k


def blocks_for(demand_tokens: int, rho: float, max_model_len: int, block_size: int) -> int:
    """Pages for a target pressure, never fewer than one request of full length plus the scheduler's three spare pages."""
    return max(math.ceil(demand_tokens / rho / block_size), math.ceil(max_model_len / block_size) + 3)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="tinyserve_llm_b200.cli.multiturn", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model*.safetensors")
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="draw the weights from this seed instead of reading them (the folder needs only config.json)")
    p.add_argument("--trace", help="a trace file in tinyserve-llm's layout; default: synthetic conversations")
    p.add_argument("--conversations", type=int, required=True, help="the first n of the trace, or how many to make up")
    p.add_argument("--turns", default="2,5", help="synthetic: turns per conversation, lo,hi")
    p.add_argument("--user-tokens", default="50,600", help="synthetic: tokens per user message, lo,hi")
    p.add_argument("--reply-tokens", default="20,200", help="synthetic: tokens per reply, lo,hi")
    p.add_argument("--rho", default="full", help="target memory pressure (peak demand / capacity), or 'full' for all free memory")
    p.add_argument("--caching", choices=["on", "off"], default="on")
    p.add_argument("--max-waves", type=int, default=None, help="stop early")
    p.add_argument("--temperature", type=float, default=0.6)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--block-size", type=int, default=256, help="tokens per cache page")
    p.add_argument("--max-model-len", type=int, default=4096)
    p.add_argument("--max-num-seqs", type=int, default=512)
    p.add_argument("--max-num-batched-tokens", type=int, default=16384)
    p.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    p.add_argument("--device", default="cuda")
    p.add_argument("--out", help="write one JSON record here")
    return p


def _pair(text: str) -> tuple[int, int]:
    lo, hi = (int(t) for t in text.split(","))
    return lo, hi


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    from tinyserve_llm_b200 import LLM, CacheConfig, SamplingParams, SchedulerConfig
    from tinyserve_llm_b200.config import read_config_json

    raw = read_config_json(args.model)
    max_model_len = min(args.max_model_len, raw.get("max_position_embeddings", args.max_model_len))
    if args.trace:
        meta, trace = load_trace(args.trace)
        max_model_len = min(max_model_len, meta.get("max_model_len", max_model_len))
        trace = trace[:args.conversations]
    else:
        meta = {"synthetic": True, "turns": args.turns, "user_tokens": args.user_tokens, "reply_tokens": args.reply_tokens}
        trace = synthetic_trace(args.conversations, raw["vocab_size"], max_model_len, args.seed, _pair(args.turns),
                                _pair(args.user_tokens), _pair(args.reply_tokens))
    if not trace:
        print("the trace holds no conversation that fits max_model_len", file=sys.stderr)
        return 2
    demand, demand_wave = peak_demand(trace) if max(len(c.turns) for c in trace) > 1 else (0, 0)
    num_blocks = None if args.rho == "full" else blocks_for(max(demand, 1), float(args.rho), max_model_len, args.block_size)

    scheduler_config = SchedulerConfig(max_model_len=max_model_len, max_num_seqs=args.max_num_seqs,
                                       max_num_batched_tokens=args.max_num_batched_tokens)
    cache_config = CacheConfig(block_size=args.block_size, caching=args.caching == "on", device=args.device)
    llm = LLM(args.model, scheduler_config, cache_config, dtype=args.dtype, num_blocks=num_blocks,
              gpu_memory_utilization=args.gpu_memory_utilization, seed=args.seed, random_weights_seed=args.random_weights)
    capacity = llm.cache.num_pages * args.block_size
    print(f"{len(trace)} conversations, peak demand {demand:,} tokens after wave {demand_wave}; cache {llm.cache.num_pages} "
          f"pages = {capacity:,} tokens, rho {demand / capacity:.2f}", flush=True)

    # kernels are built and graphs captured before anything is timed
    llm.generate([[7] * min(17, max_model_len - 4)], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))

    history: list[list[int]] = [[] for _ in trace]
    waves = max(len(c.turns) for c in trace)
    records = []
    started = time.time()
    for k in range(waves if args.max_waves is None else min(waves, args.max_waves)):
        live = [i for i, c in enumerate(trace) if len(c.turns) > k]
        prompts = [history[i] + trace[i].turns[k].user_ids for i in live]
        lengths = [trace[i].turns[k].reply_len for i in live]
        before = llm.scheduler.stats()
        begin = time.perf_counter()
        done = llm.generate(prompts, [SamplingParams(max_tokens=n, temperature=args.temperature, ignore_eos=True)
                                      for n in lengths])
        seconds = time.perf_counter() - begin
        after = llm.scheduler.stats()
        for i, prompt, c, n in zip(live, prompts, done, lengths, strict=True):
            assert len(c.token_ids[0]) == n, f"conversation {trace[i].id} turn {k + 1}: asked for {n} tokens, got {len(c.token_ids[0])}"
            history[i] = prompt + c.token_ids[0]
        record = {
            "wave": k + 1, "num_prompts": len(live), "prompt_tokens": sum(map(len, prompts)), "output_tokens": sum(lengths),
            "prefill_tokens": after.prefill_tokens - before.prefill_tokens,      # includes recomputation after preemption
            "preemptions": after.preemptions - before.preemptions, "seconds": seconds,
            "median_first_token_seconds": statistics.median(c.first_token_time - c.arrival_time for c in done),
        }
        records.append(record)
        print(f"wave {record['wave']:>3}: {record['num_prompts']:>4} prompts, {record['prompt_tokens']:>9,} prompt tokens, "
              f"{record['prefill_tokens']:>9,} prefilled, {record['preemptions']:>4} preempted, {seconds:7.2f} s", flush=True)

    prompt_tokens = sum(r["prompt_tokens"] for r in records)
    prefill_tokens = sum(r["prefill_tokens"] for r in records)
    output_tokens = sum(r["output_tokens"] for r in records)
    seconds = sum(r["seconds"] for r in records)
    summary = {
        "prompt_tokens": prompt_tokens, "prefill_tokens": prefill_tokens, "prefill_fraction": prefill_tokens / prompt_tokens,
        "cached_tokens": prompt_tokens - prefill_tokens, "output_tokens": output_tokens, "seconds": seconds,
        "output_tokens_per_second": output_tokens / seconds, "preemptions": sum(r["preemptions"] for r in records),
        "median_first_token_seconds_by_wave": [r["median_first_token_seconds"] for r in records],
    }
    result = {
        "engine": "tinyserve_llm_b200", "model": args.model, "trace": args.trace, "trace_meta": meta,
        "conversations": len(trace), "max_waves": args.max_waves, "caching": args.caching, "rho_requested": args.rho,
        "num_blocks": llm.cache.num_pages, "capacity_tokens": capacity, "peak_demand_tokens": demand,
        "rho": demand / capacity, "temperature": args.temperature, "seed": args.seed, "max_num_seqs": args.max_num_seqs,
        "max_num_batched_tokens": args.max_num_batched_tokens, "dtype": args.dtype, "started": started,
        "summary": summary, "cache_stats": asdict(llm.cache.stats()), "scheduler_stats": asdict(llm.scheduler.stats()),
        "waves": records, "final_histories": [len(h) for h in history],
        "final_history_digests": [hashlib.sha256(repr(h).encode()).hexdigest()[:16] for h in history],
    }
    print(f"{output_tokens:,} tokens out in {seconds:.2f} s ({summary['output_tokens_per_second']:,.0f} tok/s); "
          f"{prefill_tokens:,} of {prompt_tokens:,} prompt tokens prefilled ({100 * summary['prefill_fraction']:.1f} %)", flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(result, f)
    else:
        print(json.dumps({k: v for k, v in result.items() if k not in ("waves", "final_histories", "final_history_digests")}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
