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
import itertools
import json
import math
import random
import statistics
import sys
import time
from dataclasses import asdict, dataclass


@dataclass
class Conversation:
    """One chat: the user's messages as token ids, and how many tokens each reply has."""

    id: str
    user_ids: list[list[int]]
    reply_lens: list[int]

    @property
    def num_turns(self) -> int:
        return len(self.reply_lens)

    def lengths_after_turns(self) -> list[int]:
        """Tokens in the conversation after each turn's reply."""
        return list(itertools.accumulate(len(u) + r for u, r in zip(self.user_ids, self.reply_lens)))


def synthetic_trace(n: int, vocab: int, max_model_len: int, seed: int, turns: tuple[int, int],
                    user_tokens: tuple[int, int], reply_tokens: tuple[int, int]) -> list[Conversation]:
    """n conversations of seeded random token ids; a conversation is cut at the last turn that still fits."""
    rng = random.Random(seed)
    trace = []
    for c in range(n):
        messages, replies, total = [], [], 0
        for _ in range(rng.randint(*turns)):
            user, reply = rng.randint(*user_tokens), rng.randint(*reply_tokens)
            if total + user + reply > max_model_len:
                break
            messages.append([rng.randrange(vocab) for _ in range(user)])
            replies.append(reply)
            total += user + reply
        if replies:
            trace.append(Conversation(f"synthetic-{c}", messages, replies))
    return trace


def load_trace(path: str) -> tuple[dict, list[Conversation]]:
    """
    A trace file in tinyserve-llm's layout (benchmarks/multiturn.py:144-155):
    {"meta": {...}, "conversations": [{"id": ..., "turns": [{"user_ids": [...], "reply_len": n}, ...]}, ...]}.
    """
    with open(path) as f:
        raw = json.load(f)
    trace = []
    for item in raw["conversations"]:
        turns = item["turns"]
        trace.append(Conversation(item["id"], [list(t["user_ids"]) for t in turns], [int(t["reply_len"]) for t in turns]))
    return raw.get("meta", {}), trace


def tokens_held_between_waves(trace: list[Conversation]) -> list[int]:
    """
    Entry k - 1: the tokens of all histories that are needed again after wave k, i.e. of the
    conversations that have a turn k + 1.  One pass over the trace: each conversation adds its
    length after every turn but its last.
    """
    held = [0] * max(0, max((c.num_turns for c in trace), default=0) - 1)
    for conversation in trace:
        for k, tokens in enumerate(conversation.lengths_after_turns()[:-1]):
            held[k] += tokens
    return held


def peak_demand(trace: list[Conversation]) -> tuple[int, int]:
    """
    (tokens, wave): the most tokens the histories still needed hold between two waves, and after
    which wave (0, 0 if no conversation has a second turn).  A cache of that many tokens serves
    every next turn from its history; capacity over this is the pressure rho tinyserve-llm quotes
    (benchmarks/multiturn.py:158-170).
    """
    held = tokens_held_between_waves(trace)
    if not held:
        return 0, 0
    wave = max(range(len(held)), key=lambda k: (held[k], -k))
    return held[wave], wave + 1


def pool_pages(demand_tokens: int, rho: float, scheduler_config, block_size: int) -> int:
    """
    Pages for a target pressure, but never fewer than the scheduler wants before it takes a
    request of `max_model_len` tokens at all (its own pages, one for the source of a copied page,
    the watermark) and one to spare.
    """
    longest = -(-scheduler_config.max_model_len // block_size)
    pages = longest + 2
    while longest + 1 + math.ceil(scheduler_config.watermark * pages) > pages:
        pages += 1
    return max(math.ceil(demand_tokens / rho / block_size), pages + 1)


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
    demand, demand_wave = peak_demand(trace)
    scheduler_config = SchedulerConfig(max_model_len=max_model_len, max_num_seqs=args.max_num_seqs,
                                       max_num_batched_tokens=args.max_num_batched_tokens)
    num_blocks = None if args.rho == "full" else pool_pages(max(demand, 1), float(args.rho), scheduler_config, args.block_size)

    cache_config = CacheConfig(block_size=args.block_size, caching=args.caching == "on", device=args.device)
    llm = LLM(args.model, scheduler_config, cache_config, dtype=args.dtype, num_blocks=num_blocks,
              gpu_memory_utilization=args.gpu_memory_utilization, seed=args.seed, random_weights_seed=args.random_weights)
    capacity = llm.cache.num_pages * args.block_size
    print(f"{len(trace)} conversations, peak demand {demand:,} tokens after wave {demand_wave}; cache {llm.cache.num_pages} "
          f"pages = {capacity:,} tokens, rho {demand / capacity:.2f}", flush=True)

    # kernels are built and graphs captured before anything is timed
    llm.generate([[7] * min(17, max_model_len - 4)], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))

    history: list[list[int]] = [[] for _ in trace]
    waves = max(c.num_turns for c in trace)
    records = []
    started = time.time()
    for k in range(waves if args.max_waves is None else min(waves, args.max_waves)):
        live = [i for i, c in enumerate(trace) if c.num_turns > k]
        prompts = [history[i] + trace[i].user_ids[k] for i in live]
        lengths = [trace[i].reply_lens[k] for i in live]
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
        "steps": {"all": llm.runner.steps, "from_graphs": llm.runner.graph_replays, "graphs_captured": llm.runner.graph_captures,
                  "tokens_launched_kernel_by_kernel": llm.runner.eager_tokens},
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
