"""
Trace replay: feeds given token ids through a model step by step and writes the logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
                  [--page-tokens 64] [--caching off|on]

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, OUT/<step>.f32 receives the logits at the wanted places
(order of the entries, then of `want`) as little-endian float32 [wanted, vocab].  After every step a
line `done <step>` is printed and flushed.  Nothing is sampled.  The program owns no model code: it
drives the engine's model, step function, cache manager and kernels, with a page pool sized for
--max-tokens, so pages are used again.

A step may also carry `"fork": [{"from": "a", "to": "b"}]`: before the step's entries run, request
`b` starts as a copy of `a` (which is between steps) sharing all its pages, as parallel sampling
does; the first token either of them feeds into a shared, partly filled page copies that page.

`--caching on` keeps the pages of ended requests indexed by their tokens.  A request's first entry
then takes its leading tokens from the cache where it can, token by token, but never a token at or
past its first wanted place, so every wanted row is still computed by this step; the entry runs
only the tokens after the reused ones.  (With `--caching off`, the default, every given token is
run.)  At the end of input the cache manager's counters (evictions, copies on write, partial-page
copies, publishes, dedupes), the number of reused tokens and how often each kernel launcher was
called are written to OUT/stats.json.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--out", required=True, help="folder the logits files go to")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time, each rounded up to a multiple of the page size")
    parser.add_argument("--page-tokens", type=int, default=64, help="tokens per cache page (default 64)")
    parser.add_argument("--caching", choices=["on", "off"], default="off",
                        help="on: ended requests' pages stay indexed and new requests reuse them")
    args = parser.parse_args(argv)
    if args.page_tokens <= 0:
        parser.error("--page-tokens must be positive")

    import torch

    from tinyserve_llm_b200.engine.loading import build_cache, load_model
    from tinyserve_llm_b200.engine.step import StepEntry, StepRunner

    os.makedirs(args.out, exist_ok=True)
    model = load_model(args.model, args.dtype, "cuda")
    num_pages = max(1, -(-args.max_tokens // args.page_tokens))
    _, manager, storage = build_cache(model, args.page_tokens, num_pages, caching=args.caching == "on",
                                      num_state_slots=8)
    runner = StepRunner(model, manager, storage)
    reused_tokens = 0

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        for fork in record.get("fork", []):
            if not manager.can_fork():
                raise RuntimeError(f"step {step}: no state slot free to fork {fork['from']!r}")
            manager.fork(fork["from"], fork["to"])
        entries = []
        for item in record.get("entries", []):
            seq_id, tokens, want = item["id"], item["tokens"], list(item.get("want", []))
            if not tokens:
                continue
            if seq_id in manager.seqs:
                if not manager.can_extend(seq_id, len(tokens)):
                    raise RuntimeError(f"step {step}: request {seq_id!r} needs pages beyond --max-tokens {args.max_tokens}")
                manager.extend(seq_id, tokens)
            else:
                if not manager.admit(seq_id, tokens, reuse_limit=min(want, default=len(tokens) - 1)):
                    raise RuntimeError(f"step {step}: request {seq_id!r} does not fit in --max-tokens {args.max_tokens}")
                skipped = manager.committed_tokens(seq_id)          # leading tokens found in the cache: not run
                reused_tokens += skipped
                tokens, want = tokens[skipped:], [w - skipped for w in want]
            entries.append(StepEntry(seq_id, tokens, want))
        if entries:
            logits = runner.step(entries)
            for e in entries:
                manager.commit(e.seq_id, len(e.tokens))
            if logits.shape[0]:
                data = logits.to("cpu", torch.float32).contiguous().numpy()
                data.astype("<f4", copy=False).tofile(os.path.join(args.out, f"{step}.f32"))
        for seq_id in record.get("end", []):
            if seq_id in manager.seqs:
                manager.release(seq_id)
        print(f"done {step}", flush=True)
    with open(os.path.join(args.out, "stats.json"), "w") as f:
        json.dump(dict(dataclasses.asdict(manager.stats()), reused_tokens=reused_tokens,
                       kernel_calls=dict(model.rt.ops.calls), graph_replays=runner.graph_replays), f)
    return 0


if __name__ == "__main__":
    sys.exit(main())
