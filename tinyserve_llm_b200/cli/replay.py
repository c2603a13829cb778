"""
Trace replay: feeds given token ids through a model step by step and writes the logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, OUT/<step>.f32 receives the logits at the wanted places
(order of the entries, then of `want`) as little-endian float32 [wanted, vocab].  After every step a
line `done <step>` is printed and flushed.  Nothing is sampled.  The program owns no model code: it
drives the engine's model, step function, cache manager and kernels, with prefix reuse off (every
given token is run) and a page pool sized for --max-tokens, so pages are used again.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

PAGE_TOKENS = 64


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--out", required=True, help="folder the logits files go to")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    args = parser.parse_args(argv)

    import torch

    from tinyserve_llm_b200.engine.loading import build_cache, load_model
    from tinyserve_llm_b200.engine.step import StepEntry, StepRunner

    os.makedirs(args.out, exist_ok=True)
    model = load_model(args.model, args.dtype, "cuda")
    num_pages = max(1, -(-args.max_tokens // PAGE_TOKENS))
    _, manager, storage = build_cache(model, PAGE_TOKENS, num_pages, caching=False, num_state_slots=8)
    runner = StepRunner(model, manager, storage)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            seq_id, tokens = item["id"], item["tokens"]
            if not tokens:
                continue
            if seq_id in manager.seqs:
                if not manager.can_extend(seq_id, len(tokens)):
                    raise RuntimeError(f"step {step}: request {seq_id!r} needs pages beyond --max-tokens {args.max_tokens}")
                manager.extend(seq_id, tokens)
            elif not manager.admit(seq_id, tokens):
                raise RuntimeError(f"step {step}: request {seq_id!r} does not fit in --max-tokens {args.max_tokens}")
            entries.append(StepEntry(seq_id, tokens, item.get("want", [])))
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
    return 0


if __name__ == "__main__":
    sys.exit(main())
