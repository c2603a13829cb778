"""Builds replay traces, runs bin/trace_run on them and compares the logits with the plain implementation."""

from __future__ import annotations

import json
import os
import random
import subprocess
import sys

import numpy as np
import torch

import plain_llama as plain

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def random_ids(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def round64(n: int) -> int:
    return -(-n // 64) * 64


class Trace:
    """Steps for trace_run plus, for every step, which (request, position) each wanted row is."""

    def __init__(self) -> None:
        self.steps: list[dict] = []
        self.expect: dict[int, list[tuple[str, int]]] = {}
        self.fed: dict[str, int] = {}            # tokens fed so far per live request
        self.peak = 0                            # most tokens held at once, each request rounded up to 64

    def step(self, parts: list[tuple[str, list[int], list[int]]], end: list[str] = ()) -> None:
        """parts: (request, its next tokens, wanted places among them)."""
        number = len(self.steps)
        entries, rows = [], []
        for name, tokens, want in parts:
            start = self.fed.get(name, 0)
            entries.append({"id": name, "tokens": list(tokens), "want": list(want)})
            rows.extend((name, start + w) for w in want)
            self.fed[name] = start + len(tokens)
        self.peak = max(self.peak, sum(round64(n) for n in self.fed.values()))
        for name in end:
            self.fed.pop(name, None)
        self.steps.append({"step": number, "entries": entries, "end": list(end)})
        if rows:
            self.expect[number] = rows


def add_whole(trace: Trace, name: str, ids: list[int]) -> None:
    trace.step([(name, ids, list(range(len(ids))))], end=[name])


def add_decode_tail(trace: Trace, name: str, ids: list[int], tail: int = 32) -> None:
    head = max(1, len(ids) - tail)
    trace.step([(name, ids[:head], [head - 1])])
    for i in range(head, len(ids)):
        trace.step([(name, ids[i:i + 1], [0])], end=[name] if i == len(ids) - 1 else [])
    if head == len(ids):
        trace.step([], end=[name])


def add_portions(trace: Trace, name: str, ids: list[int], sizes: list[int]) -> None:
    pos, k = 0, 0
    while pos < len(ids):
        n = min(sizes[k % len(sizes)], len(ids) - pos)
        k += 1
        last = pos + n == len(ids)
        trace.step([(name, ids[pos:pos + n], list(range(n)))], end=[name] if last else [])
        pos += n


def add_mixed(trace: Trace, requests: dict[str, list[int]], seed: int, live_limit: int = 4) -> None:
    """
    Up to `live_limit` requests at a time; each step a random subset of them goes on: with portions
    of changing size while most of its tokens are ahead, then token by token; the rest sit the step
    out.  A finished request ends and the next one starts, so its pages are handed on.
    """
    rng = random.Random(seed)
    waiting = list(requests)
    live: dict[str, int] = {}
    while waiting or live:
        while waiting and len(live) < live_limit:
            live[waiting.pop(0)] = 0
        chosen = [n for n in live if rng.random() < 0.7] or [rng.choice(list(live))]
        parts, ended = [], []
        for name in chosen:
            ids, pos = requests[name], live[name]
            left = len(ids) - pos
            if left > 24:
                n = min(left - 20, rng.choice([2, 3, 5, 17, 31, 64, 100]))
            else:
                n = 1
            want = sorted({0, n - 1} | {rng.randrange(n)})
            parts.append((name, ids[pos:pos + n], want))
            live[name] = pos + n
            if live[name] == len(ids):
                ended.append(name)
        trace.step(parts, end=ended)
        for name in ended:
            del live[name]


def run_trace(model_dir: str, dtype: str, trace: Trace, out_dir: str, max_tokens: int | None = None,
              timeout: float = 900.0) -> dict[int, np.ndarray]:
    """Runs bin/trace_run as a child process, feeding the next step only after `done <step>`."""
    os.makedirs(out_dir, exist_ok=True)
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir, "--max-tokens",
           str(max_tokens if max_tokens is not None else trace.peak)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        for step in trace.steps:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            if line.strip() != f"done {step['step']}":
                proc.stdin.close()
                err = proc.stderr.read()
                raise AssertionError(f"trace_run answered {line!r} to step {step['step']}:\n{err[-4000:]}")
        proc.stdin.close()
        code = proc.wait(timeout=timeout)
        assert code == 0, f"trace_run exited with {code}: {proc.stderr.read()[-4000:]}"
    finally:
        if proc.poll() is None:
            proc.kill()
    vocab = json.load(open(os.path.join(model_dir, "config.json")))["vocab_size"]
    out = {}
    for number, rows in trace.expect.items():
        data = np.fromfile(os.path.join(out_dir, f"{number}.f32"), dtype="<f4")
        assert data.size == len(rows) * vocab, f"step {number}: {data.size} floats for {len(rows)} rows of {vocab}"
        out[number] = data.reshape(len(rows), vocab)
    return out


def plain_logits(model_dir: str, requests: dict[str, list[int]], act: str) -> dict[str, torch.Tensor]:
    cfg, tensors = plain.read_model_folder(model_dir)
    return {name: plain.logits(cfg, tensors, ids, act) for name, ids in requests.items()}


def compare(trace: Trace, got: dict[int, np.ndarray], want: dict[str, torch.Tensor], atol: float, rtol: float,
            alias: dict[str, str] | None = None) -> float:
    """
    Asserts every wanted row against the plain logits; on failure names the first wrong row (step,
    request, position) so the place can be looked at.  Returns the largest absolute difference.
    """
    worst = 0.0
    for number in sorted(got):
        for r, (name, pos) in enumerate(trace.expect[number]):
            ref = want[(alias or {}).get(name, name)][pos].to(torch.float64)
            row = torch.from_numpy(got[number][r].astype(np.float64))
            diff = (row - ref).abs()
            worst = max(worst, diff.max().item())
            bad = diff > atol + rtol * ref.abs()
            if bool(bad.any()) or not bool(torch.isfinite(row).all()):
                i = int(torch.nonzero(bad | ~torch.isfinite(row))[0])
                raise AssertionError(
                    f"first wrong logits: step {number}, request {name!r}, position {pos}, vocab index {i}: "
                    f"got {row[i].item():.6g}, plain {ref[i].item():.6g} (|diff| max {diff.max().item():.3g}, "
                    f"atol {atol}, rtol {rtol})")
    return worst
