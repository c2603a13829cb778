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

    def __init__(self, page: int = 64) -> None:
        self.page = page
        self.steps: list[dict] = []
        self.expect: dict[int, list[tuple[str, int]]] = {}
        self.fed: dict[str, int] = {}            # tokens fed so far per live request
        self.peak = 0                            # most tokens held at once, each request rounded up to a page

    def step(self, parts: list[tuple[str, list[int], list[int]]], end: list[str] = (),
             fork: list[tuple[str, str]] = ()) -> None:
        """parts: (request, its next tokens, wanted places among them); fork: (from, to) pairs, done before the parts."""
        number = len(self.steps)
        entries, rows = [], []
        for src, dst in fork:
            self.fed[dst] = self.fed[src]
        for name, tokens, want in parts:
            start = self.fed.get(name, 0)
            entries.append({"id": name, "tokens": list(tokens), "want": list(want)})
            rows.extend((name, start + w) for w in want)
            self.fed[name] = start + len(tokens)
        self.peak = max(self.peak, sum(-(-n // self.page) * self.page for n in self.fed.values()))
        for name in end:
            self.fed.pop(name, None)
        record = {"step": number, "entries": entries, "end": list(end)}
        if fork:
            record["fork"] = [{"from": src, "to": dst} for src, dst in fork]
        self.steps.append(record)
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


def simulate(trace: Trace, num_pages: int, caching: bool):
    """
    The cache manager's side of a replay, on the host alone: the calls bin/trace_run makes, with a
    storage that moves nothing.  Returns (the manager's counters, tokens reused per request), or
    None if some step does not fit into `num_pages` pages.
    """
    from tinyserve_llm_b200.cache.manager import CacheManager, plan_layout
    from tinyserve_llm_b200.parts.base import KVNeed
    manager = CacheManager(plan_layout([(KVNeed(1, 16, 0), 0)], trace.page), num_pages, caching=caching)
    reused: dict[str, int] = {}
    for record in trace.steps:
        for fork in record.get("fork", []):
            manager.fork(fork["from"], fork["to"])
        fed = []
        for item in record["entries"]:
            name, tokens, want = item["id"], item["tokens"], item["want"]
            if name in manager.seqs:
                if not manager.can_extend(name, len(tokens)):
                    return None
                manager.extend(name, tokens)
                fed.append((name, len(tokens)))
            else:
                if not manager.admit(name, tokens, reuse_limit=min(want, default=len(tokens) - 1)):
                    return None
                reused[name] = manager.committed_tokens(name)
                fed.append((name, len(tokens) - reused[name]))
        for name, n in fed:
            manager.commit(name, n)
        for name in record["end"]:
            if name in manager.seqs:
                manager.release(name)
    return manager.stats(), reused


def run_trace(model_dir: str, dtype: str, trace: Trace, out_dir: str, max_tokens: int | None = None,
              timeout: float = 900.0, caching: bool = False) -> dict[int, np.ndarray]:
    """Runs bin/trace_run as a child process, feeding the next step only after `done <step>`."""
    os.makedirs(out_dir, exist_ok=True)
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir, "--max-tokens",
           str(max_tokens if max_tokens is not None else trace.peak)]
    if trace.page != 64:
        cmd += ["--page-tokens", str(trace.page)]
    if caching:
        cmd += ["--caching", "on"]
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


def read_stats(out_dir: str) -> dict:
    with open(os.path.join(out_dir, "stats.json")) as f:
        return json.load(f)


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


def cached_paths_trace(vocab: int, page: int, seed: int = 70) -> tuple[Trace, dict[str, list[int]]]:
    """
    A replay for `--caching on` that takes every path by which a request comes to read keys another
    request computed: whole cached pages attached, a partly matching page copied, an identical page
    met at commit (dedupe), a fork whose two branches write different tokens into their shared last
    page (copy on write), and cached pages that were evicted, taken by others and computed again.
    Returns the trace and, for each request name, the whole token list its rows belong to.
    """
    B = page
    ids = lambda n, s: random_ids(vocab, n, seed + s)                       # noqa: E731
    trace = Trace(page)
    requests: dict[str, list[int]] = {}

    # P whole, then ended: seven full pages and half a page stay cached
    p = ids(7 * B + B // 2, 0)
    requests["p"] = p
    trace.step([("p", p, list(range(len(p))))], end=["p"])

    # R1 and R2 start with the same two pages, in the same step: the second to commit meets the first one's pages
    head = ids(2 * B, 1)
    requests["r1"] = head + ids(B // 2 + 1, 2)
    requests["r2"] = head + ids(B // 4 + 3, 3)
    n1, n2 = 2 * B + 3, 2 * B + 2
    trace.step([("r1", requests["r1"][:n1], [0, n1 - 1]), ("r2", requests["r2"][:n2], [2 * B - 1, n2 - 1])])
    trace.step([("r1", requests["r1"][n1:], [0]), ("r2", requests["r2"][n2:], [0, len(requests["r2"]) - n2 - 1])],
               end=["r1", "r2"])

    # Q shares P's first six pages and a quarter of the seventh (attached pages + a partial-page copy), then
    # goes its own way; fed in uneven portions.  R3 repeats P's first page but wants its first row, so it runs
    # everything and meets the cached page at commit.
    shared = 6 * B + B // 4
    q_own = ids(B + B // 2 + 3, 4)
    q_own[0] = (p[shared] + 1) % vocab                                      # the runs part exactly here
    q = p[:shared] + q_own
    r3 = p[:B] + ids(5, 5)
    requests["r3"] = r3
    first = shared + 10
    trace.step([("q", q[:first], list(range(shared + 3, first))), ("r3", r3[:B + 2], [0, B - 1, B + 1])])
    pos = first
    for n in (2, 7, 3):
        trace.step([("q", q[pos:pos + n], list(range(n)))] + ([("r3", r3[B + 2:], [0, 2])] if n == 7 else []),
                   end=["r3"] if n == 7 else [])
        pos += n
    trace.step([("q", q[pos:], [0, len(q) - pos - 1])])
    assert len(q) % B, "the fork must share a partly filled page"

    # Q forked between steps; the branches decode 20 different tokens each, in the same steps
    tail_a, tail_b = ids(20, 6), ids(20, 7)
    tail_b[0] = (tail_a[0] + 1) % vocab
    requests["q"], requests["q2"] = q + tail_a, q + tail_b
    for i in range(20):
        trace.step([("q", tail_a[i:i + 1], [0]), ("q2", tail_b[i:i + 1], [0])], fork=[("q", "q2")] if i == 0 else [],
                   end=["q", "q2"] if i == 19 else [])

    # two long strangers push cached pages out of a small pool ...
    for k, name in enumerate(("f1", "f2")):
        f = ids(6 * B + 5 + k, 8 + k)
        requests[name] = f
        trace.step([(name, f[:4 * B], [4 * B - 1])])
        trace.step([(name, f[4 * B:], [0, len(f) - 4 * B - 1])], end=[name])
    # ... and P comes again: what is left of it is attached, the rest computed again on pages others held meanwhile
    requests["p_again"] = p
    trace.step([("p_again", p, [len(p) - 3, len(p) - 1])], end=["p_again"])
    return trace, requests


def smallest_pool(trace: Trace, caching: bool) -> int:
    """The fewest pages with which every step of the trace fits (by the host-side simulation)."""
    pages = 1
    while simulate(trace, pages, caching) is None:
        pages += 1
        assert pages < 10_000
    return pages
