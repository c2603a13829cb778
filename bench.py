"""
Serving benchmark: decode tokens per second of a Llama 3.2 1B sized model with random weights on one
B200, bfloat16, through the engine's own step function; prefill of 2,048 tokens; decode at batch 1
and 64; the same decode measured end to end through the Python entry point.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

One JSON line goes to standard output.  `value` is decoded tokens per second at batch 8 with contexts
of the configuration's benchmark length, timed on the device with CUDA events around K decode steps
(graph replay + sampling kernel), every step reading all weights (2.5 GB, far more than the 126 MB
L2).  `e2e` is the same through LLM.step(): host token ids in, host token ids out, wall clock.
"""

from __future__ import annotations

import argparse
import contextlib
import dataclasses
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: Llama 3.2 1B
MODEL = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 128256,
    "hidden_size": 2048,
    "intermediate_size": 8192,
    "num_hidden_layers": 16,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 64,
    "hidden_act": "silu",
    "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072,
    "tie_word_embeddings": True,
    "attention_bias": False,
    "mlp_bias": False,
    "torch_dtype": "bfloat16",
}
# BASELINE.json configs[3] and configs[4]: Llama 3.2 3B and Llama 3.1 8B (--model 3b / 8b)
MODELS = {
    "1b": ("Llama-3.2-1B", {}, 2048),
    "3b": ("Llama-3.2-3B", {"hidden_size": 3072, "num_hidden_layers": 28, "num_attention_heads": 24, "head_dim": 128}, 2048),
    "8b": ("Llama-3.1-8B", {"hidden_size": 4096, "num_hidden_layers": 32, "num_attention_heads": 32, "head_dim": 128,
                            "intermediate_size": 14336, "tie_word_embeddings": False,
                            "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                             "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}}, 4096),
}
FULL_LAYERS = 16
# One metric, unit and direction for both arms (the driver divides one arm's value by the other's only if
# these agree); which model's layer sizes were run is in `config`.
METRIC = "decode tok/s at batch 8 (bf16, one B200)"
UNIT = "tokens/s"
BATCH = 8
CONTEXT = 4096            # benchmark context length of the configuration
POINT_CONTEXT = 2048      # contexts of the batch 1 / 8 / 64 points
PREFILL_TOKENS = 2048
PAGE = 256
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                data = json.load(f)
            flat = {}

            def walk(node) -> None:               # the keys may sit at the top or inside a nested record
                if isinstance(node, dict):
                    for k, v in node.items():
                        if isinstance(v, (int, float)) and not isinstance(v, bool):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
                elif isinstance(node, list):
                    for v in node:
                        walk(v)

            walk(data)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                return flat, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self.proc = None
        self.gpu = "0"
        try:                                  # the process's device 0 need not be the machine's GPU 0: ask by UUID
            import torch
            uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
            self.gpu = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:                     # noqa: BLE001
            pass

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc) -> None:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        clocks = [int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        top = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower() == "active" for r in self.rows)]
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None,
                "sm_max_mhz": max(top) if top else None, "reasons": reasons, "samples": len(clocks), "gpu": self.gpu}


def size_config(cfg: dict, model_name: str, layers: int, full_layers: int) -> dict:
    """The keys of `config` both arms share: which model's layer sizes ran, how many layers, batch and context."""
    return {
        "model": model_name, "layers": layers, "layers_of_model": full_layers, "hidden_size": cfg["hidden_size"],
        "intermediate_size": cfg["intermediate_size"], "num_attention_heads": cfg["num_attention_heads"],
        "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
        "vocab_size": cfg["vocab_size"], "global_batch": BATCH, "seq_len": CONTEXT, "page_tokens": PAGE,
        "parallelism": "single GPU",
    }


def weight_bytes(cfg: dict, layers: int) -> int:
    h, i, hd = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    nh, nkv, v = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["vocab_size"]
    per_layer = h * (nh + 2 * nkv) * hd + nh * hd * h + 3 * i * h + 2 * h
    # the vocabulary projection's matrix is read once, tied or not; the embedding rows a step gathers are noise
    return 2 * (layers * per_layer + v * h + h)


def kv_bytes(cfg: dict, layers: int, batch: int, context: int) -> int:
    return batch * context * 2 * layers * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg: dict, layers: int, tokens: int, before: int = 0) -> float:
    """A prompt portion of `tokens` tokens behind `before` cached ones, the logits of its last token wanted."""
    h, i, hd = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    nh, nkv, v = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["vocab_size"]
    gemm = 2.0 * tokens * (h * (nh + 2 * nkv) * hd + nh * hd * h + 3 * i * h)
    attention = 2.0 * 2.0 * nh * hd * tokens * (before + (tokens + 1) / 2.0)
    return layers * (gemm + attention) + 2.0 * v * h


# --sweep: decode steps (batch, context) and prompt portions (tokens, cached tokens before them)
SWEEP_DECODE = [(1, 512), (1, 4096), (1, 32768), (1, 131072 - 64), (8, 512), (8, 4096), (8, 32768),
                (64, 512), (64, 4096), (64, 16384)]
SWEEP_PREFILL = [(512, 0), (2048, 0), (8192, 0), (8192, 24576), (8192, 122880 - 64)]


def run_ours(args) -> dict:
    import torch

    from tinyserve_llm_b200 import LLM, CacheConfig, SamplingParams, SchedulerConfig
    from tinyserve_llm_b200.engine.step import StepEntry

    model_name, overrides, point_context = MODELS[args.model]
    cfg = dict(MODEL, **overrides)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    folder = tempfile.mkdtemp(prefix="bench_model_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    steps, warmup = args.steps, max(args.warmup, 3)
    max_len = CONTEXT + steps + warmup + 64 + 512
    pages = 66 * (-(-max_len // PAGE) + 1) + 16
    if args.sweep:
        max_len = cfg["max_position_embeddings"]
        pages = max(b * (c // PAGE + 2) for b, c in SWEEP_DECODE) + 16
    llm = LLM(folder, SchedulerConfig(max_model_len=max_len, max_num_seqs=96, max_num_batched_tokens=8192,
                                      prefill_chunk=2048, watermark=0.0),
              CacheConfig(block_size=PAGE, caching=False), dtype="bfloat16", num_blocks=pages, seed=0,
              random_weights_seed=0)
    ops, runner, cache = llm.model.rt.ops, llm.runner, llm.cache
    gen = torch.Generator().manual_seed(0)

    def prompts(batch: int, length: int) -> list[list[int]]:
        return torch.randint(0, cfg["vocab_size"], (batch, length), generator=gen).tolist()

    def start_decoding(batch: int, context: int, budget: int):
        """Requests with `context`-token prompts, run through the entry point until every one decodes."""
        params = SamplingParams(max_tokens=budget, temperature=0.0, ignore_eos=True)
        for p in prompts(batch, context):
            llm.add_request(p, params)
        while any(not s.output_token_ids for s in llm.scheduler.running + llm.scheduler.waiting):
            llm.step()

    def finish_all():
        for s in llm.scheduler.running + llm.scheduler.waiting:      # one more token, then done
            s.params = SamplingParams(max_tokens=len(s.output_token_ids) + 1, temperature=0.0, ignore_eos=True)
        while llm.scheduler.has_unfinished():
            llm.step()

    @contextlib.contextmanager
    def held_contexts(batch: int, context: int):
        """
        `batch` requests of `context` tokens in the cache, each with the slot of its next token reserved: the
        entries of one decode step, which the timed loops run again and again (every run rewrites the same slots).
        The step function and the cache manager are driven directly; the scheduler holds none of these requests.
        """
        ids = [("held", batch, context, i) for i in range(batch)]
        for seq_id, tokens in zip(ids, prompts(batch, context)):
            for at in range(0, context, PREFILL_TOKENS):      # the step function takes what was reserved, whole
                part = tokens[at:at + PREFILL_TOKENS]
                if at == 0:
                    assert cache.admit(seq_id, part), "the cache pool is too small for the measurement"
                else:
                    cache.extend(seq_id, part)
                runner.step([StepEntry(seq_id, part, [])])
                cache.commit(seq_id, len(part))
        entries = []
        for n, seq_id in enumerate(ids):
            cache.extend(seq_id, [n + 1])
            entries.append(StepEntry(seq_id, [n + 1], [0]))
        try:
            yield entries
        finally:
            torch.cuda.synchronize()
            for seq_id in ids:
                cache.commit(seq_id, 1)
                cache.release(seq_id)

    def device_decode(batch: int, context: int, k: int, w: int):
        """K decode steps timed on the device: graph replay + sampling kernel, no host read in between."""
        temps = torch.zeros(batch, dtype=torch.float32, device=llm.device)
        keys = torch.zeros((batch, 2), dtype=torch.int32, device=llm.device)
        with held_contexts(batch, context) as entries:
            for _ in range(w):
                ops.sample(runner.step(entries), temps, keys)
            torch.cuda.synchronize()
            before = ops.launches
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            for _ in range(k):
                ops.sample(runner.step(entries), temps, keys)
            end.record()
            torch.cuda.synchronize()
            return begin.elapsed_time(end) / k, ops.launches - before

    # ---- prefill of 2,048 tokens, whole, device timed
    def prefill_once(seq_id: int, count: int = PREFILL_TOKENS, before: int = 0) -> float:
        """One prompt portion of `count` tokens behind `before` tokens of the same request (fed untimed, in portions)."""
        tokens = prompts(1, before + count)[0]
        name = ("prefill", seq_id)
        for at in range(0, before, 8192):
            part = tokens[at:min(at + 8192, before)]
            if at == 0:
                assert cache.admit(name, part), "the cache pool is too small for the measurement"
            else:
                cache.extend(name, part)
            runner.step([StepEntry(name, part, [])])
            cache.commit(name, len(part))
        if before:
            cache.extend(name, tokens[before:])
        else:
            assert cache.admit(name, tokens)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        runner.step([StepEntry(name, tokens[before:], [count - 1])])
        end.record()
        torch.cuda.synchronize()
        cache.commit(name, count)
        cache.release(name)
        return begin.elapsed_time(end)

    for i in range(3):
        prefill_once(i)
    if args.sweep:
        peak, peak_kind = peaks()
        decode, prefill = [], []
        with ClockSampler() as clocks:
            for b, c in SWEEP_DECODE:
                ms, _ = device_decode(b, c, 20, 3)
                moved = weight_bytes(cfg, layers) + kv_bytes(cfg, layers, b, c)
                decode.append({"batch": b, "context": c, "ms": round(ms, 4), "value": round(b / ms * 1e3, 1),
                               "hbm_frac": round(moved / (ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4)})
            for n, (count, before) in enumerate(SWEEP_PREFILL):
                prefill_once(100 + 10 * n, count, before)
                ms = statistics.median(prefill_once(101 + 10 * n + i, count, before) for i in range(3))
                flops = prefill_flops(cfg, layers, count, before)
                prefill.append({"tokens": count, "cached_before": before, "ms": round(ms, 3),
                                "value": round(count / ms * 1e3, 1),
                                "frac": round(flops / (ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)})
        return {"impl": "ours", "sweep": {"decode": decode, "prefill": prefill, "unit": "tokens/s", "peaks": peak_kind},
                "config": size_config(cfg, model_name, layers, full_layers), "clocks": clocks.summary()}
    if args.timeline:
        # Where a decode step's time goes inside the replayed graph, overlaps of chained kernels included: CUPTI's
        # record of every kernel of the last of three steps (start after the step's first kernel, duration, and how
        # long after the end of everything before it the kernel itself ended: its share of the critical path).
        from torch.profiler import ProfilerActivity, profile
        tl_batch, tl_context = (int(v) for v in args.timeline.split("x"))
        temps = torch.zeros(tl_batch, dtype=torch.float32, device=llm.device)
        keys = torch.zeros((tl_batch, 2), dtype=torch.int32, device=llm.device)
        with held_contexts(tl_batch, tl_context) as entries:
            for _ in range(3):
                ops.sample(runner.step(entries), temps, keys)
            torch.cuda.synchronize()
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for _ in range(3):
                    ops.sample(runner.step(entries), temps, keys)
                torch.cuda.synchronize()
        events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
                         and "memcpy" not in e.name.lower() and "memset" not in e.name.lower()),
                        key=lambda e: e.time_range.start)
        last = events[-(len(events) // 3):]
        origin, done = last[0].time_range.start, last[0].time_range.start
        print(f"# one decode step, batch {tl_batch}, contexts of {tl_context} tokens, {layers} layers: {len(last)} kernels")
        print("#  start us   length us   ends after all before it (us)   kernel")
        for e in last:
            print(f"{e.time_range.start - origin:10.2f} {e.time_range.end - e.time_range.start:11.2f} "
                  f"{max(0.0, e.time_range.end - done):12.2f}   {e.name[:90]}")
            done = max(done, e.time_range.end)
        print(f"# the step: {done - origin:.1f} us")
        return {"impl": "ours", "profiled": "timeline of one decode step", "config": {"model": model_name, "layers": layers}}
    if args.profile_step is not None:
        if args.profile_step == "prefill":
            torch.cuda.profiler.start()
            prefill_once(99)
            torch.cuda.profiler.stop()
        else:
            temps = torch.zeros(BATCH, dtype=torch.float32, device=llm.device)
            keys = torch.zeros((BATCH, 2), dtype=torch.int32, device=llm.device)
            with held_contexts(BATCH, CONTEXT) as entries:
                for _ in range(3):
                    ops.sample(runner.step(entries), temps, keys)
                torch.cuda.synchronize()
                torch.cuda.profiler.start()
                ops.sample(runner.step(entries), temps, keys)
                torch.cuda.synchronize()
                torch.cuda.profiler.stop()
        return {"impl": "ours", "profiled": f"one {args.profile_step} step", "config": {"model": model_name, "layers": layers}}
    prefill_ms = statistics.median(prefill_once(10 + i) for i in range(5))

    peak, peak_kind = peaks()
    with ClockSampler() as clocks:
        ms, launches = device_decode(BATCH, CONTEXT, steps, warmup)
        # ---- end to end through the entry point: host token ids in, host token ids out
        start_decoding(BATCH, CONTEXT, warmup + steps + 2 + 512)
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        torch.cuda.synchronize()
        e2e_seconds = time.perf_counter() - t0
        graph = runner.last_graph      # the graph the end-to-end steps replayed
        finish_all()
    h2d = (graph.index_buffer.numel() * 4 if graph else 0) + BATCH * 3 * 4
    points = {}
    for b in (1, 8, 64):
        pms, _ = device_decode(b, point_context, max(10, steps // 2), 3)
        points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
    # a mixed step: 64 requests decoding beside one 2,048-token prompt portion
    chunk = prompts(1, PREFILL_TOKENS)[0]
    with held_contexts(64, point_context) as decodes:
        assert cache.admit(("mixed", 0), chunk)
        mixed_entries = decodes + [StepEntry(("mixed", 0), chunk, [PREFILL_TOKENS - 1])]
        for _ in range(2):
            runner.step(mixed_entries)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(5):
            runner.step(mixed_entries)
        end.record()
        torch.cuda.synchronize()
        mixed_ms = begin.elapsed_time(end) / 5
        cache.commit(("mixed", 0), PREFILL_TOKENS)
        cache.release(("mixed", 0))

    # prompts that arrive while 64 requests decode, in portions of 64 tokens: through the entry point (wall clock,
    # host token ids in and out) and the same step on the device alone
    chunk_tokens, arriving_prompt = 64, 512
    with held_contexts(64, point_context) as decodes:
        arriving = prompts(1, arriving_prompt)[0]
        assert cache.admit(("chunk", 0), arriving[:256])
        runner.step([StepEntry(("chunk", 0), arriving[:256], [])])
        cache.commit(("chunk", 0), 256)
        cache.extend(("chunk", 0), arriving[256:256 + chunk_tokens])
        chunk_entries = decodes + [StepEntry(("chunk", 0), arriving[256:256 + chunk_tokens], [])]
        for _ in range(3):
            runner.step(chunk_entries)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(10):
            runner.step(chunk_entries)
        end.record()
        torch.cuda.synchronize()
        chunk_device_ms = begin.elapsed_time(end) / 10
        cache.commit(("chunk", 0), chunk_tokens)
        cache.release(("chunk", 0))
    sched = llm.scheduler
    saved_config = sched.config
    sched.config = dataclasses.replace(saved_config, prefill_chunk=chunk_tokens)
    chunk_steps = 64
    start_decoding(64, point_context, chunk_steps + 200)
    one_token = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
    llm.add_request(prompts(1, arriving_prompt)[0], one_token)
    for _ in range(24):                                         # the shapes of these steps are captured meanwhile
        if llm.step():
            llm.add_request(prompts(1, arriving_prompt)[0], one_token)
    torch.cuda.synchronize()
    fed_before = sched.stats().prefill_tokens + sched.stats().decode_tokens
    t0 = time.perf_counter()
    for _ in range(chunk_steps):
        if llm.step():                                          # the arriving request is done: the next one arrives
            llm.add_request(prompts(1, arriving_prompt)[0], one_token)
    torch.cuda.synchronize()
    chunk_seconds = time.perf_counter() - t0
    chunk_fed = sched.stats().prefill_tokens + sched.stats().decode_tokens - fed_before
    sched.config = saved_config
    finish_all()

    value = BATCH / ms * 1e3
    moved = weight_bytes(cfg, layers) + kv_bytes(cfg, layers, BATCH, CONTEXT)
    achieved = moved / (ms * 1e-3) / 1e9
    flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
    record = {
        "metric": METRIC,
        "value": round(value, 1),
        "unit": UNIT,
        "n_gpus": 1,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": round(ms, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: uniform random token ids, random-init weights N(0, 0.02)",
        "impl": "ours",
        "config": dict(
            size_config(cfg, model_name, layers, full_layers), points_context_len=point_context,
            prefill_tokens=PREFILL_TOKENS, cuda_graphs=bool(graph),
            l2=f"inputs larger than L2 (weights {weight_bytes(cfg, layers) / 1e9:.1f} GB per step)", peaks=peak_kind),
        "prefill": {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
        "mixed": {"decodes": 64, "prefill_tokens": PREFILL_TOKENS, "ms": round(mixed_ms, 3),
                  "value": round((64 + PREFILL_TOKENS) / mixed_ms * 1e3, 1), "unit": "tokens/s"},
        "chunked": {"decodes": 64, "portion_tokens": chunk_tokens, "prompt_tokens": arriving_prompt, "steps": chunk_steps,
                    "device_ms": round(chunk_device_ms, 3), "e2e_ms": round(chunk_seconds / chunk_steps * 1e3, 3),
                    "e2e_over_device": round(chunk_seconds / chunk_steps * 1e3 / chunk_device_ms, 3),
                    "value": round(chunk_fed / chunk_seconds, 1), "unit": "tokens/s fed (decoded + prompt), end to end"},
        "e2e": {"value": round(BATCH * steps / e2e_seconds, 1), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": BATCH * 4},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
    }
    return record


def run_reference(args) -> dict:
    """The unmodified reference from baseline/_ref through its own LLM.generate, same model sizes and batch."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "tinyserve_llm")):
        return {"impl": "reference", "unavailable": "baseline/_ref holds no install of tinyserve-llm"}
    sys.path.insert(0, ref)
    try:
        import torch
        from tinyserve_llm.engine.interface import CacheConfig
        from tinyserve_llm.engine.llm_engine import LLM
        from tinyserve_llm.scheduler.scheduler import SchedulerConfig
        from tinyserve_llm.scheduler.sequence import SamplingParams

        from tinyserve_llm_b200.weights import write_random_model
    except Exception as exc:                                  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"import failed: {type(exc).__name__}: {exc}"[:300]}
    layers = args.layers or FULL_LAYERS
    cfg = dict(MODEL, num_hidden_layers=layers)
    steps, warmup = args.steps, max(args.warmup, 3)
    folder = tempfile.mkdtemp(prefix="bench_ref_model_")
    try:
        write_random_model(folder, cfg, 0)
        max_len = CONTEXT + steps + warmup + 64
        llm = LLM(folder, SchedulerConfig(max_model_len=max_len, max_num_seqs=BATCH,
                                          max_num_batched_tokens=BATCH * CONTEXT + BATCH),
                  CacheConfig(block_size=PAGE, caching=False), dtype=torch.bfloat16,
                  num_blocks=BATCH * (-(-max_len // PAGE) + 1) + 8, seed=0, load_tokenizer=False)
        gen = torch.Generator().manual_seed(0)
        prompts = torch.randint(0, cfg["vocab_size"], (BATCH, CONTEXT), generator=gen).tolist()
        with ClockSampler() as clocks:
            llm.generate(prompts, SamplingParams(max_tokens=warmup + steps + 1, temperature=0.0, ignore_eos=True))
        decode = [r for r in llm.steps if r.num_tokens == BATCH and r.num_seqs == BATCH][-steps:]
        seconds = sum(r.end - r.start for r in decode)
        value = BATCH * len(decode) / seconds
    except Exception as exc:                                  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"the reference did not run here: {type(exc).__name__}: {exc}"[:300]}
    return reference_record(value, len(decode), warmup, seconds, layers, clocks.summary())


def reference_h2d_bytes(batch: int, context: int) -> int:
    """
    Bytes tinyserve-llm copies to the device for one decode step of `batch` requests, counted from
    the tensors its engine/model_runner.py:73-92 builds: int64 ids, positions, slots and sample rows,
    float32 temperatures, two int32 offset arrays of batch + 1, and the int32 block tables.
    """
    width = -(-(context + 1) // PAGE)
    return batch * (8 + 8 + 8 + 8 + 4) + 2 * 4 * (batch + 1) + 4 * batch * width


def reference_record(value: float, steps: int, warmup: int, seconds: float, layers: int, clocks: dict) -> dict:
    """The reference arm's line: the same metric, unit and direction as `run_ours` prints."""
    return {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT,
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(seconds / max(steps, 1) * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, random-init weights N(0, 0.02)", "impl": "reference",
        "config": dict(size_config(MODEL, MODELS["1b"][0], layers, FULL_LAYERS),
                       timing="host clock around each decode step of LLM.generate (each ends in a host read)"),
        "e2e": {"value": round(value, 1), "unit": UNIT, "h2d_bytes_per_step": reference_h2d_bytes(BATCH, CONTEXT),
                "d2h_bytes_per_step": BATCH * 8,
                "how": "LLM.generate's own steps: each packs host lists into tensors, copies them and reads the tokens back"},
        "clocks": clocks,
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config); 0: all")
    parser.add_argument("--model", choices=sorted(MODELS), default="1b", help="layer sizes: Llama 3.2 1B (default), 3B, 3.1 8B")
    parser.add_argument("--profile-step", choices=["decode", "prefill"], default=None,
                        help="no measurement: warm up, then run ONE step of that kind between cudaProfilerStart and "
                             "cudaProfilerStop (for `ncu --profile-from-start off`), and exit")
    parser.add_argument("--sweep", action="store_true",
                        help="instead of the headline record: decode steps at batch 1, 8 and 64 with contexts from 512 tokens to "
                             "the model's longest, and prompt portions of 512 to 8,192 tokens behind up to 120k cached tokens, "
                             "each with its fraction of the measured peak")
    parser.add_argument("--timeline", nargs="?", const=f"{BATCH}x{CONTEXT}", default=None, metavar="BATCHxCONTEXT",
                        help="no measurement: print every kernel of one decode step (default: the headline's batch and context) "
                             "with its start, length and its share of the critical path inside the replayed graph (CUPTI "
                             "through torch.profiler), and exit")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (run with --gpus 1)")
        return 2
    record = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(record), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
