"""
The engine through its Python entry point on the GPU: greedy generation equal to the plain
implementation, unchanged by prefix reuse, portions, preemption and forks; seeded sampling; EOS;
step records; the command line.
"""

import json
import subprocess
import sys

import pytest
import torch

import plain_llama as plain
import replay_util as ru
from tiny_configs import PAGE_A, PAGE_B, TINY_A, TINY_B, TINY_D

pytestmark = pytest.mark.gpu


def make_llm(folder, page, num_blocks=64, dtype="float32", **kwargs):
    from tinyserve_llm_b200 import LLM, CacheConfig, SchedulerConfig
    sched = dict(max_model_len=200, max_num_seqs=8, max_num_batched_tokens=256, eos_token_id=-2, watermark=0.0)
    sched.update({k: kwargs.pop(k) for k in list(kwargs) if k in SchedulerConfig.__dataclass_fields__})
    caching = kwargs.pop("caching", True)
    return LLM(folder, SchedulerConfig(**sched), CacheConfig(block_size=page, caching=caching), dtype=dtype,
               num_blocks=num_blocks, **kwargs)


def greedy(max_tokens=8, **kw):
    from tinyserve_llm_b200 import SamplingParams
    return SamplingParams(max_tokens=max_tokens, temperature=0.0, ignore_eos=True, **kw)


@pytest.fixture(scope="module")
def workload_b(model_folders):
    vocab = TINY_B["vocab_size"]
    stem = ru.random_ids(vocab, 100, 7)
    prompts = [stem + ru.random_ids(vocab, 11, 8), ru.random_ids(vocab, 1, 9), stem + ru.random_ids(vocab, 40, 10),
               ru.random_ids(vocab, 150, 11), stem[:70] + ru.random_ids(vocab, 5, 12), ru.random_ids(vocab, 33, 13)]
    cfg, tensors = plain.read_model_folder(model_folders["b"])
    want = [plain.greedy_generate(cfg, tensors, p, 8) for p in prompts]
    return prompts, want


def test_greedy_equals_the_plain_implementation_and_reuses_the_shared_prefix(model_folders, workload_b):
    prompts, want = workload_b
    llm = make_llm(model_folders["b"], PAGE_B, prefill_chunk=64, max_num_batched_tokens=96)
    done = llm.generate(prompts[:1], greedy()) + llm.generate(prompts[1:], greedy())
    assert [c.token_ids[0] for c in done] == want
    assert [c.finish_reasons for c in done] == [["length"]] * len(prompts)
    stats = llm.scheduler.stats()
    # the first request's pages are found again: 3 whole pages + 4 copied slots, and 2 whole pages + 6 copied slots
    assert stats.cached_tokens == 100 + 70
    assert llm.cache.stats().partial_copies == 2
    assert llm.cache.stats().pages_in_use == 0
    later = llm.generate([prompts[0]], greedy())     # everything but the last token is cached now
    assert later[0].token_ids[0] == want[0]
    assert llm.scheduler.stats().cached_tokens - stats.cached_tokens == len(prompts[0]) - 1


@pytest.mark.parametrize("kwargs", [
    {"caching": False}, {"prefill_chunk": 7, "max_num_batched_tokens": 24}, {"num_blocks": 7, "caching": False},
    {"step_mode": "prefill_first"}, {"cuda_graphs": False}, {"max_num_seqs": 2}, {"run_ahead": False},
    {"run_ahead": False, "cuda_graphs": False}])
def test_output_does_not_depend_on_how_the_work_is_cut(model_folders, workload_b, kwargs):
    prompts, want = workload_b
    llm = make_llm(model_folders["b"], PAGE_B, **kwargs)
    done = llm.generate(prompts, greedy())
    assert [c.token_ids[0] for c in done] == want
    assert llm.cache.stats().pages_in_use == 0
    if kwargs.get("cuda_graphs", True):
        assert llm.runner.graph_replays > 0, "decode steps were meant to come from CUDA graphs"
    if kwargs.get("run_ahead", True):
        assert llm.steps_launched_ahead > 0, "decode steps were meant to be launched ahead of the samples"
    else:
        assert llm.steps_launched_ahead == 0


@pytest.mark.parametrize("caching", [True, False])
def test_running_out_of_pages_preempts_and_changes_no_token(model_folders, caching):
    """Three requests grow from one page to three in a pool of five: a decode finds no page, the lowest score gives way."""
    vocab = TINY_B["vocab_size"]
    prompts = [ru.random_ids(vocab, 15, 50 + i) for i in range(3)]
    cfg, tensors = plain.read_model_folder(model_folders["b"])
    want = [plain.greedy_generate(cfg, tensors, p, 20) for p in prompts]
    llm = make_llm(model_folders["b"], 16, num_blocks=5, caching=caching, max_model_len=64)
    done = llm.generate(prompts, greedy(20))
    stats = llm.scheduler.stats()
    assert stats.preemptions > 0 and stats.readmissions > 0
    assert [c.token_ids[0] for c in done] == want
    assert llm.cache.stats().pages_in_use == 0


def token_costs_within_bound(cfg, tensors, prompt, tokens, act="bfloat16"):
    """
    Token parity is not exact in bfloat16 (near-tied logits), so what each generated token costs in
    plain logit is bounded instead.  The replay tests hold every engine logit to the plain one
    within d = 1.2 % of the largest logit; a token that is the largest of the engine's logits can
    then lie at most 2 d under the largest plain logit (its own logit may be d too high, the plain
    winner's d too low).
    """
    ids = list(prompt)
    for token in tokens:
        row = plain.logits(cfg, tensors, ids, act)[-1]
        if row.max().item() - row[token].item() > 2 * 0.012 * row.abs().max().item():
            return False
        ids.append(token)
    return True


@pytest.mark.parametrize("name, page, kwargs", [
    ("b", PAGE_B, {}), ("d", 64, {}), ("d", 64, {"cuda_graphs": False, "run_ahead": False}),
    ("d", 64, {"prefill_chunk": 24, "max_num_batched_tokens": 40}), ("d", 64, {"num_blocks": 7, "caching": False}),
    ("d", 64, {"caching": False, "run_ahead": False})])
def test_bfloat16_generation_stays_with_the_plain_bfloat16_model(model_folders, name, page, kwargs):
    """
    bfloat16 through the whole engine: CUDA-graph decode and steps launched ahead (the default), neither,
    prompts in small portions beside decodes, and a pool so small that requests are preempted and run again.
    """
    raw = {"b": TINY_B, "d": TINY_D}[name]
    vocab = raw["vocab_size"]
    stem = ru.random_ids(vocab, 70, 17)
    prompts = [stem + ru.random_ids(vocab, 9, 18), ru.random_ids(vocab, 3, 19), stem[:50] + ru.random_ids(vocab, 30, 20),
               ru.random_ids(vocab, 130, 21)]
    cfg, tensors = plain.read_model_folder(model_folders[name])
    llm = make_llm(model_folders[name], page, dtype="bfloat16", max_model_len=260, **kwargs)
    done = llm.generate(prompts, greedy(70 if "num_blocks" in kwargs else 8))      # 70: the requests outgrow the small pool
    for prompt, c in zip(prompts, done):
        assert token_costs_within_bound(cfg, tensors, prompt, c.token_ids[0][:8]), (kwargs, c.token_ids[0])
    assert llm.cache.stats().pages_in_use == 0
    if "num_blocks" in kwargs:
        assert llm.scheduler.stats().preemptions > 0, "the pool was meant to be too small"
    if kwargs.get("cuda_graphs", True):
        assert llm.runner.graph_replays > 0
    if kwargs.get("run_ahead", True):
        assert llm.steps_launched_ahead > 0


def test_bfloat16_forks_share_and_copy_pages(model_folders):
    """n = 3 greedy samples of one prompt in bfloat16: the same tokens three times (the forks read the same pages and logits), within the bound."""
    prompt = ru.random_ids(TINY_D["vocab_size"], 75, 23)
    llm = make_llm(model_folders["d"], 64, dtype="bfloat16", max_model_len=260)
    done = llm.generate([prompt], greedy(10, n=3))[0]
    assert done.token_ids[0] == done.token_ids[1] == done.token_ids[2]
    cfg, tensors = plain.read_model_folder(model_folders["d"])
    assert token_costs_within_bound(cfg, tensors, prompt, done.token_ids[0][:6])
    assert llm.cache.stats().cow_copies >= 2 and llm.cache.stats().pages_in_use == 0


def test_forks_agree_when_greedy_and_leave_no_page_behind(model_folders):
    vocab = TINY_A["vocab_size"]
    prompt = ru.random_ids(vocab, 37, 3)
    llm = make_llm(model_folders["a"], PAGE_A)
    done = llm.generate([prompt], greedy(6, n=3))[0]
    cfg, tensors = plain.read_model_folder(model_folders["a"])
    assert done.token_ids == [plain.greedy_generate(cfg, tensors, prompt, 6)] * 3
    assert llm.cache.stats().cow_copies >= 2 and llm.cache.stats().pages_in_use == 0


def test_seeded_sampling_is_reproducible_and_independent_of_the_batch(model_folders):
    from tinyserve_llm_b200 import SamplingParams
    vocab = TINY_B["vocab_size"]
    prompts = [ru.random_ids(vocab, n, 20 + n) for n in (9, 40, 77)]
    params = SamplingParams(max_tokens=10, temperature=0.8, n=2, ignore_eos=True)
    first = make_llm(model_folders["b"], PAGE_B, seed=5).generate(prompts, params)
    again = make_llm(model_folders["b"], PAGE_B, seed=5).generate(prompts, params)
    other = make_llm(model_folders["b"], PAGE_B, seed=6).generate(prompts, params)
    assert [c.token_ids for c in first] == [c.token_ids for c in again]
    assert [c.token_ids for c in first] != [c.token_ids for c in other]
    assert all(c.token_ids[0] != c.token_ids[1] for c in first), "the two samples of a request must differ"
    # the same request alone, in portions, without graphs: the same draws (keys are per request and position)
    alone = make_llm(model_folders["b"], PAGE_B, seed=5, prefill_chunk=16, cuda_graphs=False, run_ahead=False)
    alone.generate([prompts[2]], greedy(1))                         # takes request id 0; ids key the noise
    assert alone.generate([prompts[1]], params)[0].token_ids == first[1].token_ids


def test_eos_stops_generation_and_is_kept(model_folders):
    from tinyserve_llm_b200 import SamplingParams
    prompt = ru.random_ids(TINY_B["vocab_size"], 20, 30)
    cfg, tensors = plain.read_model_folder(model_folders["b"])
    free = plain.greedy_generate(cfg, tensors, prompt, 8)
    stop = free[3]
    cut = free[:free.index(stop) + 1]
    llm = make_llm(model_folders["b"], PAGE_B, eos_token_id=stop)
    done = llm.generate([prompt, prompt], [SamplingParams(max_tokens=8, temperature=0.0),
                                           SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)])
    assert done[0].token_ids[0] == cut and done[0].finish_reasons == ["eos"]
    assert done[1].token_ids[0] == free and done[1].finish_reasons == ["length"]
    assert llm.steps_launched_ahead > 0 and llm.cache.stats().pages_in_use == 0
    alone = llm.generate([prompt], SamplingParams(max_tokens=8, temperature=0.0))[0]    # the step launched behind its end is dropped
    assert alone.token_ids[0] == cut and llm.cache.stats().pages_in_use == 0 and llm._in_flight is None
    # -1 means: take the model's own end token (the first of config.json's list)
    assert make_llm(model_folders["b"], PAGE_B, eos_token_id=-1).scheduler.config.eos_token_id == 7


def test_step_records_and_requests_the_engine_refuses(model_folders):
    llm = make_llm(model_folders["a"], PAGE_A)
    llm.generate([[1, 2, 3, 4, 5]], greedy(3))
    assert [(r.num_seqs, r.num_tokens) for r in llm.steps] == [(1, 5), (1, 1), (1, 1)]
    assert llm.steps[-1].scheduler.decode_tokens == 2 and llm.steps[0].end >= llm.steps[0].start
    with pytest.raises(ValueError, match="vocabulary"):
        llm.add_request([1, 2, 99999])
    with pytest.raises(ValueError, match="max_model_len"):
        llm.add_request([1] * 199, greedy(8))
    with pytest.raises(ValueError, match="tokenizer"):
        llm.add_request("some text")
    with pytest.raises(ValueError, match="max_position_embeddings"):
        make_llm(model_folders["a"], PAGE_A, max_model_len=100000, max_num_batched_tokens=200000)


def test_cache_sized_from_free_memory_and_random_weights_from_a_seed(model_folders, tmp_path):
    from tinyserve_llm_b200 import LLM, CacheConfig, SchedulerConfig
    from tinyserve_llm_b200.weights import write_random_model
    llm = LLM(model_folders["a"], SchedulerConfig(max_model_len=128, max_num_seqs=4, max_num_batched_tokens=128),
              CacheConfig(block_size=PAGE_A), dtype="bfloat16", gpu_memory_utilization=0.05, random_weights_seed=3)
    assert llm.cache.num_pages > 100
    out = llm.generate([[5, 6, 7]], greedy(4))
    assert len(out[0].token_ids[0]) == 4 and llm.cache.stats().pages_in_use == 0
    # one seed, one model: the folder written from the same seed holds the same weights
    folder = str(tmp_path / "seed3")
    write_random_model(folder, TINY_A, 3)
    written = LLM(folder, SchedulerConfig(max_model_len=128, max_num_seqs=4, max_num_batched_tokens=128),
                  CacheConfig(block_size=PAGE_A), dtype="bfloat16", num_blocks=16)
    assert torch.equal(written.model.embedding, llm.model.embedding)
    assert torch.equal(written.model.blocks[1].mixer.qkv.weight, llm.model.blocks[1].mixer.qkv.weight)
    assert written.generate([[5, 6, 7]], greedy(4))[0].token_ids == out[0].token_ids


def test_a_cache_sized_from_free_memory_leaves_room_for_the_widest_steps(model_folders):
    """
    `num_blocks=None` with 64 sequence slots: 64 requests decode across several buckets of batch size
    and table width (their lengths differ, they finish one after another), with logits of 64 rows
    and graphs of several shapes alive; the memory torch holds never passes the share it was given.
    """
    from tinyserve_llm_b200 import LLM, CacheConfig, SchedulerConfig
    share = 0.04
    total = torch.cuda.mem_get_info()[1]
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    llm = LLM(model_folders["d"], SchedulerConfig(max_model_len=1000, max_num_seqs=64, max_num_batched_tokens=2048,
                                                   eos_token_id=-2, prefill_chunk=256),
              CacheConfig(block_size=64), dtype="bfloat16", gpu_memory_utilization=share, seed=1)
    vocab = TINY_D["vocab_size"]
    prompts = [ru.random_ids(vocab, 5 + 11 * i, 300 + i) for i in range(64)]
    params = [greedy(20 + 3 * (i % 9)) for i in range(64)]
    out = llm.generate(prompts, params)
    assert [len(c.token_ids[0]) for c in out] == [p.max_tokens for p in params]
    assert llm.runner.graph_replays > 20 and len(llm.runner._graphs) >= 3
    assert torch.cuda.max_memory_allocated() <= share * total
    assert llm.cache.stats().pages_in_use == 0


def test_command_line_writes_one_json_record(model_folders, tmp_path):
    out = tmp_path / "result.json"
    cmd = [sys.executable, "-m", "tinyserve_llm_b200.cli.generate", "--model", model_folders["a"], "--prompt-ids",
           "1,2,3,4", "--prompt-ids", "9 8 7", "--max-tokens", "5", "--temperature", "0", "--dtype", "float32",
           "--block-size", str(PAGE_A), "--num-blocks", "32", "--max-model-len", "128", "--max-num-seqs", "4",
           "--max-num-batched-tokens", "64", "--ignore-eos", "--out", str(out)]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=ru.ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    record = json.loads(out.read_text())
    cfg, tensors = plain.read_model_folder(model_folders["a"])
    assert [c["token_ids"][0] for c in record["completions"]] == \
        [plain.greedy_generate(cfg, tensors, p, 5) for p in ([1, 2, 3, 4], [9, 8, 7])]
    assert record["output_tokens"] == 10 and "output tok/s" in proc.stdout


@pytest.mark.parametrize("cuda_graphs", [True, False])
def test_a_token_fed_on_the_device_gives_the_step_the_host_token_gives(model_folders, cuda_graphs):
    """`StepEntry.feed`: the step reads its token from a device tensor (the previous step's samples) and equals the step given the same token by the host."""
    from tinyserve_llm_b200.engine.loading import build_cache, load_model
    from tinyserve_llm_b200.engine.step import StepEntry, StepRunner
    model = load_model(model_folders["b"], "float32", "cuda")
    vocab = TINY_B["vocab_size"]
    prompts = [ru.random_ids(vocab, n, 70 + n) for n in (5, 40, 17)]
    nexts = [11, 3, vocab - 1]
    results = []
    for fed_on_device in (False, True):
        _, manager, storage = build_cache(model, PAGE_B, 16, caching=False)
        runner = StepRunner(model, manager, storage, cuda_graphs=cuda_graphs)
        for i, p in enumerate(prompts):
            assert manager.admit(i, p)
        runner.step([StepEntry(i, p, []) for i, p in enumerate(prompts)])
        for i, p in enumerate(prompts):
            manager.commit(i, len(p))
        for round_ in range(2):                                    # twice: the second decode step replays the captured graph
            for i in range(3):
                manager.extend(i, [nexts[i]])
            if fed_on_device:                                      # samples of "the step before", in another order than the entries
                device_tokens = torch.tensor([nexts[2], 0, nexts[0], nexts[1]], dtype=torch.int32, device="cuda")
                entries = [StepEntry(0, (0,), (0,), feed=2), StepEntry(1, (0,), (0,), feed=3), StepEntry(2, (0,), (0,), feed=0)]
                logits = runner.step(entries, device_tokens)
            else:
                logits = runner.step([StepEntry(i, [nexts[i]], [0]) for i in range(3)])
            results.append(logits.cpu().clone())
            for i in range(3):
                manager.commit(i, 1)
        with pytest.raises(ValueError, match="fed on the device"):
            manager.extend(0, [1])
            runner.step([StepEntry(0, (0,), (0,), feed=9)], torch.zeros(2, dtype=torch.int32, device="cuda"))
    assert torch.equal(results[0], results[2]) and torch.equal(results[1], results[3])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_follow_the_longest_request(model_folders, dtype):
    """
    A decode graph is captured for a bucket of the batch size and of the pages the step's longest request
    holds, not for the longest context the engine allows.  Decoding across the edges of those buckets
    (the tables grow from 2 pages to 8 here) gives bit for bit what steps without graphs give, and a short
    batch after a long one goes back to the small graph.
    """
    from tinyserve_llm_b200.engine.loading import build_cache, load_model
    from tinyserve_llm_b200.engine.step import StepEntry, StepRunner
    assert [StepRunner.width_bucket(n) for n in (1, 2, 3, 4, 5, 6, 7, 9, 13, 17, 25, 33)] == [1, 2, 3, 4, 6, 6, 8, 12, 16, 24, 32, 48]
    model = load_model(model_folders["b"], dtype, "cuda")
    vocab = TINY_B["vocab_size"]
    prompts = [ru.random_ids(vocab, n, 90 + n) for n in (PAGE_B + 3, 2 * PAGE_B - 2, 5)]
    steps = 5 * PAGE_B + 4
    outs = {}
    for graphs in (True, False):
        _, manager, storage = build_cache(model, PAGE_B, 40, caching=False)
        runner = StepRunner(model, manager, storage, cuda_graphs=graphs, max_model_len=30 * PAGE_B)
        for i, p in enumerate(prompts):
            assert manager.admit(i, p)
        runner.step([StepEntry(i, p, []) for i, p in enumerate(prompts)])
        for i, p in enumerate(prompts):
            manager.commit(i, len(p))
        got, expected = [], set()
        for t in range(steps):
            live = [0, 1, 2] if t < steps - 3 else [2]            # at the end the short request alone
            for i in live:
                manager.extend(i, [(7 * t + i) % vocab])
            expected.add(StepRunner.width_bucket(max(len(manager.seqs[i].tables[0]) for i in live)))
            got.append(runner.step([StepEntry(i, [(7 * t + i) % vocab], [0]) for i in live]).cpu().clone())
            for i in live:
                manager.commit(i, 1)
        outs[graphs] = got
        if graphs:
            widths = {shape.widths[0] for shape in runner._graphs}
            assert widths == expected and len(widths) >= 5, (widths, expected)    # 2 pages at first, 8 at the end
            assert runner.graph_replays == steps
    for a, b in zip(outs[True], outs[False]):
        assert torch.equal(a, b)
    # no more than `max_graphs` graphs are kept: the least recently used one is dropped, and captured again when needed
    _, manager, storage = build_cache(model, PAGE_B, 40, caching=False)
    runner = StepRunner(model, manager, storage, cuda_graphs=True, max_model_len=30 * PAGE_B, max_graphs=2)
    assert manager.admit(0, prompts[1])
    runner.step([StepEntry(0, prompts[1], [])])
    manager.commit(0, len(prompts[1]))
    for t in range(steps):
        manager.extend(0, [(7 * t + 1) % vocab])
        again = runner.step([StepEntry(0, [(7 * t + 1) % vocab], [0])]).cpu()
        manager.commit(0, 1)
        assert len(runner._graphs) <= 2
    assert runner.graph_replays == steps


@pytest.mark.parametrize("name, dtype, page", [("b", "float32", PAGE_B), ("d", "bfloat16", 64), ("d", "float32", 64)])
def test_steps_with_prompt_portions_are_replayed_from_graphs(model_folders, name, dtype, page):
    """
    Three requests decode while two more arrive in portions of 40 and 24 tokens (the last portions are
    shorter): from the second time a shape of step is met (the runner is told so here; its default is the
    third) it is captured and replayed, padded to its buckets.  float32 gives bit for bit what steps launched kernel by kernel give; bfloat16 the same
    up to the library product's choice of kernel for another number of rows.
    """
    from tinyserve_llm_b200.engine.loading import build_cache, load_model
    from tinyserve_llm_b200.engine.step import StepEntry, StepRunner
    raw = {"b": TINY_B, "d": TINY_D}[name]
    vocab = raw["vocab_size"]
    model = load_model(model_folders[name], dtype, "cuda")
    decoding = [ru.random_ids(vocab, n, 700 + n) for n in (page + 3, 9, 2 * page)]
    arriving = {"x": ru.random_ids(vocab, 190, 801), "y": ru.random_ids(vocab, 100, 802)}
    outs = {}
    for graphs in (True, False):
        _, manager, storage = build_cache(model, page, 40, caching=False)
        runner = StepRunner(model, manager, storage, cuda_graphs=graphs, sightings_before_capture=2)
        for i, p in enumerate(decoding):
            assert manager.admit(i, p)
        runner.step([StepEntry(i, p, []) for i, p in enumerate(decoding)])
        for i, p in enumerate(decoding):
            manager.commit(i, len(p))
        fed = {"x": 0, "y": 0}
        got = []
        for t in range(9):
            entries = []
            for i in range(3):
                manager.extend(i, [(11 * t + i) % vocab])
                entries.append(StepEntry(i, [(11 * t + i) % vocab], [0]))
            for key, size in (("x", 40), ("y", 24)):
                tokens = arriving[key][fed[key]:fed[key] + size]
                if not tokens:
                    continue
                if fed[key] == 0:
                    assert manager.admit(key, tokens)
                else:
                    manager.extend(key, tokens)
                last = fed[key] + len(tokens) == len(arriving[key])
                entries.append(StepEntry(key, tokens, [len(tokens) - 1] if last else []))
                fed[key] += len(tokens)
            got.append(runner.step(entries).cpu().clone())
            for e in entries:
                manager.commit(e.seq_id, len(e.tokens))
        outs[graphs] = got
        if graphs:
            shapes = [s for s in runner._graphs if s.portions]
            assert shapes and runner.graph_replays >= 3, (runner.graph_replays, list(runner._graphs))
            assert all(s.tokens % 64 == 0 and s.seqs == 8 for s in shapes)
    for a, b in zip(outs[True], outs[False]):
        assert a.shape == b.shape
        if dtype == "float32":
            assert torch.equal(a, b)
        else:
            torch.testing.assert_close(a, b, atol=0.012 * float(b.abs().max()), rtol=0.0)


def test_a_captured_step_records_no_buffer_of_the_eager_run(model_folders):
    """
    A capture runs the step once eagerly, then records it.  Scratch buffers that the parts keep in the step's
    context during the eager run belong to the ordinary allocator and are freed with the context: the recorded
    launches must get buffers of their own (from the graphs' pool), or a replay writes into freed memory.
    """
    from tinyserve_llm_b200.engine.loading import build_cache, load_model
    from tinyserve_llm_b200.engine.step import StepEntry, StepRunner
    model = load_model(model_folders["d"], "bfloat16", "cuda")
    _, manager, storage = build_cache(model, 64, 8, caching=False)
    runner = StepRunner(model, manager, storage)
    assert manager.admit(0, ru.random_ids(TINY_D["vocab_size"], 70, 5))
    runner.step([StepEntry(0, manager.seqs[0].tokens, [])])
    manager.commit(0, 70)
    manager.extend(0, [9])
    seen = []
    forward = model.forward

    def spy(ctx):
        seen.append((torch.cuda.is_current_stream_capturing(), dict(ctx.scratch)))
        return forward(ctx)

    model.forward = spy
    try:
        runner.step([StepEntry(0, [9], [0])])                  # the first decode step: eager run, then capture
    finally:
        model.forward = forward
    assert [capturing for capturing, _ in seen] == [False, True]
    assert seen[1][1] == {}, "the capture began with the eager run's scratch buffers"
    assert runner.graph_replays == 1


def test_multi_turn_replay_reuses_histories_and_changes_no_token(model_folders, tmp_path):
    """The multi-turn replay runner: with the prefix cache on, later turns prefill only what is new; the replies are the same."""
    from tinyserve_llm_b200.cli import multiturn
    results = {}
    for caching in ("on", "off"):
        out = tmp_path / f"{caching}.json"
        code = multiturn.main(["--model", model_folders["b"], "--conversations", "6", "--turns", "3,4", "--user-tokens", "20,60",
                               "--reply-tokens", "4,9", "--rho", "0.5", "--caching", caching, "--temperature", "0",
                               "--dtype", "float32", "--block-size", str(PAGE_B), "--max-model-len", "400",
                               "--max-num-seqs", "4", "--max-num-batched-tokens", "512", "--out", str(out)])
        assert code == 0
        results[caching] = json.loads(out.read_text())
    on, off = results["on"], results["off"]
    assert on["final_history_digests"] == off["final_history_digests"]
    assert off["summary"]["prefill_tokens"] == off["summary"]["prompt_tokens"] - off["scheduler_stats"]["cached_tokens"]
    assert on["summary"]["prefill_tokens"] < 0.7 * off["summary"]["prefill_tokens"]
    assert on["summary"]["cached_tokens"] > 0 and on["conversations"] == 6 and len(on["waves"]) >= 3
    assert abs(on["rho"] - 0.5) < 0.2
