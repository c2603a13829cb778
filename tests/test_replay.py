"""
Trace replay on the GPU against the plain implementation: the same requests whole, with the last 32
tokens decoded one by one, in portions of changing size (down to two tokens), and mixed (up to four
live requests, portions beside decoded tokens, so few pages that they are used again), in float32
and in bfloat16, for three tiny configurations that differ in every size and option.
"""

import json
import os

import pytest
import torch

import replay_util as ru
from tiny_configs import PAGE_A, PAGE_B, TINY_A, TINY_B, TINY_C, TINY_D

pytestmark = pytest.mark.gpu

RAW = {"a": TINY_A, "b": TINY_B, "c": TINY_C, "d": TINY_D}

# float32: both sides are exact up to float32 rounding of sums a few hundred terms long.
# bfloat16: the plain implementation rounds where the engine does, so what is left is the order of
# float32 accumulation and an occasional one-ulp flip (2^-8 relative) carried through the layers;
# the bound is 1.2 % of the largest logit.
FP32_TOL = dict(atol=1e-5, rtol=1e-5)


def bf16_tol(want):
    scale = max(v.abs().max().item() for v in want.values())
    return dict(atol=0.012 * scale, rtol=0.0)


def requests_for(name):
    raw = RAW[name]
    longest = raw["max_position_embeddings"] - 20
    vocab = raw["vocab_size"]
    single = {"whole": ru.random_ids(vocab, longest, 1), "tail": ru.random_ids(vocab, longest - 33, 2),
              "cut": ru.random_ids(vocab, longest - 7, 3), "short": ru.random_ids(vocab, 3, 4)}
    lengths = [150, 90, 200, 33, 120, 180, 64, 129, 65, 2]
    if longest > 800:                                   # the model with long positions: several decode splits
        lengths = [700, 90, 513, 33, 256, 180, 64, 129, 65, 2]
    mixed = {f"m{i}": ru.random_ids(vocab, n, 10 + i) for i, n in enumerate(lengths)}
    return single, mixed


def build_trace(single, mixed):
    trace = ru.Trace()
    ru.add_whole(trace, "whole", single["whole"])
    ru.add_whole(trace, "short", single["short"])
    ru.add_decode_tail(trace, "tail", single["tail"])
    ru.add_portions(trace, "cut", single["cut"], [64, 2, 3, 17, 100, 2, 31])
    ru.add_mixed(trace, mixed, seed=5)
    return trace


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_every_way_of_cutting_gives_the_plain_logits(name, dtype, model_folders, tmp_path):
    single, mixed = requests_for(name)
    trace = build_trace(single, mixed)
    assert trace.peak < sum(ru.round64(len(v)) for v in mixed.values()), "pages must be used again"
    got = ru.run_trace(model_folders[name], dtype, trace, str(tmp_path / "out"))
    want = ru.plain_logits(model_folders[name], {**single, **mixed}, dtype)
    tol = FP32_TOL if dtype == "float32" else bf16_tol(want)
    ru.compare(trace, got, want, **tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, page", [("a", PAGE_A), ("b", PAGE_B)])
def test_cached_prefixes_copies_forks_and_evicted_pages_give_the_plain_logits(name, page, dtype, model_folders, tmp_path):
    """
    Prefix reuse on: a request that attaches another's cached pages and copies part of a page, two
    that compute the same pages in one step (the second switches to the first one's at commit), a
    fork whose branches write different tokens into the page they share, and a request that comes
    again after strangers evicted some of its pages.  Every wanted row against the plain logits;
    the counters show that each path was taken.
    """
    trace, requests = ru.cached_paths_trace(RAW[name]["vocab_size"], page)
    pages = ru.smallest_pool(trace, caching=True) + 4
    predicted, reused = ru.simulate(trace, pages, caching=True)
    out = str(tmp_path / "out")
    got = ru.run_trace(model_folders[name], dtype, trace, out, max_tokens=pages * page, caching=True)
    stats = ru.read_stats(out)
    assert stats["partial_copies"] >= 1 and stats["cow_copies"] >= 1 and stats["dedupes"] >= 3 and stats["evictions"] > 0
    assert stats["reused_tokens"] == sum(reused.values()) > 6 * page
    for key in ("evictions", "cow_copies", "partial_copies", "publishes", "dedupes"):
        assert stats[key] == getattr(predicted, key), key
    want = ru.plain_logits(model_folders[name], requests, dtype)
    ru.compare(trace, got, want, **(FP32_TOL if dtype == "float32" else bf16_tol(want)))


def test_a_fork_without_prefix_reuse_still_shares_and_copies(model_folders, tmp_path):
    trace, requests = ru.cached_paths_trace(TINY_A["vocab_size"], PAGE_A)
    pages = ru.smallest_pool(trace, caching=False)
    out = str(tmp_path / "out")
    got = ru.run_trace(model_folders["a"], "float32", trace, out, max_tokens=pages * PAGE_A)
    stats = ru.read_stats(out)
    assert stats["cow_copies"] == 1 and stats["reused_tokens"] == 0 and stats["publishes"] == 0
    ru.compare(trace, got, ru.plain_logits(model_folders["a"], requests, "float32"), **FP32_TOL)


def _sharp_folder(model_folders, tmp_path, name, factor):
    """The same model with query and key projections scaled up, so that attention is peaked, not flat."""
    from safetensors.torch import load_file

    from tinyserve_llm_b200.weights import write_safetensors
    src = model_folders[name]
    tensors = load_file(os.path.join(src, "model.safetensors"))
    for key in tensors:
        if ".q_proj." in key or ".k_proj." in key:
            tensors[key] = (tensors[key].float() * factor).to(tensors[key].dtype)
    dst = str(tmp_path / f"sharp_{name}")
    os.makedirs(dst)
    write_safetensors(os.path.join(dst, "model.safetensors"), tensors)
    with open(os.path.join(dst, "config.json"), "w") as f:
        json.dump(RAW[name], f)
    return dst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_is_found(dtype, model_folders, tmp_path):
    """
    With peaked attention a repeated token makes one far key stand out for the query that repeats
    it.  The far key lies in the request's first page, the query hundreds of positions later, fed
    in another step, from pages taken over from a request that ended.
    """
    # float32 takes a strongly peaked model; in bfloat16 scores 36 times larger turn one-ulp flips
    # into other attended keys (plain bfloat16 and plain float32 then differ by most of a logit),
    # so the bfloat16 run sharpens by 2 only and keeps the usual bound
    factor = 6.0 if dtype == "float32" else 2.0
    folder = _sharp_folder(model_folders, tmp_path, "b", factor)
    vocab = TINY_B["vocab_size"]
    filler = ru.random_ids(vocab, 200, 21)
    ids = ru.random_ids(vocab, 470, 22)
    ids[5] = ids[460] = 777                           # the query at 460 meets its own token at 5
    trace = ru.Trace()
    ru.add_whole(trace, "filler", filler)             # its pages are reused by the request below
    trace.step([("far", ids[:70], [5, 69])])
    trace.step([("far", ids[70:455], [0, 384])])
    for i in range(455, 470):
        trace.step([("far", ids[i:i + 1], [0])], end=["far"] if i == 469 else [])
    got = ru.run_trace(folder, dtype, trace, str(tmp_path / "out"))
    want = ru.plain_logits(folder, {"filler": filler, "far": ids}, dtype)
    # the plain model itself must depend on the far key, or the test shows nothing
    without = list(ids)
    without[5] = (without[5] + 1) % vocab
    moved = (ru.plain_logits(folder, {"x": without}, dtype)["x"][460] - want["far"][460]).abs().max().item()
    # float32: scores are 36 times those of the unscaled model (tens, not tenths), so the float32
    # rounding of the rotated queries and keys (1e-6) reaches the softmax weights 36 times stronger;
    # the bound is wider than for the unscaled model by about that much.
    tol = dict(atol=3e-4, rtol=1e-4) if dtype == "float32" else bf16_tol(want)
    assert moved > 5 * tol["atol"], f"the far key moves the logits by only {moved}"
    ru.compare(trace, got, want, **tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_token_by_token(dtype, model_folders, tmp_path):
    """A request decoded one token at a time from its second token on, across many page edges."""
    ids = ru.random_ids(TINY_C["vocab_size"], 300, 31)
    trace = ru.Trace()
    trace.step([("long", ids[:1], [0])])
    for i in range(1, len(ids)):
        trace.step([("long", ids[i:i + 1], [0])], end=["long"] if i == len(ids) - 1 else [])
    got = ru.run_trace(model_folders["c"], dtype, trace, str(tmp_path / "out"))
    want = ru.plain_logits(model_folders["c"], {"long": ids}, dtype)
    ru.compare(trace, got, want, **(FP32_TOL if dtype == "float32" else bf16_tol(want)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_context_of_three_thousand_tokens(dtype, tmp_path):
    """
    A longer context than the other tests reach: 3,000 tokens in portions of up to 2,048, then 24 tokens decoded
    one by one beside a second, short request; a dozen decode splits, 47 pages, rotary scaling past its original
    window.  Logits of the last portion's end and of every decoded token against the plain implementation.
    """
    from tiny_configs import SEED_D, WEIGHTS
    from tinyserve_llm_b200.weights import write_random_model
    raw = dict(TINY_D, max_position_embeddings=4096)
    folder = str(tmp_path / "model")
    write_random_model(folder, raw, SEED_D, **WEIGHTS)
    ids = ru.random_ids(raw["vocab_size"], 3024, 61)
    other = ru.random_ids(raw["vocab_size"], 40, 62)
    trace = ru.Trace()
    trace.step([("long", ids[:2048], [2047])])
    trace.step([("long", ids[2048:2990], [0, 941])])
    trace.step([("long", ids[2990:3000], [9]), ("other", other[:30], [29])])
    for i in range(24):
        parts = [("long", ids[3000 + i:3001 + i], [0])]
        if i < 10:
            parts.append(("other", other[30 + i:31 + i], [0]))
        trace.step(parts, end=(["other"] if i == 9 else []) + (["long"] if i == 23 else []))
    got = ru.run_trace(folder, dtype, trace, str(tmp_path / "out"))
    want = ru.plain_logits(folder, {"long": ids, "other": other}, dtype)
    ru.compare(trace, got, want, **(FP32_TOL if dtype == "float32" else bf16_tol(want)))


def test_trace_run_is_a_program_with_the_documented_interface(model_folders, tmp_path):
    """Empty `want`, a request left out of a step, an `end` without entries, and exit code 0 at end of input."""
    ids = ru.random_ids(TINY_A["vocab_size"], 40, 41)
    other = ru.random_ids(TINY_A["vocab_size"], 9, 42)
    trace = ru.Trace()
    trace.step([("x", ids[:30], []), ("y", other[:4], [3])])
    trace.step([("y", other[4:], [4])])                       # x sits this step out
    trace.step([("x", ids[30:], [9])], end=["y"])
    trace.step([], end=["x"])
    got = ru.run_trace(model_folders["a"], "float32", trace, str(tmp_path / "out"), max_tokens=128)
    assert sorted(got) == [0, 1, 2] and not os.path.exists(tmp_path / "out" / "3.f32")
    want = ru.plain_logits(model_folders["a"], {"x": ids, "y": other}, "float32")
    ru.compare(trace, got, want, **FP32_TOL)
