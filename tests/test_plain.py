"""The plain implementation (tests/plain_llama.py) against tinyserve-llm's own outputs in tests/golden/."""

import json
import os

import numpy as np
import pytest
import torch

import plain_llama as plain
from tinyserve_llm_b200.weights import write_random_model

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _golden(name):
    with open(os.path.join(GOLDEN, f"golden_{name}.json")) as f:
        record = json.load(f)
    return record, np.load(os.path.join(GOLDEN, f"golden_{name}_logits.npy"))


@pytest.fixture(scope="module", params=["a", "b"])
def case(request, tmp_path_factory):
    record, logits = _golden(request.param)
    folder = str(tmp_path_factory.mktemp(f"golden_{request.param}"))
    write_random_model(folder, record["config"], record["seed"], store_dtype=record["store_dtype"],
                       **record["weights"])
    cfg, tensors = plain.read_model_folder(folder)
    return record, logits, cfg, tensors


def test_inv_freq_is_bit_equal(case):
    record, _, cfg, _ = case
    ours = [float(x).hex() for x in plain.rope_inv_freq(cfg).tolist()]
    assert ours == record["inv_freq_hex"]


def test_logits_match_reference_model(case):
    record, golden, cfg, tensors = case
    ours = plain.logits(cfg, tensors, record["ids"])[record["rows"]]
    # the golden logits are float32 products of float32 tensors; ours are float64
    torch.testing.assert_close(ours.float(), torch.from_numpy(golden), rtol=1e-5, atol=1e-5)


def test_greedy_generation_matches_reference_engine(case):
    record, _, cfg, tensors = case
    for prompt, want in zip(record["prompts"], record["greedy"]):
        assert plain.greedy_generate(cfg, tensors, prompt, len(want)) == want


def test_scaling_changes_some_frequencies_only():
    from tiny_configs import TINY_B
    scaled = plain.rope_inv_freq(TINY_B)
    unscaled = plain.rope_inv_freq({**TINY_B, "rope_scaling": None})
    changed = ~torch.isclose(scaled, unscaled)
    assert changed.any() and not changed.all()


def test_rounding_modes():
    x = torch.tensor([1.0 + 2 ** -10], dtype=torch.float64)
    assert plain.rnd(x, "float32").item() == x.item()
    assert plain.rnd(x, "bfloat16").item() == 1.0


def test_window_masks_far_keys():
    torch.manual_seed(0)
    q, k, v = (torch.randn(9, 2, 4, dtype=torch.float64) for _ in range(3))
    full = plain.causal_attention(q, k, v, 0.5, "float32")
    win = plain.causal_attention(q, k, v, 0.5, "float32", window=3)
    torch.testing.assert_close(full[:3], win[:3])          # the first three queries see everything either way
    assert not torch.allclose(full[5:], win[5:])
    short = plain.causal_attention(q[2:5], k[2:5], v[2:5], 0.5, "float32")
    torch.testing.assert_close(win[4], short[2])           # query 4 with window 3 sees keys 2, 3, 4


def test_bfloat16_rounding_places_are_those_of_the_reference_parts():
    """
    Where the plain implementation rounds in bfloat16 mode, against what tinyserve-llm's own modules
    gave in bfloat16 for the same inputs (golden_parts_bf16.npz), bit for bit: the norm rounds before
    the weight multiplies and carries the rounded sum, silu is rounded before it multiplies, the
    rotation is rounded once.
    """
    g = np.load(os.path.join(GOLDEN, "golden_parts_bf16.npz"))
    t = lambda key: torch.from_numpy(g[key]).to(plain.F64)       # noqa: E731
    eps = float(g["eps"])
    assert torch.equal(plain.rms_norm(t("x"), t("weight"), eps, "bfloat16"), t("rms_norm"))
    normed, carried = plain.add_rms_norm(t("x"), t("residual"), t("weight"), eps, "bfloat16")
    assert torch.equal(normed, t("add_rms_norm")) and torch.equal(carried, t("carried"))
    assert torch.equal(plain.swiglu(t("gate_up"), "bfloat16"), t("swiglu"))
    cos, sin = t("cos")[:, 0, :], t("sin")[:, 0, :]
    assert torch.equal(plain.rotate_half(t("q"), cos, sin, "bfloat16"), t("rotated"))
    # the test has teeth: a rounding moved by one place changes some element
    unrounded_silu = plain.rnd(t("gate_up").chunk(2, -1)[0] * torch.sigmoid(t("gate_up").chunk(2, -1)[0])
                               * t("gate_up").chunk(2, -1)[1], "bfloat16")
    assert not torch.equal(unrounded_silu, t("swiglu"))
    s = t("x") + t("residual")
    late = plain.rnd(s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * t("weight"), "bfloat16")
    assert not torch.equal(late, t("add_rms_norm"))
