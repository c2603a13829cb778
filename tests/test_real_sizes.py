"""
Replay at the layer sizes of Llama 3.2 1B (two layers of its sixteen), float32 and bfloat16, against
the plain implementation: the routes only these sizes take (256-token pages, the tcgen05 gate/up
product from 512 rows, the library product from 33 rows, the vocabulary projection over 128,256
columns with float32 output, the tcgen05 prompt attention, rotary scaling with factor 32 over an
8,192-token window) run inside the whole model here, not only as kernels alone.
"""

import pytest

import plain_llama as plain
import replay_util as ru

pytestmark = pytest.mark.gpu

LAYERS = 2
LLAMA_1B_TWO_LAYERS = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048,
    "intermediate_size": 8192, "num_hidden_layers": LAYERS, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "hidden_act": "silu", "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "tie_word_embeddings": True,
}
PAGE = 256


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    from tinyserve_llm_b200.weights import write_random_model
    path = str(tmp_path_factory.mktemp("llama_1b_sizes_2_layers"))
    write_random_model(path, LLAMA_1B_TWO_LAYERS, 7, std=0.02, unit_std=0.1)
    return path


@pytest.fixture(scope="module")
def workload():
    """A 2,100-token request: 2,048 tokens in one portion, then 20, then 32 single tokens beside a second request of 300."""
    vocab = LLAMA_1B_TWO_LAYERS["vocab_size"]
    big, small = ru.random_ids(vocab, 2100, 81), ru.random_ids(vocab, 300, 82)
    trace = ru.Trace(PAGE)
    trace.step([("big", big[:2048], [0, 1000, 2047])])
    trace.step([("big", big[2048:2068], [0, 19])])
    trace.step([("big", big[2068:2069], [0]), ("small", small[:268], [0, 267])])
    for i in range(1, 32):
        trace.step([("big", big[2068 + i:2069 + i], [0]), ("small", small[267 + i:268 + i], [0])],
                   end=["big"] if i == 31 else [])
    trace.step([("small", small[299:], [0])], end=["small"])
    return trace, {"big": big, "small": small}


@pytest.fixture(scope="module")
def plain_rows(folder, workload):
    """Plain logits of the wanted rows only (the float64 vocabulary projection of 2,100 rows would take minutes)."""
    trace, requests = workload
    cfg, tensors = plain.read_model_folder(folder)
    rows = {name: sorted({pos for wanted in trace.expect.values() for n, pos in wanted if n == name}) for name in requests}

    def compute(act):
        out = {}
        for name, ids in requests.items():
            out[name] = _Rows(rows[name], plain.logits(cfg, tensors, ids, act, rows=rows[name]))
        return out
    return compute


class _Rows:
    """Logits of some rows, indexed by position like the full matrix."""

    def __init__(self, rows, values):
        self.at = {r: i for i, r in enumerate(rows)}
        self.values = values

    def __getitem__(self, pos):
        return self.values[self.at[pos]]

    def abs(self):
        return self.values.abs()


def test_float32_at_llama_1b_layer_sizes_two_layers(folder, workload, plain_rows, tmp_path):
    """
    The true 32-bit path.  Tolerance: the engine sums in float32, the plain code in float64.  A sum
    of K products in ascending order carries a rounding error of about sqrt(K) * 2^-24 of its
    magnitude (K = 8,192 for the down projection: 5e-6), a row passes through eight such products in
    two layers and the vocabulary projection, and the norms rescale rows to unit size in between;
    so errors of up to about sqrt(9) * 5e-6 = 1.5e-5 of the largest logit can be expected (measured
    on a B200: 4e-6 of it), and the bound is 2e-5 of it, as an absolute tolerance.  The tiny models,
    whose sums have at most 512 terms, keep atol = rtol = 1e-5.
    """
    trace, requests = workload
    out = str(tmp_path / "out")
    got = ru.run_trace(folder, "float32", trace, out, max_tokens=trace.peak)
    want = plain_rows("float32")
    scale = max(v.abs().max().item() for v in want.values())
    worst = ru.compare(trace, got, want, atol=2e-5 * scale, rtol=0.0)
    print(f"float32 at 1B sizes: largest difference {worst:.3g}, largest logit {scale:.3g}")
    calls = ru.read_stats(out)["kernel_calls"]
    assert calls.get("ts_sgemm_nt", 0) >= (4 * LAYERS + 1) * 4 and "library_mm" not in calls   # decode steps replay graphs
    assert "ts_gemm_tcgen05" not in calls and "ts_skinny_linear" not in calls


def test_bfloat16_at_llama_1b_layer_sizes_two_layers(folder, workload, plain_rows, tmp_path):
    trace, requests = workload
    out = str(tmp_path / "out")
    got = ru.run_trace(folder, "bfloat16", trace, out, max_tokens=trace.peak)
    want = plain_rows("bfloat16")
    scale = max(v.abs().max().item() for v in want.values())
    worst = ru.compare(trace, got, want, atol=0.012 * scale, rtol=0.0)
    print(f"bfloat16 at 1B sizes: largest difference {worst:.3g}, largest logit {scale:.3g}")
    stats = ru.read_stats(out)
    calls = stats["kernel_calls"]
    # the routes that only these sizes take
    assert calls.get("ts_gemm_tcgen05", 0) >= LAYERS                    # gate/up with SwiGLU, 2,048 rows
    assert calls.get("ts_prefill_attention_tcgen05", 0) >= 3 * LAYERS   # the three steps with a prompt portion
    assert calls.get("library_mm", 0) >= 3 * LAYERS                     # q/k/v, output and down products of 2,048 and 268 rows
    assert calls.get("ts_skinny_linear:float32_out", 0) >= 1            # vocabulary projection of a few rows, float32 out
    assert calls.get("ts_skinny_qkv_rope_store", 0) >= LAYERS           # decode steps: projection, rotation and cache write fused
    assert stats["graph_replays"] >= 30                                 # the single-token steps ran from CUDA graphs
