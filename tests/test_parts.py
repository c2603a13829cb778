"""Each part of a block alone, built from its spec and tensors, against the plain function of the same part."""

import pytest
import torch

import plain_llama as plain
from gpu_util import DEV, make_binding, make_ctx
from tiny_configs import TINY_B, TINY_C

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def runtime(dtype):
    from tinyserve_llm_b200.ops import get_ops
    from tinyserve_llm_b200.parts.base import Runtime
    return Runtime(dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()), ops=get_ops())


def act_of(dtype):
    return "float32" if dtype == torch.float32 else "bfloat16"


def tol(dtype, scale=1.0):
    """Absolute bound relative to the size of the values compared; rtol alone would chase values near zero."""
    return dict(atol=3e-6 * scale, rtol=1e-5) if dtype == torch.float32 else dict(atol=1.5e-2 * scale, rtol=1.5e-2)


def rand(shape, seed, scale=1.0):
    return (torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale).to(torch.bfloat16)


def llama_parts(raw):
    from tinyserve_llm_b200.config import LlamaConfig, llama_model_spec
    spec = llama_model_spec(LlamaConfig.from_dict(raw))
    return spec, spec.blocks[0]


# Llama 3.2 1B's rotary settings on a small model: a table of 131,072 positions, scaled past a window of 8,192
LONG_ROPE = dict(TINY_B, head_dim=64, max_position_embeddings=131072, rope_theta=500000.0,
                 rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 8192})


@pytest.mark.parametrize("raw", [TINY_B, TINY_C, LONG_ROPE], ids=["b", "c", "llama-3.2-1b-rope"])
def test_rotary_table_equals_the_plain_angles(raw):
    from tinyserve_llm_b200.parts.base import part_class
    _, block = llama_parts(raw)
    rotary = part_class("position", block.mixer.position)(block.mixer.position, {}, runtime(torch.float32))
    last = raw["max_position_embeddings"] - 1
    positions = torch.tensor(sorted({0, 1, 63, 64, 65, last // 16, last // 16 + 1, last // 2 + 1, last}))
    cos, sin = plain.rope_cos_sin(raw, positions)
    half = block.mixer.head_dim // 2
    table = rotary.table.cpu()[positions]
    assert table.dtype == torch.float32 and rotary.table.shape == (raw["max_position_embeddings"], 2 * half)
    assert torch.equal(table[:, :half].double(), cos) and torch.equal(table[:, half:].double(), sin)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from tinyserve_llm_b200.config.spec import RMSNormSpec
    from tinyserve_llm_b200.parts.base import part_class
    spec = RMSNormSpec(size=200, eps=3e-4)
    w = (1 + rand((200,), 1, 0.3).float()).to(torch.bfloat16)
    norm = part_class("norm", spec)(spec, {"weight": w}, runtime(dtype))
    x, res = rand((6, 200), 2, 2.0), rand((6, 200), 3, 2.0)
    want, want_res = plain.add_rms_norm(x.double(), res.double(), w.double(), 3e-4, act_of(dtype))
    got, got_res = norm.forward(x.to(DEV, dtype), res.to(DEV, dtype))
    torch.testing.assert_close(got.cpu().double(), want, **tol(dtype, 4))
    torch.testing.assert_close(got_res.cpu().double(), want_res, **tol(dtype, 8))


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    from tinyserve_llm_b200.config.spec import GatedMLPSpec
    from tinyserve_llm_b200.parts.base import part_class
    spec = GatedMLPSpec(hidden_size=72, intermediate_size=200, activation="silu")
    cls = part_class("feed_forward", spec)
    tensors = {n: rand(d.shape, 10 + i, 0.1) for i, (n, d) in enumerate(cls.declare(spec).items())}
    mlp = cls(spec, tensors, runtime(dtype))
    x = rand((9, 72), 4)
    want = plain.mlp_block({"mlp." + k: v.double() for k, v in tensors.items()}, x.double(), act_of(dtype))
    got = mlp.forward(x.to(DEV, dtype), None)
    torch.testing.assert_close(got.cpu().double(), want, **tol(dtype, 0.5))
    with pytest.raises(NotImplementedError, match="gelu"):
        cls(GatedMLPSpec(hidden_size=72, intermediate_size=200, activation="gelu"), tensors, runtime(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("raw", [TINY_B, TINY_C])
def test_attention_part_in_two_steps(raw, dtype):
    """The mixer alone: a prefix in one step, the rest in a second one, against whole-sequence plain attention."""
    from tinyserve_llm_b200.parts.base import part_class
    _, block = llama_parts(raw)
    spec = block.mixer
    cls = part_class("mixer", spec)
    tensors = {n: rand(d.shape, 20 + i, 0.08) for i, (n, d) in enumerate(cls.declare(spec).items())}
    mixer = cls(spec, tensors, runtime(dtype))
    assert mixer.kv_need().num_kv_heads == spec.num_kv_heads and mixer.state_bytes() == 0
    total, first, page = 45, 29, 16
    x = rand((total, spec.hidden_size), 5)
    binding = make_binding(5, 1, spec.num_kv_heads, page, spec.head_dim, dtype, [[4, 1, 3]])
    got = []
    for q_len, ctx_len in ((first, first), (total - first, total)):
        ctx = make_ctx([q_len], [ctx_len])
        got.append(mixer.forward(x[ctx_len - q_len:ctx_len].to(DEV, dtype), ctx, binding).cpu().double())
    want, _ = plain.attention_block(raw, {"self_attn." + k: v.double() for k, v in tensors.items()}, x.double(),
                                    torch.arange(total), act_of(dtype))
    torch.testing.assert_close(torch.cat(got), want, **tol(dtype, 0.5))


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_arrangement(dtype):
    """A whole pre-norm block: the adds are deferred into the next norm, the first block starts the stream."""
    from tinyserve_llm_b200.parts.base import arrangement_class
    _, block = llama_parts(TINY_B)
    cls = arrangement_class(block.arrangement)
    decl = cls.declare(block)
    assert set(decl) == {"input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight",
                         "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                         "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"}
    tensors = {n: (1 + rand(d.shape, 40 + i, 0.2).float()).to(torch.bfloat16) if d.init == "unit"
               else rand(d.shape, 40 + i, 0.08) for i, (n, d) in enumerate(decl.items())}
    built = cls(block, tensors, runtime(dtype))
    T, act, eps = 20, act_of(dtype), TINY_B["rms_norm_eps"]
    x = rand((T, TINY_B["hidden_size"]), 6)
    spec = block.mixer
    binding = make_binding(2, 1, spec.num_kv_heads, 32, spec.head_dim, dtype, [[1]])
    ctx = make_ctx([T], [T])
    w = {k: v.double() for k, v in tensors.items()}
    # first block of a model: no residual yet
    out, res = built.forward(x.to(DEV, dtype), None, ctx, binding)
    n = plain.rms_norm(x.double(), w["input_layernorm.weight"], eps, act)
    a, _ = plain.attention_block(TINY_B, w, n, torch.arange(T), act)
    n2, want_res = plain.add_rms_norm(a, x.double(), w["post_attention_layernorm.weight"], eps, act)
    want = plain.mlp_block(w, n2, act)
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype, want.abs().max().item()))
    torch.testing.assert_close(res.cpu().double(), want_res, **tol(dtype, 4))
    # a later block: the incoming branch output is added to the stream inside the first norm
    res_in = rand((T, TINY_B["hidden_size"]), 7)
    out, res = built.forward(x.to(DEV, dtype), res_in.to(DEV, dtype), ctx, binding)
    n, r1 = plain.add_rms_norm(x.double(), res_in.double(), w["input_layernorm.weight"], eps, act)
    a, _ = plain.attention_block(TINY_B, w, n, torch.arange(T), act)
    n2, want_res = plain.add_rms_norm(a, r1, w["post_attention_layernorm.weight"], eps, act)
    want = plain.mlp_block(w, n2, act)
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype, want.abs().max().item()))
    torch.testing.assert_close(res.cpu().double(), want_res, **tol(dtype, 8))


def test_unknown_parts_are_refused_by_name():
    from tinyserve_llm_b200.config.spec import PartSpec
    from tinyserve_llm_b200.parts.base import arrangement_class, part_class

    class Other(PartSpec):
        pass
    other = Other()
    object.__setattr__(other, "kind", "hyena")
    with pytest.raises(NotImplementedError, match="hyena"):
        part_class("mixer", other)
    with pytest.raises(NotImplementedError, match="sandwich"):
        arrangement_class("sandwich")
