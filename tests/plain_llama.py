"""
A plain, slow Llama: whole sequences, no cache, one function for each part, float64 arithmetic.

It is written from the formulas of tejkas/tinyserve-llm's model code (each function cites the file
and lines, paths relative to that project) and shares no code with the engine: it reads the model
folder with the `safetensors` package and `json`, and computes with plain torch tensor arithmetic on
the CPU.  tests/golden/ holds logits that tinyserve-llm's own LlamaForCausalLM produced for two
tiny random models; tests/test_plain.py checks this file against them.

`act` is the activation dtype being imitated: "float32" computes everything in float64 without any
rounding (the reference a true 32-bit engine is judged against); "bfloat16" rounds to bfloat16
wherever the reference's bfloat16 model materialises a tensor, and is otherwise float64.
"""

from __future__ import annotations

import json
import math
import os

import torch
from safetensors import safe_open

F64 = torch.float64


# ----------------------------------------------------------------------------- reading
def read_model_folder(model_dir: str) -> tuple[dict, dict[str, torch.Tensor]]:
    """config.json as a dict and every tensor of model*.safetensors as float64 (values unchanged)."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors: dict[str, torch.Tensor] = {}
    for name in sorted(os.listdir(model_dir)):
        if name.startswith("model") and name.endswith(".safetensors"):
            with safe_open(os.path.join(model_dir, name), "pt", "cpu") as f:
                for key in f.keys():
                    tensors[key] = f.get_tensor(key).to(F64)
    return cfg, tensors


def head_dim_of(cfg: dict) -> int:
    # model/llama.py:197 -- head_dim, or hidden_size // num_attention_heads when absent
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def rope_settings(cfg: dict) -> tuple[float, dict | None]:
    # model/llama.py:86-104 -- rope_parameters (with its own rope_theta) or top-level rope_theta + rope_scaling
    params = cfg.get("rope_parameters")
    if params:
        theta, scaling = params.get("rope_theta", cfg.get("rope_theta", 10000.0)), params
    else:
        theta, scaling = cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling")
    if scaling is not None:
        kind = scaling.get("rope_type", scaling.get("type", "default"))
        if kind == "default":
            scaling = None
        elif kind != "llama3":
            raise NotImplementedError(kind)
    return float(theta), scaling


# ----------------------------------------------------------------------------- rounding
def rnd(x: torch.Tensor, act: str) -> torch.Tensor:
    """Round to the imitated activation dtype and come back to float64."""
    if act == "bfloat16":
        return x.to(torch.float32).to(torch.bfloat16).to(F64)
    assert act == "float32"
    return x


# ----------------------------------------------------------------------------- parts
def rope_inv_freq(cfg: dict) -> torch.Tensor:
    """float32 [head_dim/2].  model/llama.py:148 (base frequencies) and :107-128 (llama3 rescaling)."""
    hd = head_dim_of(cfg)
    theta, scaling = rope_settings(cfg)
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    if scaling is None:
        return inv
    orig = scaling.get("original_max_position_embeddings", cfg["max_position_embeddings"])
    factor, lo, hi = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
    out = torch.empty_like(inv)
    for i in range(inv.numel()):                      # element by element, as the formulas read
        f = inv[i]
        wavelen = 2 * math.pi / f
        scaled = f / factor if wavelen > orig / lo else f
        smooth = (orig / wavelen - lo) / (hi - lo)
        mid = (1 - smooth) * scaled / factor + smooth * scaled
        medium = (not wavelen < orig / hi) and (not wavelen > orig / lo)
        out[i] = mid if medium else scaled
    return out


def rope_cos_sin(cfg: dict, positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """cos, sin [T, head_dim/2]; angles are float32 products as in model/llama.py:157-160."""
    angles = positions.to(torch.float32)[:, None] * rope_inv_freq(cfg)[None, :]
    return angles.cos().to(F64), angles.sin().to(F64)


def rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, act: str) -> torch.Tensor:
    """x [T, heads, hd]; dim i pairs with dim i + hd/2.  model/llama.py:131-136."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return rnd(torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1), act)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, act: str) -> torch.Tensor:
    """model/llama.py:52-58: normalise in high precision, round, then multiply by the weight."""
    y = x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return rnd(rnd(y, act) * weight, act)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                 act: str) -> tuple[torch.Tensor, torch.Tensor]:
    """model/llama.py:60-67: the norm sees the unrounded sum, the carried residual is the rounded sum."""
    s = x + residual
    y = s * torch.rsqrt(s.pow(2).mean(dim=-1, keepdim=True) + eps)
    return rnd(rnd(y, act) * weight, act), rnd(s, act)


def linear(x: torch.Tensor, weight: torch.Tensor, act: str) -> torch.Tensor:
    """y = x W^T, no bias (model/llama.py:172-186, :200-201); the product is rounded once."""
    return rnd(x @ weight.T, act)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, act: str,
                     window: int = 0) -> torch.Tensor:
    """
    One whole sequence: q [T, nh, hd], k, v [T, nkv, hd] -> [T, nh, hd].
    model/attention.py:43-56 and attention/torch_paged.py:36-45: kv head j serves query heads
    j*g..(j+1)*g-1; scores * scale; query t sees keys 0..t; softmax in high precision.
    `window` > 0 keeps only the last `window` keys (the query's own included); Llama uses 0.
    """
    T, nh, hd = q.shape
    g = nh // k.shape[1]
    out = torch.empty_like(q)
    pos = torch.arange(T)
    hidden = pos[None, :] > pos[:, None]
    if window > 0:
        hidden = hidden | (pos[None, :] <= pos[:, None] - window)
    for h in range(nh):
        scores = (q[:, h] @ k[:, h // g].T) * scale
        scores = scores.masked_fill(hidden, float("-inf"))
        out[:, h] = torch.softmax(scores, dim=-1) @ v[:, h // g]
    return rnd(out, act)


def swiglu(gate_up: torch.Tensor, act: str) -> torch.Tensor:
    """model/llama.py:80-83: columns [gate | up]; silu(gate) is rounded, then the product is."""
    gate, up = gate_up.chunk(2, dim=-1)
    return rnd(rnd(gate * torch.sigmoid(gate), act) * up, act)


# ----------------------------------------------------------------------------- model
def layer_tensors(tensors: dict[str, torch.Tensor], i: int) -> dict[str, torch.Tensor]:
    p = f"model.layers.{i}."
    return {k[len(p):]: v for k, v in tensors.items() if k.startswith(p)}


def attention_block(cfg: dict, w: dict[str, torch.Tensor], n: torch.Tensor, positions: torch.Tensor, act: str,
                    shared_kv: tuple[torch.Tensor, torch.Tensor] | None = None, window: int = 0):
    """model/llama.py:204-212.  Returns (projected output, (k, v) as cached)."""
    nh, nkv, hd = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"], \
        head_dim_of(cfg)
    T = n.shape[0]
    cos, sin = rope_cos_sin(cfg, positions)
    q = rotate_half(linear(n, w["self_attn.q_proj.weight"], act).view(T, nh, hd), cos, sin, act)
    if shared_kv is None:
        k = rotate_half(linear(n, w["self_attn.k_proj.weight"], act).view(T, nkv, hd), cos, sin, act)
        v = linear(n, w["self_attn.v_proj.weight"], act).view(T, nkv, hd)
    else:
        k, v = shared_kv
    o = causal_attention(q, k, v, hd ** -0.5, act, window)
    return linear(o.reshape(T, nh * hd), w["self_attn.o_proj.weight"], act), (k, v)


def mlp_block(w: dict[str, torch.Tensor], n: torch.Tensor, act: str) -> torch.Tensor:
    """model/llama.py:215-225."""
    gate_up = torch.cat((linear(n, w["mlp.gate_proj.weight"], act), linear(n, w["mlp.up_proj.weight"], act)), dim=-1)
    return linear(swiglu(gate_up, act), w["mlp.down_proj.weight"], act)


def hidden_states(cfg: dict, tensors: dict[str, torch.Tensor], ids: list[int], act: str = "float32",
                  run: list[tuple[int, int, bool]] | None = None) -> torch.Tensor:
    """
    Final normalised hidden states [T, H] of one whole sequence.  model/llama.py:270-276 (model) and
    :238-253 (layer: the add is deferred into the next norm; layer 0's input is the first residual).
    `run` lists (layer, cache entry, writes) executions; None is every layer once, in order.
    """
    eps = cfg["rms_norm_eps"]
    positions = torch.arange(len(ids))
    if run is None:
        run = [(i, i, True) for i in range(cfg["num_hidden_layers"])]
    x = rnd(tensors["model.embed_tokens.weight"][torch.tensor(ids)], act)
    residual = None
    caches: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
    for layer, entry, writes in run:
        w = layer_tensors(tensors, layer)
        if residual is None:
            n, residual = rms_norm(x, w["input_layernorm.weight"], eps, act), x
        else:
            n, residual = add_rms_norm(x, residual, w["input_layernorm.weight"], eps, act)
        a, kv = attention_block(cfg, w, n, positions, act, None if writes else caches[entry])
        if writes:
            caches[entry] = kv
        n, residual = add_rms_norm(a, residual, w["post_attention_layernorm.weight"], eps, act)
        x = mlp_block(w, n, act)
    h, _ = add_rms_norm(x, residual, tensors["model.norm.weight"], eps, act)
    return h


def logits(cfg: dict, tensors: dict[str, torch.Tensor], ids: list[int], act: str = "float32",
           run: list[tuple[int, int, bool]] | None = None, rows: list[int] | None = None) -> torch.Tensor:
    """
    [T, vocab] float64 ([len(rows), vocab] with `rows`).  model/llama.py:293-304: lm_head, tied to the
    embedding when the config says so; engine/model_runner.py:126-127 projects chosen rows only.
    """
    h = hidden_states(cfg, tensors, ids, act, run)
    if rows is not None:
        h = h[torch.tensor(rows, dtype=torch.int64)]
    w = tensors["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else tensors["lm_head.weight"]
    return h @ w.T


def greedy_generate(cfg: dict, tensors: dict[str, torch.Tensor], prompt: list[int], num_tokens: int,
                    act: str = "float32", eos: int = -1) -> list[int]:
    """engine/sampler.py:14 (argmax) over engine/llm_engine.py:159-168: recompute the whole sequence each token."""
    ids, out = list(prompt), []
    for _ in range(num_tokens):
        token = int(torch.argmax(logits(cfg, tensors, ids, act)[-1]))
        out.append(token)
        ids.append(token)
        if token == eos:
            break
    return out


def sampling_distribution(logit_row: torch.Tensor, temperature: float) -> torch.Tensor:
    """engine/sampler.py:16-17: the distribution a draw at `temperature` > 0 follows."""
    return torch.softmax(logit_row.to(F64) / temperature, dim=-1)
