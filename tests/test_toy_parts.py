"""
Generality of the parts: a toy mixer with fixed-size per-request state of its own is defined here,
registered, built into a model beside attention layers and stepped through the engine (portions,
decoding, several requests, a fork) without any change to the framework's files.  The run list of
that model also names a block twice and lets one execution read the cache another one wrote.
Further down: layers with a window in a layer group of their own, and two more toy parts, a
feed-forward with routing and a position encoding that edits q and k itself.
"""

from dataclasses import dataclass, field

import pytest
import torch

pytestmark = pytest.mark.gpu

HIDDEN, HEADS, KV, HD, INTER, VOCAB = 48, 3, 1, 16, 80, 101


def build_toy():
    from tinyserve_llm_b200.config.spec import (AttentionSpec, BlockSpec, GatedMLPSpec, ModelSpec, PartSpec,
                                                RMSNormSpec, RotarySpec, RunEntry)
    from tinyserve_llm_b200.parts.base import Mixer, TensorDecl, register_part

    @dataclass(frozen=True)
    class DecaySpec(PartSpec):
        kind: str = field(init=False, default="toy_decay")
        hidden_size: int = 0
        decay: float = 0.9

    @register_part("mixer", "toy_decay")
    class DecayMixer(Mixer):
        """y_t = W s_t with s_t = decay * s_{t-1} + x_t: the state s is the request's fixed-size slot."""

        @classmethod
        def declare(cls, spec):
            return {"mix.weight": TensorDecl((spec.hidden_size, spec.hidden_size))}

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            self.weight = tensors["mix.weight"].to(rt.device, torch.float32)

        def state_bytes(self):
            return self.spec.hidden_size * 4

        def forward(self, x, ctx, binding):
            out = torch.empty_like(x)
            state = binding.state.view(torch.float32)               # [slots, hidden]
            for s, slot in enumerate(ctx.host.state_slots):
                a, b = ctx.host.cu_q[s], ctx.host.cu_q[s + 1]
                cur = state[slot].clone()
                for t in range(a, b):
                    cur = self.spec.decay * cur + x[t].float()
                    out[t] = (self.weight @ cur).to(x.dtype)
                state[slot] = cur
            return out

    rotary = RotarySpec(head_dim=HD, theta=1000.0, max_positions=128)
    attn = AttentionSpec(hidden_size=HIDDEN, num_heads=HEADS, num_kv_heads=KV, head_dim=HD, scale=HD ** -0.5,
                         position=rotary)
    mlp = GatedMLPSpec(hidden_size=HIDDEN, intermediate_size=INTER)
    norm = RMSNormSpec(size=HIDDEN, eps=1e-5)
    blocks = (
        BlockSpec("pre_norm", attn, mlp, norm, norm, prefix="layers.0."),
        BlockSpec("pre_norm", DecaySpec(hidden_size=HIDDEN, decay=0.8), mlp, norm, norm, prefix="layers.1.",
                  mixer_prefix="decay."),
        BlockSpec("pre_norm", attn, mlp, norm, norm, prefix="layers.2."),
    )
    # block 0 runs twice (shared weights, caches 0 and 3), block 2 reads the cache entry block 0 wrote first
    run = (RunEntry(0, 0), RunEntry(1, 1), RunEntry(2, 0, writes_cache=False), RunEntry(0, 3))
    spec = ModelSpec("ToyForTests", VOCAB, HIDDEN, blocks, run, norm, "embed.weight", "final_norm.", None, 128, -1)
    return spec, DecaySpec


def plain_toy(tensors, ids):
    """The toy model over a whole sequence in float64, from tests/plain_llama.py's part functions."""
    import plain_llama as plain
    cfg = {"num_attention_heads": HEADS, "num_key_value_heads": KV, "head_dim": HD, "hidden_size": HIDDEN,
           "rope_theta": 1000.0, "max_position_embeddings": 128}
    w = {k: v.double() for k, v in tensors.items()}
    positions = torch.arange(len(ids))
    x, residual = w["embed.weight"][torch.tensor(ids)], None
    caches = {}
    for block, entry, writes in ((0, 0, True), (1, 1, True), (2, 0, False), (0, 3, True)):
        p = f"layers.{block}."
        lw = {k[len(p):]: v for k, v in w.items() if k.startswith(p)}
        if residual is None:
            n, residual = plain.rms_norm(x, lw["input_layernorm.weight"], 1e-5, "float32"), x
        else:
            n, residual = plain.add_rms_norm(x, residual, lw["input_layernorm.weight"], 1e-5, "float32")
        if block == 1:
            state, rows = torch.zeros(HIDDEN, dtype=torch.float64), []
            for t in range(len(ids)):
                state = 0.8 * state + n[t]
                rows.append(lw["decay.mix.weight"] @ state)
            a = torch.stack(rows)
        else:
            a, kv = plain.attention_block(cfg, lw, n, positions, "float32", None if writes else caches[entry])
            if writes:
                caches[entry] = kv
        n, residual = plain.add_rms_norm(a, residual, lw["post_attention_layernorm.weight"], 1e-5, "float32")
        x = plain.mlp_block(lw, n, "float32")
    h, _ = plain.add_rms_norm(x, residual, w["final_norm.weight"], 1e-5, "float32")
    return h @ w["embed.weight"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    from tinyserve_llm_b200.engine.loading import build_cache
    from tinyserve_llm_b200.engine.step import StepEntry, StepRunner
    from tinyserve_llm_b200.ops import get_ops
    from tinyserve_llm_b200.parts.base import Runtime
    from tinyserve_llm_b200.parts.model import DecoderModel, declared_tensors
    from tinyserve_llm_b200.weights import random_tensors

    spec, _ = build_toy()
    declared = declared_tensors(spec)
    assert "layers.1.decay.mix.weight" in declared and "layers.0.self_attn.q_proj.weight" in declared
    tensors = dict(random_tensors(declared, 7, std=0.08, unit_std=0.2))
    device = torch.device("cuda", torch.cuda.current_device())
    model = DecoderModel(spec, {k: v.to(device) for k, v in tensors.items()},
                         Runtime(dtype=torch.float32, device=device, ops=get_ops()))
    assert not model.graph_safe                                    # the toy runs host code per request
    needs = model.cache_needs()
    assert [n[1] for n in needs] == [0, HIDDEN * 4, 0, 0] and needs[1][0] is None and needs[2][0] is None
    layout, manager, storage = build_cache(model, 16, 12, num_state_slots=4)
    assert [g.entries for g in layout.groups] == [(0, 3)] and not manager.caching
    runner = StepRunner(model, manager, storage)

    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, VOCAB, (50,), generator=g).tolist()
    b = torch.randint(0, VOCAB, (21,), generator=g).tolist()
    want_a, want_b = plain_toy(tensors, a), plain_toy(tensors, b)

    def feed(parts):
        entries = []
        for name, tokens in parts:
            if name in manager.seqs:
                manager.extend(name, tokens)
            else:
                assert manager.admit(name, tokens)
            entries.append(StepEntry(name, tokens, list(range(len(tokens)))))
        logits = runner.step(entries).cpu().double()
        for e in entries:
            manager.commit(e.seq_id, len(e.tokens))
        return logits

    got_a = [feed([("a", a[:20])])]                                # a alone, then a and b side by side
    both = feed([("a", a[20:37]), ("b", b[:9])])
    got_a.append(both[:17])
    got_b = [both[17:]]
    both = feed([("b", b[9:10]), ("a", a[37:38])])                 # single tokens of both
    got_b.append(both[:1]), got_a.append(both[1:])
    manager.fork("b", "b2")                                        # the fork gets a copy of b's state
    both = feed([("b", b[10:]), ("a", a[38:]), ("b2", b[10:])])
    got_b.append(both[:11]), got_a.append(both[11:23])
    torch.testing.assert_close(torch.cat(got_a), want_a, atol=2e-5, rtol=1e-5)
    torch.testing.assert_close(torch.cat(got_b), want_b, atol=2e-5, rtol=1e-5)
    torch.testing.assert_close(both[23:], want_b[10:], atol=2e-5, rtol=1e-5)
    for name in ("a", "b", "b2"):
        manager.release(name)
    assert manager.stats().pages_in_use == 0 and manager.free_state_slots() == 4


def test_run_list_mistakes_are_refused():
    from tinyserve_llm_b200.config.spec import RunEntry
    from tinyserve_llm_b200.ops import get_ops
    from tinyserve_llm_b200.parts.base import Runtime
    from tinyserve_llm_b200.parts.model import DecoderModel, declared_tensors
    from tinyserve_llm_b200.weights import random_tensors
    import dataclasses

    spec, _ = build_toy()
    device = torch.device("cuda", torch.cuda.current_device())
    tensors = {k: v.to(device) for k, v in random_tensors(declared_tensors(spec), 7)}
    rt = Runtime(dtype=torch.float32, device=device, ops=get_ops())
    for run, needle in (((RunEntry(2, 0, writes_cache=False), RunEntry(0, 0)), "before anything wrote"),
                        ((RunEntry(0, 0), RunEntry(2, 0)), "written by run entries"),
                        ((RunEntry(7, 0),), "names block 7")):
        with pytest.raises(ValueError, match=needle):
            DecoderModel(dataclasses.replace(spec, run=run), tensors, rt)


@pytest.mark.parametrize("dtype, hd, page", [(torch.float32, 16, 16), (torch.bfloat16, 64, 64)])
def test_window_layers_have_pages_of_their_own_and_give_them_back(dtype, hd, page):
    """
    A toy model whose second layer sees only the last `window` keys: its cache entry lands in a layer
    group of its own, whose pages are given back as the window passes and are taken again, while the
    full-attention layer keeps all of its pages.  Logits equal the plain implementation with the
    same window, in portions that cross the window's edge and token by token.
    """
    import plain_llama as plain
    from tinyserve_llm_b200.config.spec import (AttentionSpec, BlockSpec, GatedMLPSpec, ModelSpec, RMSNormSpec,
                                                RotarySpec, RunEntry)
    from tinyserve_llm_b200.engine.loading import build_cache
    from tinyserve_llm_b200.engine.step import StepEntry, StepRunner
    from tinyserve_llm_b200.ops import get_ops
    from tinyserve_llm_b200.parts.base import Runtime
    from tinyserve_llm_b200.parts.model import DecoderModel, declared_tensors
    from tinyserve_llm_b200.weights import random_tensors

    hidden, heads, kv, inter, vocab, window, length = 64, 2, 1, 96, 97, 40, 5 * page + 9
    rotary = RotarySpec(head_dim=hd, theta=10000.0, max_positions=512)
    full = AttentionSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=hd, scale=hd ** -0.5, position=rotary)
    local = AttentionSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=hd, scale=hd ** -0.5, window=window,
                          position=rotary)
    mlp, norm = GatedMLPSpec(hidden_size=hidden, intermediate_size=inter), RMSNormSpec(size=hidden, eps=1e-5)
    blocks = (BlockSpec("pre_norm", full, mlp, norm, norm, prefix="layers.0."),
              BlockSpec("pre_norm", local, mlp, norm, norm, prefix="layers.1."))
    spec = ModelSpec("ToyWindow", vocab, hidden, blocks, (RunEntry(0, 0), RunEntry(1, 1)), norm, "embed.weight",
                     "final_norm.", None, 512, -1)
    tensors = dict(random_tensors(declared_tensors(spec), 3, std=0.08, unit_std=0.2))
    device = torch.device("cuda", torch.cuda.current_device())
    model = DecoderModel(spec, {k: v.to(device) for k, v in tensors.items()}, Runtime(dtype=dtype, device=device, ops=get_ops()))
    pages_full = -(-length // page) + 1
    layout, manager, storage = build_cache(model, page, pages_full)
    assert [(g.entries, g.window) for g in layout.groups] == [((0,), 0), ((1,), window)] and not manager.caching
    runner = StepRunner(model, manager, storage)

    ids = torch.randint(0, vocab, (length,), generator=torch.Generator().manual_seed(5)).tolist()
    act = "float32" if dtype == torch.float32 else "bfloat16"
    cfg = {"num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": hd, "hidden_size": hidden,
           "rope_theta": 10000.0, "max_position_embeddings": 512}
    w = {k: v.double() for k, v in tensors.items()}
    x, residual = plain.rnd(w["embed.weight"][torch.tensor(ids)], act), None
    for layer, win in ((0, 0), (1, window)):
        lw = {k[len(f"layers.{layer}."):]: v for k, v in w.items() if k.startswith(f"layers.{layer}.")}
        if residual is None:
            n, residual = plain.rms_norm(x, lw["input_layernorm.weight"], 1e-5, act), x
        else:
            n, residual = plain.add_rms_norm(x, residual, lw["input_layernorm.weight"], 1e-5, act)
        a, _ = plain.attention_block(cfg, lw, n, torch.arange(length), act, None, win)
        n, residual = plain.add_rms_norm(a, residual, lw["post_attention_layernorm.weight"], 1e-5, act)
        x = plain.mlp_block(lw, n, act)
    want = plain.add_rms_norm(x, residual, w["final_norm.weight"], 1e-5, act)[0] @ w["embed.weight"].T

    got, pos = [], 0
    for n in [window - 3, 2, page + 1, 1, 1, 30, 1] + [1] * 400:
        n = min(n, length - pos)
        if n == 0:
            break
        tokens = ids[pos:pos + n]
        if "w" in manager.seqs:
            manager.extend("w", tokens)
        else:
            assert manager.admit("w", tokens)
        got.append(runner.step([StepEntry("w", tokens, list(range(n)))]).cpu().double())
        manager.commit("w", n)
        pos += n
    tolerance = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.012 * want.abs().max().item(), rtol=0.0)
    torch.testing.assert_close(torch.cat(got), want, **tolerance)
    table_full, table_local = manager.block_table("w", 0), manager.block_table("w", 1)
    assert all(p >= 0 for p in table_full) and len(table_full) == -(-length // page)
    passed = (length - window + 1) // page
    assert table_local[:passed] == [-1] * passed and all(p >= 0 for p in table_local[passed:])
    assert manager.counters.window_releases == passed
    assert manager.available_pages()[1] > manager.available_pages()[0]
    manager.release("w")
    assert manager.stats().pages_in_use == 0


def test_toy_routed_feed_forward_and_toy_position_encoding_are_registered_built_and_stepped():
    """
    Two more toy parts, defined here and nowhere in the framework: a feed-forward that routes each
    token to two of three experts (router logits and softmax in float32), and a position encoding
    that rotates adjacent pairs of dims and so edits q and k itself instead of handing the kernels a
    table.  A model with one layer of each beside a stock layer is stepped in portions and token by
    token, two requests side by side, and equals a float64 calculation of the same formulas.
    """
    import plain_llama as plain
    from tinyserve_llm_b200.config.spec import (AttentionSpec, BlockSpec, GatedMLPSpec, ModelSpec, PartSpec,
                                                RMSNormSpec, RotarySpec, RunEntry)
    from tinyserve_llm_b200.engine.loading import build_cache
    from tinyserve_llm_b200.engine.step import StepEntry, StepRunner
    from tinyserve_llm_b200.ops import get_ops
    from tinyserve_llm_b200.parts.base import FeedForward, PositionEncoding, Runtime, TensorDecl, register_part
    from tinyserve_llm_b200.parts.model import DecoderModel, declared_tensors
    from tinyserve_llm_b200.weights import random_tensors

    hidden, heads, kv, hd, inter, vocab, experts, base = 64, 4, 2, 16, 48, 89, 3, 500.0

    @dataclass(frozen=True)
    class RoutedSpec(PartSpec):
        kind: str = field(init=False, default="toy_routed")
        hidden_size: int = 0
        intermediate_size: int = 0
        num_experts: int = 0
        top_k: int = 1

    @register_part("feed_forward", "toy_routed")
    class RoutedFeedForward(FeedForward):
        @classmethod
        def declare(cls, spec):
            out = {"router.weight": TensorDecl((spec.num_experts, spec.hidden_size))}
            for e in range(spec.num_experts):
                out[f"experts.{e}.up.weight"] = TensorDecl((spec.intermediate_size, spec.hidden_size))
                out[f"experts.{e}.down.weight"] = TensorDecl((spec.hidden_size, spec.intermediate_size))
            return out

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            self.router = tensors["router.weight"].to(rt.device, torch.float32)
            self.up = [tensors[f"experts.{e}.up.weight"].to(rt.device, rt.dtype) for e in range(spec.num_experts)]
            self.down = [tensors[f"experts.{e}.down.weight"].to(rt.device, rt.dtype) for e in range(spec.num_experts)]

        def forward(self, x, ctx):
            probs = torch.softmax(x.float() @ self.router.T, dim=-1)
            top, chosen = probs.topk(self.spec.top_k, dim=-1)
            top = top / top.sum(-1, keepdim=True)
            out = torch.zeros_like(x, dtype=torch.float32)
            for e in range(self.spec.num_experts):
                weight = (top * (chosen == e)).sum(-1, keepdim=True)          # 0 for tokens not routed to e
                out += weight * (torch.relu(x @ self.up[e].T) @ self.down[e].T).float()
            return out.to(x.dtype)

    @dataclass(frozen=True)
    class PairRotarySpec(PartSpec):
        kind: str = field(init=False, default="toy_pair_rotary")
        head_dim: int = 0
        base: float = 10000.0

    @register_part("position", "toy_pair_rotary")
    class PairRotary(PositionEncoding):
        """Rotates dims (2i, 2i+1) of every head by position * base^(-2i / head_dim); no table for the kernels."""

        def apply(self, q, k, ctx):
            hd_ = self.spec.head_dim
            inv = self.spec.base ** (-torch.arange(0, hd_, 2, device=q.device, dtype=torch.float32) / hd_)
            ang = ctx.positions.float()[:, None] * inv[None, :]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            for t in (q, k):
                v = t.view(t.shape[0], -1, hd_ // 2, 2).float()
                a, b = v[..., 0].clone(), v[..., 1].clone()
                v2 = torch.stack((a * cos - b * sin, b * cos + a * sin), dim=-1)
                t.copy_(v2.view(t.shape[0], -1).to(t.dtype))

    rotary = RotarySpec(head_dim=hd, theta=1000.0, max_positions=256)
    attn = AttentionSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=hd, scale=hd ** -0.5, position=rotary)
    attn_pairs = AttentionSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=hd, scale=hd ** -0.5,
                               position=PairRotarySpec(head_dim=hd, base=base))
    mlp, norm = GatedMLPSpec(hidden_size=hidden, intermediate_size=inter), RMSNormSpec(size=hidden, eps=1e-5)
    routed = RoutedSpec(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=2)
    blocks = (BlockSpec("pre_norm", attn_pairs, routed, norm, norm, prefix="layers.0.", feed_forward_prefix="moe."),
              BlockSpec("pre_norm", attn, mlp, norm, norm, prefix="layers.1."))
    spec = ModelSpec("ToyRouted", vocab, hidden, blocks, (RunEntry(0, 0), RunEntry(1, 1)), norm, "embed.weight",
                     "final_norm.", None, 256, -1)
    declared = declared_tensors(spec)
    assert "layers.0.moe.router.weight" in declared and "layers.0.moe.experts.2.down.weight" in declared
    tensors = dict(random_tensors(declared, 11, std=0.1, unit_std=0.2))
    device = torch.device("cuda", torch.cuda.current_device())
    model = DecoderModel(spec, {k: v.to(device) for k, v in tensors.items()},
                         Runtime(dtype=torch.float32, device=device, ops=get_ops()))
    assert not model.graph_safe
    layout, manager, storage = build_cache(model, 16, 16)
    runner = StepRunner(model, manager, storage)

    def plain_logits(ids):
        w = {k: v.double() for k, v in tensors.items()}
        T, positions = len(ids), torch.arange(len(ids))
        x, residual = w["embed.weight"][torch.tensor(ids)], None
        # layer 0: pair rotary + routed feed-forward
        lw = {k[len("layers.0."):]: v for k, v in w.items() if k.startswith("layers.0.")}
        n, residual = plain.rms_norm(x, lw["input_layernorm.weight"], 1e-5, "float32"), x
        inv = base ** (-torch.arange(0, hd, 2, dtype=torch.float64) / hd)
        ang = positions.double()[:, None] * inv[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

        def rotate(t):
            v = t.view(T, -1, hd // 2, 2)
            return torch.stack((v[..., 0] * cos - v[..., 1] * sin, v[..., 1] * cos + v[..., 0] * sin), dim=-1).view(T, -1, hd)

        q = rotate(plain.linear(n, lw["self_attn.q_proj.weight"], "float32"))
        k = rotate(plain.linear(n, lw["self_attn.k_proj.weight"], "float32"))
        v = plain.linear(n, lw["self_attn.v_proj.weight"], "float32").view(T, kv, hd)
        o = plain.causal_attention(q, k, v, hd ** -0.5, "float32", 0).reshape(T, heads * hd)
        a = plain.linear(o, lw["self_attn.o_proj.weight"], "float32")
        n, residual = plain.add_rms_norm(a, residual, lw["post_attention_layernorm.weight"], 1e-5, "float32")
        probs = torch.softmax(n @ lw["moe.router.weight"].T, dim=-1)
        top, chosen = probs.topk(2, dim=-1)
        top = top / top.sum(-1, keepdim=True)
        x = torch.zeros_like(n)
        for e in range(experts):
            weight = (top * (chosen == e)).sum(-1, keepdim=True)
            x += weight * (torch.relu(n @ lw[f"moe.experts.{e}.up.weight"].T) @ lw[f"moe.experts.{e}.down.weight"].T)
        # layer 1: the stock parts
        lw = {k[len("layers.1."):]: v for k, v in w.items() if k.startswith("layers.1.")}
        cfg = {"num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": hd, "hidden_size": hidden,
               "rope_theta": 1000.0, "max_position_embeddings": 256}
        n, residual = plain.add_rms_norm(x, residual, lw["input_layernorm.weight"], 1e-5, "float32")
        a, _ = plain.attention_block(cfg, lw, n, positions, "float32")
        n, residual = plain.add_rms_norm(a, residual, lw["post_attention_layernorm.weight"], 1e-5, "float32")
        x = plain.mlp_block(lw, n, "float32")
        return plain.add_rms_norm(x, residual, w["final_norm.weight"], 1e-5, "float32")[0] @ w["embed.weight"].T

    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, vocab, (45,), generator=g).tolist()
    b = torch.randint(0, vocab, (30,), generator=g).tolist()

    def feed(parts):
        entries = []
        for name, tokens in parts:
            if name in manager.seqs:
                manager.extend(name, tokens)
            else:
                assert manager.admit(name, tokens)
            entries.append(StepEntry(name, tokens, list(range(len(tokens)))))
        logits = runner.step(entries).cpu().double()
        for e in entries:
            manager.commit(e.seq_id, len(e.tokens))
        return logits

    got_a = [feed([("a", a[:17])])]
    both = feed([("a", a[17:19]), ("b", b[:20])])                  # two tokens of a beside a portion of b
    got_a.append(both[:2])
    got_b = [both[2:]]
    for i in range(10):                                            # token by token, side by side
        both = feed([("b", b[20 + i:21 + i]), ("a", a[19 + i:20 + i])])
        got_b.append(both[:1]), got_a.append(both[1:])
    got_a.append(feed([("a", a[29:])]))
    torch.testing.assert_close(torch.cat(got_a), plain_logits(a), atol=3e-5, rtol=1e-5)
    torch.testing.assert_close(torch.cat(got_b), plain_logits(b), atol=3e-5, rtol=1e-5)
    manager.release("a"), manager.release("b")
    assert manager.stats().pages_in_use == 0


def test_a_toy_norm_brings_a_cuda_kernel_of_its_own():
    """
    A toy norm whose arithmetic runs in a CUDA kernel that lives beside this test (tests/toy_kernels.cu),
    not in the framework: the part compiles it as an extension of the kernel library, registers its
    launcher and calls it through `Ops.call`; it is graph safe, so decode steps of the model built
    from it are replayed from CUDA graphs.  No file of the framework names the kernel.
    """
    import os

    import plain_llama as plain
    from tinyserve_llm_b200.config.spec import (AttentionSpec, BlockSpec, GatedMLPSpec, ModelSpec, PartSpec,
                                                RMSNormSpec, RotarySpec, RunEntry)
    from tinyserve_llm_b200.engine.loading import build_cache
    from tinyserve_llm_b200.engine.step import StepEntry, StepRunner
    from tinyserve_llm_b200.ops import KernelError, get_ops
    from tinyserve_llm_b200.parts.base import Norm, Runtime, TensorDecl, register_part
    from tinyserve_llm_b200.parts.model import DecoderModel, declared_tensors
    from tinyserve_llm_b200.weights import random_tensors

    hidden, heads, kv, hd, inter, vocab, shift = 64, 4, 2, 16, 48, 97, 0.125
    source = os.path.join(os.path.dirname(os.path.abspath(__file__)), "toy_kernels.cu")

    @dataclass(frozen=True)
    class GainSpec(PartSpec):
        kind: str = field(init=False, default="toy_gain")
        size: int = 0
        shift: float = 0.0

    @register_part("norm", "toy_gain")
    class GainNorm(Norm):
        """(x + residual) * gain + shift, no statistics: the sum is the new residual stream."""

        graph_safe = True

        @classmethod
        def declare(cls, spec):
            return {"gain": TensorDecl((spec.size,), init="unit")}

        def __init__(self, spec, tensors, rt):
            super().__init__(spec, tensors, rt)
            self.gain = tensors["gain"].to(rt.device, torch.float32).contiguous()
            rt.ops.load_extension("toy", [source], {"toy_gain": ("int", "ppfpiip")})

        def forward(self, x, residual, rows=None):
            s = x if residual is None else x + residual
            picked = s if rows is None else s.index_select(0, rows.long())
            out = torch.empty_like(picked)
            self.rt.ops.call("toy_gain", picked.data_ptr(), self.gain.data_ptr(), self.spec.shift, out.data_ptr(),
                             picked.shape[0], picked.shape[1], self.rt.ops.stream())
            return out, s

    rotary = RotarySpec(head_dim=hd, theta=1000.0, max_positions=128)
    attn = AttentionSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=hd, scale=hd ** -0.5, position=rotary)
    mlp, rms = GatedMLPSpec(hidden_size=hidden, intermediate_size=inter), RMSNormSpec(size=hidden, eps=1e-5)
    gain = GainSpec(size=hidden, shift=shift)
    blocks = (BlockSpec("pre_norm", attn, mlp, rms, gain, prefix="layers.0."),)
    spec = ModelSpec("ToyGain", vocab, hidden, blocks, (RunEntry(0, 0),), rms, "embed.weight", "final_norm.", None, 128, -1)
    tensors = dict(random_tensors(declared_tensors(spec), 13, std=0.1, unit_std=0.2))
    device = torch.device("cuda", torch.cuda.current_device())
    ops = get_ops()
    model = DecoderModel(spec, {k: v.to(device) for k, v in tensors.items()}, Runtime(dtype=torch.float32, device=device, ops=ops))
    assert model.graph_safe and ops.calls.get("toy_gain", 0) == 0
    _, manager, storage = build_cache(model, 16, 8)
    runner = StepRunner(model, manager, storage)

    def plain_logits(ids):
        w = {k: v.double() for k, v in tensors.items()}
        lw = {k[len("layers.0."):]: v for k, v in w.items() if k.startswith("layers.0.")}
        cfg = {"num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": hd, "hidden_size": hidden,
               "rope_theta": 1000.0, "max_position_embeddings": 128}
        x = w["embed.weight"][torch.tensor(ids)]
        n, residual = plain.rms_norm(x, lw["input_layernorm.weight"], 1e-5, "float32"), x
        a, _ = plain.attention_block(cfg, lw, n, torch.arange(len(ids)), "float32")
        residual = a + residual
        x = plain.mlp_block(lw, residual * lw["post_attention_layernorm.gain"] + shift, "float32")
        return plain.add_rms_norm(x, residual, w["final_norm.weight"], 1e-5, "float32")[0] @ w["embed.weight"].T

    ids = torch.randint(0, vocab, (40,), generator=torch.Generator().manual_seed(3)).tolist()
    got = []
    assert manager.admit("r", ids[:25])
    got.append(runner.step([StepEntry("r", ids[:25], list(range(25)))]).cpu().double())
    manager.commit("r", 25)
    for t in ids[25:]:                                              # token by token: replayed from a CUDA graph
        manager.extend("r", [t])
        got.append(runner.step([StepEntry("r", [t], [0])]).cpu().double().clone())
        manager.commit("r", 1)
    torch.testing.assert_close(torch.cat(got), plain_logits(ids), atol=3e-5, rtol=1e-5)
    assert runner.graph_replays == 15 and ops.calls["toy_gain"] >= 2
    with pytest.raises(KernelError, match="toy_gain: bad sizes"):   # the extension reports errors like the library does
        ops.call("toy_gain", 0, 0, 0.0, 0, 1, 0, ops.stream())
    with pytest.raises(KernelError, match="not a registered kernel"):
        ops.call("toy_unknown", 0)
    manager.release("r")
