"""
Generality of the parts: a toy mixer with fixed-size per-request state of its own is defined here,
registered, built into a model beside attention layers and stepped through the engine (portions,
decoding, several requests, a fork) without any change to the framework's files.  The run list of
that model also names a block twice and lets one execution read the cache another one wrote.
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
