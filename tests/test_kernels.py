"""
Each CUDA kernel alone against a plain float64 reference of the same operation, at sizes other than
the tiny models' (widths and vocabularies that are no power of two, head sizes in steps of 16, odd
groups), with cache pools poisoned with NaN so that a read of a slot nobody wrote shows.
"""

import math

import pytest
import torch

import plain_llama as plain
from gpu_util import DEV, fill_cache, i32, make_binding, make_ctx

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from tinyserve_llm_b200.ops import get_ops
    return get_ops()


def act_of(dtype):
    return "float32" if dtype == torch.float32 else "bfloat16"


def tol(dtype, scale=1.0):
    return dict(atol=2e-6 * scale, rtol=2e-6) if dtype == torch.float32 else dict(atol=1e-2 * scale, rtol=1e-2)


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, vocab", [(64, 10), (200, 1001), (4104, 37)])
def test_embedding(ops, dtype, hidden, vocab):
    table = rand((vocab, hidden), dtype, 1)
    ids = [0, vocab - 1, 3, 3, -1, vocab // 2]
    out = ops.embedding(table.to(DEV), i32(ids)).cpu()
    for row, i in zip(out, ids):
        assert torch.equal(row, table[i] if i >= 0 else torch.zeros(hidden, dtype=dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [5, 300])                     # a few rows: a CTA a row; many: rows held in registers
@pytest.mark.parametrize("hidden, eps", [(48, 1e-5), (777, 1e-6), (4096, 1e-3), (13000, 1e-5), (3072, 1e-5), (8192, 1e-6)])
def test_add_rmsnorm(ops, dtype, hidden, eps, rows):
    act = act_of(dtype)
    x, res, w = rand((rows, hidden), dtype, 1, 3.0), rand((rows, hidden), dtype, 2, 3.0), (1 + rand((hidden,), dtype, 3, 0.3))
    w = w.to(dtype)
    want, want_res = plain.add_rms_norm(x.double(), res.double(), w.double(), eps, act)
    xd, rd = x.to(DEV), res.to(DEV)
    got, got_res = ops.add_rmsnorm(xd, rd, w.to(DEV), eps)
    assert got.data_ptr() == xd.data_ptr() and got_res.data_ptr() == rd.data_ptr()      # in place
    torch.testing.assert_close(got.cpu().double(), want, **tol(dtype, 4))
    torch.testing.assert_close(got_res.cpu().double(), want_res, **tol(dtype, 8))
    # no residual: x starts the stream and is left untouched
    xd = x.to(DEV)
    got, stream = ops.add_rmsnorm(xd, None, w.to(DEV), eps)
    assert stream.data_ptr() == xd.data_ptr() and torch.equal(xd.cpu(), x)
    torch.testing.assert_close(got.cpu().double(), plain.rms_norm(x.double(), w.double(), eps, act), **tol(dtype, 4))
    # chosen rows only, compact output, inputs untouched
    xd, rd = x.to(DEV), res.to(DEV)
    got, _ = ops.add_rmsnorm(xd, rd, w.to(DEV), eps, i32([4, 0, 4]))
    torch.testing.assert_close(got.cpu().double(), want[[4, 0, 4]], **tol(dtype, 4))
    assert torch.equal(xd.cpu(), x) and torch.equal(rd.cpu(), res)
    if rows > 256:                                             # many chosen rows, some twice, some padding (-1: left alone)
        pick = [(7 * i) % rows for i in range(290)] + [-1, 3]
        got, _ = ops.add_rmsnorm(xd, rd, w.to(DEV), eps, i32(pick))
        keep = [i for i, p in enumerate(pick) if p >= 0]
        torch.testing.assert_close(got.cpu().double()[keep], want[[pick[i] for i in keep]], **tol(dtype, 4))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [6, 300])
@pytest.mark.parametrize("hidden, vocab", [(48, 11), (2048, 1000), (777, 37)])
def test_first_norm_gathers_the_embedding_rows_itself(ops, dtype, rows, hidden, vocab):
    """One kernel for the embedding gather and the model's first norm: bit for bit what the two kernels give; an id outside the table is a row of zeros."""
    table, w = rand((vocab, hidden), dtype, 5, 2.0).to(DEV), (1 + rand((hidden,), dtype, 6, 0.3)).to(dtype).to(DEV)
    ids = torch.randint(0, vocab, (rows,), generator=torch.Generator().manual_seed(7)).tolist()
    ids[1], ids[-1] = -1, vocab + 3
    got, stream = ops.embed_rmsnorm(table, i32(ids), w, 1e-5)
    rows_of = ops.embedding(table, i32(ids))
    assert torch.equal(stream, rows_of) and torch.equal(stream[1], torch.zeros_like(stream[1]))
    want, _ = ops.add_rmsnorm(rows_of.clone(), None, w, 1e-5)
    assert torch.equal(got, want)
    ok = [i for i, t in enumerate(ids) if 0 <= t < vocab]
    ref = plain.rms_norm(table.cpu().double()[[ids[i] for i in ok]], w.cpu().double(), 1e-5, act_of(dtype))
    torch.testing.assert_close(got.cpu().double()[ok], ref, **tol(dtype, 4))


def test_add_rmsnorm_keeps_a_float32_weight_beside_bfloat16_rows(ops):
    x, res = rand((3, 96), torch.bfloat16, 1), rand((3, 96), torch.bfloat16, 2)
    w = 1 + rand((96,), torch.float32, 3, 0.3)
    s = x.double() + res.double()
    y = plain.rnd(s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5), "bfloat16")
    want = plain.rnd(y * w.double(), "bfloat16")
    got, _ = ops.add_rmsnorm(x.to(DEV), res.to(DEV), w.to(DEV), 1e-5)
    torch.testing.assert_close(got.cpu().double(), want, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, inter", [(1, 16), (7, 1000), (130, 5504)])
def test_silu_mul(ops, dtype, tokens, inter):
    gu = rand((tokens, 2 * inter), dtype, 4, 2.0)
    got = ops.silu_mul(gu.to(DEV)).cpu().double()
    torch.testing.assert_close(got, plain.swiglu(gu.double(), act_of(dtype)), **tol(dtype, 4))


@pytest.mark.parametrize("m, n, k", [(1, 1, 1), (3, 130, 70), (65, 64, 17), (200, 1000, 192), (128, 257, 1024)])
def test_float32_matrix_product(ops, m, n, k):
    from tinyserve_llm_b200.ops.library import KernelError
    x, w = rand((m, k), torch.float32, 5), rand((n, k), torch.float32, 6)
    got = ops.linear(x.to(DEV), w.to(DEV)).cpu().double()
    torch.testing.assert_close(got, x.double() @ w.double().T, atol=1e-6 * math.sqrt(k) * 4, rtol=1e-6)
    # a row's result does not depend on the rows beside it
    alone = ops.linear(x[:1].contiguous().to(DEV), w.to(DEV)).cpu()
    assert torch.equal(alone[0], ops.linear(x.to(DEV), w.to(DEV)).cpu()[0])
    with pytest.raises(KernelError):
        ops.linear(x.to(DEV), rand((n, k + 1), torch.float32, 7).to(DEV))


@pytest.mark.parametrize("m, n, k", [(1, 48, 64), (9, 1000, 192), (300, 250, 520)])
def test_bfloat16_matrix_product(ops, m, n, k):
    x, w = rand((m, k), torch.bfloat16, 5), rand((n, k), torch.bfloat16, 6)
    want = x.double() @ w.double().T
    got = ops.linear(x.to(DEV), w.to(DEV)).cpu().double()
    torch.testing.assert_close(got, plain.rnd(want, "bfloat16"), atol=2e-2 * math.sqrt(k) / 8, rtol=1e-2)
    wide = ops.linear(x.to(DEV), w.to(DEV), out_dtype=torch.float32).cpu().double()
    torch.testing.assert_close(wide, want, atol=1e-3 * math.sqrt(k), rtol=1e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh, nkv, hd, rot, page", [(4, 2, 16, 16, 4), (6, 2, 32, 32, 32), (5, 1, 48, 48, 64),
                                                     (3, 3, 64, 32, 16), (8, 2, 128, 128, 256), (2, 1, 48, 24, 8)])
def test_rope_store(ops, dtype, nh, nkv, hd, rot, page):
    """q is rotated in place; k rotated and v raw land in the slots the block table names, nowhere else."""
    act = act_of(dtype)
    q_lens, ctx_lens = [3, 1, 5], [3, page + 2, 2 * page + 1]
    ctx = make_ctx(q_lens, ctx_lens)
    tables = [[7], [2, 9], [5, 0, 3]]
    binding = make_binding(10, 2, nkv, page, hd, dtype, tables, entry=1)
    T = ctx.num_tokens
    qkv = rand((T, (nh + 2 * nkv) * hd), dtype, 8)
    g = torch.Generator().manual_seed(9)
    angles = torch.rand((3 * page + 8, rot // 2), generator=g) * 6.0
    table = torch.cat((angles.cos(), angles.sin()), dim=-1).float()
    dev_qkv = qkv.to(DEV)
    ops.rope_store(dev_qkv, ctx, binding, table.to(DEV), nh, nkv, hd)
    positions = ctx.positions.cpu().long()
    cos, sin = table[positions, : rot // 2].double(), table[positions, rot // 2:].double()

    def rotate(x):                                     # [T, heads, hd]; dims past `rot` pass through
        out = x.double().clone()
        out[..., :rot] = plain.rotate_half(x.double()[..., :rot], cos, sin, act)
        return out

    q = qkv[:, : nh * hd].view(T, nh, hd)
    k = qkv[:, nh * hd: (nh + nkv) * hd].view(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)
    got_q = dev_qkv.cpu()[:, : nh * hd].view(T, nh, hd).double()
    torch.testing.assert_close(got_q, rotate(q), **tol(dtype, 4))
    want_k, expected_slots = rotate(k), set()
    kp, vp = binding.k_pool.cpu(), binding.v_pool.cpu()
    for t in range(T):
        s, pos = int(ctx.seq_of_token[t]), int(positions[t])
        pg, off = tables[s][pos // page], pos % page
        expected_slots.add((pg, off))
        torch.testing.assert_close(kp[pg, 1, :, off].double(), want_k[t], **tol(dtype, 4))
        assert torch.equal(vp[pg, 1, :, off], v[t])
    written = {(p, o) for p in range(10) for o in range(page) if not torch.isnan(kp[p, 1, :, o].float()).all()}
    assert written == expected_slots, "a slot outside the block table was written"
    assert torch.isnan(kp[:, 0].float()).all(), "the other cache entry of the group was touched"


@pytest.mark.parametrize("nh, nkv, hd, page, hidden", [(4, 2, 16, 4, 64), (6, 2, 32, 32, 96), (5, 1, 48, 64, 160),
                                                       (32, 8, 64, 16, 256), (8, 2, 128, 256, 512)])
@pytest.mark.parametrize("q_lens, ctx_lens", [([1, 1, 1], [3, 70, 600]), ([3, 1, 5], [3, 66, 513]),
                                              ([1] * 17, list(range(5, 22))), ([20, 12], [20, 300])])
def test_projection_with_rotation_and_cache_write_in_its_epilogue(ops, nh, nkv, hd, page, hidden, q_lens, ctx_lens):
    """The fused kernel for steps of a few tokens leaves exactly what the product and the rotary + store kernels leave."""
    ctx = make_ctx(q_lens, ctx_lens)
    pages_of = [-(-c // page) for c in ctx_lens]
    order = torch.randperm(sum(pages_of) + 3, generator=torch.Generator().manual_seed(3)).tolist()
    tables, used = [], 0
    for n in pages_of:
        tables.append(order[used:used + n])
        used += n
    T = ctx.num_tokens
    x = rand((T, hidden), torch.bfloat16, 21).to(DEV)
    w = rand(((nh + 2 * nkv) * hd, hidden), torch.bfloat16, 22, 0.1).to(DEV)
    angles = torch.rand((max(ctx_lens) + 8, hd // 2), generator=torch.Generator().manual_seed(9)) * 6.0
    table = torch.cat((angles.cos(), angles.sin()), dim=-1).float().to(DEV)
    for use_table in (table, None):
        apart = make_binding(len(order), 2, nkv, page, hd, torch.bfloat16, tables, entry=1)
        fused = make_binding(len(order), 2, nkv, page, hd, torch.bfloat16, tables, entry=1)
        want = ops.linear(x, w)
        ops.rope_store(want, ctx, apart, use_table, nh, nkv, hd)
        got = ops.linear_rope_store(x, w, ctx, fused, use_table, nh, nkv, hd)
        assert got is not None, "the fused kernel takes up to 32 tokens of any head size in steps of 16"
        assert torch.equal(got[:, : nh * hd], want[:, : nh * hd])
        for a, b in ((apart.k_pool, fused.k_pool), (apart.v_pool, fused.v_pool)):
            assert torch.equal(torch.isnan(a.float()), torch.isnan(b.float())), "other slots were written"
            assert torch.equal(torch.nan_to_num(a.float()), torch.nan_to_num(b.float()))
    # more tokens than the decode product takes: the caller falls back to the two kernels
    many = rand((ops.skinny_max_rows + 1, hidden), torch.bfloat16, 23).to(DEV)
    assert ops.linear_rope_store(many, w, ctx, fused, table, nh, nkv, hd) is None


def plain_paged_attention(q, keys, values, ctx_lens, q_lens, scale, window):
    """q [T, nh, hd] float64; keys/values per sequence [ctx, nkv, hd]: whole-sequence attention, last q_len rows kept."""
    outs = []
    start = 0
    for s, (c, n) in enumerate(zip(ctx_lens, q_lens)):
        full_q = torch.zeros((c, q.shape[1], q.shape[2]), dtype=torch.float64)
        full_q[c - n:] = q[start:start + n]
        outs.append(plain.causal_attention(full_q, keys[s].double(), values[s].double(), scale, "float32", window)[c - n:])
        start += n
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("nh, nkv, hd, page, window", [
    (4, 2, 16, 4, 0), (6, 2, 32, 32, 0), (5, 1, 48, 64, 0), (8, 8, 64, 16, 0), (3, 1, 80, 8, 0),
    (12, 4, 128, 256, 0), (2, 1, 256, 32, 0), (6, 3, 32, 8, 5), (4, 1, 64, 16, 40),
    # sizes the tensor-core kernels take in bfloat16: head 64 or 128, pages of a multiple of 64
    (8, 2, 64, 64, 0), (32, 8, 64, 256, 0), (6, 2, 128, 64, 0), (5, 5, 64, 128, 0), (16, 1, 128, 128, 0),
    (4, 1, 64, 64, 40), (8, 2, 128, 128, 300), (6, 3, 64, 64, 1)])
def test_paged_attention(ops, dtype, generic, nh, nkv, hd, page, window):
    """
    A whole prompt, a portion over a cached prefix, a decode over a long context and a single first
    token in one batch, pages scattered and out of order; one score is made to stand out.
    `generic` forces the generic kernel where the tensor-core kernels would be chosen.
    """
    if generic and not (dtype == torch.bfloat16 and hd in (64, 128) and page % 64 == 0):
        pytest.skip("the generic kernel is what runs for these sizes anyway")
    q_lens = [page + 3, 7, 1, 1]
    ctx_lens = [page + 3, 3 * page + 5, 2 * page + 1, 1]
    ctx = make_ctx(q_lens, ctx_lens)
    pages_needed = [-(-c // page) for c in ctx_lens]
    order = torch.randperm(sum(pages_needed) + 3, generator=torch.Generator().manual_seed(3)).tolist()
    tables, at = [], 0
    for n in pages_needed:
        tables.append(order[at:at + n])
        at += n
    binding = make_binding(len(order), 1, nkv, page, hd, dtype, tables)
    keys = [rand((c, nkv, hd), dtype, 20 + s) for s, c in enumerate(ctx_lens)]
    values = [rand((c, nkv, hd), dtype, 30 + s) for s, c in enumerate(ctx_lens)]
    T = ctx.num_tokens
    qkv = rand((T, (nh + 2 * nkv) * hd), dtype, 11)
    # the decode query of sequence 2 and one far key agree strongly: that key must dominate its row
    far = 1 if window == 0 else ctx_lens[2] - min(window, ctx_lens[2])
    row = q_lens[0] + q_lens[1]
    qkv[row, :hd] = (keys[2][far, 0].float() * 4).to(dtype)
    for s in range(len(ctx_lens)):
        fill_cache(binding, s, keys[s], values[s])
    scale = hd ** -0.5
    got = ops.paged_attention(qkv.to(DEV), ctx, binding, nh, nkv, hd, scale, window, generic=generic)
    got = got.cpu().double().view(T, nh, hd)
    q = qkv[:, : nh * hd].view(T, nh, hd).double()
    want = plain_paged_attention(q, keys, values, ctx_lens, q_lens, scale, window)
    assert torch.isfinite(got).all(), "a slot nobody wrote was read"
    torch.testing.assert_close(got, plain.rnd(want, act_of(dtype)), **tol(dtype, 2))


@pytest.mark.parametrize("hd, g", [(64, 4), (128, 3)])
def test_tensor_core_attention_on_long_batches(ops, hd, g):
    """Decode over many splits (contexts up to 2,300 keys), prompts of several tiles, and a decode-only batch."""
    nkv, page = 2, 128
    nh = nkv * g
    for q_lens, ctx_lens in (([1, 1, 1, 1, 1], [2300, 1, 255, 256, 257]), ([200, 1, 130, 64], [200, 900, 1000, 64])):
        ctx = make_ctx(q_lens, ctx_lens)
        tables, at = [], 0
        for c in ctx_lens:
            n = -(-c // page)
            tables.append(list(range(at + n - 1, at - 1, -1)))          # pages in descending order
            at += n
        binding = make_binding(at + 1, 1, nkv, page, hd, torch.bfloat16, tables)
        keys = [rand((c, nkv, hd), torch.bfloat16, 40 + s) for s, c in enumerate(ctx_lens)]
        values = [rand((c, nkv, hd), torch.bfloat16, 50 + s) for s, c in enumerate(ctx_lens)]
        for s in range(len(ctx_lens)):
            fill_cache(binding, s, keys[s], values[s])
        T = ctx.num_tokens
        qkv = rand((T, (nh + 2 * nkv) * hd), torch.bfloat16, 12)
        qkv[0, :hd] = (keys[0][3, 0].float() * 3).to(torch.bfloat16)   # row 0 attends to its key 3 above all
        scale = hd ** -0.5
        got = ops.paged_attention(qkv.to(DEV), ctx, binding, nh, nkv, hd, scale, 0).cpu().double().view(T, nh, hd)
        want = plain_paged_attention(qkv[:, : nh * hd].view(T, nh, hd).double(), keys, values, ctx_lens, q_lens, scale, 0)
        assert torch.isfinite(got).all()
        torch.testing.assert_close(got, plain.rnd(want, "bfloat16"), **tol(torch.bfloat16, 2))
        same = ops.paged_attention(qkv.to(DEV), ctx, binding, nh, nkv, hd, scale, 0, generic=True).cpu().double()
        torch.testing.assert_close(got.view(T, -1), same, **tol(torch.bfloat16, 2))


@pytest.mark.parametrize("hd, g, page, ctx_lens, far", [(64, 4, 256, [4097, 9000, 5000, 1], 4100), (128, 2, 64, [4097, 9000, 5000, 1], 4100),
                                                        (64, 4, 256, [4097, 131000, 5000, 1], 70001)],
                         ids=["head64", "head128", "131000-tokens"])
def test_decode_attention_over_many_splits(ops, hd, g, page, ctx_lens, far):
    """
    Contexts of 17, 20 and 36 decode splits (the combination kernel takes 16 at a time), beside a first token; and one
    of 131,000 tokens (512 splits), about the longest a Llama 3.2 model takes.  One query is made to attend to a far
    key above all.
    """
    nkv = 2
    nh = nkv * g
    q_lens = [1, 1, 1, 1]
    ctx = make_ctx(q_lens, ctx_lens)
    tables, at = [], 0
    for c in ctx_lens:
        n = -(-c // page)
        tables.append(list(range(at, at + n)))
        at += n
    binding = make_binding(at + 1, 1, nkv, page, hd, torch.bfloat16, tables)
    keys = [rand((c, nkv, hd), torch.bfloat16, 60 + s) for s, c in enumerate(ctx_lens)]
    values = [rand((c, nkv, hd), torch.bfloat16, 70 + s) for s, c in enumerate(ctx_lens)]
    for s in range(len(ctx_lens)):
        table = binding.block_table[s].tolist()                        # whole pages at once: a slot at a time is slow here
        for i in range(-(-ctx_lens[s] // page)):
            n = min(page, ctx_lens[s] - i * page)
            binding.k_pool[table[i], 0, :, :n] = keys[s][i * page:i * page + n].transpose(0, 1).to(DEV)
            binding.v_pool[table[i], 0, :, :n] = values[s][i * page:i * page + n].transpose(0, 1).to(DEV)
    qkv = rand((4, (nh + 2 * nkv) * hd), torch.bfloat16, 13)
    qkv[1, :hd] = (keys[1][far, 0].float() * 3).to(torch.bfloat16)       # request 1, head 0 attends to a key in its seventeenth split or further
    scale = hd ** -0.5
    got = ops.paged_attention(qkv.to(DEV), ctx, binding, nh, nkv, hd, scale, 0).cpu().double().view(4, nh, hd)
    want = torch.zeros_like(got)
    for s in range(4):
        q = qkv[s, : nh * hd].view(nh, hd).double()
        for h in range(nh):
            k, v = keys[s][:, h // g].double(), values[s][:, h // g].double()
            p = torch.softmax(k @ q[h] * scale, dim=0)
            want[s, h] = plain.rnd(p, "bfloat16") @ v
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, plain.rnd(want, "bfloat16"), **tol(torch.bfloat16, 2))
    same = ops.paged_attention(qkv.to(DEV), ctx, binding, nh, nkv, hd, scale, 0, generic=True).cpu().double()
    torch.testing.assert_close(got.view(4, -1), same, **tol(torch.bfloat16, 2))
    # How a request's splits are merged depends on its own length only: alone or beside the 9,000-token request
    # (where the combination runs with more threads a block) it gives the same bits.  4,097 tokens are 17 splits.
    for s, c in ((0, 4097), (2, 5000), (3, 1)):
        alone_ctx = make_ctx([1], [c])
        alone = make_binding(at + 1, 1, nkv, page, hd, torch.bfloat16, [tables[s]])
        alone.k_pool.copy_(binding.k_pool)
        alone.v_pool.copy_(binding.v_pool)
        one = ops.paged_attention(qkv[s:s + 1].to(DEV), alone_ctx, alone, nh, nkv, hd, scale, 0).cpu().double()
        assert torch.equal(one.view(nh, hd), got[s]), f"request {s} depends on its neighbours"
    short_ctx = make_ctx([1, 1], [5000 - 4000, 1])        # up to 16 splits everywhere: the combination with one group
    few = make_binding(at + 1, 1, nkv, page, hd, torch.bfloat16, [tables[2], tables[3]])
    few.k_pool.copy_(binding.k_pool)
    few.v_pool.copy_(binding.v_pool)
    long_ctx = make_ctx([1, 1], [5000 - 4000, 9000])
    many = make_binding(at + 1, 1, nkv, page, hd, torch.bfloat16, [tables[2], tables[1]])
    many.k_pool.copy_(binding.k_pool)
    many.v_pool.copy_(binding.v_pool)
    a = ops.paged_attention(qkv[2:4].to(DEV), short_ctx, few, nh, nkv, hd, scale, 0)[0]
    b = ops.paged_attention(qkv[2:4].to(DEV), long_ctx, many, nh, nkv, hd, scale, 0)[0]
    assert torch.equal(a, b), "a short request is merged the same way whatever the step's longest request is"


def test_kernels_refuse_sizes_they_do_not_take(ops):
    from tinyserve_llm_b200.ops.library import KernelError
    ctx = make_ctx([1], [1])
    binding = make_binding(2, 1, 1, 8, 24, torch.float32, [[0]])
    with pytest.raises(KernelError, match="head_dim 24"):
        ops.paged_attention(torch.zeros((1, 3 * 24), device=DEV), ctx, binding, 1, 1, 24, 1.0, 0)
    binding = make_binding(2, 1, 1, 8, 272, torch.float32, [[0]])
    with pytest.raises(KernelError, match="head_dim 272"):
        ops.paged_attention(torch.zeros((1, 3 * 272), device=DEV), ctx, binding, 1, 1, 272, 1.0, 0)
    with pytest.raises(KernelError, match="not a multiple"):
        ops.paged_attention(torch.zeros((1, 5 * 16), device=DEV), ctx, make_binding(2, 1, 2, 8, 16, torch.float32, [[0]]),
                            3, 2, 16, 1.0, 0)
    with pytest.raises(KernelError, match="CUDA tensor"):
        ops.silu_mul(torch.zeros((2, 8)))
    with pytest.raises(KernelError, match="contiguous"):
        ops.silu_mul(torch.zeros((2, 16), device=DEV)[:, ::2])


@pytest.mark.parametrize("vocab", [11, 1000, 8196, 9001, 128256])       # one chunk and several; 16-byte loads and single ones
def test_sampling_greedy_and_ties(ops, vocab):
    logits = rand((4, vocab), torch.float32, 12)
    logits[1, 5] = logits[1, vocab - 2] = 50.0                     # a tie: the lowest index wins
    logits[2] = -1e30
    zeros = torch.zeros(4, dtype=torch.float32, device=DEV)
    keys = torch.zeros((4, 2), dtype=torch.int32, device=DEV)
    got = ops.sample(logits.to(DEV), zeros, keys).tolist()
    want = [int(torch.argmax(r)) for r in logits]
    want[1], want[2] = 5, 0
    assert got == want


def test_sampling_follows_the_softmax_and_its_keys(ops):
    from tinyserve_llm_b200.sampling import draw_key
    vocab, draws, temp = 37, 20000, 0.7
    row = rand((vocab,), torch.float32, 13, 2.0)
    logits = row.expand(draws, vocab).contiguous().to(DEV)
    temps = torch.full((draws,), temp, device=DEV)
    keys = torch.tensor([draw_key(1, 0, 0, i) for i in range(draws)], dtype=torch.int32, device=DEV)
    tokens = ops.sample(logits, temps, keys)
    freq = torch.bincount(tokens.long().cpu(), minlength=vocab).double() / draws
    assert (freq - plain.sampling_distribution(row, temp)).abs().max() < 0.01
    assert torch.equal(tokens, ops.sample(logits, temps, keys)), "the same keys must draw the same tokens"
    shuffled = torch.randperm(draws)
    again = ops.sample(logits, temps, keys[shuffled.to(DEV)].contiguous())
    assert torch.equal(again.cpu(), tokens.cpu()[shuffled]), "a draw depends on its key only, not on its row"
    other = ops.sample(logits, temps, torch.tensor([draw_key(2, 0, 0, i) for i in range(draws)], dtype=torch.int32, device=DEV))
    assert (other != tokens).float().mean() > 0.5
    # the noise of a logit depends on its index and the key only: the same row at the head of a vocabulary of several
    # chunks, the rest far below, draws the same tokens (another load path, other CTAs, the second kernel's pick)
    for wide_vocab in (10000, 9001):
        wide = torch.full((draws, wide_vocab), -1e30)
        wide[:, :vocab] = row
        assert torch.equal(ops.sample(wide.to(DEV), temps, keys), tokens)


def test_sampling_never_draws_what_has_no_probability(ops):
    """One logit carries all the probability (the rest: 1e-14 together): every draw over a large vocabulary is that token."""
    from tinyserve_llm_b200.sampling.sampler import draw_keys
    vocab, draws = 50000, 4000
    row = torch.zeros(vocab)
    row[123] = 30.0
    logits = row.expand(draws, vocab).contiguous().to(DEV)
    temps = torch.full((draws,), 0.7, device=DEV)
    keys = torch.from_numpy(draw_keys(3, [(r, 0, 0) for r in range(draws)])).to(DEV)
    assert ops.sample(logits, temps, keys).eq(123).all()


@pytest.mark.parametrize("dtype", DTYPES)
def test_copy_page_slots(ops, dtype):
    shape = (6, 3, 2, 8, 16)
    k, v = rand(shape, dtype, 14).to(DEV), rand(shape, dtype, 15).to(DEV)
    k0, v0 = k.clone(), v.clone()
    ops.copy_page_slots(k, v, 4, 1, 5)
    assert torch.equal(k[1, :, :, :5], k0[4, :, :, :5]) and torch.equal(v[1, :, :, :5], v0[4, :, :, :5])
    assert torch.equal(k[1, :, :, 5:], k0[1, :, :, 5:]) and torch.equal(v[1, :, :, 5:], v0[1, :, :, 5:])
    keep = [0, 2, 3, 4, 5]
    assert torch.equal(k[keep], k0[keep]) and torch.equal(v[keep], v0[keep])


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("n, k", [(48, 64), (1000, 192), (250, 512), (3072, 2048), (2048, 8192), (16, 32)])
def test_skinny_bfloat16_product(ops, m, n, k):
    """The weight-streaming kernel for a few rows of x: any N (also no multiple of 16), K a multiple of 32."""
    x, w = rand((m, k), torch.bfloat16, 5), rand((n, k), torch.bfloat16, 6, 0.05)
    want = x.double() @ w.double().T
    scale = want.abs().max().item()
    got = ops.linear(x.to(DEV), w.to(DEV)).cpu().double()
    torch.testing.assert_close(got, plain.rnd(want, "bfloat16"), atol=scale * 2 ** -8, rtol=2 ** -7)
    wide = ops.linear(x.to(DEV), w.to(DEV), out_dtype=torch.float32).cpu().double()
    torch.testing.assert_close(wide, want, atol=scale * 1e-5, rtol=1e-4)
    # a row's result does not depend on the rows beside it
    alone = ops.linear(x[:1].contiguous().to(DEV), w.to(DEV), out_dtype=torch.float32).cpu()
    assert torch.equal(alone[0], ops.linear(x.to(DEV), w.to(DEV), out_dtype=torch.float32).cpu()[0])


@pytest.mark.parametrize("m", [1, 8, 20, 40, 1500])
@pytest.mark.parametrize("inter, k", [(176, 64), (500, 192), (8192, 2048), (5, 32)])
def test_linear_with_swiglu_epilogue(ops, m, inter, k):
    """Every route: the decode product (up to 32 rows), the library product plus activation, the tcgen05 product (many rows)."""
    x, w = rand((m, k), torch.bfloat16, 7), rand((2 * inter, k), torch.bfloat16, 8, 0.2)
    gate_up = plain.rnd(x.double() @ w.double().T, "bfloat16")
    want = plain.swiglu(gate_up, "bfloat16")
    got = ops.linear_swiglu(x.to(DEV), w.to(DEV)).cpu().double()
    scale = want.abs().max().item()
    torch.testing.assert_close(got, want, atol=scale * 2 ** -7, rtol=2 ** -6)


@pytest.mark.parametrize("m, n, k", [(128, 128, 64), (1, 16, 8), (100, 200, 72), (130, 130, 136), (300, 1000, 192),
                                      (2048, 3072, 2048), (257, 4096, 520), (64, 2048, 8192), (1300, 5000, 200), (2048, 2048, 8192)])
def test_tcgen05_matrix_product(ops, m, n, k):
    """
    TMA-fed tcgen05 product: tiles that run over the edges of M, N and K, narrow and wide tile shapes, and (the large
    ones) two CTAs on a tile of 256 x 256.
    """
    x, w = rand((m, k), torch.bfloat16, 5), rand((n, k), torch.bfloat16, 6, 0.05)
    want = x.double() @ w.double().T
    scale = want.abs().max().item()
    got = ops.gemm_tcgen05(x.to(DEV), w.to(DEV)).cpu().double()
    torch.testing.assert_close(got, plain.rnd(want, "bfloat16"), atol=scale * 2 ** -8, rtol=2 ** -7)
    wide = ops.gemm_tcgen05(x.to(DEV), w.to(DEV), out_dtype=torch.float32).cpu().double()
    torch.testing.assert_close(wide, want, atol=scale * 1e-5, rtol=1e-4)
    torch.cuda.synchronize()
    ops.check_device_errors()


@pytest.mark.parametrize("m, inter, k", [(33, 64, 64), (100, 176, 72), (64, 8192, 2048), (2048, 8192, 2048), (300, 500, 192),
                                         (1300, 2500, 136)])
def test_tcgen05_product_with_swiglu_epilogue(ops, m, inter, k):
    x, w = rand((m, k), torch.bfloat16, 7), rand((2 * inter, k), torch.bfloat16, 8, 0.2)
    gate_up = plain.rnd(x.double() @ w.double().T, "bfloat16")
    want = plain.swiglu(gate_up, "bfloat16")
    got = ops.gemm_tcgen05(x.to(DEV), w.to(DEV), swiglu=True).cpu().double()
    scale = want.abs().max().item()
    torch.testing.assert_close(got, want, atol=scale * 2 ** -7, rtol=2 ** -6)
    torch.cuda.synchronize()
    ops.check_device_errors()


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("nh, nkv, page", [(8, 2, 64), (32, 8, 256), (5, 5, 128), (3, 1, 64)])
def test_tcgen05_prompt_attention(ops, nh, nkv, page, hd):
    """
    Prompt portions on the tcgen05 kernel (TMA tiles, S and O in tensor memory): whole prompts of
    several query tiles, a portion over a long cached prefix that ends inside a page, a two-token
    portion, beside requests that decode; against the plain reference and against the mma.sync
    kernel on the same inputs.  Pools are poisoned with NaN: the unwritten tail of a last page must
    not reach the result.  Head sizes 64 (tiles of 128 keys) and 128 (two sub-tiles of 64 dims, tiles of 64 keys).
    """
    q_lens = [300, 1, 130, 2, 128, 1]
    ctx_lens = [300, 700, 1000, 2, 128, 65]
    ctx = make_ctx(q_lens, ctx_lens)
    tables, at = [], 0
    for c in ctx_lens:
        n = -(-c // page)
        tables.append(list(range(at + n - 1, at - 1, -1)))
        at += n
    binding = make_binding(at + 1, 2, nkv, page, hd, torch.bfloat16, tables, entry=1)
    keys = [rand((c, nkv, hd), torch.bfloat16, 40 + s) for s, c in enumerate(ctx_lens)]
    values = [rand((c, nkv, hd), torch.bfloat16, 50 + s) for s, c in enumerate(ctx_lens)]
    for s in range(len(ctx_lens)):
        fill_cache(binding, s, keys[s], values[s], entry=1)
    T = ctx.num_tokens
    qkv = rand((T, (nh + 2 * nkv) * hd), torch.bfloat16, 12)
    qkv[5, :hd] = (keys[0][2, 0].float() * 3).to(torch.bfloat16)      # token 5 of the first prompt attends to key 2 above all
    scale = hd ** -0.5
    if not ops.tcgen05_attention:
        pytest.skip("TINYSERVE_B200_PREFILL=mma keeps prompt attention off the tcgen05 kernel in this run")
    got = ops.paged_attention(qkv.to(DEV), ctx, binding, nh, nkv, hd, scale, 0).cpu().double().view(T, nh, hd)
    torch.cuda.synchronize()
    ops.check_device_errors()
    want = plain_paged_attention(qkv[:, : nh * hd].view(T, nh, hd).double(), keys, values, ctx_lens, q_lens, scale, 0)
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, plain.rnd(want, "bfloat16"), **tol(torch.bfloat16, 2))
    ops.tcgen05_attention = False
    try:
        legacy = ops.paged_attention(qkv.to(DEV), ctx, binding, nh, nkv, hd, scale, 0).cpu().double().view(T, nh, hd)
    finally:
        ops.tcgen05_attention = True
    torch.testing.assert_close(got, legacy, **tol(torch.bfloat16, 2))


@pytest.mark.parametrize("hd", [64, 128])
def test_tcgen05_prompt_attention_behind_a_hundred_thousand_cached_tokens(ops, hd):
    """
    A portion of 130 tokens at the end of a context of 100,003: some 800 key tiles per query tile, 391 pages, the
    last one partly filled.  One query attends to a key 88,000 tokens back above all.
    """
    if not ops.tcgen05_attention:
        pytest.skip("TINYSERVE_B200_PREFILL=mma keeps prompt attention off the tcgen05 kernel in this run")
    nh, nkv, page, c, n = 4, 1, 256, 100003, 130
    pages = -(-c // page)
    ctx = make_ctx([n], [c])
    binding = make_binding(pages + 1, 1, nkv, page, hd, torch.bfloat16, [list(range(pages - 1, -1, -1))])
    keys, values = rand((c, nkv, hd), torch.bfloat16, 80), rand((c, nkv, hd), torch.bfloat16, 81)
    table = binding.block_table[0].tolist()
    for i in range(pages):
        m = min(page, c - i * page)
        binding.k_pool[table[i], 0, :, :m] = keys[i * page:i * page + m].transpose(0, 1).to(DEV)
        binding.v_pool[table[i], 0, :, :m] = values[i * page:i * page + m].transpose(0, 1).to(DEV)
    qkv = rand((n, (nh + 2 * nkv) * hd), torch.bfloat16, 82)
    qkv[7, hd:2 * hd] = (keys[12345, 0].float() * 3).to(torch.bfloat16)      # token 7, head 1
    scale = hd ** -0.5
    got = ops.paged_attention(qkv.to(DEV), ctx, binding, nh, nkv, hd, scale, 0).cpu().double().view(n, nh, hd)
    torch.cuda.synchronize()
    ops.check_device_errors()
    q = qkv[:, : nh * hd].view(n, nh, hd).double()
    k, v = keys[:, 0].double(), values[:, 0].double()
    seen = torch.arange(c)[None, :] <= (c - n + torch.arange(n))[:, None]          # [n, c]: causal, bottom-right aligned
    want = torch.zeros_like(got)
    for h in range(nh):
        scores = (q[:, h] @ k.T * scale).masked_fill(~seen, float("-inf"))
        want[:, h] = plain.rnd(torch.softmax(scores, dim=1), "bfloat16") @ v
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, plain.rnd(want, "bfloat16"), **tol(torch.bfloat16, 2))
    assert torch.softmax((q[7, 1] @ k.T * scale)[: c - n + 8], dim=0)[12345] > 0.5    # the case is what it says


@pytest.mark.parametrize("hd", [64, 128])
def test_tcgen05_prompt_attention_when_the_maximum_grows_from_tile_to_tile(ops, hd):
    """
    The kernel rescales O only when a row's maximum has grown by more than 2^8 since its reference was
    taken.  Keys are scaled so that the scores of one query direction grow along the sequence: by small steps
    (the reference stays, P holds values above one), then by a jump of hundreds (the reference moves and what
    was summed before all but vanishes), then fall again.  Random inputs alone never leave the first case.
    """
    if not ops.tcgen05_attention:
        pytest.skip("TINYSERVE_B200_PREFILL=mma keeps prompt attention off the tcgen05 kernel in this run")
    nh, nkv, page, T = 4, 2, 128, 1500
    ctx = make_ctx([T], [T])
    binding = make_binding(-(-T // page) + 1, 1, nkv, page, hd, torch.bfloat16, [list(range(-(-T // page)))], entry=0)
    direction = torch.nn.functional.normalize(rand((hd,), torch.float32, 70), dim=0)
    keys = rand((T, nkv, hd), torch.bfloat16, 71).float() * 0.3
    at = torch.arange(T, dtype=torch.float32)
    # the score against `direction` (log2 units after the scale): +1.5 a tile of 128 keys up to key 900, +400 from
    # key 900 to 1100, back to nothing after it
    ramp = torch.where(at < 900, at / 128 * 1.5, torch.where(at < 1100, torch.full_like(at, 400.0), torch.zeros_like(at)))
    scale = hd ** -0.5
    keys[:, 0, :] += (ramp / (scale * math.log2(math.e)))[:, None] * direction[None, :] / 8.0
    keys = keys.to(torch.bfloat16)
    values = rand((T, nkv, hd), torch.bfloat16, 72)
    fill_cache(binding, 0, keys, values, entry=0)
    qkv = rand((T, (nh + 2 * nkv) * hd), torch.bfloat16, 73) * 0.3
    qkv[:, :hd] += (direction * 8.0).to(torch.bfloat16)                 # head 0 (kv head 0) looks along the direction
    got = ops.paged_attention(qkv.to(DEV), ctx, binding, nh, nkv, hd, scale, 0).cpu().double().view(T, nh, hd)
    torch.cuda.synchronize()
    ops.check_device_errors()
    want = plain_paged_attention(qkv[:, : nh * hd].view(T, nh, hd).double(), [keys], [values], [T], [T], scale, 0)
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, plain.rnd(want, "bfloat16"), **tol(torch.bfloat16, 2))
    # the case is what it says: along head 0 the largest score of a row grows by more than 2^8 in one step
    s0 = (qkv[1099, :hd].double() @ keys[:1100, 0].double().T) * scale * math.log2(math.e)
    assert s0[900:].max() - s0[:900].max() > 100 and 2 < s0[:900].max() - s0[:128].max() < 40


def test_environment_switches(ops, monkeypatch):
    """The library's switches are read when it is loaded; serialised launches give the same bits as chained ones."""
    from tinyserve_llm_b200.ops.library import Ops
    as_found = ops.chaining                        # the flag lives in the shared library: it is handed back as it was
    x, res = rand((8, 256), torch.bfloat16, 1).to(DEV), rand((8, 256), torch.bfloat16, 2).to(DEV)
    w, norm_w = rand((512, 256), torch.bfloat16, 3, 0.1).to(DEV), (1 + rand((256,), torch.bfloat16, 4, 0.2)).to(DEV)

    def chain(o):
        h, _ = o.add_rmsnorm(x.clone(), res.clone(), norm_w, 1e-5)
        return o.linear_swiglu(h, w)

    try:
        monkeypatch.setenv("TINYSERVE_B200_CHAINING", "0")
        monkeypatch.setenv("TINYSERVE_B200_PREFILL", "mma")
        monkeypatch.setenv("TINYSERVE_B200_SWIGLU_ROWS", "77")
        plain_launches = Ops(ops.lib_path)
        assert not plain_launches.chaining and not plain_launches.tcgen05_attention and plain_launches.tcgen05_swiglu_min_rows == 77
        serial = chain(plain_launches)
        for name in ("TINYSERVE_B200_CHAINING", "TINYSERVE_B200_PREFILL", "TINYSERVE_B200_SWIGLU_ROWS"):
            monkeypatch.delenv(name)
        defaults = Ops(ops.lib_path)
        assert defaults.chaining and defaults.tcgen05_attention and defaults.tcgen05_swiglu_min_rows == 512
        chained = chain(defaults)
    finally:
        ops.set_chaining(as_found)
    assert torch.equal(serial, chained)
