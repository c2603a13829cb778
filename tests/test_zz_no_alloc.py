"""
The decode-attention entry point that brings its own scratch (csrc/attention_decode_noalloc.h), for
hosts that cannot allocate device memory at step time.  It is called here the way such a host would
call it: through the exported C symbol of the shared library, with raw pointers.  It runs the same
kernels with the same splits as the ordinary entry point, which is handed a scratch buffer, so its
output must equal that one's bit for bit, on two calls in a row; the second call is smaller than the
first, so whatever the first left in the shared scratch array would show if a stale value were read.
Both calls are also held to the plain attention, within the bfloat16 bound of tests/test_kernels.py.
This file sorts last on purpose: a run that stops at the first failure has then run every other
test already.
"""

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

import plain_llama as plain
from gpu_util import DEV, fill_cache, make_binding, make_ctx

pytestmark = pytest.mark.gpu


def _rand(shape, seed):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)


def _batch(ctx_lens, nh, nkv, hd, page, seed):
    ctx = make_ctx([1] * len(ctx_lens), ctx_lens)
    tables, at = [], 0
    for c in ctx_lens:
        n = -(-c // page)
        tables.append(list(range(at, at + n)))
        at += n
    binding = make_binding(at + 2, 1, nkv, page, hd, torch.bfloat16, tables)
    keys = [_rand((c, nkv, hd), seed + 2 * s) for s, c in enumerate(ctx_lens)]
    values = [_rand((c, nkv, hd), seed + 2 * s + 1) for s, c in enumerate(ctx_lens)]
    for s in range(len(ctx_lens)):
        fill_cache(binding, s, keys[s], values[s])
    qkv = _rand((len(ctx_lens), (nh + 2 * nkv) * hd), seed + 100).to(DEV)
    return ctx, binding, qkv, keys, values


def _plain(qkv, keys, values, nh, hd, scale):
    """Each request's one query over all its keys (plain_llama.causal_attention on the whole sequence, last row)."""
    rows = []
    for s, (k, v) in enumerate(zip(keys, values)):
        q = torch.zeros((k.shape[0], nh, hd), dtype=torch.float64)
        q[-1] = qkv[s, :nh * hd].cpu().double().view(nh, hd)
        rows.append(plain.causal_attention(q, k.double(), v.double(), scale, "float32")[-1].reshape(-1))
    return plain.rnd(torch.stack(rows), "bfloat16")


def _call_no_alloc(lib, ctx, binding, qkv, nh, nkv, hd, scale, max_ctx_len):
    out = torch.full((qkv.shape[0], nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    fn = lib.ts_decode_attention_bf16_noalloc
    fn.restype = c_int
    code = fn(c_void_p(qkv.data_ptr()), c_void_p(out.data_ptr()), c_void_p(binding.k_pool.data_ptr()),
              c_void_p(binding.v_pool.data_ptr()), c_longlong(binding.page_stride), c_longlong(binding.entry_offset),
              c_int(binding.page_tokens), c_int(binding.num_pages), c_void_p(binding.block_table.data_ptr()),
              c_int(binding.table_width), c_void_p(ctx.cu_q.data_ptr()), c_void_p(ctx.ctx_lens.data_ptr()),
              c_int(ctx.ctx_lens.shape[0]), c_int(max_ctx_len), c_int(nh), c_int(nkv), c_int(hd), c_float(scale),
              c_int(0), c_void_p(torch.cuda.current_stream().cuda_stream))
    return code, out


def test_entry_point_without_allocation_agrees_with_the_ordinary_one():
    from tinyserve_llm_b200.ops import get_ops
    ops = get_ops()
    lib = ctypes.CDLL(ops.lib_path)                       # the exported symbol, as a C host would find it
    lib.ts_last_error.restype = ctypes.c_char_p
    nh, nkv, hd, page = 8, 2, 64, 128
    scale = hd ** -0.5
    for ctx_lens, seed in (([1500, 700, 1, 256, 257, 90], 1), ([300, 5], 50)):     # the second call is the smaller one
        ctx, binding, qkv, keys, values = _batch(ctx_lens, nh, nkv, hd, page, seed)
        want = ops.paged_attention(qkv.clone(), ctx, binding, nh, nkv, hd, scale, 0)
        code, got = _call_no_alloc(lib, ctx, binding, qkv, nh, nkv, hd, scale, max(ctx_lens))
        assert code == 0, lib.ts_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want), "the same kernels with the same splits must give the same bits"
        torch.testing.assert_close(got.cpu().double(), _plain(qkv, keys, values, nh, hd, scale), atol=2e-2, rtol=1e-2)   # the bound of test_paged_attention
    # beyond the built-in scratch: refused with the need and the limit, nothing launched
    lib.ts_decode_attention_noalloc_max_floats.restype = c_longlong
    limit = lib.ts_decode_attention_noalloc_max_floats()
    code, _ = _call_no_alloc(lib, ctx, binding, qkv, nh, nkv, hd, scale, 200_000_000)
    message = lib.ts_last_error().decode()
    assert code != 0 and str(limit) in message and "scratch" in message
