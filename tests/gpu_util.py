"""Small helpers for GPU tests that drive kernels and parts directly."""

from __future__ import annotations

from types import SimpleNamespace

import torch

from tinyserve_llm_b200.cache.storage import EntryBinding

DEV = "cuda"


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def make_ctx(q_lens: list[int], ctx_lens: list[int]):
    """A step context as the kernels see it: flat positions and sequence index per token."""
    positions, seq_of_token, cu_q = [], [], [0]
    for s, (q, c) in enumerate(zip(q_lens, ctx_lens)):
        positions += list(range(c - q, c))
        seq_of_token += [s] * q
        cu_q.append(cu_q[-1] + q)
    return SimpleNamespace(positions=i32(positions), seq_of_token=i32(seq_of_token), num_tokens=len(positions),
                           cu_q=i32(cu_q), ctx_lens=i32(ctx_lens), max_q_len=max(q_lens), min_q_len=min(q_lens),
                           max_ctx_len=max(ctx_lens), scratch={},
                           host=SimpleNamespace(cu_q=cu_q, ctx_lens=list(ctx_lens), start=[c - q for q, c in zip(q_lens, ctx_lens)]))


def make_binding(num_pages, entries, nkv, page_tokens, hd, dtype, tables: list[list[int]], entry=0, poison=True,
                 writes=True) -> EntryBinding:
    shape = (num_pages, entries, nkv, page_tokens, hd)
    k = torch.full(shape, float("nan") if poison else 0.0, dtype=dtype, device=DEV)
    v = torch.full(shape, float("nan") if poison else 0.0, dtype=dtype, device=DEV)
    width = max(len(t) for t in tables)
    table = i32([t + [-1] * (width - len(t)) for t in tables])
    per_entry = nkv * page_tokens * hd
    return EntryBinding(k, v, per_entry * entries, per_entry * entry, page_tokens, num_pages, table, width, writes)


def fill_cache(binding: EntryBinding, seq: int, keys: torch.Tensor, values: torch.Tensor, entry=0) -> None:
    """Writes keys/values [ctx, nkv, hd] of sequence `seq` into the pages its table names."""
    table = binding.block_table[seq].tolist()
    B = binding.page_tokens
    for pos in range(keys.shape[0]):
        page = table[pos // B]
        binding.k_pool[page, entry, :, pos % B] = keys[pos].to(binding.k_pool.dtype)
        binding.v_pool[page, entry, :, pos % B] = values[pos].to(binding.v_pool.dtype)
