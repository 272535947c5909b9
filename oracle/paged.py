"""Paged KV-cache indexing on the CPU (test oracle only).

Logical token ``t`` of sequence ``b`` lives at physical row
``block_tables[b, t // page_size] * page_size + t % page_size`` of a cache
whose second dimension is ``num_pages * page_size``
(construction by scatter: tests/test_tree_attention.py:375-409; page-swap
invariance: tests/test_mem_eff_attention.py:2690-2738).  Integer arithmetic
only; numpy int64.
"""

from __future__ import annotations

import numpy as np
import torch


def physical_rows(block_tables, page_size: int, b: int, n_tokens: int) -> np.ndarray:
    bt = np.asarray(block_tables.cpu() if isinstance(block_tables, torch.Tensor) else block_tables, dtype=np.int64)
    t = np.arange(n_tokens, dtype=np.int64)
    return bt[b, t // page_size] * page_size + t % page_size


def gather_paged(cache: torch.Tensor, block_tables, page_size: int, kv_seqlens, padding: int) -> torch.Tensor:
    """``cache [1, num_pages*page_size, ...]`` -> padded ``[1, B*padding, ...]``
    with sequence ``b`` at rows ``[b*padding, b*padding+kv_seqlens[b])`` and
    zeros elsewhere."""
    B = len(kv_seqlens)
    cache = cache.cpu()
    out = torch.zeros((1, B * padding) + tuple(cache.shape[2:]), dtype=cache.dtype)
    for b, n in enumerate(kv_seqlens):
        rows = torch.from_numpy(physical_rows(block_tables, page_size, b, int(n)))
        out[0, b * padding : b * padding + int(n)] = cache[0, rows]
    return out


def scatter_to_pages(padded: torch.Tensor, block_tables, page_size: int, kv_seqlens, padding: int, num_pages: int) -> torch.Tensor:
    """Inverse of :func:`gather_paged` (rows not owned by any token are zero)."""
    padded = padded.cpu()
    out = torch.zeros((1, num_pages * page_size) + tuple(padded.shape[2:]), dtype=padded.dtype)
    for b, n in enumerate(kv_seqlens):
        rows = torch.from_numpy(physical_rows(block_tables, page_size, b, int(n)))
        out[0, rows] = padded[0, b * padding : b * padding + int(n)]
    return out
