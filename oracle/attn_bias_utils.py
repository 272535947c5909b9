"""Test helpers under the names the reference's tests use
(xformers/attn_bias_utils.py:7-12: ``ref_attention``, ``ref_attention_bmhk``,
``create_attn_bias``, ``pack_kv_cache``).  TEST INFRASTRUCTURE ONLY.

The reference's own bodies live in the un-vendored ``mslk`` package; what is
stated here is their contract as the reference's tests use it
(tests/test_mem_eff_attention.py:446-459 builds every bias through
``create_attn_bias``; :2660-2665 packs a padded cache into pages with
``pack_kv_cache``), written independently.  ``create_attn_bias`` returns
instances of the bias classes of the package under test, because those objects
are what an operator receives; the arithmetic they are checked against stays in
``oracle/masks.py`` and ``oracle/ref_attention.py``.
"""

from __future__ import annotations

import random
from typing import Any, List, Optional, Sequence, Tuple

import torch

from .ref_attention import ref_attention, ref_attention_bmhk  # noqa: F401  (re-exported under the reference's module name)


def _split_total(r: random.Random, total: int, parts: int, at_least: int = 1) -> List[int]:
    """``parts`` lengths >= ``at_least`` that add up to ``total`` (seeded)."""
    assert total >= parts * at_least, f"cannot cut {total} into {parts} parts of at least {at_least}"
    spare = total - parts * at_least
    cuts = sorted(r.randint(0, spare) for _ in range(parts - 1))
    edges = [0] + cuts + [spare]
    return [at_least + edges[i + 1] - edges[i] for i in range(parts)]


def _seqlens_q_kv(r: random.Random, batch_size: int, q_len: int, kv_len: int, more_keys_than_queries: bool) -> Tuple[List[int], List[int]]:
    """Lengths of ``batch_size`` sequences whose queries fill ``q_len`` rows and whose keys fill ``kv_len`` rows.
    With ``more_keys_than_queries`` no sequence has fewer keys than queries (bottom-right aligned masks need that
    to leave every query a key)."""
    n = max(1, min(batch_size, q_len, kv_len))
    q = _split_total(r, q_len, n)
    if more_keys_than_queries:
        assert kv_len >= q_len
        extra = _split_total(r, kv_len - q_len, n, at_least=0)
        return q, [a + b for a, b in zip(q, extra)]
    return q, _split_total(r, kv_len, n)


def _seqlens_padded(r: random.Random, batch_size: int, q_len: int, kv_len: int) -> Tuple[List[int], List[int]]:
    """``batch_size`` sequences of ``q_len`` queries each in slots of ``kv_len`` key rows: key counts are random but
    never below the number of queries."""
    assert kv_len >= q_len
    return [q_len] * batch_size, [r.randint(q_len, kv_len) for _ in range(batch_size)]


def create_attn_bias(
    bias_type,
    batch_size: int,
    num_heads: int,
    num_heads_groups: int,
    q_len: int,
    kv_len: int,
    device,
    dtype,
    requires_grad: bool,
    fmt: str,
    op=None,
    page_size: Optional[int] = None,
):
    """A bias of type ``bias_type`` for inputs of ``batch_size`` x ``q_len`` queries and ``kv_len`` keys in layout
    ``fmt`` ("BMK", "BMHK" or "BMGHK"); seeded by its arguments, so the same call gives the same bias.

    * ``None`` / ``type(None)``: no bias.
    * ``torch.Tensor``: an additive tensor ``[B, (G,) H, Mq, Mkv]`` (``[B*H, Mq, Mkv]`` for BMK), N(0, 3^2).
    * mask classes without tensors: an instance (window sizes drawn from {3, 128, 300}).
    * block-diagonal classes: the query and key rows are cut into ``batch_size`` sequences; the inputs must then be
      reshaped to batch 1 (tests/test_mem_eff_attention.py:460-475 does that for every varlen bias).
    * padded-keys classes: every sequence has ``q_len`` queries and a slot of ``kv_len`` key rows; their paged
      forms get the identity block table over ``page_size`` pages (``kv_len`` must divide into pages).
    * gappy-keys classes: as padded keys, the slot of sequence b starting at row ``b * kv_len``.
    """
    from xformers_b200.ops.fmha import attn_bias as ab

    if bias_type is None or bias_type is type(None):
        return None
    r = random.Random("-".join(map(str, [batch_size, q_len, kv_len, dtype, fmt])))
    window = (3, 128, 300)[r.randint(0, 2)]
    if bias_type is torch.Tensor:
        g = torch.Generator().manual_seed(r.randint(0, 2**31 - 1))
        if fmt == "BMK":
            shape: Tuple[int, ...] = (batch_size * num_heads, q_len, kv_len)
        elif fmt == "BMHK":
            shape = (batch_size, num_heads, q_len, kv_len)
        else:
            shape = (batch_size, num_heads_groups, num_heads, q_len, kv_len)
        # rows start 16-byte aligned whatever kv_len is: allocate padded, then slice
        padded = -(-kv_len // 8) * 8
        t = (torch.randn(shape[:-1] + (padded,), generator=g) * 3).to(dtype).to(device)[..., :kv_len]
        if requires_grad:
            t.requires_grad_(True)
        return t
    if bias_type is ab.LowerTriangularMask:
        return ab.LowerTriangularMask()
    if bias_type is ab.LowerTriangularFromBottomRightMask:
        return ab.LowerTriangularFromBottomRightMask()
    if bias_type is ab.LowerTriangularMaskLocalAttention:
        return ab.LowerTriangularMaskLocalAttention(window)
    if bias_type is ab.LowerTriangularFromBottomRightLocalAttentionMask:
        return ab.LowerTriangularFromBottomRightLocalAttentionMask(window)
    if bias_type is ab.LocalAttentionFromBottomRightMask:
        return ab.LocalAttentionFromBottomRightMask(window_left=r.randint(0, 5), window_right=r.randint(0, 5))
    if bias_type is ab.LowerTriangularMaskWithTensorBias:
        t = create_attn_bias(torch.Tensor, batch_size, num_heads, num_heads_groups, q_len, kv_len, device, dtype, requires_grad, fmt, op)
        return ab.LowerTriangularMaskWithTensorBias(t)

    if fmt == "BMK":
        raise ValueError(f"{bias_type.__name__} needs a head axis (BMHK or BMGHK inputs)")
    if issubclass(bias_type, ab.BlockDiagonalMask):
        bottom_right = issubclass(bias_type, ab.BlockDiagonalCausalFromBottomRightMask)
        q, k = _seqlens_q_kv(r, batch_size, q_len, kv_len, bottom_right)
        base = ab.BlockDiagonalMask.from_seqlens(q, k, device=device)
        if bias_type is ab.BlockDiagonalMask:
            return base
        if bias_type is ab.BlockDiagonalCausalMask:
            return base.make_causal()
        if bias_type is ab.BlockDiagonalCausalFromBottomRightMask:
            return base.make_causal_from_bottomright()
        if bias_type is ab.BlockDiagonalCausalLocalAttentionMask:
            return base.make_local_attention(window)
        if bias_type is ab.BlockDiagonalCausalLocalAttentionFromBottomRightMask:
            return base.make_local_attention_from_bottomright(window)
        raise NotImplementedError(bias_type)

    paged = issubclass(bias_type, ab.PagedBlockDiagonalPaddedKeysMask)
    flat_type = bias_type._UNPAGED_TYPE if paged else bias_type
    if not issubclass(flat_type, ab.BlockDiagonalPaddedKeysMask):
        raise NotImplementedError(f"create_attn_bias: {bias_type}")
    q, k = _seqlens_padded(r, batch_size, q_len, kv_len)
    if issubclass(flat_type, ab.BlockDiagonalGappyKeysMask):
        starts = [b * kv_len for b in range(batch_size + 1)]
        if hasattr(flat_type, "from_seqlens_local") and "window_left" in flat_type.__dataclass_fields__:
            flat = flat_type.from_seqlens_local(q, starts, k, r.randint(0, window), r.randint(0, 5), device=device)
        else:
            flat = flat_type.from_seqlens(q, starts, k, device=device)
    elif "window_left" in getattr(flat_type, "__dataclass_fields__", {}):
        flat = flat_type.from_seqlens_local(q, kv_len, k, r.randint(0, window), r.randint(0, 5), device=device)
    elif "_window_size" in getattr(flat_type, "__dataclass_fields__", {}):
        flat = flat_type.from_seqlens_local(q, kv_len, k, min(window, min(k)), device=device)
    else:
        flat = flat_type.from_seqlens(q_seqlen=q, kv_padding=kv_len, kv_seqlen=k, device=device)
    if not paged:
        return flat
    if not page_size or kv_len % page_size:
        raise ValueError(f"a paged bias needs page_size dividing kv_len, got page_size={page_size}, kv_len={kv_len}")
    per_row = kv_len // page_size
    block_tables = torch.arange(batch_size * per_row, dtype=torch.int32, device=device).reshape(batch_size, per_row)
    kwargs = {"notional_padding": kv_len} if issubclass(flat_type, ab.BlockDiagonalGappyKeysMask) else {}
    return flat.make_paged(block_tables, page_size, bias_type, **kwargs)


def pack_kv_cache(
    cache_k: torch.Tensor,
    cache_v: torch.Tensor,
    kv_seqlens: Sequence[int],
    page_size: int,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Padded caches ``[B, MAX_T, H_kv, D]`` (heads not expanded) -> ``(block_tables [B, max pages of a sequence]
    int32, packed_k, packed_v [1, pages * page_size, H_kv, D])`` in which only the pages a sequence really uses
    exist, handed out in order (tests/test_mem_eff_attention.py:2660-2665; page placement as
    tests/test_tree_attention.py:375-409).  Table entries past a sequence's last page are 0 and never read."""
    B, max_t = cache_k.shape[:2]
    assert cache_v.shape[:2] == (B, max_t) and len(kv_seqlens) == B
    pages = [-(-int(n) // page_size) for n in kv_seqlens]
    total = sum(pages)
    block_tables = torch.zeros((B, max(max(pages), 1)), dtype=torch.int32, device=cache_k.device)
    packed_k = torch.zeros((1, total * page_size) + tuple(cache_k.shape[2:]), dtype=cache_k.dtype, device=cache_k.device)
    packed_v = torch.zeros((1, total * page_size) + tuple(cache_v.shape[2:]), dtype=cache_v.dtype, device=cache_v.device)
    nxt = 0
    for b, n in enumerate(kv_seqlens):
        n = int(n)
        block_tables[b, : pages[b]] = torch.arange(nxt, nxt + pages[b], dtype=torch.int32)
        packed_k[0, nxt * page_size : nxt * page_size + n] = cache_k[b, :n]
        packed_v[0, nxt * page_size : nxt * page_size + n] = cache_v[b, :n]
        nxt += pages[b]
    return block_tables, packed_k, packed_v
