"""Additive-mask materialisers built from plain integer lists (test oracle only).

Each function returns a float32 ``[Mq, Mkv]`` tensor holding 0 where a key is
visible and ``-inf`` where it is not.  They are deliberately independent of
the bias classes shipped in the package so that the two can be compared.

Semantics follow the known-answer tests of the reference:
  * top-left causal .............. tests/test_mem_eff_attention.py:1427-1439
  * block diagonal ............... tests/test_mem_eff_attention.py:1452-1538
  * bottom-right causal blocks ... tests/test_mem_eff_attention.py:1555-1587
  * padded keys, causal offset ... tests/test_mem_eff_attention.py:1617-1626
  * local windows ................ tests/test_mem_eff_attention.py:1997-2028,2389-2399
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

NEG_INF = -math.inf


def _visible_to_additive(visible: torch.Tensor) -> torch.Tensor:
    out = torch.full(visible.shape, NEG_INF, dtype=torch.float32)
    out[visible] = 0.0
    return out


def causal_mask(
    mq: int,
    mkv: int,
    *,
    from_bottom_right: bool = False,
    kv_offset: int = 0,
    window_left: Optional[int] = None,
    window_right: Optional[int] = None,
) -> torch.Tensor:
    """Key ``j`` (global index ``j + kv_offset``) is visible to query ``i`` iff
    ``j + kv_offset <= i + shift`` with ``shift = 0`` (top-left aligned) or
    ``mkv - mq`` (bottom-right aligned).  ``window_left`` keeps only keys with
    ``j >= i + shift - window_left``; ``window_right`` replaces the causal
    upper limit by ``j <= i + shift + window_right``."""
    i = torch.arange(mq).view(-1, 1)
    j = torch.arange(mkv).view(1, -1) + kv_offset
    shift = (mkv - mq) if from_bottom_right else 0
    upper = i + shift + (0 if window_right is None else window_right)
    vis = j <= upper
    if window_left is not None:
        vis &= j >= i + shift - window_left
    return _visible_to_additive(vis)


def local_mask(mq: int, mkv: int, window_left: int, window_right: int) -> torch.Tensor:
    """Bottom-right aligned band: |offset| limited on both sides
    (tests/test_mem_eff_attention.py:2389-2399)."""
    return causal_mask(
        mq,
        mkv,
        from_bottom_right=True,
        window_left=window_left,
        window_right=window_right,
    )


def block_diagonal_mask(
    q_seqlens: Sequence[int],
    kv_seqlens: Optional[Sequence[int]] = None,
    *,
    causal: bool = False,
    from_bottom_right: bool = False,
    window_size: Optional[int] = None,
) -> torch.Tensor:
    """Sequences concatenated along both axes; block ``b`` couples its own
    queries with its own keys only.  ``causal`` is applied inside each block.
    ``window_size`` w keeps keys ``j > i - w`` of the (causal) block
    (tests/test_mem_eff_attention.py:1997-2028)."""
    if kv_seqlens is None:
        kv_seqlens = q_seqlens
    assert len(q_seqlens) == len(kv_seqlens)
    out = torch.full((sum(q_seqlens), sum(kv_seqlens)), NEG_INF, dtype=torch.float32)
    qs = ks = 0
    for ql, kl in zip(q_seqlens, kv_seqlens):
        if causal or window_size is not None:
            blk = causal_mask(
                ql,
                kl,
                from_bottom_right=from_bottom_right,
                window_left=None if window_size is None else window_size - 1,
            )
        else:
            blk = torch.zeros((ql, kl), dtype=torch.float32)
        out[qs : qs + ql, ks : ks + kl] = blk
        qs += ql
        ks += kl
    return out


def padded_keys_mask(
    q_seqlens: Sequence[int],
    kv_seqlens: Sequence[int],
    kv_padding: int,
    *,
    causal: bool,
) -> torch.Tensor:
    """Keys of sequence ``b`` occupy ``[b*P, b*P + kv_seqlens[b])`` of a cache
    of ``len(kv_seqlens)*P`` rows.  The causal form is bottom-right aligned
    with respect to ``kv_seqlens[b]``: exactly ``triu(diagonal=1+slen-qlen)``
    of the reference's hand-built mask
    (tests/test_mem_eff_attention.py:1617-1626)."""
    n = len(q_seqlens)
    assert len(kv_seqlens) == n
    out = torch.full((sum(q_seqlens), n * kv_padding), NEG_INF, dtype=torch.float32)
    qs = 0
    for b, (ql, kl) in enumerate(zip(q_seqlens, kv_seqlens)):
        assert kl <= kv_padding
        if causal:
            blk = causal_mask(ql, kl, from_bottom_right=True)
        else:
            blk = torch.zeros((ql, kl), dtype=torch.float32)
        out[qs : qs + ql, b * kv_padding : b * kv_padding + kl] = blk
        qs += ql
    return out
