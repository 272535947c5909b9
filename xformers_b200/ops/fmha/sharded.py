"""Long-context attention with the key/value sequence sharded across ranks.

The reference has no ring or context-parallel attention; its long-context
primitive is algebraic: attention over parts of the keys
(``memory_efficient_attention_partial``) followed by ``merge_attentions``
(tests/test_fmha_merge_attentions.py:234-363).  Here the parts live on
different GPUs of one NVSwitch box: rank r holds the contiguous key range
``[kv_offset_r, kv_offset_r + len_r)``, runs the prefill kernel over all
queries against its shard with the causal diagonal shifted by ``kv_offset_r``,
and the per-rank ``(O_r, LSE_r)`` are exchanged with one NCCL all-gather over
NVLink and combined by the same LSE-merge kernel.  Query rows that lie before a
shard see none of its keys and arrive with ``LSE = -inf`` (weight 0).  For
balanced causal work a rank may hold the two key ranges of :func:`zigzag_bounds`
instead; it then merges its own two partials before the exchange.
"""

from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from .attn_bias import LowerTriangularMask
from .common import Inputs


def shard_bounds(total: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous, 128-aligned shards of ``total`` keys (the last may be short)."""
    per = -(-total // world_size)
    per = -(-per // 128) * 128
    lo = min(total, rank * per)
    return lo, min(total, lo + per)


def zigzag_bounds(total: int, world_size: int, rank: int) -> List[Tuple[int, int]]:
    """Two 128-aligned key ranges per rank: chunks ``rank`` and ``2 * world_size -
    1 - rank`` of ``2 * world_size``.  Under a causal mask every query sees all of
    an early chunk and little of a late one; pairing them gives every rank the
    same number of visible (query, key) pairs, which contiguous shards do not
    (their slowest rank does about twice the average)."""
    per = -(-total // (2 * world_size))
    per = -(-per // 128) * 128

    def span(c: int) -> Tuple[int, int]:
        lo = min(total, c * per)
        return lo, min(total, lo + per)

    return [span(rank), span(2 * world_size - 1 - rank)]


def _partial_on_gpu(q, k, v, causal: bool, kv_offset: int, scale, partial_dtype):
    from . import b200

    inp = Inputs(q, k, v, LowerTriangularMask() if causal else None, scale=scale, output_dtype=partial_dtype, is_partial=True)
    inp.validate_inputs()
    reasons = b200.FwOp.not_supported_reasons(inp)
    if reasons:
        raise ValueError("sharded attention: " + "; ".join(reasons))
    out, ctx = b200.FwOp._apply(inp, want_lse=True, kv_offset=kv_offset if causal else 0)
    return out, ctx.lse


def _merge_on_gpu(outs, lses, out_dtype):
    from .merge import merge_attentions

    return merge_attentions(outs, lses, write_lse=True, output_dtype=out_dtype)


def sharded_kv_attention_forward(
    query: torch.Tensor,
    key_shard: Union[torch.Tensor, Sequence[torch.Tensor]],
    value_shard: Union[torch.Tensor, Sequence[torch.Tensor]],
    *,
    kv_offset: Union[int, Sequence[int]],
    causal: bool = True,
    scale: Optional[float] = None,
    group: Optional[dist.ProcessGroup] = None,
    partial_dtype: Optional[torch.dtype] = None,
    partial_fn: Callable = _partial_on_gpu,
    merge_fn: Callable = _merge_on_gpu,
    exchange: str = "all_to_all",
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Every rank passes the full ``query`` ``[B, Mq, (G,) H, D]`` and its own
    key/value shard ``[B, len_r, (G,) H, D]`` starting at global key index
    ``kv_offset``.  Returns the full ``(out, lse)`` on every rank.  Several key
    ranges per rank are passed as sequences of shards and offsets (empty ranges
    are skipped); the rank merges their partials before the exchange.

    ``exchange="all_to_all"`` (when the number of queries divides by the number of
    ranks): every rank receives the partials of its slice of the queries, merges
    them and the merged slices are all-gathered; ``"all_gather"``: every rank
    receives every partial and merges all queries itself.

    ``partial_fn`` / ``merge_fn`` exist so that the exchange logic can be
    exercised with CPU stand-ins under the gloo backend.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if isinstance(key_shard, torch.Tensor):
        key_shard, value_shard, kv_offset = [key_shard], [value_shard], [kv_offset]
    if not (len(key_shard) == len(value_shard) == len(kv_offset)) or not len(key_shard):
        raise ValueError("sharded attention: key shards, value shards and offsets must pair up")
    parts = [
        partial_fn(query, k, v, causal, off, scale, partial_dtype)
        for k, v, off in zip(key_shard, value_shard, kv_offset)
        if k.shape[1] > 0
    ]
    if not parts:
        # this rank holds no keys at all: a partial of weight 0, shaped like a neighbour's (one key, then discarded)
        k0, v0 = key_shard[0], value_shard[0]
        one = lambda t: t.new_zeros((t.shape[0], 1) + tuple(t.shape[2:]))
        out_r, lse_r = partial_fn(query, one(k0), one(v0), False, 0, scale, partial_dtype)
        out_r, lse_r = torch.zeros_like(out_r), torch.full_like(lse_r, float("-inf"))
    elif len(parts) == 1:
        out_r, lse_r = parts[0]
    else:
        out_r, lse_r = merge_fn([p[0] for p in parts], [p[1] for p in parts], parts[0][0].dtype)
    if world == 1:
        return merge_fn([out_r], [lse_r], query.dtype)
    out_r = out_r.contiguous()
    lse_r = lse_r.contiguous()
    mq = out_r.shape[1]
    if exchange == "all_to_all" and mq % world == 0 and lse_r.shape[-1] == mq:
        # Every rank merges one slice of the queries: the partials of that slice come
        # in by all-to-all (1/world of an all-gather's volume), the merged slices in the
        # output dtype go round by all-gather.
        ms = mq // world
        send_o = out_r.view(out_r.shape[0], world, ms, *out_r.shape[2:]).transpose(0, 1).contiguous()      # [world, B, ms, ...]
        send_l = lse_r.view(*lse_r.shape[:-1], world, ms).movedim(-2, 0).contiguous()                        # [world, B, .., ms]
        recv_o, recv_l = torch.empty_like(send_o), torch.empty_like(send_l)
        dist.all_to_all_single(recv_o, send_o, group=group)
        dist.all_to_all_single(recv_l, send_l, group=group)
        out_s, lse_s = merge_fn(recv_o, recv_l, query.dtype)                                               # [B, ms, ...], [B, .., ms]
        out_s, lse_s = out_s.contiguous(), lse_s.contiguous()
        all_o = torch.empty((world,) + tuple(out_s.shape), dtype=out_s.dtype, device=out_s.device)
        all_l = torch.empty((world,) + tuple(lse_s.shape), dtype=lse_s.dtype, device=lse_s.device)
        dist.all_gather_into_tensor(all_o.view(-1, *out_s.shape[1:]), out_s, group=group)
        dist.all_gather_into_tensor(all_l.view(-1, *lse_s.shape[1:]), lse_s, group=group)
        out = all_o.transpose(0, 1).reshape(out_s.shape[0], mq, *out_s.shape[2:])
        lse = all_l.movedim(0, -2).reshape(*lse_s.shape[:-1], mq)
        return out, lse
    outs = torch.empty((world,) + tuple(out_r.shape), dtype=out_r.dtype, device=out_r.device)
    lses = torch.empty((world,) + tuple(lse_r.shape), dtype=lse_r.dtype, device=lse_r.device)
    # the flat form (ranks concatenated along dim 0) is the one every backend takes
    dist.all_gather_into_tensor(outs.view(-1, *out_r.shape[1:]), out_r, group=group)
    dist.all_gather_into_tensor(lses.view(-1, *lse_r.shape[1:]), lse_r, group=group)
    return merge_fn(outs, lses, query.dtype)
