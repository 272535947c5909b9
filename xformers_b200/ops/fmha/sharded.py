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
shard see none of its keys and arrive with ``LSE = -inf`` (weight 0).
"""

from __future__ import annotations

from typing import Callable, List, Optional, Tuple

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
    key_shard: torch.Tensor,
    value_shard: torch.Tensor,
    *,
    kv_offset: int,
    causal: bool = True,
    scale: Optional[float] = None,
    group: Optional[dist.ProcessGroup] = None,
    partial_dtype: Optional[torch.dtype] = None,
    partial_fn: Callable = _partial_on_gpu,
    merge_fn: Callable = _merge_on_gpu,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Every rank passes the full ``query`` ``[B, Mq, (G,) H, D]`` and its own
    key/value shard ``[B, len_r, (G,) H, D]`` starting at global key index
    ``kv_offset``.  Returns the full ``(out, lse)`` on every rank.

    ``partial_fn`` / ``merge_fn`` exist so that the exchange logic can be
    exercised with CPU stand-ins under the gloo backend.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    out_r, lse_r = partial_fn(query, key_shard, value_shard, causal, kv_offset, scale, partial_dtype)
    if world == 1:
        return merge_fn([out_r], [lse_r], query.dtype)
    out_r = out_r.contiguous()
    lse_r = lse_r.contiguous()
    outs = torch.empty((world,) + tuple(out_r.shape), dtype=out_r.dtype, device=out_r.device)
    lses = torch.empty((world,) + tuple(lse_r.shape), dtype=lse_r.dtype, device=lse_r.device)
    # the flat form (ranks concatenated along dim 0) is the one every backend takes
    dist.all_gather_into_tensor(outs.view(-1, *out_r.shape[1:]), out_r, group=group)
    dist.all_gather_into_tensor(lses.view(-1, *lse_r.shape[1:]), lse_r, group=group)
    return merge_fn(outs, lses, query.dtype)
