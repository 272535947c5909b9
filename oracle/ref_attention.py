"""fp32 reference attention on the CPU (test oracle only).

``O = softmax(Q K^T * scale + bias) V`` and ``LSE = logsumexp(Q K^T * scale +
bias)`` in natural log, computed densely in float32, following
tests/test_mem_eff_attention.py:664-682 (scores from ``q / sqrt(K)``, additive
materialised bias, ``logsumexp(-1)``) and benchmarks/benchmark_attn_decoding.py:335-343.

``attn_bias`` may be ``None``, an additive tensor broadcastable to
``[B, H, Mq, Mkv]`` (4-D inputs) / ``[B*H, Mq, Mkv]`` (3-D inputs), or any
object with ``materialize(shape, dtype=, device=)``.

Rows without a visible key produce ``out = 0`` and ``lse = -inf``.
"""

from __future__ import annotations

from typing import Any, Optional, Tuple

import torch


def _materialize(attn_bias: Any, shape, device) -> Optional[torch.Tensor]:
    if attn_bias is None:
        return None
    if isinstance(attn_bias, torch.Tensor):
        return attn_bias.to(device=device, dtype=torch.float32)
    return attn_bias.materialize(shape, dtype=torch.float32, device=device)


def _attention_bmk(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    bias: Optional[torch.Tensor],
    scale: Optional[float],
) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [N, Mq, K], k [N, Mkv, K], v [N, Mkv, Kv] -> out [N, Mq, Kv], lse [N, Mq]."""
    q = q.float()
    k = k.float()
    v = v.float()
    if scale is None:
        scale = q.shape[-1] ** -0.5
    s = (q * scale) @ k.transpose(-2, -1)
    if bias is not None:
        # masked-out keys may hold NaN or garbage (padding): they must not
        # leak, so mask by select, never by arithmetic
        # (tests/test_mem_eff_attention.py:3104-3111)
        hidden = torch.isneginf(bias).expand_as(s)
        s = torch.where(hidden, torch.full_like(s, -float("inf")), s + bias)
        dead_keys = hidden.all(dim=-2)  # [N, Mkv]: visible to no query at all
        v = torch.where(dead_keys.unsqueeze(-1), torch.zeros_like(v), v)
    lse = torch.logsumexp(s, dim=-1)
    if s.shape[-1]:
        row_max = s.max(dim=-1, keepdim=True).values
    else:
        row_max = s.new_zeros(s.shape[:-1] + (1,))
    row_max = torch.where(torch.isfinite(row_max), row_max, torch.zeros_like(row_max))
    p = torch.exp(s - row_max)
    denom = p.sum(dim=-1, keepdim=True)
    out = (p @ v) / torch.where(denom > 0, denom, torch.ones_like(denom))
    if s.shape[-1] == 0:
        lse = torch.full(s.shape[:-1], -float("inf"))
    return out, lse


def ref_attention_with_lse(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    attn_bias: Any = None,
    scale: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Layouts as in the reference API (tests/test_mem_eff_attention.py:420-440):
    3-D BMK ``[B*H, M, K]``, 4-D BMHK ``[B, M, H, K]``, 5-D BMGHK
    ``[B, M, G, H, K]``.  Returns ``out`` in q's layout (float32) and ``lse``
    as ``[B*H, Mq]``, ``[B, H, Mq]`` or ``[B, G, H, Mq]``."""
    q = q.detach().cpu()
    k = k.detach().cpu()
    v = v.detach().cpu()
    if q.ndim == 3:
        bias = _materialize(attn_bias, (q.shape[0], q.shape[1], k.shape[1]), q.device)
        return _attention_bmk(q, k, v, bias, scale)
    if q.ndim == 5:
        B, Mq, G, H, K = q.shape
        outs, lses = [], []
        for g in range(G):
            bg = attn_bias
            if isinstance(attn_bias, torch.Tensor) and attn_bias.ndim == 5:
                bg = attn_bias[:, g]
            o, l = ref_attention_with_lse(q[:, :, g], k[:, :, g], v[:, :, g], bg, scale)
            outs.append(o)
            lses.append(l)
        return torch.stack(outs, dim=2), torch.stack(lses, dim=1)
    assert q.ndim == 4
    B, Mq, H, K = q.shape
    Mkv = k.shape[1]
    bias = _materialize(attn_bias, (B, H, Mq, Mkv), q.device)
    if bias is not None:
        while bias.ndim < 4:
            bias = bias.unsqueeze(0)
        bias = bias.expand(B, H, Mq, Mkv).reshape(B * H, Mq, Mkv)
    tq = q.permute(0, 2, 1, 3).reshape(B * H, Mq, K)
    tk = k.permute(0, 2, 1, 3).reshape(B * H, Mkv, K)
    tv = v.permute(0, 2, 1, 3).reshape(B * H, Mkv, v.shape[-1])
    out, lse = _attention_bmk(tq, tk, tv, bias, scale)
    out = out.reshape(B, H, Mq, -1).permute(0, 2, 1, 3).contiguous()
    return out, lse.reshape(B, H, Mq)


def ref_attention(q, k, v, attn_bias=None, drop_mask=None, p=0.0, scale=None) -> torch.Tensor:
    """Positional signature of the reference helper
    (xformers/attn_bias_utils.py:7-12; positional use tests/test_mem_eff_attention.py:1026).
    Dropout is outside the forward hot path and is rejected."""
    assert drop_mask is None and p == 0.0, "dropout is not part of the forward hot path"
    return ref_attention_with_lse(q, k, v, attn_bias, scale)[0]


def ref_attention_bmhk(q, k, v, attn_bias=None, scale=None) -> torch.Tensor:
    assert q.ndim == 4
    return ref_attention_with_lse(q, k, v, attn_bias, scale)[0]
