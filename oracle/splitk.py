"""Split-K (flash-decoding) attention algebra on the CPU (test oracle only).

The key axis is cut into ``split_k`` equal chunks; each chunk yields an
un-normalised partial ``(acc, row_max, row_sumexp)``; partials are folded in
order with the running-max rescale.  Follows tests/test_splitk_reference.py:42-154,
including the NaN guard for chunks without visible keys (:142-144).
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from .ref_attention import _materialize


def _splitk_bmk(q, k, v, bias, scale, split_k):
    q = q.float()
    k = k.float()
    v = v.float()
    if scale is None:
        scale = q.shape[-1] ** -0.5
    q = q * scale
    n = k.shape[-2]
    size = max(1, -(-n // split_k))
    acc = torch.zeros(q.shape[:-1] + (v.shape[-1],))
    g_max = torch.full(q.shape[:-1] + (1,), -float("inf"))
    g_sum = torch.zeros(q.shape[:-1] + (1,))
    for lo in range(0, n, size):
        hi = min(n, lo + size)
        s = q @ k[..., lo:hi, :].transpose(-2, -1)
        vv = v[..., lo:hi, :]
        if bias is not None:
            hidden = torch.isneginf(bias[..., lo:hi]).expand_as(s)
            s = torch.where(hidden, torch.full_like(s, -float("inf")), s + bias[..., lo:hi])
            vv = torch.where(hidden.all(dim=-2).unsqueeze(-1), torch.zeros_like(vv), vv)
        l_max = s.max(dim=-1, keepdim=True).values
        p = torch.exp(s - torch.where(torch.isfinite(l_max), l_max, torch.zeros_like(l_max)))
        l_sum = p.sum(dim=-1, keepdim=True)
        l_acc = p @ vv
        alpha = torch.exp(-torch.abs(l_max - g_max)).nan_to_num(1.0)
        pick_new = l_max < g_max
        new_c = torch.where(pick_new, alpha, torch.ones_like(alpha))
        cur_c = torch.where(pick_new, torch.ones_like(alpha), alpha)
        acc = acc * cur_c + l_acc * new_c
        g_sum = g_sum * cur_c + l_sum * new_c
        g_max = torch.maximum(l_max, g_max)
    return acc / torch.where(g_sum > 0, g_sum, torch.ones_like(g_sum))


def ref_attention_splitk(q, k, v, attn_bias: Any = None, scale: Optional[float] = None, split_k: int = 2) -> torch.Tensor:
    """Same layouts as :func:`oracle.ref_attention`; float32 output in q's layout."""
    q, k, v = q.detach().cpu(), k.detach().cpu(), v.detach().cpu()
    if q.ndim == 5:
        return torch.stack(
            [ref_attention_splitk(q[:, :, g], k[:, :, g], v[:, :, g], attn_bias, scale, split_k) for g in range(q.shape[2])],
            dim=2,
        )
    if q.ndim == 3:
        bias = _materialize(attn_bias, (q.shape[0], q.shape[1], k.shape[1]), q.device)
        return _splitk_bmk(q, k, v, bias, scale, split_k)
    B, Mq, H, K = q.shape
    Mkv = k.shape[1]
    bias = _materialize(attn_bias, (B, H, Mq, Mkv), q.device)
    if bias is not None:
        while bias.ndim < 4:
            bias = bias.unsqueeze(0)
        bias = bias.expand(B, H, Mq, Mkv).reshape(B * H, Mq, Mkv)
    f = lambda t: t.permute(0, 2, 1, 3).reshape(B * H, t.shape[1], t.shape[-1])
    out = _splitk_bmk(f(q), f(k), f(v), bias, scale, split_k)
    return out.reshape(B, H, Mq, -1).permute(0, 2, 1, 3).contiguous()
