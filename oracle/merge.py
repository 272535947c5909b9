"""LSE-weighted merge of partial attentions on the CPU (test oracle only).

``m = max_s LSE_s; w_s = exp(LSE_s - m); out = sum_s w_s O_s / sum_s w_s;
lse = m + log sum_s w_s`` -- tests/test_fmha_merge_attentions.py:513-538 and
benchmarks/benchmark_merge_attentions.py:12-31.  A partial whose LSE is
``-inf`` (no visible key) gets weight exactly 0 by select; if every partial of
a row is ``-inf`` the row is ``out = 0, lse = -inf``
(tests/test_fmha_merge_attentions.py:401-405,464-485).
"""

from __future__ import annotations

from typing import Tuple

import torch


def merge_attentions_ref(attn_split: torch.Tensor, lse_split: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``attn_split [S, B, M, (G,) H, D]``, ``lse_split [S, B, (G,) H, M]`` ->
    ``out [B, M, (G,) H, D]`` float32, ``lse [B, (G,) H, M]`` float32."""
    attn_split = attn_split.detach().cpu().float()
    lse_split = lse_split.detach().cpu().float()
    bmghk = attn_split.ndim == 6
    if not bmghk:
        attn_split = attn_split.unsqueeze(3)
        lse_split = lse_split.unsqueeze(2)
    lse_t = lse_split.permute(0, 1, 4, 2, 3).unsqueeze(-1)  # [S, B, M, G, H, 1]
    m = lse_t.max(dim=0).values
    m_safe = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    w = torch.exp(lse_t - m_safe)
    w = torch.where(torch.isneginf(lse_t), torch.zeros_like(w), w)
    den = w.sum(dim=0)
    contrib = torch.where(w > 0, w * attn_split, torch.zeros_like(attn_split))
    num = contrib.sum(dim=0)
    out = num / torch.where(den > 0, den, torch.ones_like(den))
    lse = torch.where(den > 0, m_safe + torch.log(den), torch.full_like(den, -float("inf")))
    lse = lse.squeeze(-1).permute(0, 2, 3, 1).contiguous()  # [B, G, H, M]
    if not bmghk:
        out = out.squeeze(2)
        lse = lse.squeeze(1)
    return out, lse
