"""xFormers' int4 row-wise KV-cache format on the CPU (test oracle only).

Quantiser: benchmarks/benchmark_attn_decoding.py:38-72.  For each row (last
dim, length D) and each of ``num_groups`` equal groups: ``scale = (max-min)/15``
and ``shift = min`` stored as fp16; ``q = uint8((x - shift)/scale + 0.5) & 0xF``.
Row layout in bytes: ``[scale_0, shift_0, ..., scale_{G-1}, shift_{G-1}]``
(fp16 each, so one int32 per group with scale in the low half) followed by
``D/2`` bytes of nibbles with the even element in the low nibble.  Viewed as
int32 a row has ``num_groups + D/8`` words and element ``e`` of a word sits at
bits ``[4e, 4e+4)`` (tests/test_mem_eff_attention.py:1730-1738).

Dequantiser: ``x = q * scale + shift``.
"""

from __future__ import annotations

import numpy as np
import torch


def quantize_kv_int4(x: torch.Tensor, num_groups: int = 1) -> torch.Tensor:
    """``x [..., D]`` float -> int32 ``[..., num_groups + D/8]``."""
    D = x.shape[-1]
    assert D % (8 * num_groups) == 0
    xf = x.detach().cpu().float().reshape(*x.shape[:-1], num_groups, D // num_groups)
    mx = xf.max(dim=-1, keepdim=True).values
    mn = xf.min(dim=-1, keepdim=True).values
    scale = ((mx - mn) / 15).to(torch.float16)
    shift = mn.to(torch.float16)
    qv = ((xf - shift.float()) / scale.float() + 0.5).to(torch.uint8) & 0xF
    packed = qv[..., ::2] + (qv[..., 1::2] << 4)  # uint8 [..., G, D/G/2]
    ss = torch.cat([scale.view(torch.uint8), shift.view(torch.uint8)], dim=-1)  # [..., G, 4]
    row = torch.cat([ss.flatten(start_dim=-2), packed.flatten(start_dim=-2)], dim=-1)
    return row.contiguous().view(torch.int32)


def dequantize_kv_int4(xq: torch.Tensor, num_groups: int = 1) -> torch.Tensor:
    """int32 ``[..., num_groups + D/8]`` -> float32 ``[..., D]``; integer
    unpacking done in numpy on the raw words."""
    w = xq.detach().cpu().contiguous().numpy().view(np.uint32)
    meta = w[..., :num_groups]
    scale = (meta & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float32)
    shift = (meta >> 16).astype(np.uint16).view(np.float16).astype(np.float32)
    body = w[..., num_groups:]
    sh = (4 * np.arange(8, dtype=np.uint32)).reshape((1,) * body.ndim + (8,))
    nib = ((body[..., None] >> sh) & 0xF).astype(np.float32)  # [..., D/8, 8]
    nib = nib.reshape(*body.shape[:-1], num_groups, -1)
    out = nib * scale[..., None] + shift[..., None]
    return torch.from_numpy(out.reshape(*body.shape[:-1], -1).copy())
