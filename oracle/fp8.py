"""Row-wise fp8 KV cache format -- TEST INFRASTRUCTURE ONLY.

CPU restatement of the helpers the reference's tests use to build and read the
format (tests/utils.py:311-340): asymmetric per-row quantisation to e4m3 with a
shift (the row mean) and a scale, both carried as fp16 and packed into one int32
per row ``[scale | shift << 16]``; values are packed four to an int32 word.
"""

from __future__ import annotations

from typing import Tuple

import torch

FP8 = torch.float8_e4m3fn


def quantize_fp8_asymmetric(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``x`` [rows, D] -> (e4m3 values [rows, D], scale [rows] fp32, shift [rows])
    with ``x ~ fp8 * scale + shift``, exactly as the reference's test helper
    does it (tests/utils.py:320-333): shift = row mean, scale = fp8_max /
    max|x - shift| (1 where that is infinite), values = (x - shift) / scale."""
    max_fp8 = torch.finfo(FP8).max
    shift = x.float().mean(dim=1)
    centered = x.float() - shift[:, None]
    row_max = centered.abs().max(dim=-1)[0]
    scale = max_fp8 * row_max.float().pow(-1)
    scale = torch.nan_to_num(scale, posinf=1)
    q = (centered / scale[:, None]).to(FP8)
    return q, scale, shift


def dequantize_fp8_asymmetric(q: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    """tests/utils.py:336-340."""
    return q.float() * scale.float()[..., None] + shift.float()[..., None]


def combine_scale_shift(scale: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    """One int32 per row: fp16 scale in the low half, fp16 shift in the high
    half (tests/utils.py:311-317)."""
    return torch.stack([scale.half(), shift.half()], dim=-1).contiguous().view(torch.int32).squeeze(-1)


def split_scale_shift(words: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    h = words.contiguous().view(torch.int32).unsqueeze(-1).view(torch.float16)
    return h[..., 0].float(), h[..., 1].float()


def pack_fp8_words(q: torch.Tensor) -> torch.Tensor:
    """e4m3 [.., D] -> int32 [.., D/4] (tests/utils.py:168)."""
    return q.contiguous().view(torch.int32)


def unpack_fp8_words(words: torch.Tensor) -> torch.Tensor:
    return words.contiguous().view(FP8)
