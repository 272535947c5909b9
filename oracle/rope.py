"""CPU restatement of rotary embeddings with KV-cache emplacement.  TEST
INFRASTRUCTURE ONLY: nothing of the product imports this module.

Follows the reference's own slow implementations and cache bookkeeping:
  * frequencies and rotation: tests/test_rope_padded.py:53-104 (``_slow_rope``)
    and :106-145 (``_slow_rope2``, float64);
  * wavelength-dependent rescaling: tests/test_rope_padded.py:24-50
    (``apply_scaling``), with the kernel's strict lower bound of the middle band
    (xformers/ops/_triton/rope_padded_kernels.py:190-203);
  * which cache rows are written and which position a token has:
    xformers/ops/_triton/rope_padded_kernels.py:103-139.
Everything is computed in float64 and rounded once to the input dtype."""

from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch


def rope_frequencies(
    dim: int,
    theta: float = 10000.0,
    use_dynamic_scaling: bool = False,
    dynamic_old_context_len: float = 8192.0,
    dynamic_scale_factor: float = 16.0,
    dynamic_low_freq_factor: float = 1.0,
    dynamic_high_freq_factor: float = 32.0,
) -> torch.Tensor:
    """``theta^(-2j/dim)`` for j < dim/2 (float64), optionally rescaled per wavelength."""
    assert dim % 2 == 0
    freqs = [float(theta) ** (-(2.0 * j) / dim) for j in range(dim // 2)]
    if use_dynamic_scaling:
        lo = dynamic_old_context_len / dynamic_low_freq_factor
        hi = dynamic_old_context_len / dynamic_high_freq_factor
        assert lo >= hi
        for j, f in enumerate(freqs):
            wavelen = 2.0 * math.pi / f
            if wavelen > lo:
                freqs[j] = f / dynamic_scale_factor
            elif hi < wavelen <= lo:
                smooth = (dynamic_old_context_len / wavelen - dynamic_low_freq_factor) / (dynamic_high_freq_factor - dynamic_low_freq_factor)
                freqs[j] = (1.0 - smooth) * f / dynamic_scale_factor + smooth * f
    return torch.tensor(freqs, dtype=torch.float64)


def rope_rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, *, linear_scale: float = 1.0, adjacents: bool = True) -> torch.Tensor:
    """Rotate ``x [M, ..., dim]`` by ``positions [M]``: pair j turns by the angle
    ``positions / linear_scale * freqs[j]``."""
    M, dim = x.shape[0], x.shape[-1]
    ang = (positions.double() / linear_scale)[:, None] * freqs[None, :]  # [M, dim/2]
    ang = ang.reshape((M,) + (1,) * (x.ndim - 2) + (dim // 2,))
    cs, sn = ang.cos(), ang.sin()
    xd = x.double()
    if adjacents:
        re, im = xd[..., 0::2], xd[..., 1::2]
    else:
        re, im = xd[..., : dim // 2], xd[..., dim // 2 :]
    out_re, out_im = re * cs - im * sn, im * cs + re * sn
    out = torch.empty_like(xd)
    if adjacents:
        out[..., 0::2], out[..., 1::2] = out_re, out_im
    else:
        out[..., : dim // 2], out[..., dim // 2 :] = out_re, out_im
    return out.to(x.dtype)


def rope_padded(
    xq: torch.Tensor,
    xk: torch.Tensor,
    xv: torch.Tensor,
    cache_k: torch.Tensor,
    cache_v: torch.Tensor,
    q_seqlen: Sequence[int],
    kv_seqstart: Sequence[int],
    kv_seqlen: Sequence[int],
    *,
    first_seqpos: Optional[Sequence[int]] = None,
    seqpos: Optional[Sequence[int]] = None,
    linear_scale: float = 1.0,
    adjacents: bool = True,
    block_tables: Optional[Sequence[Sequence[int]]] = None,
    page_size: int = 0,
    **freq_kwargs,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``xq/xk/xv [1, M, (G,) H, dim]``, caches ``[1, rows, (G,) Hkv, dim]``.
    Returns (out_q, new cache_k, new cache_v); the inputs are not modified.
    The queries of sequence b are its last ``q_seqlen[b]`` keys: token i of them
    goes to cache row ``kv_seqstart[b] + kv_seqlen[b] - q_seqlen[b] + i``; with
    ``block_tables`` key t of sequence b is instead row
    ``block_tables[b][t // page_size] * page_size + t % page_size`` of a page pool
    (the paged layout of oracle/paged.py)."""
    assert first_seqpos is None or seqpos is None
    freqs = rope_frequencies(xq.shape[-1], **freq_kwargs)
    rows, pos = [], []
    t = 0
    for b, (ql, ks, kl) in enumerate(zip(q_seqlen, kv_seqstart, kv_seqlen)):
        for i in range(ql):
            key = kl - ql + i
            rows.append(ks + key if block_tables is None else int(block_tables[b][key // page_size]) * page_size + key % page_size)
            if seqpos is not None:
                pos.append(int(seqpos[t]))
            else:
                pos.append(key + (int(first_seqpos[b]) if first_seqpos is not None else 0))
            t += 1
    assert t == xq.shape[1]
    rows_t, pos_t = torch.tensor(rows, dtype=torch.long), torch.tensor(pos, dtype=torch.long)
    out_q = rope_rotate(xq[0], pos_t, freqs, linear_scale=linear_scale, adjacents=adjacents)[None]
    new_k, new_v = cache_k.clone(), cache_v.clone()
    new_k[0, rows_t] = rope_rotate(xk[0], pos_t, freqs, linear_scale=linear_scale, adjacents=adjacents)
    new_v[0, rows_t] = xv[0]
    return out_q, new_k, new_v
