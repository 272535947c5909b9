"""Rotary embeddings + KV-cache emplacement for a concatenated batch, behind the
reference's ``xformers.ops.rope_padded`` signature (xformers/ops/rope_padded.py:16-36).

The work is one CUDA kernel (``csrc/rope_padded.cu``) reached through the C
entry point ``xfb200_rope_padded``; there is no other implementation behind
this function."""

from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple, Union

import torch

from .. import _lib
from .fmha.attn_bias import BlockDiagonalCausalWithOffsetPaddedKeysMask, PagedBlockDiagonalCausalWithOffsetPaddedKeysMask

_DTYPES = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}


def _strides3(t: torch.Tensor, ndim: int) -> Tuple[int, int, int]:
    """(token, group, head) strides in elements of a [1, M, (G,) H, D] tensor."""
    s = t.stride()
    return s[1], (s[2] if ndim == 5 else 0), s[-2]


def rope_padded(
    xq: torch.Tensor,
    xk: torch.Tensor,
    xv: torch.Tensor,
    cache_k: torch.Tensor,
    cache_v: torch.Tensor,
    attn_bias: Union[BlockDiagonalCausalWithOffsetPaddedKeysMask, PagedBlockDiagonalCausalWithOffsetPaddedKeysMask],
    *,
    theta: float = 10000.0,
    linear_scale: float = 1.0,
    use_dynamic_scaling: bool = False,
    dynamic_old_context_len: float = 8192.0,
    dynamic_scale_factor: float = 16.0,
    dynamic_low_freq_factor: float = 1.0,
    dynamic_high_freq_factor: float = 32.0,
    out_q: Optional[torch.Tensor] = None,
    first_seqpos: Optional[torch.Tensor] = None,
    seqpos: Optional[torch.Tensor] = None,
    adjacents: bool = True,
    internal_dtype: str = "",
    cache_k_scale_shift: Optional[torch.Tensor] = None,
    cache_v_scale_shift: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Rotate ``xq`` into ``out_q`` (returned), rotate ``xk`` into its rows of
    ``cache_k`` and copy ``xv`` into the same rows of ``cache_v`` (both caches
    MODIFIED IN PLACE), so that ``memory_efficient_attention_forward(out_q,
    cache_k, cache_v, attn_bias)`` can follow.

    Shapes: ``xq [1, M, (G,) Hq, D]``, ``xk``/``xv`` ``[1, M, (G,) Hkv, D]``,
    caches ``[1, rows, (G,) Hkv, D]`` with ``M`` / ``rows`` the totals of
    ``attn_bias``; a single kv head may be given expanded (head stride 0).  The
    queries of a sequence are its last keys.  ``first_seqpos [batch]`` shifts a
    sequence's positions, ``seqpos [M]`` gives every token's position;
    ``adjacents`` pairs features (2j, 2j+1), otherwise (j, j + D/2);
    ``linear_scale`` divides positions; ``use_dynamic_scaling`` rescales
    frequencies per wavelength; ``internal_dtype`` "" / "f32" computes angles in
    float32, "f64" in float64.  Errors follow xformers/ops/rope_padded.py:97-233.

    Beyond the reference: with a ``PagedBlockDiagonalCausalWithOffsetPaddedKeysMask``
    the caches are page pools ``[1, pages * page_size, (G,) Hkv, D]`` and key t of
    sequence b is written to row ``block_tables[b, t // page_size] * page_size +
    t % page_size``, the layout the paged decode operator reads; and int32 caches
    ``[..., 1 + D // 8]`` are int4 row-wise caches (one quantisation group,
    benchmarks/benchmark_attn_decoding.py:38-72): the rotated keys and the values
    are quantised as they are written (bf16 / f16 inputs).  With
    ``cache_k_scale_shift`` / ``cache_v_scale_shift`` (int32, the caches' shape
    without the last axis) int32 caches ``[..., D // 4]`` are fp8 row-wise caches
    (``InputsFp8``, tests/utils.py:134-222): four e4m3 values per word, ``x ~ fp8 *
    scale + shift`` with the row's (fp16 scale | fp16 shift << 16) word written to
    those tensors (shift = row mean, scale = max |x - shift| / 448).
    """
    if torch.is_grad_enabled() and (
        xq.requires_grad or xk.requires_grad or xv.requires_grad or cache_k.requires_grad or cache_v.requires_grad or out_q is not None
    ):
        raise ValueError("Gradients not supported.")
    n_total_queries = attn_bias.q_seqinfo.seqstart_py[-1]
    paged = isinstance(attn_bias, PagedBlockDiagonalCausalWithOffsetPaddedKeysMask)
    if paged:
        if cache_k.ndim < 2 or cache_k.shape[1] % attn_bias.page_size:
            raise ValueError(f"unexpected cache_k shape {tuple(cache_k.shape)}: rows must be a whole number of pages of {attn_bias.page_size}")
        cache_length = cache_k.shape[1]
    else:
        cache_length = attn_bias.k_seqinfo.seqstart_py[-1]
    ndim = xq.ndim
    if ndim not in [4, 5]:
        raise ValueError("Unexpected xq dimension")
    n_kv_heads = xk.shape[-2]
    expected_kv_heads = n_kv_heads
    if xk.stride(-2) == 0:
        n_kv_heads = 1
    expected_cache_heads = n_kv_heads
    if n_kv_heads == 1 and cache_k.stride(-2) == 0:
        expected_cache_heads = cache_k.shape[-2]  # one kv head: expanded before or after, either is fine

    bsz, q_len = xq.shape[:2]
    n_q_heads, dim = xq.shape[-2:]
    n_groups = xq.shape[2] if ndim == 5 else 1
    mid = (n_groups,) if ndim == 5 else ()
    assert q_len == n_total_queries
    want_x = (1, n_total_queries) + mid + (expected_kv_heads, dim)
    # int32 caches are int4 row-wise caches with one quantisation group: a scale/shift word and dim / 8 words of nibbles
    fp8_cache = cache_k_scale_shift is not None or cache_v_scale_shift is not None
    int4_cache = cache_k.dtype == torch.int32 and not fp8_cache
    want_cache = (1, cache_length) + mid + (expected_cache_heads, dim // 4 if fp8_cache else 1 + dim // 8 if int4_cache else dim)
    if tuple(xk.shape) != want_x:
        raise ValueError(f"unexpected k shape {tuple(xk.shape)}: expected {want_x}")
    if tuple(xv.shape) != want_x:
        raise ValueError(f"unexpected v shape {tuple(xv.shape)}: expected {want_x}")
    if tuple(cache_k.shape) != want_cache:
        raise ValueError(f"unexpected cache_k shape {tuple(cache_k.shape)}: expected {want_cache}")
    if tuple(cache_v.shape) != want_cache:
        raise ValueError(f"unexpected cache_v shape {tuple(cache_v.shape)}: expected {want_cache}")
    if bsz != 1:
        raise ValueError("Expected batch size dimension to be 1 as batches should be concatenated.")
    for name, t in (("q", xq), ("k", xk), ("v", xv), ("cache_k", cache_k), ("cache_v", cache_v)):
        if t.stride(-1) != 1:
            raise ValueError(f"Each {name} head must be contiguous")
    if out_q is None:
        out_q = xq.new_empty(xq.shape)
    else:
        if out_q.shape != xq.shape:
            raise ValueError("Unexpected shape of out_q")
        if out_q.stride(-1) != 1:
            raise ValueError("Each out_q head must be contiguous")

    logical_bsz = len(attn_bias.q_seqinfo.seqstart_py) - 1
    if first_seqpos is not None and seqpos is not None:
        raise ValueError("seqpos and first_seqpos may not both be provided")
    positions = first_seqpos if first_seqpos is not None else seqpos
    if first_seqpos is not None and first_seqpos.shape != (logical_bsz,):
        raise ValueError(f"first_seqpos.shape {tuple(first_seqpos.shape)} but ({logical_bsz},) expected.")
    if seqpos is not None and seqpos.shape != (n_total_queries,):
        raise ValueError(f"seqpos.shape {tuple(seqpos.shape)} but ({n_total_queries},) expected.")
    if positions is not None and positions.dtype not in (torch.int32, torch.int64):
        raise ValueError(f"sequence positions must be int32 or int64, got {positions.dtype}")

    device = xq.device
    seqstartq = attn_bias.q_seqinfo.seqstart
    seqstartk = attn_bias.k_seqinfo.seqstart
    seqlenk = attn_bias.k_seqinfo.seqlen
    if seqstartq.device != device or seqstartk.device != device or seqlenk.device != device:
        raise ValueError("`attn_bias` must be on the same device as the other inputs")
    if internal_dtype not in ("", "f32", "f64"):
        raise ValueError(f"internal_dtype {internal_dtype!r}: expected '', 'f32' or 'f64'")
    if device.type != "cuda":
        raise ValueError(f"rope_padded needs CUDA tensors, got device={device}")
    tensors = (xq, xk, xv, cache_k, cache_v, out_q)
    if xq.dtype not in _DTYPES or any(t.dtype != xq.dtype for t in (xk, xv, out_q)):
        raise ValueError(f"rope_padded: xq, xk, xv and out_q must share one dtype of bf16 / f16 / f32, got {[t.dtype for t in tensors]}")
    if cache_v.dtype != cache_k.dtype or cache_k.dtype not in (xq.dtype, torch.int32):
        raise ValueError(f"rope_padded: the caches must have the dtype of the inputs or be int32 (int4 row-wise), got {cache_k.dtype}, {cache_v.dtype}")
    if (int4_cache or fp8_cache) and (xq.dtype == torch.float32 or dim % 8):
        raise ValueError("rope_padded: a quantised cache needs bf16 / f16 inputs and dim a multiple of 8")
    if fp8_cache:
        if cache_k.dtype != torch.int32:
            raise ValueError("rope_padded: fp8 caches are int32 tensors of four e4m3 values per word")
        for name, t in (("cache_k_scale_shift", cache_k_scale_shift), ("cache_v_scale_shift", cache_v_scale_shift)):
            if t is None or t.dtype != torch.int32 or tuple(t.shape) != tuple(cache_k.shape[:-1]) or t.device != device:
                raise ValueError(f"rope_padded: {name} must be an int32 tensor of shape {tuple(cache_k.shape[:-1])} on the device of the caches")
    if any(t.device != device for t in tensors) or (positions is not None and positions.device != device):
        raise ValueError("rope_padded: all tensors must be on one device")
    for t in (seqstartq, seqstartk, seqlenk):
        assert t.dtype == torch.int32 and t.is_contiguous()

    p = _lib.RopeParams()
    p.xq, p.xk, p.xv, p.cache_k, p.cache_v, p.out_q = (t.data_ptr() for t in tensors)
    p.seqstart_q, p.seqstart_k, p.seqlen_k = seqstartq.data_ptr(), seqstartk.data_ptr(), seqlenk.data_ptr()
    p.first_seqpos = first_seqpos.data_ptr() if first_seqpos is not None else None
    p.seqpos = seqpos.data_ptr() if seqpos is not None else None
    p.seqpos_stride = positions.stride(0) if positions is not None else 0
    p.seqpos_i64 = int(positions is not None and positions.dtype == torch.int64)
    p.dtype = _DTYPES[xq.dtype]
    p.batch, p.max_q_per_seq = logical_bsz, attn_bias.q_seqinfo.max_seqlen
    p.q_heads, p.kv_heads, p.groups, p.dim = n_q_heads, n_kv_heads, n_groups, dim
    p.adjacents, p.use_dynamic_scaling, p.internal_f64 = int(adjacents), int(use_dynamic_scaling), int(internal_dtype == "f64")
    p.cache_format = 2 if fp8_cache else int(int4_cache)
    if fp8_cache:
        p.k_scale_shift, p.v_scale_shift = cache_k_scale_shift.data_ptr(), cache_v_scale_shift.data_ptr()
        p.kss_m, p.kss_g, p.kss_h = _strides3(cache_k_scale_shift.unsqueeze(-1), ndim)
        p.vss_m, p.vss_g, p.vss_h = _strides3(cache_v_scale_shift.unsqueeze(-1), ndim)
    p.theta, p.linear_scale = theta, linear_scale
    p.dynamic_old_context_len, p.dynamic_scale_factor = dynamic_old_context_len, dynamic_scale_factor
    p.dynamic_low_freq_factor, p.dynamic_high_freq_factor = dynamic_low_freq_factor, dynamic_high_freq_factor
    p.xq_m, p.xq_g, p.xq_h = _strides3(xq, ndim)
    p.xk_m, p.xk_g, p.xk_h = _strides3(xk, ndim)
    p.xv_m, p.xv_g, p.xv_h = _strides3(xv, ndim)
    p.oq_m, p.oq_g, p.oq_h = _strides3(out_q, ndim)
    p.ck_m, p.ck_g, p.ck_h = _strides3(cache_k, ndim)
    p.cv_m, p.cv_g, p.cv_h = _strides3(cache_v, ndim)
    if paged:
        tables = attn_bias.block_tables
        if tables.device != device or tables.dtype != torch.int32 or tables.ndim != 2 or tables.shape[0] != logical_bsz or tables.stride(1) != 1:
            raise ValueError("`attn_bias.block_tables` must be an int32 [batch, pages] tensor with unit inner stride on the same device as the other inputs")
        p.block_tables, p.block_tables_stride, p.page_size = tables.data_ptr(), tables.stride(0), attn_bias.page_size
        p.pages_per_seq = tables.shape[1]
    with torch.cuda.device(device):
        rc = _lib.load().xfb200_rope_padded(C.byref(p), C.c_void_p(torch.cuda.current_stream(device).cuda_stream))
    _lib.check(rc, "rope_padded")
    return out_q
