"""Split-K decode operator for B200 (``fmha.b200_splitk.FwOp``).

CUDA replacement of the reference's Triton flash-decoding operator
(``fmha.triton_splitk.FwOp`` and its fixed-split variants ``FwOp_S1 .. FwOp_S128``,
xformers/ops/fmha/triton_splitk.py:18-27): few queries per sequence against a
long KV cache, padded or paged, in bf16/f16 or in the int4 row-wise format
(K/V of dtype int32 whose last dim is ``D/8 + NUM_GROUPS``,
tests/test_mem_eff_attention.py:1700-1707) or in the row-wise fp8 format
(``InputsFp8``, tests/utils.py:134-340).  The split count is chosen from
static shape quantities only, never from device-side lengths, so a call can be
captured in a CUDA graph and replayed after the lengths changed.
"""

from __future__ import annotations

import ctypes as C
from typing import Any, List, Optional, Tuple

import torch

from ... import _lib
from .attn_bias import (
    BlockDiagonalCausalLocalAttentionPaddedKeysMask,
    PagedBlockDiagonalCausalLocalPaddedKeysMask,
    BlockDiagonalCausalWithOffsetGappyKeysMask,
    BlockDiagonalCausalWithOffsetPaddedKeysMask,
    BlockDiagonalGappyKeysMask,
    BlockDiagonalPaddedKeysMask,
    PagedBlockDiagonalCausalWithOffsetGappyKeysMask,
    PagedBlockDiagonalCausalWithOffsetPaddedKeysMask,
    PagedBlockDiagonalGappyKeysMask,
    PagedBlockDiagonalPaddedKeysMask,
)
from .common import AttentionFwOpBase, Context, Inputs, InputsFp8, check_lastdim_alignment_stride1

_DTYPE_CODE = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}
_SM_COUNT = 148
_MAX_ROWS_PER_KV_HEAD = 64


def _geometry(inp: Inputs):
    """Normalise to: q [rows, kv_heads, q_per_kv, D], k/v [rows, kv_heads, W].

    BMGHK with K/V broadcast over H (stride 0)  -> kv_heads = G, q_per_kv = H (GQA)
    BMHK  with K/V broadcast over H (stride 0)  -> kv_heads = 1, q_per_kv = H (MQA)
    otherwise every query head has its own KV head -> kv_heads = G*H, q_per_kv = 1
    """
    q, k, v = inp.get_qkv_in_bmghk()
    B, Mq, G, H, D = q.shape
    broadcast = H > 1 and k.stride(3) == 0 and v.stride(3) == 0
    return q, k, v, broadcast


_LOCAL_BIASES = (BlockDiagonalCausalLocalAttentionPaddedKeysMask, PagedBlockDiagonalCausalLocalPaddedKeysMask)


def _debug_check_decode(bias, p, k: torch.Tensor) -> None:
    """Host-side validation of the device arrays a decode call trusts
    (``XFB200_DEBUG_CHECKS=1``): lengths within their slots, page ids within the pool."""
    if not isinstance(bias, (BlockDiagonalPaddedKeysMask, PagedBlockDiagonalPaddedKeysMask)):
        return
    lens = bias.k_seqinfo.seqlen.cpu().tolist()
    if any(n < 0 or n > p.kv_padding for n in lens):
        raise ValueError(f"kv_seqlen {lens} does not fit the slot of {p.kv_padding} keys")
    if isinstance(bias, PagedBlockDiagonalPaddedKeysMask):
        num_pages = k.shape[1] // bias.page_size
        table = bias.block_tables.cpu()
        for b, n in enumerate(lens):
            first = 0
            if isinstance(bias, PagedBlockDiagonalGappyKeysMask):
                first = int(bias.slot_starts()[b])
            used = table[b, first // bias.page_size : -(-(first + n) // bias.page_size)] if n > 0 else table[b, :0]
            if used.numel() and (int(used.min()) < 0 or int(used.max()) >= num_pages):
                raise ValueError(f"block_tables[{b}] names a page outside the pool of {num_pages} pages")
    else:
        starts = bias.k_seqinfo.seqstart.cpu().tolist()
        for b, n in enumerate(lens):
            if starts[b] < 0 or starts[b] + n > k.shape[1]:
                raise ValueError(f"sequence {b}: keys [{starts[b]}, {starts[b] + n}) leave the {k.shape[1]} rows of the cache")


def decode_device_status(device=None) -> int:
    """Code of the first wait a decode kernel gave up on ``device`` since the last
    call (0 = none), cleared by the call.  Synchronises the current stream."""
    dev = torch.device("cuda" if device is None else device)
    with torch.cuda.device(dev):
        st = C.c_int32(0)
        rc = _lib.load().xfb200_decode_device_status(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(st))
        if rc != _lib.XFB200_E_DEVICE:
            _lib.check(rc, "decode_device_status")
    return st.value


def check_device_status(device=None) -> None:
    """Raises ``RuntimeError`` when a decode kernel gave up a wait on ``device``; clears the status."""
    dev = torch.device("cuda" if device is None else device)
    with torch.cuda.device(dev):
        st = C.c_int32(0)
        rc = _lib.load().xfb200_decode_device_status(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(st))
        _lib.check(rc, "b200_splitk.FwOp")


class FwOp(AttentionFwOpBase):
    """Flash-decoding on sm_100a.  ``SPLIT_K = None`` picks the split count."""

    OPERATOR = _lib.load().xfb200_decode_forward if _lib.is_built() else None
    NAME = "b200_splitKF"
    SUPPORTED_DTYPES = {torch.bfloat16, torch.half}
    SUPPORTED_MAX_K = 128
    SUPPORTED_MIN_K = 64
    SUPPORTED_ATTN_BIAS_TYPES = (
        type(None),
        BlockDiagonalPaddedKeysMask,
        BlockDiagonalCausalWithOffsetPaddedKeysMask,
        PagedBlockDiagonalPaddedKeysMask,
        PagedBlockDiagonalCausalWithOffsetPaddedKeysMask,
        BlockDiagonalGappyKeysMask,
        BlockDiagonalCausalWithOffsetGappyKeysMask,
        PagedBlockDiagonalGappyKeysMask,
        PagedBlockDiagonalCausalWithOffsetGappyKeysMask,
        BlockDiagonalCausalLocalAttentionPaddedKeysMask,
        PagedBlockDiagonalCausalLocalPaddedKeysMask,
        torch.Tensor,
    )
    SUPPORTS_DROPOUT = False
    SUPPORTS_CUSTOM_SCALE = True
    SUPPORTS_BMGHK = True
    SUPPORTS_OUTPUT_DTYPE = True
    SUPPORTS_PARTIAL = True
    VARLEN_LSE_PACKED = True
    _TEST_K = [64, 128]

    SPLIT_K: Optional[int] = None
    NUM_GROUPS = 1  # quantisation groups per int4 row
    AUTOTUNE = False  # kept for API parity; there is nothing to autotune

    @classmethod
    def shape_not_supported_reasons(cls, Mq: int, Mkv: int, K: int, Kv: int) -> List[str]:
        reasons = super().shape_not_supported_reasons(Mq, Mkv, K, Kv)
        if K not in (64, 128):
            reasons.append(f"head dim {K} not in (64, 128)")
        return reasons

    @classmethod
    def not_supported_reasons(cls, d: Inputs) -> List[str]:
        reasons = super().not_supported_reasons(d)
        if d.query.ndim not in (4, 5):
            reasons.append("needs BMHK or BMGHK inputs")
            return reasons
        quantized = d.key.dtype == torch.int32
        K = d.query.shape[-1]
        if K not in (64, 128):
            reasons.append(f"head dim {K} not in (64, 128)")
        fp8 = isinstance(d, InputsFp8)
        if fp8:
            if not quantized or d.value.dtype != torch.int32:
                reasons.append("fp8 K/V must be passed as int32 words of four e4m3 values")
            elif d.key.shape[-1] != K // 4 or d.value.shape[-1] != K // 4:
                reasons.append(f"fp8 K/V rows must have {K // 4} int32 words, got {d.key.shape[-1]}")
            if K != 128:
                reasons.append("fp8 caches are supported for head dim 128 only")
            for name, t in (("k_fp8_scale_shift", d.k_fp8_scale_shift), ("v_fp8_scale_shift", d.v_fp8_scale_shift)):
                if t is None or t.dtype != torch.int32 or tuple(t.shape) != tuple(d.key.shape[:-1]):
                    reasons.append(f"{name} must be an int32 tensor of shape key.shape[:-1]")
        elif quantized:
            if d.value.dtype != torch.int32:
                reasons.append("key is int32 (quantised) but value is not")
            if cls.NUM_GROUPS not in (1, 2, 4, 8) or K // cls.NUM_GROUPS < 16:
                reasons.append(f"int4 caches need 1, 2, 4 or 8 quantisation groups of at least 16 elements per row, got NUM_GROUPS={cls.NUM_GROUPS}")
            elif d.key.shape[-1] != K // 8 + cls.NUM_GROUPS or d.value.shape[-1] != d.key.shape[-1]:
                reasons.append(f"int4 K/V rows must have {K // 8 + cls.NUM_GROUPS} int32 words, got {d.key.shape[-1]}")
        else:
            check_lastdim_alignment_stride1(reasons, "key", d.key, 8)
            check_lastdim_alignment_stride1(reasons, "value", d.value, 8)
        check_lastdim_alignment_stride1(reasons, "query", d.query, 8)
        if d.query.numel() and d.query.data_ptr() % 16:
            reasons.append("query is not 16-byte aligned")
        if d.key.numel() == 0:
            reasons.append("empty key/value")
            return reasons
        q, k, v, broadcast = _geometry(d)
        B, Mq, G, H, _ = q.shape
        bias = d.attn_bias
        if isinstance(bias, (BlockDiagonalPaddedKeysMask, PagedBlockDiagonalPaddedKeysMask)):
            qs = bias.q_seqinfo
            if qs.max_seqlen != qs.min_seqlen:
                reasons.append("every sequence must have the same number of queries")
            mq = qs.max_seqlen
            if B != 1:
                reasons.append("padded/paged biases need batch 1")
            if isinstance(bias, _LOCAL_BIASES):
                if mq != 1 and quantized:
                    reasons.append("local attention over a quantised cache is supported for one query per sequence")
                if fp8 and isinstance(bias, PagedBlockDiagonalPaddedKeysMask):
                    reasons.append("a paged fp8 cache cannot be read through a window")
        else:
            mq = Mq
            if B > 1 and (q.stride(0) != Mq * q.stride(1) or k.stride(0) != k.shape[1] * k.stride(1) or v.stride(0) != v.shape[1] * v.stride(1)):
                reasons.append("batched inputs must be contiguous along batch and sequence")
        rows = mq * (H if broadcast else 1)
        if rows > _MAX_ROWS_PER_KV_HEAD:
            reasons.append(f"{rows} query rows per KV head (more than {_MAX_ROWS_PER_KV_HEAD}): this is a prefill")
        if not broadcast and G > 1 and H > 1 and (k.stride(2) != H * k.stride(3) or q.stride(2) != H * q.stride(3)):
            reasons.append("head axes (G, H) of non-broadcast K/V must flatten to one stride")
        if isinstance(bias, PagedBlockDiagonalPaddedKeysMask):
            if bias.block_tables.dtype != torch.int32 or bias.block_tables.stride(-1) != 1:
                reasons.append("block_tables must be contiguous int32")
            if k.shape[1] % bias.page_size:
                reasons.append("the cache length is not a multiple of page_size")
        if d.output_dtype is not None and d.output_dtype not in _DTYPE_CODE:
            reasons.append(f"output_dtype={d.output_dtype}")
        if isinstance(bias, torch.Tensor):
            # the bias in the query layout: [B, G, H, Mq, Mkv]
            want = (B, G, H, Mq, k.shape[1])
            shape5 = tuple(bias.shape) if bias.ndim == 5 else (tuple(bias.shape[:1]) + (1,) + tuple(bias.shape[1:]) if bias.ndim == 4 else
                                                                tuple(bias.shape[:1]) + (1, 1) + tuple(bias.shape[1:]) if bias.ndim == 3 else None)
            if shape5 != want:
                reasons.append(f"additive bias of shape {tuple(bias.shape)}: expected [B, (G,) H, Mq, Mkv] = {want}")
            elif bias.stride(-1) != 1:
                reasons.append("additive bias needs unit stride on its last axis")
            if bias.dtype not in _DTYPE_CODE:
                reasons.append(f"additive bias dtype {bias.dtype}")
            if quantized or fp8:
                reasons.append("additive biases need a 16-bit cache")
            if d.scale is not None and not d.scale > 0:
                reasons.append("additive biases need a positive scale")
            if not broadcast and G > 1 and H > 1 and bias.ndim == 5 and bias.stride(1) != H * bias.stride(2):
                reasons.append("additive bias: head axes (G, H) of non-broadcast K/V must flatten to one stride")
        return reasons

    # ------------------------------------------------------------------ split
    @classmethod
    def get_split_k(cls, batch: int, kv_bound: int, kv_heads: int, row_bytes: int) -> int:
        """Static heuristic: chunks of 1280 tokens per CTA (measured optimum
        for both cache formats at 8 kv heads per CTA: 24-32 chunks of a 32k
        context), halved while the grid would not fill the machine four times
        over."""
        if cls.SPLIT_K is not None:
            return max(1, int(cls.SPLIT_K))
        hb = 8
        while kv_heads % hb:
            hb //= 2
        head_blocks = kv_heads // hb
        bound = -(-kv_bound // 128) * 128
        chunk = max(128, min(bound, 1280))
        while chunk > 128 and batch * head_blocks * (-(-bound // chunk)) < 4 * _SM_COUNT:
            chunk = max(128, (chunk // 2) // 128 * 128)
        return -(-bound // chunk)

    @classmethod
    def apply(cls, inp: Inputs, needs_gradient: bool) -> Tuple[torch.Tensor, Optional[Context]]:
        if cls.OPERATOR is None:
            raise RuntimeError("libxfb200.so is not built; there is no fallback")
        q, k, v, broadcast = _geometry(inp)
        if q.device.type != "cuda":
            raise ValueError("b200_splitk.FwOp runs on CUDA tensors only")
        B, Mq, G, H, D = q.shape
        want_lse = needs_gradient or inp.is_partial
        out_dtype = inp.output_dtype or q.dtype
        out = torch.empty((B, Mq, G, H, D), dtype=out_dtype, device=q.device)
        # packed [G, H, sequences * queries]; viewed as [B, G, H, Mq] on return
        lse = torch.empty((G, H, B * Mq), dtype=torch.float32, device=q.device) if want_lse else None
        bias = inp.attn_bias
        quantized = k.dtype == torch.int32

        if out.numel() > 0:
            p = _lib.DecodeParams()
            p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
            p.lse = lse.data_ptr() if lse is not None else None
            p.dtype = _DTYPE_CODE[q.dtype]
            p.out_dtype = _DTYPE_CODE[out_dtype]
            fp8 = isinstance(inp, InputsFp8)
            p.kv_format = _lib.KV_FP8_ROWWISE if fp8 else _lib.KV_INT4_ROWWISE if quantized else _lib.KV_PLAIN
            p.num_quant_groups = cls.NUM_GROUPS if quantized and not fp8 else 0
            if fp8:
                kss, vss = inp.k_fp8_scale_shift, inp.v_fp8_scale_shift
                # same axes as key without the last one: [B, M, G, H] (or [B, M, H])
                if kss.ndim == 3:
                    kss, vss = kss.unsqueeze(2), vss.unsqueeze(2)
                p.k_scale_shift, p.v_scale_shift = kss.data_ptr(), vss.data_ptr()
                p.ks_stride_m, p.vs_stride_m = kss.stride(1), vss.stride(1)
            p.head_dim = D
            if broadcast:
                p.kv_heads, p.q_per_kv = G, H
                p.q_stride_g, p.q_stride_h = q.stride(2), q.stride(3)
                p.k_stride_g, p.v_stride_g = k.stride(2), v.stride(2)
                if fp8:
                    p.ks_stride_g, p.vs_stride_g = kss.stride(2), vss.stride(2)
                    # the word is laid out once per query head of the group: H consecutive int32 per entry
                    p.ss_words = H if kss.stride(3) == 1 and vss.stride(3) == 1 else 1
                p.o_stride_g, p.o_stride_h = out.stride(2), out.stride(3)
                lse_g, lse_h = (lse.stride(0), lse.stride(1)) if lse is not None else (0, 0)
            else:
                # one KV head per query head: flatten (G, H)
                p.kv_heads, p.q_per_kv = G * H, 1
                hs = lambda t: t.stride(3) if H > 1 else t.stride(2)
                p.q_stride_g, p.q_stride_h = hs(q), 0
                p.k_stride_g, p.v_stride_g = hs(k), hs(v)
                if fp8:
                    p.ks_stride_g, p.vs_stride_g = hs(kss), hs(vss)
                p.o_stride_g, p.o_stride_h = hs(out), 0
                lse_g, lse_h = (lse.stride(1), 0) if lse is not None else (0, 0)
            p.lse_stride_g, p.lse_stride_h = lse_g, lse_h
            p.q_stride_m, p.k_stride_m, p.v_stride_m, p.o_stride_m = q.stride(1), k.stride(1), v.stride(1), out.stride(1)
            p.mask_type = _lib.MASK_NONE
            if isinstance(bias, (BlockDiagonalPaddedKeysMask, PagedBlockDiagonalPaddedKeysMask)):
                p.batch = len(bias.k_seqinfo.seqlen_py)
                p.mq = bias.q_seqinfo.max_seqlen
                p.seqlen_k = bias.k_seqinfo.seqlen.data_ptr()
                kv_start = None  # keeps the tensor alive until the launch
                if isinstance(bias, PagedBlockDiagonalPaddedKeysMask):
                    p.block_tables = bias.block_tables.data_ptr()
                    p.page_size = bias.page_size
                    p.block_table_stride = bias.block_tables.stride(0)
                    p.kv_padding = bias.block_tables.shape[1] * bias.page_size
                    if isinstance(bias, PagedBlockDiagonalGappyKeysMask):
                        kv_start = bias.slot_starts()
                        p.kv_padding = bias.notional_padding
                else:
                    p.kv_padding = bias.k_seqinfo.padding
                    if isinstance(bias, BlockDiagonalGappyKeysMask):
                        kv_start = bias.k_seqinfo.seqstart
                if kv_start is not None:
                    p.kv_seqstart = kv_start.data_ptr()
                if isinstance(
                    bias,
                    (
                        BlockDiagonalCausalWithOffsetPaddedKeysMask,
                        PagedBlockDiagonalCausalWithOffsetPaddedKeysMask,
                        BlockDiagonalCausalWithOffsetGappyKeysMask,
                        PagedBlockDiagonalCausalWithOffsetGappyKeysMask,
                    )
                    + _LOCAL_BIASES,
                ):
                    p.mask_type = _lib.MASK_CAUSAL_BOTTOM_RIGHT
                if isinstance(bias, _LOCAL_BIASES):
                    p.window_size = bias._window_size
            else:
                p.batch, p.mq = B, Mq
                p.seqlen_k = None
                p.kv_padding = k.shape[1]
                if isinstance(bias, torch.Tensor):
                    b5 = bias if bias.ndim == 5 else bias.unsqueeze(1) if bias.ndim == 4 else bias.unsqueeze(1).unsqueeze(1)
                    p.bias, p.bias_dtype = b5.data_ptr(), _DTYPE_CODE[b5.dtype]
                    p.bias_stride_b, p.bias_stride_m = b5.stride(0), b5.stride(3)
                    if broadcast:
                        p.bias_stride_kvh, p.bias_stride_q = b5.stride(1), b5.stride(2)
                    else:
                        # one KV head per query head: (G, H) flattened
                        p.bias_stride_kvh, p.bias_stride_q = (b5.stride(2) if H > 1 else b5.stride(1)), 0
            # token rows of the cache tensors: bounds the tiled copies, so that a bad page-table entry reads zeros
            p.kv_rows = B * k.shape[1]
            if _lib.debug_checks():
                _debug_check_decode(bias, p, k)
            row_bytes = D if fp8 else (D // 8 + cls.NUM_GROUPS) * 4 if quantized else D * 2
            p.split_k = cls.get_split_k(p.batch, min(p.kv_padding, p.window_size + p.mq - 1) if p.window_size else p.kv_padding, p.kv_heads, row_bytes)
            lib = _lib.load()
            nbytes = lib.xfb200_decode_scratch_bytes(p.batch, p.mq, p.kv_heads, p.q_per_kv, D, p.split_k)
            scratch = torch.empty((nbytes,), dtype=torch.uint8, device=q.device) if nbytes else None
            p.scratch = scratch.data_ptr() if scratch is not None else None
            p.scale = inp.scale_float
            with torch.cuda.device(q.device):
                rc = lib.xfb200_decode_forward(C.byref(p), C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream))
                _lib.check(rc, cls.NAME)
                if _lib.check_status_after_every_call():
                    check_device_status(q.device)

        if lse is not None:
            lse = lse.view(G, H, B, Mq).permute(2, 0, 1, 3)
            if out.numel() == 0:
                lse = lse.contiguous()
        if inp.query.ndim == 4:
            out = out[:, :, 0]
            lse = lse[:, 0] if lse is not None else None
        ctx = Context(out=out, lse=lse) if lse is not None else None
        return out, ctx


def _make_split(n: int):
    return type(f"FwOp_S{n}", (FwOp,), {"SPLIT_K": n, "NAME": f"b200_splitK{n}"})


FwOp_S1 = _make_split(1)
FwOp_S2 = _make_split(2)
FwOp_S4 = _make_split(4)
FwOp_S8 = _make_split(8)
FwOp_S16 = _make_split(16)
FwOp_S32 = _make_split(32)
FwOp_S64 = _make_split(64)
FwOp_S128 = _make_split(128)
FwOp_Map = {k: _make_split(k) for k in range(1, 129)}
for _n, _op in ((1, FwOp_S1), (2, FwOp_S2), (4, FwOp_S4), (8, FwOp_S8), (16, FwOp_S16), (32, FwOp_S32), (64, FwOp_S64), (128, FwOp_S128)):
    FwOp_Map[_n] = _op
