"""Prefill attention-forward operator for B200 (``fmha.b200.FwOp``).

Slots into the dispatcher next to the reference's forward operators
(``fmha.cutlass_blackwell.FwOp``, ``fmha.flash.FwOp``; registration record as
tests/test_mem_eff_attention.py:104-111 reads it).  The arithmetic is done by
``xfb200_prefill_forward`` of libxfb200.so: a persistent TMA + tcgen05/TMEM
kernel for head dims 64 and 128 (every mask, additive tensor biases included),
an mma.sync kernel for the other head dims.
"""

from __future__ import annotations

import ctypes as C
from typing import Any, List, Optional, Tuple

import torch

from ... import _lib
from .attn_bias import (
    BlockDiagonalLocalAttentionFromBottomRightGappyKeysMask,
    BlockDiagonalLocalAttentionPaddedKeysMask,
    LocalAttentionFromBottomRightMask,
    BlockDiagonalCausalFromBottomRightMask,
    BlockDiagonalCausalLocalAttentionFromBottomRightMask,
    BlockDiagonalCausalLocalAttentionMask,
    BlockDiagonalCausalLocalAttentionPaddedKeysMask,
    LowerTriangularFromBottomRightLocalAttentionMask,
    BlockDiagonalCausalMask,
    BlockDiagonalCausalWithOffsetGappyKeysMask,
    BlockDiagonalCausalWithOffsetPaddedKeysMask,
    BlockDiagonalGappyKeysMask,
    BlockDiagonalMask,
    BlockDiagonalPaddedKeysMask,
    LowerTriangularFromBottomRightMask,
    LowerTriangularMask,
    LowerTriangularMaskLocalAttention,
    LowerTriangularMaskWithTensorBias,
)
from .common import AttentionFwOpBase, Context, Inputs, check_lastdim_alignment_stride1

_DTYPE_CODE = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}


def _strides4(t: torch.Tensor) -> _lib.Strides:
    """(b, m, g, h) element strides of a 5-D BMGHK tensor."""
    return _lib.Strides(t.stride(0), t.stride(1), t.stride(2), t.stride(3))


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _bias_tensor(bias: Any) -> Optional[torch.Tensor]:
    """The additive tensor of a bias, if it carries one."""
    if isinstance(bias, torch.Tensor):
        return bias
    if isinstance(bias, LowerTriangularMaskWithTensorBias):
        return bias._bias
    return None


def _mask_of(bias: Any) -> Tuple[int, int, int]:
    """(mask_type, window_left, window_right) of a bias object."""
    if bias is None or type(bias) in (BlockDiagonalMask, BlockDiagonalPaddedKeysMask, BlockDiagonalGappyKeysMask):
        return _lib.MASK_NONE, -1, 0
    if isinstance(bias, torch.Tensor):
        return _lib.MASK_NONE, -1, 0
    if type(bias) in (LowerTriangularMask, BlockDiagonalCausalMask, LowerTriangularMaskWithTensorBias):
        return _lib.MASK_CAUSAL_TOP_LEFT, -1, 0
    if type(bias) in (
        LowerTriangularFromBottomRightMask,
        BlockDiagonalCausalFromBottomRightMask,
        BlockDiagonalCausalWithOffsetPaddedKeysMask,
        BlockDiagonalCausalWithOffsetGappyKeysMask,
    ):
        return _lib.MASK_CAUSAL_BOTTOM_RIGHT, -1, 0
    if type(bias) in (LowerTriangularMaskLocalAttention, BlockDiagonalCausalLocalAttentionMask):
        return _lib.MASK_CAUSAL_TOP_LEFT, bias._window_size - 1, 0
    if type(bias) in (
        BlockDiagonalCausalLocalAttentionFromBottomRightMask,
        BlockDiagonalCausalLocalAttentionPaddedKeysMask,
        LowerTriangularFromBottomRightLocalAttentionMask,
    ):
        return _lib.MASK_CAUSAL_BOTTOM_RIGHT, bias._window_size - 1, 0
    if type(bias) in (
        LocalAttentionFromBottomRightMask,
        BlockDiagonalLocalAttentionPaddedKeysMask,
        BlockDiagonalLocalAttentionFromBottomRightGappyKeysMask,
    ):
        return _lib.MASK_LOCAL_BOTTOM_RIGHT, bias.window_left, bias.window_right
    raise NotImplementedError(f"bias {type(bias)}")


def _debug_check_varlen(bias, total_q: int, total_k: int) -> None:
    """Host-side validation of the device arrays a varlen bias carries
    (``XFB200_DEBUG_CHECKS=1``): the kernels trust them."""
    qs = bias.q_seqinfo.seqstart.cpu().tolist()
    ks = bias.k_seqinfo.seqstart.cpu().tolist()
    if any(b < a for a, b in zip(qs, qs[1:])) or qs[0] < 0 or qs[-1] > total_q:
        raise ValueError(f"q_seqinfo.seqstart {qs} is not a monotone partition of {total_q} query rows")
    if any(x < 0 or x > total_k for x in ks):
        raise ValueError(f"k_seqinfo.seqstart {ks} leaves the {total_k} key rows")
    if isinstance(bias, BlockDiagonalPaddedKeysMask):
        lens = bias.k_seqinfo.seqlen.cpu().tolist()
        for i, n in enumerate(lens):
            slot = (ks[i + 1] if i + 1 < len(ks) else total_k) - ks[i]
            if n < 0 or n > slot:
                raise ValueError(f"k_seqinfo.seqlen[{i}] = {n} does not fit its slot of {slot} rows")
    elif any(b < a for a, b in zip(ks, ks[1:])):
        raise ValueError(f"k_seqinfo.seqstart {ks} is not monotone")


class FwOp(AttentionFwOpBase):
    """softmax(Q K^T * scale + mask) V on sm_100a, with optional LSE."""

    OPERATOR = _lib.load().xfb200_prefill_forward if _lib.is_built() else None
    NAME = "b200F"
    SUPPORTED_DTYPES = {torch.bfloat16, torch.half}
    SUPPORTED_MAX_K = 256
    SUPPORTED_MIN_K = 8
    SUPPORTED_ATTN_BIAS_TYPES = (
        type(None),
        LowerTriangularMask,
        LowerTriangularFromBottomRightMask,
        LowerTriangularMaskLocalAttention,
        BlockDiagonalMask,
        BlockDiagonalCausalMask,
        BlockDiagonalCausalFromBottomRightMask,
        BlockDiagonalCausalLocalAttentionMask,
        BlockDiagonalCausalLocalAttentionFromBottomRightMask,
        BlockDiagonalPaddedKeysMask,
        BlockDiagonalCausalWithOffsetPaddedKeysMask,
        BlockDiagonalCausalLocalAttentionPaddedKeysMask,
        LowerTriangularFromBottomRightLocalAttentionMask,
        BlockDiagonalGappyKeysMask,
        BlockDiagonalCausalWithOffsetGappyKeysMask,
        LocalAttentionFromBottomRightMask,
        BlockDiagonalLocalAttentionPaddedKeysMask,
        BlockDiagonalLocalAttentionFromBottomRightGappyKeysMask,
        torch.Tensor,
        LowerTriangularMaskWithTensorBias,
    )
    SUPPORTS_DROPOUT = False
    SUPPORTS_CUSTOM_SCALE = True
    SUPPORTS_DIFFERENT_VALUE_EMBED = False
    SUPPORTS_OUTPUT_DTYPE = True
    SUPPORTS_PARTIAL = True
    SUPPORTS_BMGHK = True
    VARLEN_LSE_PACKED = True
    _TEST_K = [32, 64, 128, 256]
    # which kernel may run the call (XFB200_PREFILL_* of the C ABI): 0 = automatic
    KERNEL_PATH = _lib.PREFILL_AUTO
    # testing aids of the bounded waits (see include/xfb200.h); 0 in production
    _WAIT_BUDGET_KCYCLES = 0
    _DEBUG_FLAGS = 0

    @classmethod
    def shape_not_supported_reasons(cls, Mq: int, Mkv: int, K: int, Kv: int) -> List[str]:
        reasons = super().shape_not_supported_reasons(Mq, Mkv, K, Kv)
        if K % 8 != 0:
            reasons.append(f"query.shape[-1] = {K} is not a multiple of 8")
        return reasons

    @classmethod
    def not_supported_reasons(cls, d: Inputs) -> List[str]:
        reasons = super().not_supported_reasons(d)
        if d.key.dtype == torch.int32:
            reasons.append("quantised K/V caches are read by the split-K decode operator only")
            return reasons
        check_lastdim_alignment_stride1(reasons, "query", d.query, 8)
        check_lastdim_alignment_stride1(reasons, "key", d.key, 8)
        check_lastdim_alignment_stride1(reasons, "value", d.value, 8)
        for name, t in (("query", d.query), ("key", d.key), ("value", d.value)):
            if t.numel() and any(s % 8 for s in t.stride()[:-1]):
                reasons.append(f"{name}: every stride but the last must be a multiple of 8 elements, got {t.stride()}")
            if t.numel() and t.data_ptr() % 16:
                reasons.append(f"{name} is not 16-byte aligned")
        if d.scale is not None and not d.scale > 0:
            pass  # handled by the mma.sync kernel
        if d.output_dtype is not None and d.output_dtype not in _DTYPE_CODE:
            reasons.append(f"output_dtype={d.output_dtype}")
        bt = _bias_tensor(d.attn_bias)
        if bt is not None:
            q5 = d.get_qkv_in_bmghk()[0]
            want = tuple(q5.shape[:1]) + tuple(q5.shape[2:4]) + (q5.shape[1], d.key.shape[1])
            if bt.ndim == 5:
                shape5 = tuple(bt.shape)
            elif bt.ndim == 4:
                shape5 = tuple(bt.shape[:1]) + (1,) + tuple(bt.shape[1:])
            elif bt.ndim == 3:  # BMK inputs before they are brought to BMHK
                shape5 = tuple(bt.shape[:1]) + (1, 1) + tuple(bt.shape[1:])
            else:
                shape5 = None
            if shape5 != want:
                reasons.append(f"additive bias of shape {tuple(bt.shape)}: expected [B, (G,) H, Mq, Mkv] = {want}")
            elif bt.stride(-1) != 1:
                reasons.append("additive bias needs unit stride on its last axis")
            if bt.dtype not in _DTYPE_CODE:
                reasons.append(f"additive bias dtype {bt.dtype}")
            if cls.KERNEL_PATH == _lib.PREFILL_TCGEN05_CTA:
                reasons.append("additive biases run on the persistent tcgen05 kernel or on the mma.sync kernel")
        return reasons

    @classmethod
    def apply(cls, inp: Inputs, needs_gradient: bool) -> Tuple[torch.Tensor, Optional[Context]]:
        return cls._apply(inp, needs_gradient or inp.is_partial, kv_offset=0)

    @classmethod
    def _apply(cls, inp: Inputs, want_lse: bool, kv_offset: int = 0, kv_split: int = 0, kv_offset2: int = 0,
               sm_margin: int = 0) -> Tuple[torch.Tensor, Optional[Context]]:
        """``kv_offset``: global index of the first key (causal masks of a sharded key axis).  ``kv_split`` /
        ``kv_offset2``: the key tensor holds two ranges back to back, the second one (rows from ``kv_split`` on)
        starting at global key ``kv_offset2``.  ``sm_margin``: SMs the persistent kernel leaves free for kernels
        of other streams."""
        if cls.OPERATOR is None:
            raise RuntimeError("libxfb200.so is not built; there is no fallback")
        q, k, v = inp.get_qkv_in_bmghk()
        if q.device.type != "cuda":
            raise ValueError("b200.FwOp runs on CUDA tensors only")
        B, Mq, G, H, D = q.shape
        Mkv = k.shape[1]
        out_dtype = inp.output_dtype or q.dtype
        out = torch.empty((B, Mq, G, H, D), dtype=out_dtype, device=q.device)
        bias = inp.attn_bias
        varlen = isinstance(bias, (BlockDiagonalMask, BlockDiagonalPaddedKeysMask))
        lse = torch.empty((B, G, H, Mq), dtype=torch.float32, device=q.device) if want_lse else None

        if out.numel() > 0:
            if Mkv == 0:
                out.zero_()
                if lse is not None:
                    lse.fill_(float("-inf"))
            else:
                mask_type, window_left, window_right = _mask_of(bias)
                if varlen and _lib.debug_checks():
                    _debug_check_varlen(bias, Mq, Mkv)
                p = _lib.PrefillParams()
                p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
                p.lse = _ptr(lse)
                p.dtype = _DTYPE_CODE[q.dtype]
                p.out_dtype = _DTYPE_CODE[out_dtype]
                if varlen:
                    qi, ki = bias.q_seqinfo, bias.k_seqinfo
                    p.seqstart_q = qi.seqstart.data_ptr()
                    p.seqstart_k = ki.seqstart.data_ptr()
                    p.seqlen_k = ki.seqlen.data_ptr() if isinstance(bias, BlockDiagonalPaddedKeysMask) else None
                    p.batch = len(qi.seqstart_py) - 1
                    p.mq = max(qi.max_seqlen, 0)
                else:
                    p.batch, p.mq = B, Mq
                p.mkv, p.total_q = Mkv, Mq
                p.groups, p.heads_per_group, p.head_dim = G, H, D
                p.q_strides, p.k_strides, p.v_strides, p.o_strides = _strides4(q), _strides4(k), _strides4(v), _strides4(out)
                if lse is not None:
                    p.lse_stride_b, p.lse_stride_g, p.lse_stride_h = lse.stride(0), lse.stride(1), lse.stride(2)
                bt = _bias_tensor(bias)
                if bt is not None:
                    b5 = bt if bt.ndim == 5 else bt.unsqueeze(1)  # [B, G, H, Mq, Mkv]
                    p.bias, p.bias_dtype = b5.data_ptr(), _DTYPE_CODE[b5.dtype]
                    p.bias_stride_b, p.bias_stride_g, p.bias_stride_h, p.bias_stride_m = b5.stride(0), b5.stride(1), b5.stride(2), b5.stride(3)
                p.mask_type, p.kv_offset, p.window_left, p.window_right = mask_type, kv_offset, window_left, window_right
                p.scale = inp.scale_float
                p.kv_split, p.kv_offset2, p.sm_margin = kv_split, kv_offset2, sm_margin
                p.kernel_path = cls.KERNEL_PATH
                p.wait_budget_kcycles, p.debug_flags = cls._WAIT_BUDGET_KCYCLES, cls._DEBUG_FLAGS
                lib = _lib.load()
                # launch on q's device, whatever the current one is
                with torch.cuda.device(q.device):
                    rc = lib.xfb200_prefill_forward(C.byref(p), C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream))
                    _lib.check(rc, "b200.FwOp")
                    if _lib.check_status_after_every_call():
                        check_device_status(q.device)

        if inp.query.ndim == 4:
            out = out[:, :, 0]
            lse = lse[:, 0] if lse is not None else None
        elif inp.query.ndim == 3:
            out = out[:, :, 0, 0]
            lse = lse[:, 0, 0] if lse is not None else None
        ctx = Context(out=out, lse=lse) if lse is not None else None
        return out, ctx


class FwOp_Generic(FwOp):
    """Same operator pinned to the mma.sync kernel (tests, comparisons)."""

    NAME = "b200F-mma"
    KERNEL_PATH = _lib.PREFILL_MMA_SYNC


class FwOp_Tcgen05(FwOp):
    """Same operator, failing unless a tcgen05 kernel covers the input."""

    NAME = "b200F-tc5"
    KERNEL_PATH = _lib.PREFILL_TCGEN05
    SUPPORTED_MAX_K = 128
    _TEST_K = [64, 128]


class FwOp_Tcgen05_Persistent(FwOp_Tcgen05):
    """tcgen05 kernel, one persistent CTA per SM pulling blocks of 256 query rows (the default)."""

    NAME = "b200F-tc5-persistent"
    KERNEL_PATH = _lib.PREFILL_TCGEN05_PERSISTENT


class FwOp_Tcgen05_M256(FwOp_Tcgen05):
    """tcgen05 kernel with one CTA per block of 256 query rows."""

    NAME = "b200F-tc5-m256"
    KERNEL_PATH = _lib.PREFILL_TCGEN05_CTA


def prefill_device_status(device=None) -> int:
    """Code of the first wait a tcgen05 prefill kernel gave up on ``device`` since the
    last call (0 = none), cleared by the call.  Synchronises the current stream."""
    dev = torch.device("cuda" if device is None else device)
    with torch.cuda.device(dev):
        st = C.c_int32(0)
        rc = _lib.load().xfb200_prefill_device_status(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(st))
        if rc != _lib.XFB200_E_DEVICE:
            _lib.check(rc, "prefill_device_status")
    return st.value


def check_device_status(device=None) -> None:
    """Raises ``RuntimeError`` when a prefill kernel gave up a wait on ``device``
    (its output is not valid); clears the status.  Synchronises the current stream."""
    dev = torch.device("cuda" if device is None else device)
    with torch.cuda.device(dev):
        st = C.c_int32(0)
        rc = _lib.load().xfb200_prefill_device_status(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(st))
        _lib.check(rc, "b200.FwOp")
