"""``fmha.merge_attentions``: LSE-weighted combination of partial attentions.

API of the reference (xformers/ops/fmha/__init__.py:49,
xformers/ops/fmha/triton_splitk.py:29-33; calls
tests/test_fmha_merge_attentions.py:128,319-325,507): ``attn_split`` is a
tensor ``[S, B, M, (G,) H, D]`` or a list of S tensors ``[B, M, (G,) H, D]``,
``lse_split`` is ``[S, B, (G,) H, M]`` or a list of ``[B, (G,) H, M]``.  The
list form is merged in place of a stack: the kernel takes up to 32 separate
base pointers, so no copy is made.  No autograd.
"""

from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple, Union

import torch

from ... import _lib

_DTYPE_CODE = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}


def merge_attentions(
    attn_split: Union[torch.Tensor, Sequence[torch.Tensor]],
    lse_split: Union[torch.Tensor, Sequence[torch.Tensor]],
    write_lse: bool = True,
    output_dtype: Optional[torch.dtype] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Returns ``(out [B, M, (G,) H, D], lse [B, (G,) H, M] or None)``."""
    attn_is_list = not isinstance(attn_split, torch.Tensor)
    lse_is_list = not isinstance(lse_split, torch.Tensor)
    if attn_is_list != lse_is_list:
        raise ValueError("attn_split and lse_split must both be tensors or both be lists")
    if attn_is_list:
        attn_list, lse_list = list(attn_split), list(lse_split)
        if len(attn_list) == 0 or len(attn_list) != len(lse_list):
            raise ValueError("attn_split and lse_split need the same, non-zero number of partials")
        if len(attn_list) > _lib.MERGE_MAX_PTRS:
            return merge_attentions(torch.stack(attn_list), torch.stack(lse_list), write_lse, output_dtype)
        ref_a, ref_l = attn_list[0], lse_list[0]
        for a_, l_ in zip(attn_list, lse_list):
            if a_.shape != ref_a.shape or l_.shape != ref_l.shape or a_.dtype != ref_a.dtype:
                raise ValueError("all partials must have the same shape and dtype")
        # one set of strides is passed for all partials
        if any(a_.stride() != ref_a.stride() for a_ in attn_list):
            attn_list = [a_.contiguous() for a_ in attn_list]
        lse_list = [l_.float() if l_.dtype != torch.float32 else l_ for l_ in lse_list]
        if any(l_.stride() != lse_list[0].stride() or (l_.shape[-1] > 1 and l_.stride(-1) != 1) for l_ in lse_list):
            lse_list = [l_.contiguous() for l_ in lse_list]
        num_splits = len(attn_list)
        a0, l0 = attn_list[0], lse_list[0]
        stacked = False
    else:
        if attn_split.ndim not in (5, 6):
            raise ValueError(f"attn_split must be [S, B, M, (G,) H, D], got {tuple(attn_split.shape)}")
        if lse_split.dtype != torch.float32:
            lse_split = lse_split.float()
        if lse_split.shape[-1] > 1 and lse_split.stride(-1) != 1:
            lse_split = lse_split.contiguous()
        num_splits = attn_split.shape[0]
        if num_splits == 0:
            raise ValueError("no partial to merge")
        a0, l0 = attn_split[0], lse_split[0]
        attn_list, lse_list = [a0], [l0]
        stacked = True

    bmghk = a0.ndim == 5
    if a0.ndim not in (4, 5) or l0.ndim != a0.ndim - 1:
        raise ValueError(f"bad ranks: attn {tuple(a0.shape)}, lse {tuple(l0.shape)}")
    if not bmghk:
        a5 = a0.unsqueeze(2)
        l4 = l0.unsqueeze(1)
    else:
        a5, l4 = a0, l0
    B, M, G, H, D = a5.shape
    if tuple(l4.shape) != (B, G, H, M):
        raise ValueError(f"lse shape {tuple(l0.shape)} does not match attn shape {tuple(a0.shape)}")
    if a0.device.type != "cuda":
        raise ValueError("merge_attentions runs on CUDA tensors only")
    if a0.dtype not in _DTYPE_CODE:
        raise ValueError(f"unsupported dtype {a0.dtype}")
    if D > 1 and a5.stride(-1) != 1:
        raise ValueError("the last dim of attn_split must be contiguous")
    out_dtype = output_dtype or a0.dtype
    if out_dtype not in _DTYPE_CODE:
        raise ValueError(f"unsupported output dtype {out_dtype}")
    out5 = torch.empty((B, M, G, H, D), dtype=out_dtype, device=a0.device)
    lse_out = torch.empty((B, G, H, M), dtype=torch.float32, device=a0.device) if write_lse else None

    if out5.numel() > 0 or (lse_out is not None and lse_out.numel() > 0):
        p = _lib.MergeParams()
        n_ptr = 1 if stacked else num_splits
        attn_arr = (C.c_void_p * n_ptr)(*[t.data_ptr() for t in attn_list])
        lse_arr = (C.c_void_p * n_ptr)(*[t.data_ptr() for t in lse_list])
        p.attn_ptrs, p.lse_ptrs = attn_arr, lse_arr
        p.num_splits, p.stacked = num_splits, int(stacked)
        if stacked:
            p.attn_stride_s, p.lse_stride_s = attn_split.stride(0), lse_split.stride(0)
        p.attn_strides = _lib.Strides(a5.stride(0), a5.stride(1), a5.stride(2), a5.stride(3))
        p.lse_in_stride_b, p.lse_in_stride_g, p.lse_in_stride_h = l4.stride(0), l4.stride(1), l4.stride(2)
        p.out, p.lse_out = out5.data_ptr(), (lse_out.data_ptr() if lse_out is not None else None)
        p.out_strides = _lib.Strides(out5.stride(0), out5.stride(1), out5.stride(2), out5.stride(3))
        if lse_out is not None:
            p.lse_out_stride_b, p.lse_out_stride_g, p.lse_out_stride_h = lse_out.stride(0), lse_out.stride(1), lse_out.stride(2)
        p.B, p.M, p.G, p.H, p.D = B, M, G, H, D
        p.in_dtype, p.out_dtype = _DTYPE_CODE[a0.dtype], _DTYPE_CODE[out_dtype]
        with torch.cuda.device(a0.device):
            rc = _lib.load().xfb200_merge_attentions(C.byref(p), C.c_void_p(torch.cuda.current_stream(a0.device).cuda_stream))
        _lib.check(rc, "merge_attentions")

    if not bmghk:
        return out5[:, :, 0], (lse_out[:, 0] if lse_out is not None else None)
    return out5, lse_out


def _merge_varargs_impl(
    attn_split: List[torch.Tensor],
    lse_split: List[torch.Tensor],
    write_lse: bool = True,
    output_dtype: Optional[torch.dtype] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    out, lse = merge_attentions(list(attn_split), list(lse_split), write_lse, output_dtype)
    if lse is None:  # a custom op returns tensors only: an empty one stands for "not written"
        lse = out.new_empty((0,), dtype=torch.float32)
    return out, lse


def _merge_varargs_fake(attn_split, lse_split, write_lse=True, output_dtype=None):
    a0, l0 = attn_split[0], lse_split[0]
    out = a0.new_empty(a0.shape, dtype=output_dtype or a0.dtype)
    lse = l0.new_empty(l0.shape if write_lse else (0,), dtype=torch.float32)
    return out, lse


# The list form as a custom operator with a fake implementation, so that a graph traced by
# torch.compile(fullgraph=True) keeps the merge as one opaque node (the reference registers
# ``xformers::fmha_merge_attentions_varargs`` for the same purpose, xformers/ops/fmha/triton_splitk.py:42-53).
_merge_varargs_op = torch.library.custom_op(
    "xformers_b200::fmha_merge_attentions_varargs", _merge_varargs_impl, mutates_args=(), device_types=["cuda"]
)
torch.library.register_fake("xformers_b200::fmha_merge_attentions_varargs", _merge_varargs_fake)


def merge_attentions_varargs(attn_split: List[torch.Tensor], lse_split: List[torch.Tensor], write_lse: bool = True,
                             output_dtype: Optional[torch.dtype] = None):
    """List form under the name the reference registers as a custom op
    (xformers/ops/fmha/triton_splitk.py:42-53): ``(out, lse)``, ``lse`` ``None`` when not written."""
    out, lse = _merge_varargs_op(list(attn_split), list(lse_split), write_lse, output_dtype)
    return out, (lse if write_lse else None)
