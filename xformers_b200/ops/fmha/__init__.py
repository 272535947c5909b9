"""Attention forward behind the reference's fmha API
(xformers/ops/fmha/__init__.py:12-58): the same entry points, bias classes,
operator base classes and dispatcher, with B200-native operators registered.

Out of scope and therefore absent: the backward pass
(``memory_efficient_attention`` raises when autograd would have to record the
call; ``*BwOp``), dropout, and the reference's other backends (``cutlass``,
``flash``, ``flash3``, ``ck``).
"""

from __future__ import annotations

from typing import Any, List, Optional, Sequence, Tuple, Type, Union

import torch

from . import attn_bias, b200, b200_splitk, common, dispatch, merge, triton_splitk  # noqa: F401
from .attn_bias import (  # noqa: F401
    VARLEN_BIASES,
    AttentionBias,
    BlockDiagonalMask,
    LowerTriangularMask,
)
from .common import (  # noqa: F401
    AttentionBwOpBase,
    AttentionFwOpBase,
    AttentionOp,
    AttentionOpBase,
    Context,
    Inputs,
    bmk2bmhk,
)
from .dispatch import _dispatch_fw, _dispatch_fw_priority_list, _ensure_op_supports_or_raise  # noqa: F401
from .merge import merge_attentions, merge_attentions_varargs  # noqa: F401

MemoryEfficientAttentionB200Op = (b200.FwOp, None)
MemoryEfficientAttentionB200SplitKOp = (b200_splitk.FwOp, None)

ALL_FW_OPS: List[Type[AttentionFwOpBase]] = [b200.FwOp, b200_splitk.FwOp]
ALL_BW_OPS: List[Type[AttentionBwOpBase]] = []
_OPS_LOOKUP = {op.NAME: op for op in ALL_FW_OPS + [b200.FwOp_Generic, b200.FwOp_Tcgen05, b200.FwOp_Tcgen05_M256, b200.FwOp_Tcgen05_Persistent] + list(b200_splitk.FwOp_Map.values())}


def _serialize_op(op):
    return op.NAME if op is not None else None


def _unserialize_op(name):
    return _OPS_LOOKUP[name] if name is not None else None


def _fw_op_of(op) -> Optional[Type[AttentionFwOpBase]]:
    """``op=`` accepts a forward operator class or the reference's
    ``(fw_op, bw_op)`` tuple."""
    if op is None:
        return None
    if isinstance(op, tuple):
        return op[0]
    return op


def _run_forward(inp: Inputs, op, needs_lse: bool) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    inp.validate_inputs()
    if inp.query.device.type != "cuda":
        raise ValueError(f"memory_efficient_attention_forward needs CUDA tensors, got device={inp.query.device}")
    output_shape = inp.normalize_bmhk()
    fw = _fw_op_of(op)
    if fw is None:
        fw = _dispatch_fw(inp, needs_lse and not inp.is_partial)
    else:
        _ensure_op_supports_or_raise(ValueError, "memory_efficient_attention", fw, inp)
    out, ctx = fw.apply(inp, needs_gradient=needs_lse)
    out = out.reshape(output_shape)
    lse = ctx.lse if ctx is not None else None
    if lse is not None and len(output_shape) == 3:
        lse = lse.reshape(output_shape[0], output_shape[1])  # BMK: [B*H, M]
    return out, lse


def memory_efficient_attention_forward(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_bias: Optional[Union[torch.Tensor, AttentionBias]] = None,
    p: float = 0.0,
    scale: Optional[float] = None,
    *,
    op=None,
    output_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """``softmax(Q K^T * scale + bias) V`` (xformers/ops/__init__.py:18)."""
    return _run_forward(Inputs(query, key, value, attn_bias, p, scale, output_dtype), op, needs_lse=False)[0]


def memory_efficient_attention_forward_requires_grad(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_bias: Optional[Union[torch.Tensor, AttentionBias]] = None,
    p: float = 0.0,
    scale: Optional[float] = None,
    *,
    op=None,
    output_dtype: Optional[torch.dtype] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same, also returning the log-sum-exp ``[B, (G,) H, Mq]`` in natural log
    (tests/test_mem_eff_attention.py:657-663)."""
    if p != 0.0:
        raise NotImplementedError("dropout is outside the forward hot path")
    out, lse = _run_forward(Inputs(query, key, value, attn_bias, p, scale, output_dtype), op, needs_lse=True)
    assert lse is not None
    return out, lse


def _memory_efficient_attention_forward(inp: Inputs, op=None) -> torch.Tensor:
    """Forward on a prepared :class:`Inputs` (or :class:`InputsFp8`) object
    (used as ``fmha._memory_efficient_attention_forward`` by the reference's tests)."""
    return _run_forward(inp, op, needs_lse=False)[0]


def _memory_efficient_attention_forward_requires_grad(inp: Inputs, op=None) -> Tuple[torch.Tensor, Context]:
    """Same, returning ``(out, Context)`` with the log-sum-exp
    (tests/test_mem_eff_attention.py:2843-2848)."""
    out, lse = _run_forward(inp, op, needs_lse=True)
    return out, Context(out=out, lse=lse)


def memory_efficient_attention_partial(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_bias: Optional[Union[torch.Tensor, AttentionBias]] = None,
    p: float = 0.0,
    scale: Optional[float] = None,
    *,
    op=None,
    output_dtype: Optional[torch.dtype] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention over a part of the keys, to be combined with
    :func:`merge_attentions` (tests/test_fmha_merge_attentions.py:117-122)."""
    inp = Inputs(query, key, value, attn_bias, p, scale, output_dtype, is_partial=True)
    out, lse = _run_forward(inp, op, needs_lse=True)
    assert lse is not None
    return out, lse


def memory_efficient_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attn_bias: Optional[Union[torch.Tensor, AttentionBias]] = None,
    p: float = 0.0,
    scale: Optional[float] = None,
    *,
    op=None,
    output_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """The reference's main entry point (xformers/ops/__init__.py:16; called as
    such by examples/llama_inference/model.py:142 and in the docstring of
    xformers/ops/rope_padded.py:49-53).  When no input asks for a gradient, or
    gradient mode is off, it is the forward pass and runs here; the backward
    pass is outside this library, so a call that autograd would have to record
    raises ``NotImplementedError``."""
    if torch.is_grad_enabled() and any(t.requires_grad for t in (query, key, value)):
        raise NotImplementedError(
            "memory_efficient_attention: an input requires grad, and the backward pass is outside this library; "
            "call it under torch.no_grad(), or use memory_efficient_attention_forward"
        )
    if isinstance(attn_bias, torch.Tensor) and torch.is_grad_enabled() and attn_bias.requires_grad:
        raise NotImplementedError("memory_efficient_attention: attn_bias requires grad; the backward pass is outside this library")
    if p != 0.0:
        raise NotImplementedError("dropout is outside the forward hot path")
    return _run_forward(Inputs(query, key, value, attn_bias, p, scale, output_dtype), op, needs_lse=False)[0]


from . import torch_library  # noqa: E402,F401  (defines torch.ops.xformers_b200.memory_efficient_attention_forward[_with_bias])
