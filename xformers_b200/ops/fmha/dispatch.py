"""Operator selection (mirrors ``xformers.ops.fmha.dispatch``,
xformers/ops/fmha/dispatch.py:6-10).

Priority list: the split-K decode operator comes first when the input looks
like decoding -- few queries, few sequences, K/V shared by several query heads
(MQA/GQA as a stride-0 head axis) -- which are the rules pinned by
tests/test_mem_eff_attention.py:2189-2236; otherwise the prefill operator.
The first operator whose ``supports(inp)`` holds wins.
"""

from __future__ import annotations

import textwrap
from typing import List, Type

import torch

from . import b200, b200_splitk
from .attn_bias import PagedBlockDiagonalPaddedKeysMask
from .common import AttentionFwOpBase, Inputs

_DECODE_MAX_QUERIES = 16
_DECODE_MAX_BATCH = 64


def _is_decoding(inp: Inputs) -> bool:
    if inp.query.ndim not in (4, 5):
        return False
    if inp.key.dtype == torch.int32 or isinstance(inp.attn_bias, PagedBlockDiagonalPaddedKeysMask):
        return True  # only the decode operator reads these caches
    H = inp.query.shape[-2]
    shared_kv = H > 1 and inp.key.stride(-2) == 0 and inp.value.stride(-2) == 0
    if not shared_kv:
        return False  # one query row per KV head cannot feed the tensor cores
    bias = inp.attn_bias
    if hasattr(bias, "q_seqinfo"):
        mq, batch = bias.q_seqinfo.max_seqlen, len(bias.q_seqinfo.seqstart_py) - 1
    else:
        mq, batch = inp.query.shape[1], inp.query.shape[0]
    return mq <= _DECODE_MAX_QUERIES and batch <= _DECODE_MAX_BATCH


def _dispatch_fw_priority_list(inp: Inputs, needs_gradient: bool) -> List[Type[AttentionFwOpBase]]:
    if _is_decoding(inp) and not needs_gradient:
        return [b200_splitk.FwOp, b200.FwOp]
    return [b200.FwOp, b200_splitk.FwOp]


def _format_inputs_description(inp: Inputs) -> str:
    return f"""query       : shape={tuple(inp.query.shape)} ({inp.query.dtype})
key         : shape={tuple(inp.key.shape)} ({inp.key.dtype})
value       : shape={tuple(inp.value.shape)} ({inp.value.dtype})
attn_bias   : {type(inp.attn_bias)}
p           : {inp.p}"""


def _ensure_op_supports_or_raise(exc_type, name: str, op, inp: Inputs) -> None:
    reasons = op.not_supported_reasons(inp)
    if not reasons:
        return
    raise exc_type(
        f"""Operator `{name}` does not support inputs:
{textwrap.indent(_format_inputs_description(inp), '     ')}
{_format_not_supported_reasons(op, reasons)}"""
    )


def _format_not_supported_reasons(op, reasons: List[str]) -> str:
    return f"`{op.NAME}` is not supported because:\n    " + "\n    ".join(reasons)


def _run_priority_list(name: str, priority_list, inp: Inputs):
    not_supported = []
    for op in priority_list:
        reasons = op.not_supported_reasons(inp)
        if not reasons:
            return op
        not_supported.append(_format_not_supported_reasons(op, reasons))
    msg = f"No operator found for `{name}` with inputs:\n{textwrap.indent(_format_inputs_description(inp), '     ')}"
    for m in not_supported:
        msg += "\n" + m
    raise NotImplementedError(msg)


def _dispatch_fw(inp: Inputs, needs_gradient: bool) -> Type[AttentionFwOpBase]:
    """Pick the forward operator; ``NotImplementedError`` with every
    operator's reasons if none applies (benchmarks/utils.py:532-536)."""
    return _run_priority_list("memory_efficient_attention_forward", _dispatch_fw_priority_list(inp, needs_gradient), inp)
