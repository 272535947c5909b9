"""``torch.library`` registration of the forward operator, so that graphs
captured with ``torch.compile(fullgraph=True)`` or traced with fake tensors keep
a single opaque node for it (the reference defines the same two schemas under
``xformer::``, xformers/ops/fmha/__init__.py:72-103).

The operators live in the ``xformers_b200`` namespace; the same definitions are
also placed under ``xformer::`` when that name is still free, i.e. when the
reference package has not been imported into the process.  Implementations:
``CUDA`` calls :func:`memory_efficient_attention_forward`, ``Meta`` returns an
empty tensor of the output shape.  A FLOP formula (2 * B * H * Mq * Mkv *
(Kqk + Kv), the dense count a tensor-bias call performs) is registered with
``torch.utils.flop_counter``.
"""

from __future__ import annotations

from typing import Optional

import torch

_SCHEMA = "(Tensor q, Tensor k, Tensor v, Tensor? b = None, float? p = 0.0, float? scale = None) -> Tensor"
_SCHEMA_BIAS = "(Tensor q, Tensor k, Tensor v, Tensor b, float? p = 0.0, float? scale = None) -> Tensor"
NAMESPACES = []


def _forward(q, k, v, b=None, p=0.0, scale=None):
    from . import memory_efficient_attention_forward

    return memory_efficient_attention_forward(q, k, v, b, 0.0 if p is None else p, scale)


def _forward_meta(q, k, v, b=None, p=0.0, scale=None):
    return q.new_empty(tuple(q.shape[:-1]) + (v.shape[-1],))


def _flops(q_shape, k_shape, v_shape, *args, out_shape=None, **kwargs) -> int:
    """Dense count for BMK / BMHK / BMGHK inputs: one multiply-add = 2 FLOPs."""
    mq, kqk = q_shape[1], q_shape[-1]
    mkv, kv = k_shape[1], v_shape[-1]
    heads = 1
    for n in q_shape[2:-1]:
        heads *= n
    return 2 * q_shape[0] * heads * mq * mkv * (kqk + kv)


def _register(ns: str) -> bool:
    try:
        torch.library.define(f"{ns}::memory_efficient_attention_forward", _SCHEMA)
        torch.library.define(f"{ns}::memory_efficient_attention_forward_with_bias", _SCHEMA_BIAS)
    except RuntimeError:
        return False  # the names are taken (the reference package defined them first)
    for name in ("memory_efficient_attention_forward", "memory_efficient_attention_forward_with_bias"):
        torch.library.impl(f"{ns}::{name}", "Meta", _forward_meta)
        torch.library.impl(f"{ns}::{name}", "CUDA", _forward)
    try:
        from torch.utils.flop_counter import register_flop_formula

        ops = getattr(torch.ops, ns)
        register_flop_formula([ops.memory_efficient_attention_forward, ops.memory_efficient_attention_forward_with_bias])(_flops)
    except Exception:  # older torch without the registry: the ops still work
        pass
    NAMESPACES.append(ns)
    return True


_register("xformers_b200")
_register("xformer")
