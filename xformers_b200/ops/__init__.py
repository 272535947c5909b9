"""Operator namespace mirroring ``xformers.ops`` for the attention-forward path
(xformers/ops/__init__.py:9-25)."""

from . import fmha  # noqa: F401
from .rope_padded import rope_padded  # noqa: F401
from .fmha import (  # noqa: F401
    AttentionBias,
    AttentionOpBase,
    LowerTriangularMask,
    memory_efficient_attention,
    memory_efficient_attention_forward,
    memory_efficient_attention_forward_requires_grad,
    memory_efficient_attention_partial,
    merge_attentions,
)
