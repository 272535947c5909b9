"""Names of ``xformers.ops.fmha.triton_splitk`` kept for drop-in use
(xformers/ops/fmha/triton_splitk.py:7-34).  Nothing here uses Triton: the
classes are the CUDA split-K decode operator of :mod:`.b200_splitk`."""

from .b200_splitk import (  # noqa: F401
    FwOp,
    FwOp_Map,
    FwOp_S1,
    FwOp_S2,
    FwOp_S4,
    FwOp_S8,
    FwOp_S16,
    FwOp_S32,
    FwOp_S64,
    FwOp_S128,
)
from .common import InputsFp8  # noqa: F401
from .merge import merge_attentions, merge_attentions_varargs  # noqa: F401
