"""Argument bundle, context and operator base classes of the fmha API.

Mirrors ``xformers.ops.fmha.common`` (xformers/ops/fmha/common.py:6-20): the
names and the class attributes that callers and tests read
(tests/test_mem_eff_attention.py:104-111,145-181,227,264,476,609-610).
Only the forward path exists here.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Sequence, Set, Tuple, Type, Union

import torch

from .attn_bias import (
    AttentionBias,
    BlockDiagonalMask,
    BlockDiagonalPaddedKeysMask,
    LowerTriangularMask,
    PagedBlockDiagonalPaddedKeysMask,
    VARLEN_BIASES,
)


def _is_bias_type_supported_in_BMK(attn_bias_type: Any) -> bool:
    # NoneType, tensors and the dense causal mask make sense without a head axis
    if isinstance(None, attn_bias_type) or issubclass(attn_bias_type, torch.Tensor):
        return True
    return attn_bias_type in (LowerTriangularMask,)


def bmk2bmhk(tensor: torch.Tensor, num_heads: int) -> torch.Tensor:
    """``[B*H, M, K]`` -> ``[B, M, H, K]`` view (xformers/ops/fmha/common.py:13)."""
    if tensor.ndim == 4:
        return tensor
    return tensor.reshape([-1, num_heads, tensor.shape[1], tensor.shape[2]]).permute((0, 2, 1, 3))


def check_lastdim_alignment_stride1(reasons: List[str], name: str, x: torch.Tensor, alignment: int) -> None:
    """Append reasons when rows of ``x`` cannot be read with ``alignment``-element
    vector loads (tests/test_mem_eff_attention.py:1378-1407)."""
    if x.shape[-1] % alignment != 0:
        reasons.append(f"{name}.shape[-1] % {alignment} != 0")
    elif x.stride(-2) % alignment != 0:
        reasons.append(f"{name}.stride(-2) % {alignment} != 0 ({name}.stride() = {x.stride()})")
    if x.shape[-1] > 1 and x.stride(-1) != 1:
        reasons.append(f"expect {name}.stride(-1) == 1 ({name}.stride() = {x.stride()})")


@dataclass
class Inputs:
    """Arguments of one attention call (tests/test_mem_eff_attention.py:474,1007)."""

    query: torch.Tensor
    key: torch.Tensor
    value: torch.Tensor
    attn_bias: Optional[Union[torch.Tensor, AttentionBias]] = None
    p: float = 0.0
    scale: Optional[float] = None
    output_dtype: Optional[torch.dtype] = None
    is_partial: bool = False

    @property
    def device(self) -> torch.device:
        return self.query.device

    @property
    def scale_float(self) -> float:
        return self.query.shape[-1] ** (-0.5) if self.scale is None else self.scale

    def get_qkv_in_bmghk(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        if self.query.ndim == 5:
            return self.query, self.key, self.value
        if self.query.ndim == 4:
            return self.query.unsqueeze(2), self.key.unsqueeze(2), self.value.unsqueeze(2)
        if self.value.ndim == 3:
            return self.query[:, :, None, None], self.key[:, :, None, None], self.value[:, :, None, None]
        assert False

    def normalize_bmhk(self) -> Tuple[int, ...]:
        """Bring 3-D BMK inputs to BMHK (one head) and return the shape the
        output must be given back in."""
        if self.query.ndim not in (3, 4, 5):
            raise ValueError(f"Invalid shape for query: {self.query.shape}. Expected shape [batch, seqlen, head_groups, num_heads_per_group, K], [batch, seqlen, num_heads, K], or [batch, seqlen, K].")
        if self.value.dtype == torch.int32:
            # quantised K/V carry packed words: the output takes q's last dim
            output_shape = tuple(self.query.shape)
        else:
            output_shape = self.query.shape[:-1] + (self.value.shape[-1],)
        if self.query.ndim == 3:
            self.query = self.query.unsqueeze(2)
            self.key = self.key.unsqueeze(2)
            self.value = self.value.unsqueeze(2)
            if isinstance(self.attn_bias, torch.Tensor):
                if self.attn_bias.ndim != 3:
                    raise ValueError(f"Expected BMK format for attn_bias, but got {self.attn_bias.shape}")
                self.attn_bias = self.attn_bias.unsqueeze(1)
        return output_shape

    def validate_inputs(self) -> None:
        qkv = (self.query, self.key, self.value)
        if self.query.ndim not in (3, 4, 5) or any(x.ndim != self.query.ndim for x in qkv):
            raise ValueError(
                f"Query/Key/Value should all have BMGHK, BMHK or BMK shape.\n  query.shape: {self.query.shape}\n"
                f"  key.shape  : {self.key.shape}\n  value.shape: {self.value.shape}"
            )
        if any(x.device != self.query.device for x in qkv):
            raise ValueError("Query/Key/Value should all be on the same device")
        if isinstance(self.attn_bias, (BlockDiagonalMask, BlockDiagonalPaddedKeysMask, PagedBlockDiagonalPaddedKeysMask)):
            bias_device = self.attn_bias.q_seqinfo.seqstart.device
            if bias_device != self.query.device:
                raise ValueError(
                    f"Attention bias and Query/Key/Value should be on the same device\n"
                    f"  query.device: {self.query.device}\n  attn_bias   : {bias_device}\n"
                )
        quantized = self.key.dtype == torch.int32
        if not quantized and any(x.dtype != self.query.dtype for x in qkv):
            raise ValueError(
                f"Query/Key/Value should all have the same dtype\n  query.dtype: {self.query.dtype}\n"
                f"  key.dtype  : {self.key.dtype}\n  value.dtype: {self.value.dtype}"
            )
        if isinstance(self.attn_bias, VARLEN_BIASES) and self.query.shape[0] != 1:
            raise ValueError(
                f"Expected batch_size=1 when using block-diagonal bias\n  query.shape: {self.query.shape}"
            )
        if self.p < 0.0 or self.p > 1.0:
            raise ValueError(f"Invalid dropout probability: p={self.p}")
        # shapes
        B, Mq = self.query.shape[:2]
        K = self.query.shape[-1]
        Bk, Mkv = self.key.shape[:2]
        Kv = self.value.shape[-1]
        ok = self.key.shape[:2] == self.value.shape[:2] and B == Bk
        if not quantized:
            ok = ok and self.key.shape[-1] == K
        if self.query.ndim in (4, 5):
            ok = ok and self.query.shape[2:-1] == self.key.shape[2:-1] == self.value.shape[2:-1]
        if not ok:
            raise ValueError(
                f"Incompatible shapes for attention inputs:\n  query.shape: {self.query.shape}\n"
                f"  key.shape  : {self.key.shape}\n  value.shape: {self.value.shape}\n"
                "HINT: We don't support broadcasting, please use `expand` yourself before calling `memory_efficient_attention` if you need to"
            )


@dataclass
class InputsFp8(Inputs):
    """Inputs of the split-K operator with a row-wise fp8 KV cache
    (xformers/ops/fmha/triton_splitk.py:28; built in tests/utils.py:215-222):
    ``key`` / ``value`` are int32 words of four e4m3 values, element
    ``x = fp8 * scale + shift`` with one ``(fp16 scale | fp16 shift << 16)``
    int32 per token and head in ``k_fp8_scale_shift`` / ``v_fp8_scale_shift``
    (shape of ``key`` without its last axis)."""

    k_fp8_scale_shift: Optional[torch.Tensor] = None
    v_fp8_scale_shift: Optional[torch.Tensor] = None


@dataclass
class Context:
    """What a forward call leaves behind for its caller: the log-sum-exp
    (tests/test_mem_eff_attention.py:2860-2861) and the output."""

    lse: torch.Tensor
    out: torch.Tensor
    op_bw: Any = None
    rng_state: Any = None

    def get_padded_lse(self, pad_to: int, force_pad_inf: bool = False) -> torch.Tensor:
        pad_amount = (pad_to - (self.lse.shape[2] % pad_to)) % pad_to
        lse = self.lse
        if pad_amount > 0:
            lse = torch.nn.functional.pad(lse, [0, pad_amount], value=math.inf if force_pad_inf else 0.0)
        return lse


class BaseOperator:
    OPERATOR: Any = None
    NAME: str = ""
    OPERATOR_CATEGORY: str = "memory_efficient_attention"

    @classmethod
    def is_available(cls) -> bool:
        return cls.OPERATOR is not None


class AttentionOpBase(BaseOperator):
    """Registration record of an attention operator: what it supports, as
    class attributes; stateless classmethods only."""

    SUPPORTED_DEVICES: Set[str] = {"cuda"}
    CUDA_MINIMUM_COMPUTE_CAPABILITY: Tuple[int, int] = (10, 0)
    CUDA_MAXIMUM_COMPUTE_CAPABILITY: Optional[Tuple[int, int]] = (10, 0)
    SUPPORTED_DTYPES: Set[torch.dtype] = {torch.bfloat16, torch.half}
    SUPPORTED_MAX_K: float = 256
    SUPPORTED_MIN_K: int = 0
    SUPPORTED_ATTN_BIAS_TYPES: Tuple[Any, ...] = (type(None),)
    SUPPORTS_DROPOUT = False
    SUPPORTS_CUSTOM_SCALE = True
    SUPPORTS_DIFFERENT_VALUE_EMBED = False
    SUPPORTS_OUTPUT_DTYPE = True
    SUPPORTS_PARTIAL = True
    IS_DETERMINISTIC = True
    SUPPORTS_BMGHK = True
    VARLEN_LSE_PACKED = True
    _TEST_BATCH_SIZES: List[int] = [1, 3]
    _TEST_K: List[int] = [64, 128]

    ERROR_ATOL: Mapping[torch.dtype, float] = {torch.float: 3e-4, torch.half: 4e-3, torch.bfloat16: 2e-2}
    ERROR_RTOL: Mapping[torch.dtype, float] = {torch.float: 2e-5, torch.half: 4e-4, torch.bfloat16: 5e-3}

    @classmethod
    def supports(cls, d: Inputs) -> bool:
        return not cls.not_supported_reasons(d)

    @classmethod
    def shape_not_supported_reasons(cls, Mq: int, Mkv: int, K: int, Kv: int) -> List[str]:
        reasons = []
        if not cls.SUPPORTS_DIFFERENT_VALUE_EMBED and K != Kv:
            reasons.append("query.shape[-1] != value.shape[-1]")
        if max(K, Kv) > cls.SUPPORTED_MAX_K:
            reasons.append(f"max(query.shape[-1], value.shape[-1]) > {cls.SUPPORTED_MAX_K}")
        if min(K, Kv) < cls.SUPPORTED_MIN_K:
            reasons.append(f"min(query.shape[-1], value.shape[-1]) < {cls.SUPPORTED_MIN_K}")
        return reasons

    @classmethod
    def not_supported_reasons(cls, d: Inputs) -> List[str]:
        """Human-readable reasons why this operator cannot run ``d``; empty
        list = supported (tests/test_mem_eff_attention.py:476-481)."""
        query_shape = d.query.shape
        quantized = d.key.dtype == torch.int32
        reasons = []
        if not quantized:
            reasons += cls.shape_not_supported_reasons(
                Mq=query_shape[1], Mkv=d.key.shape[1], K=query_shape[-1], Kv=d.value.shape[-1]
            )
        device_type = d.query.device.type
        dtype = d.query.dtype
        if device_type not in cls.SUPPORTED_DEVICES:
            reasons.append(f"device={device_type} (supported: {cls.SUPPORTED_DEVICES})")
        if device_type == "cuda" and torch.cuda.is_available():
            cap = torch.cuda.get_device_capability(d.query.device)
            if cap < cls.CUDA_MINIMUM_COMPUTE_CAPABILITY:
                reasons.append(f"requires device with capability >= {cls.CUDA_MINIMUM_COMPUTE_CAPABILITY} but your GPU has capability {cap} (too old)")
            elif cls.CUDA_MAXIMUM_COMPUTE_CAPABILITY is not None and cap > cls.CUDA_MAXIMUM_COMPUTE_CAPABILITY:
                reasons.append(f"requires device with capability <= {cls.CUDA_MAXIMUM_COMPUTE_CAPABILITY} but your GPU has capability {cap} (too new)")
        if dtype not in cls.SUPPORTED_DTYPES:
            reasons.append(f"dtype={dtype} (supported: {cls.SUPPORTED_DTYPES})")
        if type(d.attn_bias) not in cls.SUPPORTED_ATTN_BIAS_TYPES:
            reasons.append(f"attn_bias type is {type(d.attn_bias)}")
        if not cls.SUPPORTS_OUTPUT_DTYPE and d.output_dtype is not None:
            reasons.append("Custom output dtype not supported")
        if d.is_partial and not cls.SUPPORTS_PARTIAL:
            reasons.append("Partial attention not supported")
        if d.p != 0.0 and not cls.SUPPORTS_DROPOUT:
            reasons.append("dropout > 0.0")
        if d.scale is not None and not cls.SUPPORTS_CUSTOM_SCALE:
            reasons.append("has custom scale")
        if not cls.SUPPORTS_BMGHK and d.query.ndim == 5:
            reasons.append("operator does not support BMGHK format")
        if not cls.is_available():
            reasons.append("operator wasn't built - libxfb200.so is missing (python -m xformers_b200.build)")
        return reasons


class AttentionFwOpBase(AttentionOpBase):
    """Base class of forward operators: ``apply(inp, needs_gradient) -> (out, ctx)``
    (benchmarks/benchmark_attn_decoding.py:435)."""

    @classmethod
    def apply(cls, inp: Inputs, needs_gradient: bool) -> Tuple[torch.Tensor, Optional[Context]]:
        raise NotImplementedError()


class AttentionBwOpBase(AttentionOpBase):
    """The backward pass is outside this library."""


AttentionOp = Tuple[Optional[Type[AttentionFwOpBase]], Optional[Type[AttentionBwOpBase]]]
