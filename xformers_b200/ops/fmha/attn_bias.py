"""Attention-bias descriptors of the fmha API.

Mirrors the public names of ``xformers.ops.fmha.attn_bias``
(xformers/ops/fmha/attn_bias.py:21-49).  A bias object never holds an
``[Mq, Mkv]`` tensor: it is a *description* (sequence starts, key lengths,
page tables) that the kernels consume directly from device memory, plus a
``materialize`` method that expands it to an additive mask for tests.

Mask semantics (pinned by the reference's known-answer tests):
  * ``LowerTriangularMask``: key j visible to query i iff j <= i (top-left
    aligned; tests/test_mem_eff_attention.py:1427-1439).
  * block-diagonal biases: tensors carry batch 1 with all sequences
    concatenated; block b couples q rows ``[sq[b], sq[b+1])`` with k rows
    ``[sk[b], sk[b+1])``; causal variants are top-left aligned per block
    unless "FromBottomRight" (tests/test_mem_eff_attention.py:1452-1587).
  * padded-keys biases: keys of sequence b live at ``[b*P, b*P+kv_seqlen[b])``;
    the causal-with-offset form is bottom-right aligned w.r.t. ``kv_seqlen[b]``
    (tests/test_mem_eff_attention.py:1590-1646).
  * paged biases: logical token t of sequence b is physical row
    ``block_tables[b, t // page_size] * page_size + t % page_size``
    (tests/test_tree_attention.py:375-409).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, ClassVar, Iterable, List, Optional, Sequence, Tuple, Type, Union

import torch


def _additive(visible: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    out = torch.zeros(visible.shape, dtype=dtype, device=visible.device)
    return out.masked_fill_(~visible, -math.inf)


def _band(
    mq: int,
    mkv: int,
    device,
    *,
    shift: int,
    window_left: Optional[int] = None,
    window_right: Optional[int] = 0,
) -> torch.Tensor:
    """Boolean ``[mq, mkv]``: key j visible to query i iff
    ``i + shift - window_left <= j <= i + shift + window_right`` (a bound set
    to ``None`` is absent)."""
    i = torch.arange(mq, device=device).view(-1, 1)
    j = torch.arange(mkv, device=device).view(1, -1)
    vis = torch.ones((mq, mkv), dtype=torch.bool, device=device)
    if window_right is not None:
        vis &= j <= i + shift + window_right
    if window_left is not None:
        vis &= j >= i + shift - window_left
    return vis


class AttentionBias:
    """Base class.  ``HOLDS_DENSE_TENSOR`` is False for every bias the kernels
    accept: they are implicit masks, not tensors."""

    HOLDS_DENSE_TENSOR: ClassVar[bool] = False

    def materialize(
        self,
        shape: Tuple[int, ...],
        dtype: torch.dtype = torch.float32,
        device: Union[str, torch.device] = "cpu",
    ) -> torch.Tensor:
        raise NotImplementedError()

    def to(self, device) -> "AttentionBias":
        return self


class LowerTriangularMask(AttentionBias):
    """Top-left aligned causal mask; holds no tensor and allocates nothing."""

    def to(self, device) -> "LowerTriangularMask":
        return self

    def materialize(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        vis = _band(shape[-2], shape[-1], device, shift=0)
        return _additive(vis, dtype).expand(*shape)

    def add_bias(self, bias: torch.Tensor) -> "LowerTriangularMaskWithTensorBias":
        return LowerTriangularMaskWithTensorBias(bias)

    def make_local_attention(self, window_size: int) -> "LowerTriangularMaskLocalAttention":
        return LowerTriangularMaskLocalAttention(window_size)


@dataclass
class LowerTriangularMaskLocalAttention(LowerTriangularMask):
    _window_size: int = 0

    def materialize(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        vis = _band(shape[-2], shape[-1], device, shift=0, window_left=self._window_size - 1)
        return _additive(vis, dtype).expand(*shape)


class LowerTriangularFromBottomRightMask(AttentionBias):
    """Causal mask whose diagonal ends in the bottom-right corner."""

    def materialize(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        vis = _band(shape[-2], shape[-1], device, shift=shape[-1] - shape[-2])
        return _additive(vis, dtype).expand(*shape)


@dataclass
class LowerTriangularFromBottomRightLocalAttentionMask(LowerTriangularFromBottomRightMask):
    """Bottom-right causal mask that also hides keys more than ``_window_size - 1``
    positions left of the diagonal: each query sees at most ``_window_size`` keys
    (xformers/ops/fmha/attn_bias.py:42; listed as a bottom-right mask in
    tests/test_mem_eff_attention.py:384-396)."""

    _window_size: int = 0

    def __post_init__(self) -> None:
        if self._window_size <= 0:
            raise ValueError(f"Expected `window_size > 0`, but window_size={self._window_size}")

    def materialize(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        vis = _band(shape[-2], shape[-1], device, shift=shape[-1] - shape[-2], window_left=self._window_size - 1)
        return _additive(vis, dtype).expand(*shape)


@dataclass
class LocalAttentionFromBottomRightMask(AttentionBias):
    """Bottom-right aligned band (tests/test_mem_eff_attention.py:2389-2399)."""

    window_left: int
    window_right: int

    def materialize(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        vis = _band(
            shape[-2],
            shape[-1],
            device,
            shift=shape[-1] - shape[-2],
            window_left=self.window_left,
            window_right=self.window_right,
        )
        return _additive(vis, dtype).expand(*shape)


class LowerTriangularMaskWithTensorBias(LowerTriangularMask):
    """Causal mask plus an additive tensor ``[B, (G,) H, Mq, Mkv]``
    (tests/test_mem_eff_attention.py:1431-1449); runs on the mma.sync prefill kernel."""

    HOLDS_DENSE_TENSOR = True

    def __init__(self, bias: torch.Tensor) -> None:
        self._bias = bias

    def materialize(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        return super().materialize(shape, dtype=dtype, device=device) + self._bias.to(device=device, dtype=dtype)


# ---------------------------------------------------------------------------
# sequence-length records
# ---------------------------------------------------------------------------


@dataclass
class _SeqLenInfo:
    """Where each sequence starts inside a concatenated ``[1, sum(len), ...]``
    tensor.  ``seqstart`` is an int32 tensor ``[n+1]`` that the kernels read
    from device memory at run time; ``seqstart_py`` is its host copy, used only
    when the object is built (rope_padded.py:110,233; generate.py:119-126)."""

    seqstart: torch.Tensor
    max_seqlen: int
    min_seqlen: int
    seqstart_py: List[int]

    def to(self, device) -> "_SeqLenInfo":
        if self.seqstart.device == torch.device(device):
            return self
        return _SeqLenInfo(self.seqstart.to(device), self.max_seqlen, self.min_seqlen, self.seqstart_py)

    def intervals(self) -> Iterable[Tuple[int, int]]:
        yield from zip(self.seqstart_py, self.seqstart_py[1:])

    @classmethod
    def _starts(cls, seqlens: Iterable[int]) -> Tuple[List[int], int, int]:
        starts = [0]
        mx, mn = -1, -1
        for n in seqlens:
            n = int(n)
            mx = max(mx, n)
            mn = n if mn < 0 else min(mn, n)
            starts.append(starts[-1] + n)
        return starts, mx, mn

    @classmethod
    def from_seqlens(cls, seqlens: Iterable[int], *, device=None) -> "_SeqLenInfo":
        starts, mx, mn = cls._starts(seqlens)
        return cls(
            seqstart=torch.tensor(starts, dtype=torch.int32, device=device),
            max_seqlen=mx,
            min_seqlen=mn,
            seqstart_py=starts,
        )

    def split(self, x: torch.Tensor, batch_sizes: Optional[Sequence[int]] = None) -> List[torch.Tensor]:
        if self.seqstart_py[-1] != x.shape[1] or x.shape[0] != 1:
            raise ValueError(
                f"Invalid `torch.Tensor` of shape {tuple(x.shape)}, expected "
                f"(1, {self.seqstart_py[-1]}, ...): it does not match this sequence layout"
            )
        if batch_sizes is None:
            batch_sizes = [1] * (len(self.seqstart_py) - 1)
        out, it = [], 0
        for bs in batch_sizes:
            lo, hi = self.seqstart_py[it], self.seqstart_py[it + bs]
            out.append(x[:, lo:hi].reshape(bs, -1, *x.shape[2:]))
            it += bs
        return out


@dataclass
class _PaddedSeqLenInfo(_SeqLenInfo):
    """Sequence b owns the slot ``[b*padding, (b+1)*padding)`` of the key cache
    and fills its first ``seqlen[b]`` rows.  ``seqlen`` is a device int32
    tensor ``[n]`` that callers mutate in place between CUDA-graph replays
    (generate.py:179-185), so kernels never read the host copy."""

    seqlen: torch.Tensor = None  # type: ignore[assignment]
    seqlen_py: Sequence[int] = ()
    padding: int = 0

    def to(self, device) -> "_PaddedSeqLenInfo":
        if self.seqlen.device == torch.device(device):
            return self
        return _PaddedSeqLenInfo(
            seqstart=self.seqstart.to(device),
            max_seqlen=self.max_seqlen,
            min_seqlen=self.min_seqlen,
            seqstart_py=self.seqstart_py,
            seqlen=self.seqlen.to(device),
            seqlen_py=self.seqlen_py,
            padding=self.padding,
        )

    def intervals(self) -> Iterable[Tuple[int, int]]:
        for start, length in zip(self.seqstart_py, self.seqlen_py):
            yield start, start + length

    @classmethod
    def from_seqlens(cls, seqlens, *, device=None):  # type: ignore[override]
        raise RuntimeError("use from_seqlens_padded")

    @classmethod
    def from_seqlens_padded(cls, seqlens: Sequence[int], padding: int, *, device=None) -> "_PaddedSeqLenInfo":
        seqlens = [int(s) for s in seqlens]
        if any(s > padding for s in seqlens):
            raise ValueError(f"Seqlens {seqlens} Padding {padding}: a sequence is longer than its slot")
        starts = list(range(0, len(seqlens) * padding + 1, padding)) if padding > 0 else [0] * (len(seqlens) + 1)
        return cls(
            seqstart=torch.tensor(starts, dtype=torch.int32, device=device),
            max_seqlen=max(seqlens) if seqlens else -1,
            min_seqlen=min(seqlens) if seqlens else -1,
            seqstart_py=starts,
            seqlen=torch.tensor(seqlens, dtype=torch.int32, device=device),
            seqlen_py=seqlens,
            padding=padding,
        )

    def split(self, x, batch_sizes=None):
        raise NotImplementedError("a padded cache is not split back into sequences")


@dataclass
class _GappySeqInfo(_PaddedSeqLenInfo):
    """Sequence b owns the key rows ``[seqstart[b], seqstart[b] + seqlen[b])``;
    ``seqstart`` has ``n + 1`` entries (the last one closes the last slot) and
    the slots need not be equally long (fmha/attn_bias.py:21, ``_GappySeqInfo``;
    tests/test_fmha_merge_attentions.py:406-414).  ``padding`` is the longest slot."""

    def to(self, device) -> "_GappySeqInfo":
        if self.seqlen.device == torch.device(device):
            return self
        return _GappySeqInfo(
            seqstart=self.seqstart.to(device),
            max_seqlen=self.max_seqlen,
            min_seqlen=self.min_seqlen,
            seqstart_py=self.seqstart_py,
            seqlen=self.seqlen.to(device),
            seqlen_py=self.seqlen_py,
            padding=self.padding,
        )

    @classmethod
    def from_seqlens_gappy(cls, seqstarts: Sequence[int], seqlens: Sequence[int], *, device=None) -> "_GappySeqInfo":
        seqstarts, seqlens = [int(s) for s in seqstarts], [int(s) for s in seqlens]
        if len(seqstarts) != len(seqlens) + 1:
            raise ValueError(f"kv_seqstarts needs one entry more than kv_seqlen, got {len(seqstarts)} and {len(seqlens)}")
        slots = [seqstarts[i + 1] - seqstarts[i] for i in range(len(seqlens))]
        if any(n < 0 or n > slot for n, slot in zip(seqlens, slots)):
            raise ValueError(f"Seqlens {seqlens} do not fit the slots between the starts {seqstarts}")
        return cls(
            seqstart=torch.tensor(seqstarts, dtype=torch.int32, device=device),
            max_seqlen=max(seqlens) if seqlens else -1,
            min_seqlen=min(seqlens) if seqlens else -1,
            seqstart_py=seqstarts,
            seqlen=torch.tensor(seqlens, dtype=torch.int32, device=device),
            seqlen_py=seqlens,
            padding=max(slots) if slots else 0,
        )


# ---------------------------------------------------------------------------
# block-diagonal family (queries and keys concatenated, batch 1)
# ---------------------------------------------------------------------------


@dataclass
class BlockDiagonalMask(AttentionBias):
    q_seqinfo: _SeqLenInfo
    k_seqinfo: _SeqLenInfo
    _batch_sizes: Optional[Sequence[int]] = None

    def to(self, device) -> "BlockDiagonalMask":
        return type(self)(
            q_seqinfo=self.q_seqinfo.to(device),
            k_seqinfo=self.k_seqinfo.to(device),
            _batch_sizes=self._batch_sizes,
        )

    # -- what a single block looks like -------------------------------------
    def _block(self, ql: int, kl: int, device) -> torch.Tensor:
        return torch.ones((ql, kl), dtype=torch.bool, device=device)

    def materialize(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        if shape[-1] != self.k_seqinfo.seqstart_py[-1]:
            raise ValueError(f"key axis {shape[-1]} != {self.k_seqinfo.seqstart_py[-1]}")
        if shape[-2] != self.q_seqinfo.seqstart_py[-1]:
            raise ValueError(f"query axis {shape[-2]} != {self.q_seqinfo.seqstart_py[-1]}")
        vis = torch.zeros(shape[-2:], dtype=torch.bool, device=device)
        for (qs, qe), (ks, ke) in zip(self.q_seqinfo.intervals(), self.k_seqinfo.intervals()):
            vis[qs:qe, ks:ke] = self._block(qe - qs, ke - ks, device)
        return _additive(vis, dtype).expand(*shape)

    # -- constructors ---------------------------------------------------------
    @classmethod
    def from_seqlens(
        cls,
        q_seqlen: Sequence[int],
        kv_seqlen: Optional[Sequence[int]] = None,
        *,
        device=None,
    ) -> "BlockDiagonalMask":
        if kv_seqlen is not None and len(q_seqlen) != len(kv_seqlen):
            raise ValueError("q_seqlen and kv_seqlen must describe the same number of sequences")
        q_info = _SeqLenInfo.from_seqlens(q_seqlen, device=device)
        k_info = q_info if kv_seqlen is None or list(q_seqlen) == list(kv_seqlen) else _SeqLenInfo.from_seqlens(kv_seqlen, device=device)
        return cls(q_seqinfo=q_info, k_seqinfo=k_info)

    @classmethod
    def from_tensor_list(cls, tensors: Sequence[torch.Tensor]) -> Tuple["BlockDiagonalMask", torch.Tensor]:
        batch_sizes = [t.shape[0] for t in tensors]
        seqlens: List[int] = []
        for t in tensors:
            seqlens += [t.shape[1]] * t.shape[0]
        bias = cls.from_seqlens(seqlens)
        bias._batch_sizes = batch_sizes
        cat = torch.cat([t.reshape(1, -1, *t.shape[2:]) for t in tensors], dim=1)
        return bias, cat

    @classmethod
    def from_tensor_lists_qkv(
        cls,
        tensors_q: Sequence[torch.Tensor],
        tensors_k: Sequence[torch.Tensor],
        tensors_v: Optional[Sequence[torch.Tensor]] = None,
    ) -> Tuple["BlockDiagonalMask", torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
        assert len(tensors_q) == len(tensors_k)
        assert tensors_v is None or len(tensors_v) == len(tensors_q)
        batch_sizes = [t.shape[0] for t in tensors_q]
        q_lens: List[int] = []
        k_lens: List[int] = []
        for tq, tk in zip(tensors_q, tensors_k):
            assert tq.shape[0] == tk.shape[0]
            q_lens += [tq.shape[1]] * tq.shape[0]
            k_lens += [tk.shape[1]] * tk.shape[0]
        bias = cls.from_seqlens(q_lens, k_lens)
        bias._batch_sizes = batch_sizes
        cat = lambda ts: torch.cat([t.reshape(1, -1, *t.shape[2:]) for t in ts], dim=1)
        return bias, cat(tensors_q), cat(tensors_k), (cat(tensors_v) if tensors_v is not None else None)

    # -- inverse of the concatenation -----------------------------------------
    def split_queries(self, tensor: torch.Tensor) -> List[torch.Tensor]:
        return self.q_seqinfo.split(tensor, self._batch_sizes)

    def split_kv(self, tensor: torch.Tensor) -> List[torch.Tensor]:
        return self.k_seqinfo.split(tensor, self._batch_sizes)

    def split(self, tensor: torch.Tensor) -> List[torch.Tensor]:
        assert self.q_seqinfo is self.k_seqinfo or self.q_seqinfo.seqstart_py == self.k_seqinfo.seqstart_py
        return self.q_seqinfo.split(tensor, self._batch_sizes)

    # -- derived masks --------------------------------------------------------
    def make_causal(self) -> "BlockDiagonalCausalMask":
        return BlockDiagonalCausalMask(self.q_seqinfo, self.k_seqinfo, self._batch_sizes)

    def make_causal_from_bottomright(self) -> "BlockDiagonalCausalFromBottomRightMask":
        return BlockDiagonalCausalFromBottomRightMask(self.q_seqinfo, self.k_seqinfo, self._batch_sizes)

    def make_local_attention(self, window_size: int) -> "BlockDiagonalCausalLocalAttentionMask":
        return BlockDiagonalCausalLocalAttentionMask(self.q_seqinfo, self.k_seqinfo, self._batch_sizes, window_size)

    def make_local_attention_from_bottomright(self, window_size: int) -> "BlockDiagonalCausalLocalAttentionFromBottomRightMask":
        return BlockDiagonalCausalLocalAttentionFromBottomRightMask(self.q_seqinfo, self.k_seqinfo, self._batch_sizes, window_size)


@dataclass
class BlockDiagonalCausalMask(BlockDiagonalMask):
    """Each block is top-left aligned causal."""

    def _block(self, ql, kl, device):
        return _band(ql, kl, device, shift=0)


@dataclass
class BlockDiagonalCausalFromBottomRightMask(BlockDiagonalMask):
    """Each block is causal with its diagonal ending bottom-right; every
    sequence needs at least as many keys as queries
    (tests/test_mem_eff_attention.py:1541-1552)."""

    def __post_init__(self) -> None:
        for i, ((qs, qe), (ks, ke)) in enumerate(zip(self.q_seqinfo.intervals(), self.k_seqinfo.intervals())):
            if qe - qs > ke - ks:
                raise ValueError(
                    f"Block #{i} has {qe - qs} queries and only {ke - ks} keys: a "
                    "bottom-right causal block would leave queries without any key"
                )

    def _block(self, ql, kl, device):
        return _band(ql, kl, device, shift=kl - ql)


@dataclass
class BlockDiagonalCausalLocalAttentionMask(BlockDiagonalCausalMask):
    _window_size: int = 0

    def __post_init__(self) -> None:
        if self._window_size <= 0:
            raise ValueError(f"Expected `window_size > 0`, got {self._window_size}")

    def to(self, device):
        return type(self)(self.q_seqinfo.to(device), self.k_seqinfo.to(device), self._batch_sizes, self._window_size)

    def _block(self, ql, kl, device):
        return _band(ql, kl, device, shift=0, window_left=self._window_size - 1)


@dataclass
class BlockDiagonalCausalLocalAttentionFromBottomRightMask(BlockDiagonalCausalFromBottomRightMask):
    _window_size: int = 0

    def to(self, device):
        return type(self)(self.q_seqinfo.to(device), self.k_seqinfo.to(device), self._batch_sizes, self._window_size)

    def _block(self, ql, kl, device):
        return _band(ql, kl, device, shift=kl - ql, window_left=self._window_size - 1)


# ---------------------------------------------------------------------------
# padded-keys family (decode / KV cache with one fixed-size slot per sequence)
# ---------------------------------------------------------------------------


@dataclass
class BlockDiagonalPaddedKeysMask(AttentionBias):
    q_seqinfo: _SeqLenInfo
    k_seqinfo: _PaddedSeqLenInfo

    _CAUSAL: ClassVar[bool] = False

    def to(self, device):
        return type(self)(q_seqinfo=self.q_seqinfo.to(device), k_seqinfo=self.k_seqinfo.to(device))

    def _block(self, ql: int, kl: int, device) -> torch.Tensor:
        if self._CAUSAL:
            return _band(ql, kl, device, shift=kl - ql)
        return torch.ones((ql, kl), dtype=torch.bool, device=device)

    def materialize(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        if shape[-1] != self.k_seqinfo.seqstart_py[-1]:
            raise ValueError(f"key axis {shape[-1]} != {self.k_seqinfo.seqstart_py[-1]}")
        if shape[-2] != self.q_seqinfo.seqstart_py[-1]:
            raise ValueError(f"query axis {shape[-2]} != {self.q_seqinfo.seqstart_py[-1]}")
        vis = torch.zeros(shape[-2:], dtype=torch.bool, device=device)
        for (qs, qe), (ks, ke) in zip(self.q_seqinfo.intervals(), self.k_seqinfo.intervals()):
            vis[qs:qe, ks:ke] = self._block(qe - qs, ke - ks, device)
        return _additive(vis, dtype).expand(*shape)

    @classmethod
    def from_seqlens(
        cls,
        q_seqlen: Sequence[int],
        kv_padding: int,
        kv_seqlen: Sequence[int],
        causal_diagonal: Any = None,
        *,
        device=None,
    ):
        if len(q_seqlen) != len(kv_seqlen):
            raise ValueError("q_seqlen and kv_seqlen must describe the same number of sequences")
        return cls(
            q_seqinfo=_SeqLenInfo.from_seqlens(q_seqlen, device=device),
            k_seqinfo=_PaddedSeqLenInfo.from_seqlens_padded(kv_seqlen, kv_padding, device=device),
        )

    def make_paged(
        self,
        block_tables: torch.Tensor,
        page_size: int,
        paged_type: Type["PagedBlockDiagonalPaddedKeysMask"],
        notional_padding: Optional[int] = None,
    ) -> "PagedBlockDiagonalPaddedKeysMask":
        """Same sequences, but keys are reached through ``block_tables``
        (tests/test_mem_eff_attention.py:2595-2599)."""
        max_row_len = block_tables.shape[1] * page_size
        k_info = _PaddedSeqLenInfo.from_seqlens_padded(
            self.k_seqinfo.seqlen_py, notional_padding or max_row_len, device=self.k_seqinfo.seqlen.device
        )
        # share the device tensor so that in-place length updates stay visible
        k_info.seqlen = self.k_seqinfo.seqlen
        extra = {"_window_size": self._window_size} if hasattr(self, "_window_size") else {}
        return paged_type(q_seqinfo=self.q_seqinfo, k_seqinfo=k_info, block_tables=block_tables, page_size=page_size, **extra)


@dataclass
class BlockDiagonalCausalWithOffsetPaddedKeysMask(BlockDiagonalPaddedKeysMask):
    """Bottom-right causal w.r.t. each sequence's current key length: query i
    of a block of ql queries sees key t iff ``t <= i + kv_seqlen[b] - ql``."""

    _CAUSAL: ClassVar[bool] = True


@dataclass
class BlockDiagonalCausalLocalAttentionPaddedKeysMask(BlockDiagonalPaddedKeysMask):
    """:class:`BlockDiagonalCausalWithOffsetPaddedKeysMask` with a window: query
    i of a block of ql queries sees key t of its sequence iff ``t <= i +
    kv_seqlen[b] - ql`` and ``t > i + kv_seqlen[b] - ql - _window_size``
    (xformers/ops/fmha/attn_bias.py:29; tests/test_mem_eff_attention.py:283)."""

    _window_size: int = 0

    def to(self, device):
        return type(self)(q_seqinfo=self.q_seqinfo.to(device), k_seqinfo=self.k_seqinfo.to(device), _window_size=self._window_size)

    def _block(self, ql: int, kl: int, device) -> torch.Tensor:
        return _band(ql, kl, device, shift=kl - ql, window_left=self._window_size - 1)

    @classmethod
    def from_seqlens_local(cls, q_seqlen: Sequence[int], kv_padding: int, kv_seqlen: Sequence[int], window_size: int, *, device=None):
        if window_size <= 0:
            raise ValueError(f"Expected `window_size > 0`, but window_size={window_size}")
        if len(q_seqlen) != len(kv_seqlen):
            raise ValueError("q_seqlen and kv_seqlen must describe the same number of sequences")
        return cls(
            q_seqinfo=_SeqLenInfo.from_seqlens(q_seqlen, device=device),
            k_seqinfo=_PaddedSeqLenInfo.from_seqlens_padded(kv_seqlen, kv_padding, device=device),
            _window_size=window_size,
        )


@dataclass
class BlockDiagonalLocalAttentionPaddedKeysMask(BlockDiagonalPaddedKeysMask):
    """Padded-keys block-diagonal mask with a band around the bottom-right
    diagonal instead of a causal one: query i of a block of ql queries sees key
    t of its sequence iff ``i + kv_seqlen[b] - ql - window_left <= t <= i +
    kv_seqlen[b] - ql + window_right`` (xformers/ops/fmha/attn_bias.py:35; the
    band of ``LocalAttentionFromBottomRightMask``, tests/test_mem_eff_attention.py:2389-2399,
    per sequence)."""

    window_left: int = 0
    window_right: int = 0

    def __post_init__(self) -> None:
        if self.window_left < 0 or self.window_right < 0:
            raise ValueError(f"Expected non-negative windows, got ({self.window_left}, {self.window_right})")

    def to(self, device):
        return type(self)(q_seqinfo=self.q_seqinfo.to(device), k_seqinfo=self.k_seqinfo.to(device),
                          window_left=self.window_left, window_right=self.window_right)

    def _block(self, ql: int, kl: int, device) -> torch.Tensor:
        return _band(ql, kl, device, shift=kl - ql, window_left=self.window_left, window_right=self.window_right)

    @classmethod
    def from_seqlens_local(cls, q_seqlen: Sequence[int], kv_padding: int, kv_seqlen: Sequence[int], window_left: int,
                           window_right: int, *, device=None):
        if len(q_seqlen) != len(kv_seqlen):
            raise ValueError("q_seqlen and kv_seqlen must describe the same number of sequences")
        return cls(
            q_seqinfo=_SeqLenInfo.from_seqlens(q_seqlen, device=device),
            k_seqinfo=_PaddedSeqLenInfo.from_seqlens_padded(kv_seqlen, kv_padding, device=device),
            window_left=window_left,
            window_right=window_right,
        )


@dataclass
class BlockDiagonalGappyKeysMask(BlockDiagonalPaddedKeysMask):
    """Keys of sequence b are the rows ``[kv_seqstarts[b], kv_seqstarts[b] +
    kv_seqlen[b])`` of the flat key tensor: like the padded-keys mask, but the
    first row of every sequence is free (tests/test_fmha_merge_attentions.py:406-414,
    tests/test_mem_eff_attention.py:2521-2525)."""

    k_seqinfo: _GappySeqInfo

    @classmethod
    def from_seqlens(cls, q_seqlen: Sequence[int], kv_seqstarts: Sequence[int], kv_seqlen: Sequence[int], *, device=None):  # type: ignore[override]
        if len(q_seqlen) != len(kv_seqlen):
            raise ValueError("q_seqlen and kv_seqlen must describe the same number of sequences")
        return cls(
            q_seqinfo=_SeqLenInfo.from_seqlens(q_seqlen, device=device),
            k_seqinfo=_GappySeqInfo.from_seqlens_gappy(kv_seqstarts, kv_seqlen, device=device),
        )

    def make_paged(self, block_tables, page_size, paged_type, notional_padding=None):  # type: ignore[override]
        """Keys reached through ``block_tables``; sequence b's logical rows are
        those of the slot ``[b * notional_padding, (b+1) * notional_padding)``
        (tests/test_mem_eff_attention.py:2516-2525)."""
        if notional_padding is None:
            raise ValueError("make_paged of a gappy bias needs notional_padding")
        starts = self.k_seqinfo.seqstart_py
        for b, n in enumerate(self.k_seqinfo.seqlen_py):
            if not (b * notional_padding <= starts[b] and starts[b] + n <= (b + 1) * notional_padding):
                raise ValueError(f"sequence {b} does not lie inside its notional slot of {notional_padding} rows")
        return paged_type(
            q_seqinfo=self.q_seqinfo, k_seqinfo=self.k_seqinfo, block_tables=block_tables, page_size=page_size,
            notional_padding=notional_padding,
        )


@dataclass
class BlockDiagonalCausalWithOffsetGappyKeysMask(BlockDiagonalGappyKeysMask):
    _CAUSAL: ClassVar[bool] = True


@dataclass
class BlockDiagonalLocalAttentionFromBottomRightGappyKeysMask(BlockDiagonalGappyKeysMask):
    """Gappy-keys block-diagonal mask with a band around the bottom-right
    diagonal of every block: query i of a block of ql queries sees key t of its
    sequence iff ``i + kv_seqlen[b] - ql - window_left <= t <= i + kv_seqlen[b] -
    ql + window_right`` (xformers/ops/fmha/attn_bias.py:34)."""

    window_left: int = 0
    window_right: int = 0

    def __post_init__(self) -> None:
        if self.window_left < 0 or self.window_right < 0:
            raise ValueError(f"Expected non-negative windows, got ({self.window_left}, {self.window_right})")

    def to(self, device):
        return type(self)(q_seqinfo=self.q_seqinfo.to(device), k_seqinfo=self.k_seqinfo.to(device),
                          window_left=self.window_left, window_right=self.window_right)

    def _block(self, ql: int, kl: int, device) -> torch.Tensor:
        return _band(ql, kl, device, shift=kl - ql, window_left=self.window_left, window_right=self.window_right)

    @classmethod
    def from_seqlens_local(cls, q_seqlen: Sequence[int], kv_seqstarts: Sequence[int], kv_seqlen: Sequence[int],
                           window_left: int, window_right: int, *, device=None):
        if len(q_seqlen) != len(kv_seqlen):
            raise ValueError("q_seqlen and kv_seqlen must describe the same number of sequences")
        return cls(
            q_seqinfo=_SeqLenInfo.from_seqlens(q_seqlen, device=device),
            k_seqinfo=_GappySeqInfo.from_seqlens_gappy(kv_seqstarts, kv_seqlen, device=device),
            window_left=window_left,
            window_right=window_right,
        )


@dataclass
class PagedBlockDiagonalPaddedKeysMask(AttentionBias):
    q_seqinfo: _SeqLenInfo
    k_seqinfo: _PaddedSeqLenInfo
    block_tables: torch.Tensor
    page_size: int

    _UNPAGED_TYPE: ClassVar[Type[BlockDiagonalPaddedKeysMask]] = BlockDiagonalPaddedKeysMask

    def to(self, device):
        return type(self)(
            q_seqinfo=self.q_seqinfo.to(device),
            k_seqinfo=self.k_seqinfo.to(device),
            block_tables=self.block_tables.to(device),
            page_size=self.page_size,
        )

    def materialize(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        """Mask over *physical* key rows: shape[-1] = num_pages * page_size."""
        max_row_len = self.block_tables.shape[1] * self.page_size
        bias_nonpaged = self._UNPAGED_TYPE(
            q_seqinfo=self.q_seqinfo,
            k_seqinfo=_PaddedSeqLenInfo.from_seqlens_padded(self.k_seqinfo.seqlen_py, max_row_len),
        )
        logical = bias_nonpaged.materialize(
            (self.q_seqinfo.seqstart_py[-1], len(self.k_seqinfo.seqlen_py) * max_row_len), dtype=dtype, device=device
        )
        n_rows = shape[-1]
        out = torch.full((logical.shape[0], n_rows), -math.inf, dtype=dtype, device=device)
        bt = self.block_tables.to(device).long()
        for b, ((qs, qe), n) in enumerate(zip(self.q_seqinfo.intervals(), self.k_seqinfo.seqlen_py)):
            t = torch.arange(n, device=device)
            rows = bt[b, t // self.page_size] * self.page_size + t % self.page_size
            out[qs:qe, rows] = logical[qs:qe, b * max_row_len : b * max_row_len + n]
        return out.expand(*shape)

    @classmethod
    def from_seqlens(
        cls,
        q_seqlen: Sequence[int],
        kv_seqlen: Sequence[int],
        block_tables: torch.Tensor,
        page_size: int,
        *,
        device=None,
    ):
        if len(q_seqlen) != len(kv_seqlen):
            raise ValueError("q_seqlen and kv_seqlen must describe the same number of sequences")
        device = block_tables.device if device is None else device
        return cls(
            q_seqinfo=_SeqLenInfo.from_seqlens(q_seqlen, device=device),
            k_seqinfo=_PaddedSeqLenInfo.from_seqlens_padded(kv_seqlen, block_tables.shape[1] * page_size, device=device),
            block_tables=block_tables,
            page_size=page_size,
        )


@dataclass
class PagedBlockDiagonalCausalWithOffsetPaddedKeysMask(PagedBlockDiagonalPaddedKeysMask):
    _UNPAGED_TYPE: ClassVar[Type[BlockDiagonalPaddedKeysMask]] = BlockDiagonalCausalWithOffsetPaddedKeysMask


@dataclass
class PagedBlockDiagonalCausalLocalPaddedKeysMask(PagedBlockDiagonalPaddedKeysMask):
    """:class:`BlockDiagonalCausalLocalAttentionPaddedKeysMask` behind a block table
    (xformers/ops/fmha/attn_bias.py:43; tests/test_mem_eff_attention.py:395)."""

    _window_size: int = 0

    _UNPAGED_TYPE: ClassVar[Type[BlockDiagonalPaddedKeysMask]] = BlockDiagonalCausalLocalAttentionPaddedKeysMask

    def to(self, device):
        return type(self)(
            q_seqinfo=self.q_seqinfo.to(device), k_seqinfo=self.k_seqinfo.to(device),
            block_tables=self.block_tables.to(device), page_size=self.page_size, _window_size=self._window_size,
        )

    def materialize(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        """Mask over *physical* key rows: shape[-1] = num_pages * page_size."""
        out = torch.full((self.q_seqinfo.seqstart_py[-1], shape[-1]), -math.inf, dtype=dtype, device=device)
        bt = self.block_tables.to(device).long()
        for b, ((qs, qe), n) in enumerate(zip(self.q_seqinfo.intervals(), self.k_seqinfo.seqlen_py)):
            t = torch.arange(n, device=device)
            rows = bt[b, t // self.page_size] * self.page_size + t % self.page_size
            vis = _band(qe - qs, n, device, shift=n - (qe - qs), window_left=self._window_size - 1)
            out[qs:qe, rows] = _additive(vis, dtype)
        return out.expand(*shape)

    @classmethod
    def from_seqlens_local(cls, q_seqlen: Sequence[int], kv_seqlen: Sequence[int], block_tables: torch.Tensor, page_size: int,
                           window_size: int, *, device=None):
        if window_size <= 0:
            raise ValueError(f"Expected `window_size > 0`, but window_size={window_size}")
        base = PagedBlockDiagonalPaddedKeysMask.from_seqlens(q_seqlen, kv_seqlen, block_tables, page_size, device=device)
        return cls(q_seqinfo=base.q_seqinfo, k_seqinfo=base.k_seqinfo, block_tables=block_tables, page_size=page_size, _window_size=window_size)


@dataclass
class PagedBlockDiagonalGappyKeysMask(PagedBlockDiagonalPaddedKeysMask):
    """Gappy keys behind a block table: the logical row ``kv_seqstarts[b] - b *
    notional_padding + t`` of sequence b is the physical row
    ``block_tables[b, row // page_size] * page_size + row % page_size``."""

    k_seqinfo: _GappySeqInfo
    notional_padding: int = 0

    _UNPAGED_TYPE: ClassVar[Type[BlockDiagonalPaddedKeysMask]] = BlockDiagonalGappyKeysMask

    def to(self, device):
        return type(self)(
            q_seqinfo=self.q_seqinfo.to(device), k_seqinfo=self.k_seqinfo.to(device),
            block_tables=self.block_tables.to(device), page_size=self.page_size, notional_padding=self.notional_padding,
        )

    def slot_starts(self) -> torch.Tensor:
        """int32 ``[n]`` on the device of the lengths: first logical row of every sequence inside its block table."""
        n = len(self.k_seqinfo.seqlen_py)
        base = torch.arange(n, dtype=torch.int32, device=self.k_seqinfo.seqstart.device) * self.notional_padding
        return (self.k_seqinfo.seqstart[:n] - base).contiguous()

    def materialize(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        """Mask over *physical* key rows: shape[-1] = num_pages * page_size."""
        out = torch.full((self.q_seqinfo.seqstart_py[-1], shape[-1]), -math.inf, dtype=dtype, device=device)
        bt = self.block_tables.to(device).long()
        causal = self._UNPAGED_TYPE._CAUSAL
        for b, ((qs, qe), n) in enumerate(zip(self.q_seqinfo.intervals(), self.k_seqinfo.seqlen_py)):
            t = torch.arange(n, device=device) + (self.k_seqinfo.seqstart_py[b] - b * self.notional_padding)
            rows = bt[b, t // self.page_size] * self.page_size + t % self.page_size
            block = _band(qe - qs, n, device, shift=n - (qe - qs)) if causal else torch.ones((qe - qs, n), dtype=torch.bool, device=device)
            out[qs:qe, rows] = _additive(block, dtype)
        return out.expand(*shape)


@dataclass
class PagedBlockDiagonalCausalWithOffsetGappyKeysMask(PagedBlockDiagonalGappyKeysMask):
    _UNPAGED_TYPE: ClassVar[Type[BlockDiagonalPaddedKeysMask]] = BlockDiagonalCausalWithOffsetGappyKeysMask


VARLEN_BIASES = (
    BlockDiagonalMask,
    BlockDiagonalPaddedKeysMask,
    PagedBlockDiagonalPaddedKeysMask,
)
