"""``oracle.attn_bias_utils`` (the reference's ``xformers.attn_bias_utils`` names) and the
local-attention bias classes, on the CPU."""

import pytest
import torch

import oracle
from oracle import attn_bias_utils as abu
from xformers_b200.ops.fmha import attn_bias as ab


def test_local_band_classes_materialise_like_the_integer_mask():
    # LocalAttentionFromBottomRightMask KAT: tests/test_mem_eff_attention.py:2389-2399
    m = ab.LocalAttentionFromBottomRightMask(window_left=1, window_right=2).materialize((4, 4))
    assert torch.equal(m, oracle.local_mask(4, 4, 1, 2))
    q_lens, kv_lens, pad = [3, 7, 1], [5, 7, 9], 12
    padded = ab.BlockDiagonalLocalAttentionPaddedKeysMask.from_seqlens_local(q_lens, pad, kv_lens, 2, 1)
    got = padded.materialize((sum(q_lens), len(q_lens) * pad))
    want = torch.full_like(got, float("-inf"))
    qs = 0
    for b, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        want[qs : qs + ql, b * pad : b * pad + kl] = oracle.local_mask(ql, kl, 2, 1)
        qs += ql
    assert torch.equal(got, want)
    starts = [1, 14, 25, 36]
    gappy = ab.BlockDiagonalLocalAttentionFromBottomRightGappyKeysMask.from_seqlens_local(q_lens, starts, kv_lens, 2, 1)
    got = gappy.materialize((sum(q_lens), 36))
    want = torch.full_like(got, float("-inf"))
    qs = 0
    for b, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        want[qs : qs + ql, starts[b] : starts[b] + kl] = oracle.local_mask(ql, kl, 2, 1)
        qs += ql
    assert torch.equal(got, want)
    assert type(gappy.to("cpu")) is type(gappy) and gappy.to("cpu").window_right == 1
    with pytest.raises(ValueError):
        ab.BlockDiagonalLocalAttentionPaddedKeysMask.from_seqlens_local(q_lens, pad, kv_lens, -1, 0)


BIAS_TYPES = [
    type(None), torch.Tensor, ab.LowerTriangularMask, ab.LowerTriangularFromBottomRightMask, ab.LowerTriangularMaskLocalAttention,
    ab.LowerTriangularFromBottomRightLocalAttentionMask, ab.LocalAttentionFromBottomRightMask, ab.LowerTriangularMaskWithTensorBias,
    ab.BlockDiagonalMask, ab.BlockDiagonalCausalMask, ab.BlockDiagonalCausalFromBottomRightMask, ab.BlockDiagonalCausalLocalAttentionMask,
    ab.BlockDiagonalCausalLocalAttentionFromBottomRightMask, ab.BlockDiagonalPaddedKeysMask, ab.BlockDiagonalCausalWithOffsetPaddedKeysMask,
    ab.BlockDiagonalCausalLocalAttentionPaddedKeysMask, ab.BlockDiagonalLocalAttentionPaddedKeysMask, ab.BlockDiagonalGappyKeysMask,
    ab.BlockDiagonalCausalWithOffsetGappyKeysMask, ab.BlockDiagonalLocalAttentionFromBottomRightGappyKeysMask,
    ab.PagedBlockDiagonalPaddedKeysMask, ab.PagedBlockDiagonalCausalWithOffsetPaddedKeysMask, ab.PagedBlockDiagonalCausalLocalPaddedKeysMask,
    ab.PagedBlockDiagonalGappyKeysMask, ab.PagedBlockDiagonalCausalWithOffsetGappyKeysMask,
]


@pytest.mark.parametrize("bias_type", BIAS_TYPES)
def test_create_attn_bias_builds_every_bias(bias_type):
    B, H, G, Mq, Mkv = 3, 2, 2, 16, 64
    bias = abu.create_attn_bias(bias_type, B, H, G, Mq, Mkv, "cpu", torch.float32, False, "BMGHK", None, page_size=16)
    again = abu.create_attn_bias(bias_type, B, H, G, Mq, Mkv, "cpu", torch.float32, False, "BMGHK", None, page_size=16)
    if bias_type is type(None):
        assert bias is None
        return
    assert isinstance(bias, bias_type)
    if bias_type is torch.Tensor:
        assert bias.shape == (B, G, H, Mq, Mkv) and torch.equal(bias, again)
        return
    varlen = isinstance(bias, ab.VARLEN_BIASES)
    if isinstance(bias, (ab.BlockDiagonalPaddedKeysMask, ab.PagedBlockDiagonalPaddedKeysMask)):
        shape = (B * Mq, B * Mkv)
    elif varlen:
        shape = (Mq, Mkv)  # the sequences partition the rows
    else:
        shape = (Mq, Mkv)
    m = bias.materialize(shape)
    assert m.shape[-2:] == shape and torch.equal(m, again.materialize(shape))
    assert torch.isfinite(m).any(), "some key must be visible"
    assert ((m == 0) | torch.isneginf(m)).all() or bias_type is ab.LowerTriangularMaskWithTensorBias


def test_pack_kv_cache_keeps_every_token_and_only_used_pages():
    g = torch.Generator().manual_seed(0)
    B, T, H, D, page = 4, 96, 2, 8, 16
    ck, cv = torch.randn(B, T, H, D, generator=g), torch.randn(B, T, H, D, generator=g)
    lens = [96, 1, 40, 17]
    bt, pk, pv = abu.pack_kv_cache(ck, cv, lens, page)
    assert bt.dtype == torch.int32 and bt.shape == (B, 6) and pk.shape == (1, (6 + 1 + 3 + 2) * page, H, D)
    back_k = oracle.gather_paged(pk, bt, page, lens, T)
    back_v = oracle.gather_paged(pv, bt, page, lens, T)
    for b, n in enumerate(lens):
        assert torch.equal(back_k[0, b * T : b * T + n], ck[b, :n]) and torch.equal(back_v[0, b * T : b * T + n], cv[b, :n])
    # attention through the packed pages equals attention on the padded cache
    q = torch.randn(1, B, H, D, generator=g)
    flat = ab.BlockDiagonalPaddedKeysMask.from_seqlens([1] * B, T, lens)
    paged = flat.make_paged(bt, page, ab.PagedBlockDiagonalPaddedKeysMask)
    o1, l1 = oracle.ref_attention_with_lse(q, ck.reshape(1, B * T, H, D), cv.reshape(1, B * T, H, D), flat)
    o2, l2 = oracle.ref_attention_with_lse(q, pk, pv, paged)
    torch.testing.assert_close(o1, o2)
    torch.testing.assert_close(l1, l2)
