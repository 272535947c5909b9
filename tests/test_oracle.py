"""The CPU oracle against the reference's known-answer vectors and against
independent formulas.  No GPU needed."""

import json
import math
import os

import numpy as np
import pytest
import torch

import oracle
from xformers_b200.ops.fmha import attn_bias as ab

HERE = os.path.dirname(os.path.abspath(__file__))
KATS = json.load(open(os.path.join(HERE, "golden", "mask_kats.json")))


def _vis(additive: torch.Tensor) -> torch.Tensor:
    assert ((additive == 0) | torch.isneginf(additive)).all()
    return (additive == 0).to(torch.int64)


def _t(x):
    return torch.tensor(x, dtype=torch.int64)


def both(oracle_mask, package_mask):
    """The oracle's materialiser and the package's bias class must agree."""
    assert torch.equal(_vis(oracle_mask), _vis(package_mask))
    return _vis(oracle_mask)


def test_kat_causal():
    for key in ("causal_3x2", "causal_2x3"):
        want = _t(KATS[key]["visible"])
        got = both(oracle.causal_mask(*want.shape), ab.LowerTriangularMask().materialize(tuple(want.shape)))
        assert torch.equal(got, want)


def test_kat_causal_plus_tensor_bias():
    # tests/test_mem_eff_attention.py:1431-1439
    tb = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    got = ab.LowerTriangularMask().add_bias(tb).materialize((3, 2))
    want = tb + oracle.causal_mask(3, 2)
    assert torch.equal(got, want)


def test_kat_blockdiag():
    for key in ("blockdiag_3_2_5", "blockdiag_batched"):
        lens = KATS[key]["q_seqlens"]
        n = sum(lens)
        got = both(oracle.block_diagonal_mask(lens), ab.BlockDiagonalMask.from_seqlens(lens).materialize((n, n)))
        assert int(got.sum()) == KATS[key]["num_visible"]
        s = 0
        for l in lens:
            assert got[s : s + l, s : s + l].all()
            s += l


def test_kat_blockdiag_crossattn_and_causal():
    k = KATS["blockdiag_crossattn"]
    ql, kl = k["q_seqlens"], k["kv_seqlens"]
    bias = ab.BlockDiagonalMask.from_seqlens(ql, kl)
    got = both(oracle.block_diagonal_mask(ql, kl), bias.materialize((sum(ql), sum(kl))))
    assert int(got.sum()) == k["num_visible"]
    causal = both(oracle.block_diagonal_mask(ql, kl, causal=True), bias.make_causal().materialize((sum(ql), sum(kl))))
    assert torch.equal(causal[3:4, 2:5], _t(k["causal_block_1"]))


def test_kat_bottomright():
    k = KATS["bottomright_prefix"]
    ql, kl = k["q_seqlens"], k["kv_seqlens"]
    bias = ab.BlockDiagonalMask.from_seqlens(ql, kl).make_causal_from_bottomright()
    got = both(
        oracle.block_diagonal_mask(ql, kl, causal=True, from_bottom_right=True), bias.materialize((sum(ql), sum(kl)))
    )
    for blk in k["blocks"]:
        (r0, r1), (c0, c1) = blk["rows"], blk["cols"]
        assert torch.equal(got[r0:r1, c0:c1], _t(blk["visible"]))
    bad = KATS["bottomright_needs_enough_keys"]
    with pytest.raises(ValueError):
        ab.BlockDiagonalMask.from_seqlens(bad["q_seqlens"], bad["kv_seqlens"]).make_causal_from_bottomright()


def test_kat_windows():
    k = KATS["window2_4_6"]
    lens = k["q_seqlens"]
    bias = ab.BlockDiagonalMask.from_seqlens(lens, lens).make_local_attention(k["window_size"])
    got = both(
        oracle.block_diagonal_mask(lens, causal=True, window_size=k["window_size"]),
        bias.materialize((1, 1, sum(lens), sum(lens)))[0, 0],
    )
    assert torch.equal(got, _t(k["visible"]))
    k = KATS["local_1_2_4x4"]
    got = both(
        oracle.local_mask(4, 4, k["window_left"], k["window_right"]),
        ab.LocalAttentionFromBottomRightMask(k["window_left"], k["window_right"]).materialize((4, 4)),
    )
    assert torch.equal(got, _t(k["visible"]))


def test_kat_padded_keys():
    k = KATS["padded_keys_causal"]
    ql, kl, P = k["q_seqlens"], k["kv_seqlens"], k["padding"]
    bias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=ql, kv_seqlen=kl, kv_padding=P)
    got = both(oracle.padded_keys_mask(ql, kl, P, causal=True), bias.materialize((sum(ql), len(kl) * P)))
    assert torch.equal(got[0:4, 0:5], _t(k["first_block_visible"]))
    # the reference's hand-built mask: triu(diagonal = 1 + slen - qlen) is hidden
    want = torch.zeros(sum(ql), len(kl) * P, dtype=torch.int64)
    qs = 0
    for i, (slen, qlen) in enumerate(zip(kl, ql)):
        hidden = torch.triu(torch.ones(qlen, slen), diagonal=1 + slen - qlen)
        want[qs : qs + qlen, i * P : i * P + slen] = 1 - hidden.long()
        qs += qlen
    assert torch.equal(got, want)


def test_ref_attention_against_sdpa():
    torch.manual_seed(3)
    q, k, v = (torch.randn(2, 37, 3, 32) for _ in range(3))
    k = torch.randn(2, 53, 3, 32)
    v = torch.randn(2, 53, 3, 32)
    out, lse = oracle.ref_attention_with_lse(q, k, v)
    want = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2).double(), k.transpose(1, 2).double(), v.transpose(1, 2).double()
    ).transpose(1, 2)
    assert (out.double() - want).abs().max() < 1e-5
    # test-local formula of tests/test_mem_eff_attention.py:664-682
    attn = (q.transpose(1, 2).float() / 32**0.5) @ k.transpose(1, 2).float().transpose(-2, -1)
    assert (lse - attn.logsumexp(-1)).abs().max() < 2e-5


def test_cfg1_golden():
    g = np.load(os.path.join(HERE, "golden", "cfg1_seed0.npz"))
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(2, 128, 4, 64, generator=gen)
    k = torch.randn(2, 128, 4, 64, generator=gen)
    v = torch.randn(2, 128, 4, 64, generator=gen)
    assert np.array_equal(q[0, :4, 0, :8].numpy(), g["q_head"]), "RNG stream changed: regenerate the golden file"
    out, lse = oracle.ref_attention_with_lse(q, k, v, ab.LowerTriangularMask())
    assert out.shape == (2, 128, 4, 64) and lse.shape == (2, 4, 128)
    assert np.abs(out.numpy() - g["out"]).max() < 1e-5
    assert np.abs(lse.numpy() - g["lse"]).max() < 1e-5


def test_bmk_bmghk_layouts_agree():
    torch.manual_seed(0)
    B, M, G, H, K = 2, 9, 2, 3, 16
    q = torch.randn(B, M, G, H, K)
    k = torch.randn(B, M, G, 1, K).expand(B, M, G, H, K)
    v = torch.randn(B, M, G, 1, K).expand(B, M, G, H, K)
    o5, l5 = oracle.ref_attention_with_lse(q, k, v, ab.LowerTriangularMask())
    o4, l4 = oracle.ref_attention_with_lse(q.reshape(B, M, G * H, K), k.reshape(B, M, G * H, K), v.reshape(B, M, G * H, K), ab.LowerTriangularMask())
    assert torch.allclose(o5.reshape(B, M, G * H, K), o4) and torch.allclose(l5.reshape(B, G * H, M), l4)
    q3 = q.reshape(B, M, G * H, K).permute(0, 2, 1, 3).reshape(B * G * H, M, K)
    k3 = k.reshape(B, M, G * H, K).permute(0, 2, 1, 3).reshape(B * G * H, M, K)
    v3 = v.reshape(B, M, G * H, K).permute(0, 2, 1, 3).reshape(B * G * H, M, K)
    o3 = oracle.ref_attention(q3, k3, v3, ab.LowerTriangularMask())
    assert torch.allclose(o3.reshape(B, G * H, M, K).permute(0, 2, 1, 3), o4, atol=1e-6)


@pytest.mark.parametrize("kv_heads", [None, 1, 2])
@pytest.mark.parametrize("padding,bsz", [(32, 8), (256, 1)])
@pytest.mark.parametrize("split_k", [1, 2, 4])
def test_splitk_algebra(kv_heads, padding, bsz, split_k):
    # tests/test_splitk_reference.py:165-222 (d=256 there; smaller here for speed)
    d, n_heads = 64, 16
    torch.manual_seed(1)
    if kv_heads is not None and kv_heads > 1:
        ks, qs = (1, bsz * padding, kv_heads, n_heads, d), (1, bsz, kv_heads, n_heads, d)
    else:
        ks, qs = (1, bsz * padding, n_heads, d), (1, bsz, n_heads, d)
    k, v, q = torch.rand(ks), torch.rand(ks), torch.rand(qs)
    if kv_heads is not None:
        k = k[..., :1, :].expand(ks)
        v = v[..., :1, :].expand(ks)
    lens = torch.randint(1, padding + 1, (bsz,)).tolist()
    bias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=[1] * bsz, kv_seqlen=lens, kv_padding=padding)
    full = oracle.ref_attention(q, k, v, bias)
    split = oracle.ref_attention_splitk(q, k, v, bias, split_k=split_k)
    assert (full - split).abs().max() < 1e-5


def test_int4_format_bits():
    """Word layout: word 0 = shift<<16 | scale (fp16 bits); element e of a
    nibble word at bits [4e, 4e+4) (benchmarks/benchmark_attn_decoding.py:38-72,
    tests/test_mem_eff_attention.py:1730-1738)."""
    torch.manual_seed(0)
    x = torch.randn(5, 3, 128)
    xq = oracle.quantize_kv_int4(x)
    assert xq.dtype == torch.int32 and xq.shape == (5, 3, 17)
    w = xq.numpy().view(np.uint32)
    mn, mx = x.min(-1).values, x.max(-1).values
    scale = ((mx - mn) / 15).to(torch.float16)
    shift = mn.to(torch.float16)
    assert np.array_equal((w[..., 0] & 0xFFFF).astype(np.uint16), scale.view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal((w[..., 0] >> 16).astype(np.uint16), shift.view(torch.int16).numpy().view(np.uint16))
    qv = (((x - shift.float()[..., None]) / scale.float()[..., None]) + 0.5).to(torch.uint8) & 0xF
    for e in range(8):
        assert np.array_equal((w[..., 1:] >> (4 * e)) & 0xF, qv[..., e::8].numpy().astype(np.uint32))
    # dequantiser as written in the reference test: x // 2**(4*arange(8)) % 16
    body = xq[..., 1:, None].long() & 0xFFFFFFFF
    nib = (body // (2 ** (4 * torch.arange(8)))) % 16
    want = nib.flatten(start_dim=-2).float() * scale.float()[..., None] + shift.float()[..., None]
    assert torch.equal(oracle.dequantize_kv_int4(xq), want)
    assert (oracle.dequantize_kv_int4(xq) - x).abs().max() <= (scale.float().max() / 2 + 2e-2)


@pytest.mark.parametrize("groups", [1, 8])
def test_int4_reference_test_pattern(groups):
    # tests/test_mem_eff_attention.py:1700-1707,1730-1738: scale = shift = 1.0 -> value = nibble + 1
    k = torch.zeros(4, 7, 128 // 8 + groups, dtype=torch.int32)
    k.random_()
    k[..., :groups].view(torch.float16).fill_(1.0)
    x = k[..., groups:, None].expand(4, 7, 16, 8)
    x = x // (2 ** (4 * torch.arange(8)))
    want = (x % 16).flatten(start_dim=-2).float() + 1.0
    assert torch.equal(oracle.dequantize_kv_int4(k, groups), want)


def test_paged_indexing():
    torch.manual_seed(0)
    B, P, max_pages = 3, 4, 5
    lens = [7, 20, 1]
    perm = torch.randperm(B * max_pages).view(B, max_pages).int()
    padded = torch.arange(B * max_pages * P).float().view(1, B * max_pages * P, 1)
    paged = oracle.scatter_to_pages(padded, perm, P, lens, max_pages * P, B * max_pages)
    for b, n in enumerate(lens):
        rows = oracle.physical_rows(perm, P, b, n)
        for t in range(n):
            assert rows[t] == int(perm[b, t // P]) * P + t % P
            assert paged[0, rows[t], 0] == padded[0, b * max_pages * P + t, 0]
    back = oracle.gather_paged(paged, perm, P, lens, max_pages * P)
    for b, n in enumerate(lens):
        s = b * max_pages * P
        assert torch.equal(back[0, s : s + n], padded[0, s : s + n])
    # the package's paged bias hides exactly the rows no token of the sequence owns
    bias = ab.PagedBlockDiagonalPaddedKeysMask.from_seqlens([1] * B, lens, perm, P)
    m = bias.materialize((B, B * max_pages * P))
    for b, n in enumerate(lens):
        vis = set(torch.nonzero(m[b] == 0).flatten().tolist())
        assert vis == set(oracle.physical_rows(perm, P, b, n).tolist())


def test_merge_reference_properties():
    torch.manual_seed(0)
    S, B, M, G, H, D = 4, 2, 5, 2, 3, 8
    attn = torch.randn(S, B, M, G, H, D)
    lse = torch.randn(S, B, G, H, M)
    out, lo = oracle.merge_attentions_ref(attn, lse)
    # formula of tests/test_fmha_merge_attentions.py:513-538, written out again
    l = lse.permute(0, 1, 4, 2, 3)[..., None]
    mx = l.max(0).values
    w = torch.exp(l - mx)
    assert torch.allclose(out, (w * attn).sum(0) / w.sum(0), atol=1e-6)
    assert torch.allclose(lo, (mx + torch.log(w.sum(0))).squeeze(-1).permute(0, 2, 3, 1), atol=1e-6)
    # merge with self: same output, lse + ln 2 (tests/test_fmha_merge_attentions.py:80-138)
    o2, l2 = oracle.merge_attentions_ref(torch.stack([attn[0], attn[0]]), torch.stack([lse[0], lse[0]]))
    assert torch.allclose(o2, attn[0], atol=1e-6) and torch.allclose(l2, lse[0] + math.log(2), atol=1e-6)
    # an empty partial (lse = -inf, garbage values) is ignored
    attn[1].fill_(float("nan"))
    lse[1].fill_(-float("inf"))
    o3, l3 = oracle.merge_attentions_ref(attn, lse)
    keep = [0, 2, 3]
    o4, l4 = oracle.merge_attentions_ref(attn[keep], lse[keep])
    assert torch.equal(o3, o4) and torch.equal(l3, l4)


def test_chunked_attention_merges_to_full():
    # tests/test_fmha_merge_attentions.py:234-363 in miniature, on the oracle itself
    torch.manual_seed(0)
    q = torch.randn(2, 3, 4, 16)
    k, v = torch.randn(2, 40, 4, 16), torch.randn(2, 40, 4, 16)
    full, lse_full = oracle.ref_attention_with_lse(q, k, v)
    parts = [oracle.ref_attention_with_lse(q, k[:, a:b], v[:, a:b]) for a, b in ((0, 7), (7, 8), (8, 40))]
    out, lse = oracle.merge_attentions_ref(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]))
    assert torch.allclose(out, full, atol=1e-5) and torch.allclose(lse, lse_full, atol=1e-5)


def test_nan_in_hidden_keys_does_not_leak():
    torch.manual_seed(0)
    q = torch.randn(1, 4, 2, 8)
    k, v = torch.randn(1, 32, 2, 8), torch.randn(1, 32, 2, 8)
    bias = ab.BlockDiagonalPaddedKeysMask.from_seqlens([1] * 4, 8, [3, 8, 1, 5])
    ref = oracle.ref_attention(q, k, v, bias)
    for b, n in enumerate([3, 8, 1, 5]):
        k[0, b * 8 + n : (b + 1) * 8] = float("nan")
        v[0, b * 8 + n : (b + 1) * 8] = float("nan")
    got = oracle.ref_attention(q, k, v, bias)
    assert not got.isnan().any() and torch.equal(ref, got)


def test_fp8_rowwise_format():
    """tests/utils.py:311-340: one int32 per row carries fp16 scale (low half)
    and fp16 shift (high half); four e4m3 values per int32 word, element e in
    byte e; x = fp8 * scale + shift."""
    import struct

    w = oracle.combine_scale_shift(torch.tensor([1.0, 0.5]), torch.tensor([2.0, -1.0]))
    assert w.dtype == torch.int32 and [int(x) & 0xFFFFFFFF for x in w] == [0x40003C00, 0xBC003800]
    sc, sh = oracle.split_scale_shift(w)
    assert sc.tolist() == [1.0, 0.5] and sh.tolist() == [2.0, -1.0]
    vals = torch.tensor([[1.0, -2.0, 0.5, 448.0]]).to(oracle.fp8.FP8)
    words = oracle.pack_fp8_words(vals)
    assert words.shape == (1, 1) and (int(words[0, 0]) & 0xFFFFFFFF) == struct.unpack("<I", bytes([0x38, 0xC0, 0x30, 0x7E]))[0]
    assert torch.equal(oracle.unpack_fp8_words(words).float(), vals.float())
    x = torch.randn(7, 128, generator=torch.Generator().manual_seed(0))
    q, scale, shift = oracle.quantize_fp8_asymmetric(x)
    assert torch.allclose(shift, x.mean(dim=1)) and torch.allclose(scale, 448.0 / (x - shift[:, None]).abs().max(dim=1)[0])
    back = oracle.dequantize_fp8_asymmetric(q, scale, shift)
    assert (back - x).abs().max() < 0.5  # the reference's scale choice uses little of the e4m3 range


def test_gappy_keys_mask_materialize():
    """Keys of block b are the columns [starts[b], starts[b] + len[b]); the
    causal form is bottom-right aligned inside the block."""
    from xformers_b200.ops.fmha import attn_bias as ab

    bias = ab.BlockDiagonalGappyKeysMask.from_seqlens(q_seqlen=[1, 2], kv_seqstarts=[1, 4, 8], kv_seqlen=[2, 3])
    m = bias.materialize((3, 8))
    vis = (m == 0).int().tolist()
    assert vis == [[0, 1, 1, 0, 0, 0, 0, 0], [0, 0, 0, 0, 1, 1, 1, 0], [0, 0, 0, 0, 1, 1, 1, 0]]
    cb = ab.BlockDiagonalCausalWithOffsetGappyKeysMask.from_seqlens(q_seqlen=[1, 2], kv_seqstarts=[1, 4, 8], kv_seqlen=[2, 3])
    vis = (cb.materialize((3, 8)) == 0).int().tolist()
    assert vis == [[0, 1, 1, 0, 0, 0, 0, 0], [0, 0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 0, 1, 1, 1, 0]]
    with pytest.raises(ValueError):
        ab.BlockDiagonalGappyKeysMask.from_seqlens(q_seqlen=[1], kv_seqstarts=[0, 4], kv_seqlen=[5])
    paged = bias.make_paged(torch.tensor([[1, 0], [0, 1]], dtype=torch.int32), 4, ab.PagedBlockDiagonalGappyKeysMask, notional_padding=4)
    assert paged.slot_starts().tolist() == [1, 0]
    pv = (paged.materialize((3, 8)) == 0).int().tolist()
    # sequence 0: logical rows 1, 2 of its table [1, 0] -> physical rows 5, 6; sequence 1: rows 0..2 of table [0, 1] -> 0, 1, 2
    assert pv == [[0, 0, 0, 0, 0, 1, 1, 0], [1, 1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0, 0]]


def test_causal_local_padded_keys_and_bottom_right_local_materialize():
    """Hand-built masks of the window forms: query i of a block of ql queries sees
    key t iff i + kl - ql - window < t <= i + kl - ql."""
    from xformers_b200.ops.fmha import attn_bias as ab

    bias = ab.BlockDiagonalCausalLocalAttentionPaddedKeysMask.from_seqlens_local([2, 1], 4, [4, 2], 2)
    m = bias.materialize((3, 8)) == 0
    want = torch.tensor([
        [0, 1, 1, 0, 0, 0, 0, 0],   # sequence 0, query 0 of 2, 4 keys: diagonal at key 2, window 2 -> keys 1, 2
        [0, 0, 1, 1, 0, 0, 0, 0],   # query 1: keys 2, 3
        [0, 0, 0, 0, 1, 1, 0, 0],   # sequence 1 (slot 4..7, 2 keys): its only query sees keys 0, 1 of the slot
    ], dtype=torch.bool)
    assert torch.equal(m, want)
    with pytest.raises(ValueError):
        ab.BlockDiagonalCausalLocalAttentionPaddedKeysMask.from_seqlens_local([1], 4, [1], 0)

    m = ab.LowerTriangularFromBottomRightLocalAttentionMask(2).materialize((2, 5)) == 0
    want = torch.tensor([[0, 0, 1, 1, 0], [0, 0, 0, 1, 1]], dtype=torch.bool)
    assert torch.equal(m, want)
    # window >= number of keys: the plain bottom-right causal mask
    full = ab.LowerTriangularFromBottomRightLocalAttentionMask(99).materialize((3, 5))
    assert torch.equal(full, ab.LowerTriangularFromBottomRightMask().materialize((3, 5)))
