"""Split-K decode over a row-wise fp8 KV cache (``InputsFp8``) against the
oracle on dequantised values; padded and paged caches."""

import pytest
import torch

import oracle
from gpu_utils import assert_o_lse, gpu, require_cuda
from xformers_b200.ops import fmha
from xformers_b200.ops.fmha import attn_bias as ab

S = fmha.triton_splitk


def _fp8_case(B, Mkv, Hkv, G, dtype, seed=10, mq=1, random_bytes=False):
    """Tensors of tests/utils.py:134-222: q [1, B*mq, Hkv, G, K]; K/V rows
    quantised one by one, words and scale/shift expanded over the G query heads."""
    K = 128
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, B * mq, Hkv, G, K, generator=g).to(dtype)
    if random_bytes:
        # every finite e4m3 value (0x7f / 0xff are NaN), scales and shifts of either sign
        def rnd():
            b = torch.randint(0, 256, (B * Mkv * Hkv, K), generator=g, dtype=torch.int64)
            b = torch.where((b & 0x7F) == 0x7F, b - 1, b).to(torch.uint8)
            return b.view(oracle.fp8.FP8)

        k8, v8 = rnd(), rnd()
        ksc, vsc = (torch.randn(B * Mkv * Hkv, generator=g) * 0.01 for _ in range(2))
        ksh, vsh = (torch.randn(B * Mkv * Hkv, generator=g) for _ in range(2))
    else:
        k = torch.randn(B * Mkv * Hkv, K, generator=g).to(dtype).float()
        v = torch.randn(B * Mkv * Hkv, K, generator=g).to(dtype).float()
        k8, ksc, ksh = oracle.quantize_fp8_asymmetric(k)
        v8, vsc, vsh = oracle.quantize_fp8_asymmetric(v)
    kss, vss = oracle.combine_scale_shift(ksc, ksh), oracle.combine_scale_shift(vsc, vsh)
    # what the kernel sees after the fp16 rounding of scale and shift
    ksc, ksh = oracle.split_scale_shift(kss)
    vsc, vsh = oracle.split_scale_shift(vss)
    k_deq = oracle.dequantize_fp8_asymmetric(k8, ksc, ksh).view(1, B * Mkv, Hkv, 1, K)
    v_deq = oracle.dequantize_fp8_asymmetric(v8, vsc, vsh).view(1, B * Mkv, Hkv, 1, K)
    kw = oracle.pack_fp8_words(k8).view(1, B * Mkv, Hkv, 1, K // 4)
    vw = oracle.pack_fp8_words(v8).view(1, B * Mkv, Hkv, 1, K // 4)
    kss, vss = kss.view(1, B * Mkv, Hkv, 1), vss.view(1, B * Mkv, Hkv, 1)
    return q, kw, vw, kss, vss, k_deq, v_deq


def _expand(t, G):
    return t.expand(*t.shape[:3], G, *t.shape[4:])


@gpu
@pytest.mark.parametrize("random_bytes", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("page_size", [64, 256])
@pytest.mark.parametrize("Hkv,G", [(1, 1), (1, 8), (2, 8), (8, 8), (4, 4)])
@pytest.mark.parametrize("B,Mkv", [(1, 2048), (5, 1024)])
@pytest.mark.parametrize("replicated", [True, False])
def test_rowwise_fp8(B, Mkv, Hkv, G, page_size, dtype, random_bytes, replicated):
    """tests/test_mem_eff_attention.py:2818-2881: the fp8 operator equals
    attention on the dequantised cache; the paged cache equals the padded one.
    ``replicated``: the scale/shift word of a (token, kv head) entry is laid out once per
    query head of the group, as the reference's helper does it (tests/utils.py:175-188);
    otherwise one word per entry, expanded over the query heads with stride 0 like K and V."""
    require_cuda()
    rep = (lambda t: t.contiguous()) if replicated else (lambda t: t)
    q, kw, vw, kss, vss, k_deq, v_deq = _fp8_case(B, Mkv, Hkv, G, dtype, random_bytes=random_bytes)
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(1, Mkv + 1, (B,), generator=g).tolist()
    lens[0] = Mkv
    bias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=[1] * B, kv_seqlen=lens, kv_padding=Mkv, device="cuda")
    ro, rl = oracle.ref_attention_with_lse(q.float(), _expand(k_deq, G), _expand(v_deq, G), bias.to("cpu"))
    cu = lambda t: t.cuda()
    inp = S.InputsFp8(
        query=cu(q), key=_expand(cu(kw), G), value=_expand(cu(vw), G), attn_bias=bias,
        k_fp8_scale_shift=rep(_expand(cu(kss), G)), v_fp8_scale_shift=rep(_expand(cu(vss), G)),
    )
    assert not S.FwOp.not_supported_reasons(inp)
    out, ctx = fmha._memory_efficient_attention_forward_requires_grad(inp, op=S.FwOp)
    scale = 1.0 if not random_bytes else max(1.0, float(v_deq.abs().max()))
    assert_o_lse(out, ctx.lse, ro, rl, dtype, "fp8 padded", o_scale=scale)

    # paged: the same rows scattered over pages
    pages_per_seq = Mkv // page_size
    n_pages = B * pages_per_seq
    perm = torch.randperm(n_pages, generator=g).int().view(B, pages_per_seq)
    sc = lambda t: oracle.scatter_to_pages(t, perm, page_size, [Mkv] * B, Mkv, n_pages)
    pbias = bias.make_paged(perm.cuda(), page_size, ab.PagedBlockDiagonalCausalWithOffsetPaddedKeysMask)
    inp_p = S.InputsFp8(
        query=cu(q), key=_expand(cu(sc(kw)), G), value=_expand(cu(sc(vw)), G), attn_bias=pbias,
        k_fp8_scale_shift=rep(_expand(cu(sc(kss.unsqueeze(-1)).squeeze(-1)), G)),
        v_fp8_scale_shift=rep(_expand(cu(sc(vss.unsqueeze(-1)).squeeze(-1)), G)),
    )
    out_p, ctx_p = fmha._memory_efficient_attention_forward_requires_grad(inp_p, op=S.FwOp)
    assert torch.equal(out_p, out) and torch.equal(ctx_p.lse, ctx.lse), "page placement must not change a single bit"


@gpu
def test_fp8_rejects_what_it_cannot_run():
    require_cuda()
    q, kw, vw, kss, vss, _, _ = _fp8_case(1, 256, 1, 1, torch.bfloat16)
    bias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=[1], kv_seqlen=[256], kv_padding=256, device="cuda")
    inp = S.InputsFp8(query=q.cuda(), key=kw.cuda(), value=vw.cuda(), attn_bias=bias, k_fp8_scale_shift=None, v_fp8_scale_shift=vss.cuda())
    assert any("k_fp8_scale_shift" in r for r in S.FwOp.not_supported_reasons(inp))
    with pytest.raises(ValueError):
        fmha._memory_efficient_attention_forward(inp, op=S.FwOp)


@gpu
def test_fp8_nan_bytes_in_padding_do_not_leak():
    """tests/test_mem_eff_attention.py:1750-1853 (``test_nans_in_padding``) for
    the fp8 cache: rows past a sequence's end hold the NaN byte pattern of e4m3
    and NaN scale/shift words; the outputs must not change."""
    require_cuda()
    B, Mkv, Hkv, G = 3, 256, 2, 8
    q, kw, vw, kss, vss, k_deq, v_deq = _fp8_case(B, Mkv, Hkv, G, torch.bfloat16, seed=4)
    lens = [200, 1, 129]
    bias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=[1] * B, kv_seqlen=lens, kv_padding=Mkv, device="cuda")

    def run(kw_, vw_, kss_, vss_):
        inp = S.InputsFp8(
            query=q.cuda(), key=_expand(kw_.cuda(), G), value=_expand(vw_.cuda(), G), attn_bias=bias,
            k_fp8_scale_shift=_expand(kss_.cuda(), G).contiguous(), v_fp8_scale_shift=_expand(vss_.cuda(), G).contiguous(),
        )
        out, ctx = fmha._memory_efficient_attention_forward_requires_grad(inp, op=S.FwOp)
        return out, ctx.lse

    out0, lse0 = run(kw, vw, kss, vss)
    kw2, vw2, kss2, vss2 = kw.clone(), vw.clone(), kss.clone(), vss.clone()
    for b, n in enumerate(lens):
        sl = slice(b * Mkv + n, (b + 1) * Mkv)
        kw2[:, sl], vw2[:, sl] = 0x7F7F7F7F, 0x7F7F7F7F  # e4m3 NaN in every byte
        kss2[:, sl], vss2[:, sl] = 0x7E007E00, 0x7E007E00  # fp16 NaN scale and shift
    out1, lse1 = run(kw2, vw2, kss2, vss2)
    assert not out1.isnan().any() and not lse1.isnan().any()
    assert torch.equal(out0, out1) and torch.equal(lse0, lse1)


@gpu
@pytest.mark.parametrize("Hkv,G", [(2, 8), (1, 4), (8, 2)])
def test_scale_shift_layouts_agree(Hkv, G):
    """The scale/shift words may be laid out once per query head of the group
    (tests/utils.py:175-188; fetched by tiled copies when a group has at least 4
    heads) or given expanded with stride 0 (fetched word by word): same bits out."""
    require_cuda()
    B, Mkv = 3, 512
    q, kw, vw, kss, vss, _, _ = _fp8_case(B, Mkv, Hkv, G, torch.bfloat16, seed=9)
    lens = [512, 77, 300]
    bias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=[1] * B, kv_seqlen=lens, kv_padding=Mkv, device="cuda")
    outs = []
    for contiguous in (True, False):
        ks, vs = _expand(kss.cuda(), G), _expand(vss.cuda(), G)
        if contiguous:
            ks, vs = ks.contiguous(), vs.contiguous()
        assert (ks.stride(3) == 1) == contiguous or G == 1
        inp = S.InputsFp8(query=q.cuda(), key=_expand(kw.cuda(), G), value=_expand(vw.cuda(), G), attn_bias=bias,
                          k_fp8_scale_shift=ks, v_fp8_scale_shift=vs)
        out, ctx = fmha._memory_efficient_attention_forward_requires_grad(inp, op=S.FwOp)
        outs.append((out, ctx.lse))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
