"""Gappy-key biases (keys of a sequence start at an arbitrary row of the
cache) on both operators, padded and paged, against the oracle."""

import pytest
import torch

import oracle
from gpu_utils import assert_o_lse, gpu, require_cuda
from xformers_b200.ops import fmha
from xformers_b200.ops.fmha import attn_bias as ab


def _case(B, slot, Hkv, G, D, dtype, seed, quant=False):
    g = torch.Generator().manual_seed(seed)
    total = B * slot + 40  # a tail that belongs to nobody
    starts = [b * slot + int(torch.randint(0, slot // 2, (1,), generator=g)) for b in range(B)] + [total]
    lens = [int(torch.randint(1, starts[b + 1] - starts[b] + 1, (1,), generator=g)) for b in range(B)]
    lens[0] = min(lens[0], slot // 2)
    kf = torch.randn(1, total, Hkv, 1, D, generator=g)
    vf = torch.randn(1, total, Hkv, 1, D, generator=g)
    if quant:
        k, v = oracle.quantize_kv_int4(kf), oracle.quantize_kv_int4(vf)
        k_ref, v_ref = oracle.dequantize_kv_int4(k), oracle.dequantize_kv_int4(v)
    else:
        k, v = kf.to(dtype), vf.to(dtype)
        k_ref, v_ref = k.float(), v.float()
    return starts, lens, k, v, k_ref, v_ref, g


@gpu
@pytest.mark.parametrize("quant", [False, True])
@pytest.mark.parametrize("causal,mq", [(False, 1), (True, 1), (True, 3)])
@pytest.mark.parametrize("Hkv,G", [(1, 8), (8, 8), (2, 4)])
def test_decode_gappy(Hkv, G, causal, mq, quant):
    """tests/test_fmha_merge_attentions.py:406-414: keys of sequence b are the
    rows [kv_seqstarts[b], kv_seqstarts[b] + kv_seqlen[b])."""
    require_cuda()
    B, slot, D, dtype = 4, 512, 128, torch.bfloat16
    starts, lens, k, v, k_ref, v_ref, g = _case(B, slot, Hkv, G, D, dtype, seed=21, quant=quant)
    lens = [max(n, mq) for n in lens]
    q = torch.randn(1, B * mq, Hkv, G, D, generator=g).to(dtype)
    cls = ab.BlockDiagonalCausalWithOffsetGappyKeysMask if causal else ab.BlockDiagonalGappyKeysMask
    bias = cls.from_seqlens(q_seqlen=[mq] * B, kv_seqstarts=starts, kv_seqlen=lens, device="cuda")
    ex = lambda t: t.expand(-1, -1, -1, G, -1)
    ro, rl = oracle.ref_attention_with_lse(q.float(), ex(k_ref), ex(v_ref), bias.to("cpu"))
    for op in (fmha.b200_splitk.FwOp, fmha.b200_splitk.FwOp_S1, fmha.b200_splitk.FwOp_S4):
        assert not op.not_supported_reasons(fmha.Inputs(q.cuda(), ex(k.cuda()), ex(v.cuda()), bias))
        out, lse = fmha.memory_efficient_attention_forward_requires_grad(q.cuda(), ex(k.cuda()), ex(v.cuda()), bias, op=op)
        assert_o_lse(out, lse, ro, rl, dtype, f"gappy decode {op.NAME}")


@gpu
@pytest.mark.parametrize("quant", [False, True])
@pytest.mark.parametrize("page_size", [16, 64, 256])
def test_decode_paged_gappy(page_size, quant):
    """tests/test_mem_eff_attention.py:2516-2525: the paged form of a gappy
    bias reads the same keys through a block table."""
    require_cuda()
    B, slot, Hkv, G, D, dtype = 3, 512, 2, 8, 128, torch.bfloat16
    g = torch.Generator().manual_seed(5)
    offs = [0, 37, 300]
    lens = [500, 100, 212]
    starts = [b * slot + offs[b] for b in range(B)] + [B * slot]
    kf = torch.randn(1, B * slot, Hkv, 1, D, generator=g)
    vf = torch.randn(1, B * slot, Hkv, 1, D, generator=g)
    if quant:
        k, v = oracle.quantize_kv_int4(kf), oracle.quantize_kv_int4(vf)
    else:
        k, v = kf.to(dtype), vf.to(dtype)
    q = torch.randn(1, B, Hkv, G, D, generator=g).to(dtype).cuda()
    bias = ab.BlockDiagonalGappyKeysMask.from_seqlens(q_seqlen=[1] * B, kv_seqstarts=starts, kv_seqlen=lens, device="cuda")
    ex = lambda t: t.cuda().expand(-1, -1, -1, G, -1)
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, ex(k), ex(v), bias, op=fmha.b200_splitk.FwOp)
    pages_per_seq = slot // page_size
    n_pages = B * pages_per_seq
    perm = torch.randperm(n_pages, generator=g).int().view(B, pages_per_seq)
    k_pg = oracle.scatter_to_pages(k, perm, page_size, [slot] * B, slot, n_pages)
    v_pg = oracle.scatter_to_pages(v, perm, page_size, [slot] * B, slot, n_pages)
    pbias = bias.make_paged(perm.cuda(), page_size, ab.PagedBlockDiagonalGappyKeysMask, notional_padding=slot)
    assert not fmha.b200_splitk.FwOp.not_supported_reasons(fmha.Inputs(q, ex(k_pg), ex(v_pg), pbias))
    out_p, lse_p = fmha.memory_efficient_attention_forward_requires_grad(q, ex(k_pg), ex(v_pg), pbias, op=fmha.b200_splitk.FwOp)
    assert torch.equal(out_p, out) and torch.equal(lse_p, lse), "the paged gappy cache must give the same bits as the flat one"
    if not quant:
        ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), ex(k_pg).float().cpu(), ex(v_pg).float().cpu(), pbias.to("cpu"))
        assert_o_lse(out_p, lse_p, ro, rl, dtype, "paged gappy")


@gpu
@pytest.mark.parametrize("op", [fmha.b200.FwOp_Tcgen05, fmha.b200.FwOp_Generic])
@pytest.mark.parametrize("causal", [False, True])
def test_prefill_gappy(causal, op):
    require_cuda()
    B, slot, H, D, dtype = 3, 384, 4, 128, torch.bfloat16
    starts, lens, k, v, k_ref, v_ref, g = _case(B, slot, H, 1, D, dtype, seed=9)
    q_lens = [min(n, 150) for n in lens]
    q = torch.randn(1, sum(q_lens), H, D, generator=g).to(dtype)
    cls = ab.BlockDiagonalCausalWithOffsetGappyKeysMask if causal else ab.BlockDiagonalGappyKeysMask
    bias = cls.from_seqlens(q_seqlen=q_lens, kv_seqstarts=starts, kv_seqlen=lens, device="cuda")
    k4, v4, kr, vr = k[:, :, :, 0], v[:, :, :, 0], k_ref[:, :, :, 0], v_ref[:, :, :, 0]
    ro, rl = oracle.ref_attention_with_lse(q.float(), kr, vr, bias.to("cpu"))
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q.cuda(), k4.cuda(), v4.cuda(), bias, op=op)
    assert_o_lse(out, lse, ro, rl, dtype, f"gappy prefill {op.NAME}")
