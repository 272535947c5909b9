"""The benchmark's own configurations, at their full shapes, against the oracle.

`bench.py` times causal prefill (B=4, 4096 x 4096, 32 heads), packed varlen
GQA prefill (16 sequences of 256..4096 tokens, Hq=32 / Hkv=8), split-K decode
over a paged cache (64 sequences of up to 32768 keys, page 256, Hq=64 / Hkv=8;
bf16, int4 and fp8 caches) and one 131072-token causal sequence.  The dense
fp32 oracle cannot run those whole, so each case runs at full size on the GPU
-- the grid order, the number of row blocks per head, the 128-page tables and
the split counts are the benchmark's -- and slices of the result are compared
with the oracle on the same slices of the inputs.  Tolerances are the
suite's: O 2e-2 (bf16), LSE 1e-3.
"""

import pytest
import torch

import bench
import oracle
from gpu_utils import assert_o_lse, gpu, require_cuda
from xformers_b200.ops import fmha
from xformers_b200.ops.fmha import attn_bias as ab
from xformers_b200.ops.fmha.sharded import zigzag_bounds

P = fmha.b200


def _status_ok():
    assert P.prefill_device_status() == 0, "a wait inside the tcgen05 kernel ran out"
    assert fmha.b200_splitk.decode_device_status() == 0, "a wait inside the decode kernel ran out"


@gpu
@pytest.mark.parametrize("op", [P.FwOp, P.FwOp_Tcgen05_M256])
def test_cfg2_causal_prefill_full_shape(op):
    require_cuda()
    B, M, H, D = bench.CFG2["B"], bench.CFG2["M"], bench.CFG2["H"], bench.CFG2["D"]
    gd = torch.Generator(device="cuda").manual_seed(0)
    q, k, v = (torch.randn(B, M, H, D, generator=gd, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, ab.LowerTriangularMask(), op=op)
    _status_ok()
    assert out.shape == (B, M, H, D) and lse.shape == (B, H, M)
    for b in (0, 3):
        hs = [0, 13, 31]
        ro, rl = oracle.ref_attention_with_lse(q[b : b + 1, :, hs].float().cpu(), k[b : b + 1, :, hs].float().cpu(), v[b : b + 1, :, hs].float().cpu(),
                                               ab.LowerTriangularMask())
        assert_o_lse(out[b : b + 1, :, hs], lse[b : b + 1, hs], ro, rl, torch.bfloat16, f"cfg2 batch {b}")
    # every other (batch, head): finite, and the first row attends to the first key only
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    assert torch.equal(out[:, 0], v[:, 0])


@gpu
def test_cfg3_packed_varlen_gqa_full_shape():
    require_cuda()
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(256, 4097, (16,), generator=g).tolist()
    total = sum(lens)
    gd = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(1, total, 8, 4, 128, generator=gd, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, total, 8, 1, 128, generator=gd, device="cuda", dtype=torch.bfloat16).expand(-1, -1, -1, 4, -1)
    v = torch.randn(1, total, 8, 1, 128, generator=gd, device="cuda", dtype=torch.bfloat16).expand(-1, -1, -1, 4, -1)
    bias = ab.BlockDiagonalCausalMask.from_seqlens(lens, device="cuda")
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=P.FwOp)
    _status_ok()
    assert lse.shape == (1, 8, 4, total)
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    order = sorted(range(16), key=lambda i: lens[i])
    for i in (order[0], order[1], order[-1]):  # the two shortest and the longest sequence
        a, b = starts[i], starts[i + 1]
        for grp in (0, 5):
            ro, rl = oracle.ref_attention_with_lse(q[:, a:b, grp].float().cpu(), k[:, a:b, grp].float().cpu(), v[:, a:b, grp].float().cpu(),
                                                   ab.LowerTriangularMask())
            assert_o_lse(out[:, a:b, grp], lse[:, grp, :, a:b], ro, rl, torch.bfloat16, f"cfg3 seq {i} (len {lens[i]}) group {grp}")
    assert torch.isfinite(out.float()).all()


def _decode_reference(q, k_rows, v_rows, b):
    """Oracle for sequence ``b``: its query [Hkv, G, D] against its gathered, dequantised keys [L, Hkv, D]."""
    qb = q[0, b].float().cpu().unsqueeze(0).unsqueeze(0)  # [1, 1, Hkv, G, D]
    G = qb.shape[3]
    kk = k_rows.unsqueeze(0).unsqueeze(3).expand(-1, -1, -1, G, -1)
    vv = v_rows.unsqueeze(0).unsqueeze(3).expand(-1, -1, -1, G, -1)
    return oracle.ref_attention_with_lse(qb, kk, vv)


@gpu
@pytest.mark.parametrize("quant", [False, True, "fp8"])
def test_cfg4_paged_decode_full_shape(quant):
    require_cuda()
    wl = bench.decode_workload(torch.device("cuda"), quant)
    q, k, v, bias = wl[0], wl[1], wl[2], wl[3]
    if quant == "fp8":
        kss, vss = wl[5], wl[6]
        inp = fmha.triton_splitk.InputsFp8(query=q, key=k, value=v, attn_bias=bias, k_fp8_scale_shift=kss, v_fp8_scale_shift=vss)
        out, ctx = fmha._memory_efficient_attention_forward_requires_grad(inp, op=fmha.b200_splitk.FwOp)
        lse = ctx.lse
    else:
        out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=fmha.b200_splitk.FwOp)
    _status_ok()
    lens = bias.k_seqinfo.seqlen_py
    page = bias.page_size
    order = sorted(range(len(lens)), key=lambda i: lens[i])
    picks = [order[0], order[-1]] + order[7:60:9]  # the shortest, the longest and six in between
    assert len(set(picks)) == 8
    for b in picks:
        rows = torch.from_numpy(oracle.physical_rows(bias.block_tables, page, b, lens[b])).cuda()
        kb, vb = k[0, rows, :, 0].cpu(), v[0, rows, :, 0].cpu()  # [L, Hkv, words or D]
        if quant == "fp8":
            ksc, ksh = oracle.split_scale_shift(kss[0, rows, :, 0].cpu())
            vsc, vsh = oracle.split_scale_shift(vss[0, rows, :, 0].cpu())
            kr = oracle.dequantize_fp8_asymmetric(oracle.unpack_fp8_words(kb), ksc, ksh)
            vr = oracle.dequantize_fp8_asymmetric(oracle.unpack_fp8_words(vb), vsc, vsh)
        elif quant:
            kr, vr = oracle.dequantize_kv_int4(kb), oracle.dequantize_kv_int4(vb)
        else:
            kr, vr = kb.float(), vb.float()
        ro, rl = _decode_reference(q, kr, vr, b)
        assert_o_lse(out[:, b : b + 1], lse[:, :, :, b : b + 1], ro, rl, torch.bfloat16, f"cfg4 quant={quant} seq {b} (len {lens[b]})")
    assert torch.isfinite(out.float()).all()


@gpu
@pytest.mark.parametrize("ranks", [1, 8])
def test_cfg5_long_context_full_shape(ranks):
    """One 131072-token causal sequence: in one piece, and as the key ranges the
    8-rank benchmark gives its ranks (two per rank, merged), each range run at
    full size on this GPU."""
    require_cuda()
    S, Hkv, G, D = 131072, 8, 8, 128
    gd = torch.Generator(device="cuda").manual_seed(1234)
    q = torch.randn(1, S, Hkv, G, D, generator=gd, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(1, S, Hkv, 1, D, generator=gd, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(1, S, Hkv, 1, D, generator=gd, device="cuda", dtype=torch.bfloat16)
    ke, ve = k.expand(-1, -1, -1, G, -1), v.expand(-1, -1, -1, G, -1)
    stripes = [(0, 512), (S // 2 - 256, S // 2 + 256), (S - 512, S)]
    groups, heads = (0, 6), [0, 5]
    sel = torch.cat([torch.arange(a, b) for a, b in stripes]).cuda()
    if ranks == 1:
        out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, ke, ve, ab.LowerTriangularMask(), op=P.FwOp)
        out_s, lse_s = out[:, sel], lse[..., sel]
    else:
        # Every key range of the 8-rank split contributes a partial.  The ranges of the first and the last rank
        # run at full size (all 131072 queries, as in the benchmark); the others on the checked rows only,
        # with the causal diagonal shifted accordingly.
        outs, lses = [], []
        for r in range(ranks):
            for lo, hi in zigzag_bounds(S, ranks, r):
                if r in (0, ranks - 1):
                    inp = fmha.Inputs(q, ke[:, lo:hi], ve[:, lo:hi], ab.LowerTriangularMask(), output_dtype=torch.float32, is_partial=True)
                    o, ctx = P.FwOp._apply(inp, want_lse=True, kv_offset=lo)
                    outs.append(o[:, sel].clone())
                    lses.append(ctx.lse[..., sel].clone())
                    del o, ctx
                else:
                    po, pl = [], []
                    for a, b in stripes:
                        inp = fmha.Inputs(q[:, a:b], ke[:, lo:hi], ve[:, lo:hi], ab.LowerTriangularMask(), output_dtype=torch.float32, is_partial=True)
                        o, ctx = P.FwOp._apply(inp, want_lse=True, kv_offset=lo - a)
                        po.append(o)
                        pl.append(ctx.lse)
                    outs.append(torch.cat(po, dim=1))
                    lses.append(torch.cat(pl, dim=-1))
        _status_ok()
        out_s, lse_s = fmha.merge_attentions(outs, lses, output_dtype=torch.bfloat16)
    _status_ok()
    pos = 0
    for a, b in stripes:
        n = b - a
        for grp in groups:
            bias = oracle.causal_mask(n, b, kv_offset=-a)  # query i of the stripe is global row a + i
            ro, rl = oracle.ref_attention_with_lse(q[:, a:b, grp][:, :, heads].float().cpu(), ke[:, :b, grp][:, :, heads].float().cpu(),
                                                   ve[:, :b, grp][:, :, heads].float().cpu(), bias)
            assert_o_lse(out_s[:, pos : pos + n, grp][:, :, heads], lse_s[:, grp][:, heads, pos : pos + n], ro, rl, torch.bfloat16,
                         f"cfg5 ranks={ranks} rows [{a},{b}) group {grp}")
        pos += n
