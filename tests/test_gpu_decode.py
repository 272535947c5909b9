"""Split-K decode operator on the GPU against the oracle: padded and paged
caches, bf16/f16 and int4 row-wise, MQA/GQA/MHA head layouts."""

import pytest
import torch

import oracle
from gpu_utils import ATOL_LSE, ATOL_O, assert_o_lse, gpu, ref, require_cuda
from xformers_b200.ops import fmha
from xformers_b200.ops.fmha import attn_bias as ab

S = fmha.b200_splitk


def _decoder_case(n_heads, kv_heads, padding, bsz, dtype, num_queries=1, d=128, seed=1, quant=False, rand_scale=False, groups=1):
    """Tensors of tests/test_mem_eff_attention.py:1657-1747."""
    g = torch.Generator().manual_seed(seed)
    if kv_heads is not None and kv_heads > 1:
        k_shape = (1, bsz * padding, kv_heads, n_heads, d)
        q_shape = (1, bsz * num_queries, kv_heads, n_heads, d)
    else:
        k_shape = (1, bsz * padding, n_heads, d)
        q_shape = (1, bsz * num_queries, n_heads, d)
    q = torch.randn(q_shape, generator=g).to(dtype).cuda()
    k_seqlen = torch.randint(num_queries, padding + 1, (bsz,), generator=g).tolist()
    if quant:
        w_shape = k_shape[:-1] + (d // 8 + groups,)
        if rand_scale:
            kf = torch.randn(k_shape[:-2] + (1, d) if kv_heads is not None else k_shape, generator=g)
            vf = torch.randn(kf.shape, generator=g)
            k, v = oracle.quantize_kv_int4(kf, groups), oracle.quantize_kv_int4(vf, groups)
        else:
            # the reference's pattern: random words, scale = shift = 1.0
            k = torch.randint(-(2**31), 2**31 - 1, w_shape, generator=g, dtype=torch.int64).to(torch.int32)
            v = torch.randint(-(2**31), 2**31 - 1, w_shape, generator=g, dtype=torch.int64).to(torch.int32)
            k[..., :groups].view(torch.float16).fill_(1.0)
            v[..., :groups].view(torch.float16).fill_(1.0)
            if kv_heads is not None:
                k, v = k[..., :1, :], v[..., :1, :]
        k, v = k.cuda(), v.cuda()
        if kv_heads is not None:
            k, v = k.expand(w_shape), v.expand(w_shape)
        k_ref = oracle.dequantize_kv_int4(k.cpu().contiguous(), groups)
        v_ref = oracle.dequantize_kv_int4(v.cpu().contiguous(), groups)
    else:
        k = torch.randn(k_shape, generator=g).to(dtype).cuda()
        v = torch.randn(k_shape, generator=g).to(dtype).cuda()
        if kv_heads is not None:
            k = k[..., :1, :].expand(k_shape)
            v = v[..., :1, :].expand(k_shape)
        k_ref, v_ref = k.float().cpu(), v.float().cpu()
    bias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(
        q_seqlen=[num_queries] * bsz, kv_seqlen=k_seqlen, kv_padding=padding, device="cuda"
    )
    return q, k, v, bias, k_ref, v_ref


@gpu
@pytest.mark.parametrize("split_k", [None, 1, 2])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("padding,bsz", [(32, 8), (4096, 1)])
@pytest.mark.parametrize("kv_heads", [None, 1, 2])
def test_decoder(kv_heads, padding, bsz, dtype, split_k):
    require_cuda()
    op = S.FwOp if split_k is None else S.FwOp_Map[split_k]
    q, k, v, bias, k_ref, v_ref = _decoder_case(16, kv_heads, padding, bsz, dtype)
    assert not op.not_supported_reasons(fmha.Inputs(q, k, v, bias))
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k_ref, v_ref, bias.to("cpu"))
    assert_o_lse(out, lse, ro, rl, dtype, f"decode kvh={kv_heads}")
    out2 = fmha.memory_efficient_attention_forward(q, k, v, bias, op=op)
    assert torch.equal(out, out2), "decode must be bit-reproducible"


@gpu
@pytest.mark.parametrize("split_k", [1, 2])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("padding,bsz", [(32, 8), (4096, 1)])
@pytest.mark.parametrize("kv_heads", [None, 1, 2])
@pytest.mark.parametrize("rand_scale", [False, True])
def test_decoder_int4(kv_heads, padding, bsz, dtype, split_k, rand_scale):
    # tests/test_mem_eff_attention.py:1700-1707,1730-1745 (4x the op tolerance there)
    require_cuda()
    op = S.FwOp_Map[split_k]
    q, k, v, bias, k_ref, v_ref = _decoder_case(16, kv_heads, padding, bsz, dtype, quant=True, rand_scale=rand_scale)
    reasons = op.not_supported_reasons(fmha.Inputs(q, k, v, bias))
    assert not reasons, reasons
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k_ref, v_ref, bias.to("cpu"))
    # values reach 16 in the reference's pattern: tolerance scales with |V|
    assert_o_lse(out, None, ro, rl, dtype, "int4", o_scale=4.0 if not rand_scale else 1.0)
    lerr = (lse.cpu() - rl).abs().max().item()
    assert lerr <= ATOL_LSE, f"int4 LSE error {lerr:.3e} > {ATOL_LSE:.0e}"


@gpu
@pytest.mark.parametrize("rand_scale", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("padding,bsz", [(32, 8), (4096, 1)])
@pytest.mark.parametrize("kv_heads", [None, 1, 2])
@pytest.mark.parametrize("groups,d", [(2, 128), (4, 128), (8, 128), (2, 64), (4, 64)])
def test_decoder_int4_groups(groups, d, kv_heads, padding, bsz, dtype, rand_scale):
    """Several quantisation groups per row (``NUM_GROUPS``,
    tests/test_mem_eff_attention.py:1700-1707,1759)."""
    require_cuda()
    op = type(f"S2_{groups}", (S.FwOp_S2,), {"NUM_GROUPS": groups, "NAME": f"S2_{groups}"})
    q, k, v, bias, k_ref, v_ref = _decoder_case(16, kv_heads, padding, bsz, dtype, d=d, quant=True, rand_scale=rand_scale, groups=groups)
    reasons = op.not_supported_reasons(fmha.Inputs(q, k, v, bias))
    assert not reasons, reasons
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k_ref, v_ref, bias.to("cpu"))
    assert_o_lse(out, None, ro, rl, dtype, f"int4 x{groups}", o_scale=4.0 if not rand_scale else 1.0)
    lerr = (lse.cpu() - rl).abs().max().item()
    assert lerr <= ATOL_LSE, f"int4 x{groups} LSE error {lerr:.3e} > {ATOL_LSE:.0e}"


@gpu
@pytest.mark.parametrize("n_heads,num_queries", [(2, 4), (2, 5), (6, 7), (20, 3)])
@pytest.mark.parametrize("padding,bsz", [(32, 8), (48, 1)])
@pytest.mark.parametrize("kv_heads", [1, 2])
def test_decoder_many_queries(n_heads, num_queries, padding, bsz, kv_heads):
    # tests/test_mem_eff_attention.py:1820-1853: causal-with-offset across several queries
    require_cuda()
    dtype = torch.bfloat16
    q, k, v, bias, k_ref, v_ref = _decoder_case(n_heads, kv_heads, padding, bsz, dtype, num_queries=num_queries)
    op = S.FwOp_S2
    reasons = op.not_supported_reasons(fmha.Inputs(q, k, v, bias))
    if reasons:
        pytest.skip("; ".join(reasons))
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k_ref, v_ref, bias.to("cpu"))
    assert_o_lse(out, lse, ro, rl, dtype, "many queries")


@gpu
@pytest.mark.parametrize("B,Mq,Mkv,K", [(1, 8, 16384, 128), (1, 4, 16384, 128), (1, 16, 16384, 128), (1, 8, 1025, 128),
                                        (2, 8, 4096, 128), (3, 3, 16374, 128), (2, 3, 73, 128), (2, 7, 7328, 64), (2, 7, 63, 64)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_splitk_long_kv_mqa_dense(B, Mq, Mkv, K, dtype):
    # tests/test_mem_eff_attention.py:2239-2313: no bias, dense batch, MQA (stride-0 heads)
    require_cuda()
    H = 8 if Mq <= 8 else 4  # at most 64 query rows per KV head is decoding; more is a prefill
    g = torch.Generator().manual_seed(B * Mq + Mkv)
    q = torch.randn(B, Mq, H, K, generator=g).to(dtype).cuda()
    k = torch.randn(B, Mkv, 1, K, generator=g).to(dtype).cuda().expand(-1, -1, H, -1)
    v = torch.randn(B, Mkv, 1, K, generator=g).to(dtype).cuda().expand(-1, -1, H, -1)
    for op in (S.FwOp, S.FwOp_S1):
        reasons = op.not_supported_reasons(fmha.Inputs(q, k, v))
        assert not reasons, reasons
        out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, op=op)
        ro, rl = ref(q, k, v)
        assert_o_lse(out, lse, ro, rl, dtype, f"long kv {op.NAME}")
    assert fmha._dispatch_fw(fmha.Inputs(q, k, v), False) is S.FwOp


def _paged_case(B, max_t, page, quant, dtype=torch.bfloat16, Hq=8, D=128, seed=10):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, max_t + 1, (B,), generator=g).tolist()
    lens[0] = max_t
    q = torch.randn(1, B, 1, Hq, D, generator=g).to(dtype).cuda()
    kf = torch.randn(1, B * max_t, 1, 1, D, generator=g)
    vf = torch.randn(1, B * max_t, 1, 1, D, generator=g)
    if quant:
        k_pad, v_pad = oracle.quantize_kv_int4(kf), oracle.quantize_kv_int4(vf)
        k_ref, v_ref = oracle.dequantize_kv_int4(k_pad), oracle.dequantize_kv_int4(v_pad)
    else:
        k_pad, v_pad = kf.to(dtype), vf.to(dtype)
        k_ref, v_ref = k_pad.float(), v_pad.float()
    return q, k_pad, v_pad, k_ref, v_ref, lens


@gpu
@pytest.mark.parametrize("quant", [False, True])
@pytest.mark.parametrize("page", [64, 128, 256])
@pytest.mark.parametrize("B,max_t", [(1, 64), (5, 128), (5, 2048), (16, 4096)])
def test_paged_invariances(B, max_t, page, quant):
    """tests/test_mem_eff_attention.py:2402-2433,2493-2738: identity table ==
    padded; random page placement == padded; swapping two physical pages and
    patching the table changes nothing, bit for bit."""
    require_cuda()
    if max_t < page:
        pytest.skip("sequence shorter than a page")
    dtype = torch.bfloat16
    q, k_pad, v_pad, k_ref, v_ref, lens = _paged_case(B, max_t, page, quant)
    Hq = q.shape[3]
    expand = lambda t: t.cuda().expand(-1, -1, -1, Hq, -1)
    pad_bias = ab.BlockDiagonalPaddedKeysMask.from_seqlens([1] * B, max_t, lens, device="cuda")
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k_ref.expand(-1, -1, -1, Hq, -1), v_ref.expand(-1, -1, -1, Hq, -1), pad_bias.to("cpu"))
    out_pad, lse_pad = fmha.memory_efficient_attention_forward_requires_grad(q, expand(k_pad), expand(v_pad), pad_bias, op=S.FwOp)
    assert_o_lse(out_pad, lse_pad, ro, rl, dtype, "padded")

    pages_per_seq = max_t // page
    n_pages = B * pages_per_seq
    ident = torch.arange(n_pages, dtype=torch.int32).view(B, pages_per_seq).cuda()
    paged_bias = pad_bias.make_paged(ident, page, ab.PagedBlockDiagonalPaddedKeysMask)
    out_id, lse_id = fmha.memory_efficient_attention_forward_requires_grad(q, expand(k_pad), expand(v_pad), paged_bias, op=S.FwOp)
    assert torch.equal(out_id, out_pad) and torch.equal(lse_id, lse_pad), "identity block table must equal the padded cache bit for bit"

    # random placement of the pages
    g = torch.Generator().manual_seed(3)
    perm = torch.randperm(n_pages, generator=g).int().view(B, pages_per_seq)
    k_pg = oracle.scatter_to_pages(k_pad, perm, page, [max_t] * B, max_t, n_pages)
    v_pg = oracle.scatter_to_pages(v_pad, perm, page, [max_t] * B, max_t, n_pages)
    bias_r = pad_bias.make_paged(perm.cuda(), page, ab.PagedBlockDiagonalPaddedKeysMask)
    out_r, lse_r = fmha.memory_efficient_attention_forward_requires_grad(q, expand(k_pg), expand(v_pg), bias_r, op=S.FwOp)
    assert torch.equal(out_r, out_pad) and torch.equal(lse_r, lse_pad), "page placement must not change a single bit"

    if n_pages >= 2:
        # swap physical pages 0 and last, patch the table
        k2, v2 = k_pg.clone(), v_pg.clone()
        a, b = slice(0, page), slice((n_pages - 1) * page, n_pages * page)
        for t in (k2, v2):
            tmp = t[0, a].clone()
            t[0, a] = t[0, b]
            t[0, b] = tmp
        perm2 = perm.clone()
        perm2[perm == 0] = n_pages - 1
        perm2[perm == n_pages - 1] = 0
        bias_s = pad_bias.make_paged(perm2.cuda(), page, ab.PagedBlockDiagonalPaddedKeysMask)
        out_s, lse_s = fmha.memory_efficient_attention_forward_requires_grad(q, expand(k2), expand(v2), bias_s, op=S.FwOp)
        assert torch.equal(out_s, out_pad) and torch.equal(lse_s, lse_pad)


@gpu
@pytest.mark.parametrize("quant", [False, True])
@pytest.mark.parametrize("split_k", [None, 1, 3])
@pytest.mark.parametrize("page", [32, 64, 256])
@pytest.mark.parametrize("kv_heads,group", [(8, 8), (4, 4), (2, 16), (3, 8)])
def test_paged_gqa_several_kv_heads(kv_heads, group, page, split_k, quant):
    """Serving layout of benchmarks/benchmark_attn_decoding.py:241-306: several
    kv heads interleaved in every token row (so runs of tokens are contiguous
    in memory), query heads of a group broadcast with stride 0, paged cache."""
    require_cuda()
    dtype, D, B, max_t = torch.bfloat16, 128, 3, 1536
    g = torch.Generator().manual_seed(77)
    lens = [max_t, 1, 700]
    q = torch.randn(1, B, kv_heads, group, D, generator=g).to(dtype).cuda()
    kf = torch.randn(1, B * max_t, kv_heads, 1, D, generator=g)
    vf = torch.randn(1, B * max_t, kv_heads, 1, D, generator=g)
    if quant:
        k_pad, v_pad = oracle.quantize_kv_int4(kf), oracle.quantize_kv_int4(vf)
        k_ref, v_ref = oracle.dequantize_kv_int4(k_pad), oracle.dequantize_kv_int4(v_pad)
    else:
        k_pad, v_pad = kf.to(dtype), vf.to(dtype)
        k_ref, v_ref = k_pad.float(), v_pad.float()
    expand = lambda t: t.expand(-1, -1, -1, group, -1)
    pad_bias = ab.BlockDiagonalPaddedKeysMask.from_seqlens([1] * B, max_t, lens, device="cuda")
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), expand(k_ref), expand(v_ref), pad_bias.to("cpu"))
    pages_per_seq = max_t // page
    n_pages = B * pages_per_seq
    perm = torch.randperm(n_pages, generator=g).int().view(B, pages_per_seq)
    k_pg = oracle.scatter_to_pages(k_pad, perm, page, [max_t] * B, max_t, n_pages)
    v_pg = oracle.scatter_to_pages(v_pad, perm, page, [max_t] * B, max_t, n_pages)
    bias = pad_bias.make_paged(perm.cuda(), page, ab.PagedBlockDiagonalPaddedKeysMask)
    op = S.FwOp if split_k is None else type("Op", (S.FwOp,), {"SPLIT_K": split_k})
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, expand(k_pg.cuda()), expand(v_pg.cuda()), bias, op=op)
    assert_o_lse(out, lse, ro, rl, dtype, f"paged kv_heads={kv_heads}")
    out_pad, lse_pad = fmha.memory_efficient_attention_forward_requires_grad(q, expand(k_pad.cuda()), expand(v_pad.cuda()), pad_bias, op=op)
    assert torch.equal(out, out_pad) and torch.equal(lse, lse_pad), "page placement must not change a single bit"


@gpu
@pytest.mark.parametrize("quant", [False, True])
def test_nans_in_padding_do_not_leak(quant):
    # tests/test_mem_eff_attention.py:3036-3163
    require_cuda()
    B, max_kv, Hq, D = 64, 256, 8, 128
    dtype = torch.bfloat16
    q, k_pad, v_pad, k_ref, v_ref, lens = _paged_case(B, max_kv, 64, quant, seed=5)
    expand = lambda t: t.cuda().expand(-1, -1, -1, Hq, -1)
    bias = ab.BlockDiagonalPaddedKeysMask.from_seqlens([1] * B, max_kv, lens, device="cuda")
    out0, lse0 = fmha.memory_efficient_attention_forward_requires_grad(q, expand(k_pad), expand(v_pad), bias, op=S.FwOp)
    k_nan, v_nan = k_pad.clone(), v_pad.clone()
    for b, n in enumerate(lens):
        if quant:
            nan_word = torch.tensor([0x7E007E00], dtype=torch.int32)  # scale = shift = fp16 NaN
            k_nan[0, b * max_kv + n : (b + 1) * max_kv, ..., 0] = nan_word
            v_nan[0, b * max_kv + n : (b + 1) * max_kv, ..., 0] = nan_word
        else:
            k_nan[0, b * max_kv + n : (b + 1) * max_kv] = float("nan")
            v_nan[0, b * max_kv + n : (b + 1) * max_kv] = float("nan")
    out1, lse1 = fmha.memory_efficient_attention_forward_requires_grad(q, expand(k_nan), expand(v_nan), bias, op=S.FwOp)
    assert not out1.isnan().any() and not lse1.isnan().any()
    assert torch.equal(out0, out1) and torch.equal(lse0, lse1)


@gpu
def test_decode_empty_sequences_and_graph_replay():
    """kv_seqlen = 0 gives out = 0, lse = -inf; lengths are read from device
    memory at run time, so a captured graph follows in-place updates
    (examples/llama_inference/generate.py:144-187)."""
    require_cuda()
    dtype = torch.bfloat16
    B, P, Hq, D = 4, 512, 8, 128
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, B, 1, Hq, D, generator=g).to(dtype).cuda()
    k = torch.randn(1, B * P, 1, 1, D, generator=g).to(dtype).cuda().expand(-1, -1, -1, Hq, -1)
    v = torch.randn(1, B * P, 1, 1, D, generator=g).to(dtype).cuda().expand(-1, -1, -1, Hq, -1)
    lens = [0, 17, 512, 1]
    bias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens([1] * B, P, lens, device="cuda")
    for op in (S.FwOp_S1, S.FwOp_S4):
        out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
        assert (out[0, 0] == 0).all() and torch.isneginf(lse[0, :, :, 0]).all()
        ro, rl = ref(q, k, v, bias)
        assert_o_lse(out, lse, ro, rl, dtype, "empty sequence")
    # graph capture, then mutate the lengths in place and replay
    out_static = torch.empty_like(q)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        fmha.memory_efficient_attention_forward(q, k, v, bias, op=S.FwOp_S4)  # warm-up outside capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out_static = fmha.memory_efficient_attention_forward(q, k, v, bias, op=S.FwOp_S4)
    new_lens = [300, 18, 100, 2]
    bias.k_seqinfo.seqlen.copy_(torch.tensor(new_lens, dtype=torch.int32))
    graph.replay()
    torch.cuda.synchronize()
    bias_new = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens([1] * B, P, new_lens)
    ro, _ = oracle.ref_attention_with_lse(q.float().cpu(), k.float().cpu(), v.float().cpu(), bias_new)
    assert (out_static.float().cpu() - ro).abs().max() <= ATOL_O[dtype]


@gpu
def test_decode_respects_current_stream_and_custom_scale():
    require_cuda()
    dtype = torch.float16
    q, k, v, bias, k_ref, v_ref = _decoder_case(16, 2, 1024, 4, dtype)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        out = fmha.memory_efficient_attention_forward(q, k, v, bias, scale=0.05, op=S.FwOp, output_dtype=torch.float32)
    s.synchronize()
    assert out.dtype == torch.float32
    ro, _ = oracle.ref_attention_with_lse(q.float().cpu(), k_ref, v_ref, bias.to("cpu"), scale=0.05)
    assert (out.cpu() - ro).abs().max() <= ATOL_O[dtype]


@gpu
@pytest.mark.parametrize("fmt", ["bf16", "int4", "fp8"])
@pytest.mark.parametrize("split_k", [None, 1, 3])
@pytest.mark.parametrize("window", [1, 100, 640, 5000])
@pytest.mark.parametrize("kv_heads,group", [(8, 8), (1, 4)])
@pytest.mark.parametrize("Mq", [1, 3])
def test_local_window(Mq, kv_heads, group, window, split_k, fmt):
    """BlockDiagonalCausalLocalAttentionPaddedKeysMask and its paged form
    (bias list of tests/test_mem_eff_attention.py:283,395): a query sees the
    `window` keys that end at its own position (the last `window` keys of its
    sequence with one query per sequence, i.e. the sequence starts later); the
    same keys behind a block table give the same bits."""
    require_cuda()
    if Mq > 1 and fmt != "bf16":
        pytest.skip("windows with several queries per sequence: 16-bit caches")
    dtype, D, B, max_t, page = torch.bfloat16, 128, 4, 1536, 64
    g = torch.Generator().manual_seed(window)
    lens = [max_t, Mq, 700, 99]
    q = torch.randn(1, B * Mq, kv_heads, group, D, generator=g).to(dtype).cuda()
    kf = torch.randn(1, B * max_t, kv_heads, 1, D, generator=g)
    vf = torch.randn(1, B * max_t, kv_heads, 1, D, generator=g)
    expand = lambda t: t.expand(-1, -1, -1, group, -1)
    pad_bias = ab.BlockDiagonalCausalLocalAttentionPaddedKeysMask.from_seqlens_local([Mq] * B, max_t, lens, window, device="cuda")
    if fmt == "fp8":
        from oracle import fp8 as ofp8

        flat = lambda t: t.to(dtype).float().reshape(-1, D)
        (kq, ksc, ksh), (vq, vsc, vsh) = ofp8.quantize_fp8_asymmetric(flat(kf)), ofp8.quantize_fp8_asymmetric(flat(vf))
        kss_w, vss_w = ofp8.combine_scale_shift(ksc, ksh), ofp8.combine_scale_shift(vsc, vsh)
        # what the kernel sees after the fp16 rounding of scale and shift
        (ksc, ksh), (vsc, vsh) = ofp8.split_scale_shift(kss_w), ofp8.split_scale_shift(vss_w)
        k_ref = ofp8.dequantize_fp8_asymmetric(kq, ksc, ksh).reshape(kf.shape)
        v_ref = ofp8.dequantize_fp8_asymmetric(vq, vsc, vsh).reshape(vf.shape)
        k_pad = ofp8.pack_fp8_words(kq).reshape(1, B * max_t, kv_heads, 1, D // 4)
        v_pad = ofp8.pack_fp8_words(vq).reshape(1, B * max_t, kv_heads, 1, D // 4)
        kss, vss = kss_w.reshape(1, B * max_t, kv_heads, 1), vss_w.reshape(1, B * max_t, kv_heads, 1)
    elif fmt == "int4":
        k_pad, v_pad = oracle.quantize_kv_int4(kf), oracle.quantize_kv_int4(vf)
        k_ref, v_ref = oracle.dequantize_kv_int4(k_pad), oracle.dequantize_kv_int4(v_pad)
    else:
        k_pad, v_pad = kf.to(dtype), vf.to(dtype)
        k_ref, v_ref = k_pad.float(), v_pad.float()
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), expand(k_ref), expand(v_ref), pad_bias.to("cpu"))
    op = S.FwOp if split_k is None else type("Op", (S.FwOp,), {"SPLIT_K": split_k})

    def run(kc, vc, bias):
        if fmt == "fp8":
            inp = S.InputsFp8(query=q, key=expand(kc.cuda()), value=expand(vc.cuda()), attn_bias=bias,
                              k_fp8_scale_shift=kss.cuda().expand(-1, -1, -1, group).contiguous(),
                              v_fp8_scale_shift=vss.cuda().expand(-1, -1, -1, group).contiguous())
            out, ctx = fmha._memory_efficient_attention_forward_requires_grad(inp, op=op)
            return out, ctx.lse
        return fmha.memory_efficient_attention_forward_requires_grad(q, expand(kc.cuda()), expand(vc.cuda()), bias, op=op)

    out_pad, lse_pad = run(k_pad, v_pad, pad_bias)
    assert_o_lse(out_pad, lse_pad, ro, rl, dtype, f"window {window} {fmt}")
    # the plain causal mask with a window that covers everything is the same computation
    if window >= max_t:
        full = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens([Mq] * B, max_t, lens, device="cuda")
        out_f, lse_f = run(k_pad, v_pad, full)
        assert torch.equal(out_pad, out_f) and torch.equal(lse_pad, lse_f)
    if fmt == "fp8":
        paged = pad_bias.make_paged(torch.arange(B * (max_t // page), dtype=torch.int32).view(B, -1).cuda(), page, ab.PagedBlockDiagonalCausalLocalPaddedKeysMask)
        inp = S.InputsFp8(query=q, key=expand(k_pad.cuda()), value=expand(v_pad.cuda()), attn_bias=paged, k_fp8_scale_shift=kss.cuda().expand(-1, -1, -1, group).contiguous(),
                          v_fp8_scale_shift=vss.cuda().expand(-1, -1, -1, group).contiguous())
        assert any("window" in r for r in S.FwOp.not_supported_reasons(inp))
        return
    pages_per_seq = max_t // page
    n_pages = B * pages_per_seq
    perm = torch.randperm(n_pages, generator=g).int().view(B, pages_per_seq)
    k_pg = oracle.scatter_to_pages(k_pad, perm, page, [max_t] * B, max_t, n_pages)
    v_pg = oracle.scatter_to_pages(v_pad, perm, page, [max_t] * B, max_t, n_pages)
    bias = pad_bias.make_paged(perm.cuda(), page, ab.PagedBlockDiagonalCausalLocalPaddedKeysMask)
    assert bias._window_size == window
    out, lse = run(k_pg, v_pg, bias)
    assert_o_lse(out, lse, ro, rl, dtype, f"paged window {window} {fmt}")
    # and the paged bias materialises to the same visible keys as the flat one (physical rows)
    m = bias.to("cpu").materialize((B * Mq, n_pages * page)) == 0
    assert int(m.sum()) == sum(min(n - Mq + i + 1, window) for n in lens for i in range(Mq))


@gpu
@pytest.mark.parametrize("bias_dtype", [None, torch.float32])
@pytest.mark.parametrize("split_k", [None, 1, 4])
@pytest.mark.parametrize("layout,Mq", [("gqa", 1), ("gqa", 3), ("mha", 2), ("mha", 1)])
def test_decode_additive_tensor_bias(layout, Mq, split_k, bias_dtype):
    """A plain tensor as attn_bias on the split-K operator (the reference's takes one,
    xformers/ops/fmha/triton_splitk.py:18-27): added to q k^T * scale before the softmax;
    -inf entries hide keys."""
    require_cuda()
    dtype, D, B, Mkv = torch.bfloat16, 128, 2, 700
    g = torch.Generator().manual_seed(17 + Mq)
    if layout == "gqa":
        G, H = 2, 4
        q = torch.randn(B, Mq, G, H, D, generator=g).to(dtype).cuda()
        k = torch.randn(B, Mkv, G, 1, D, generator=g).to(dtype).cuda().expand(-1, -1, -1, H, -1)
        v = torch.randn(B, Mkv, G, 1, D, generator=g).to(dtype).cuda().expand(-1, -1, -1, H, -1)
        bshape = (B, G, H, Mq, Mkv)
    else:
        H = 3
        q = torch.randn(B, Mq, H, D, generator=g).to(dtype).cuda()
        k = torch.randn(B, Mkv, H, D, generator=g).to(dtype).cuda()
        v = torch.randn(B, Mkv, H, D, generator=g).to(dtype).cuda()
        bshape = (B, H, Mq, Mkv)
    bias = (torch.randn(bshape, generator=g) * 2).to(bias_dtype or dtype)
    bias[..., 0, : Mkv // 3] = float("-inf")
    bias = bias.cuda()
    op = S.FwOp if split_k is None else type("Op", (S.FwOp,), {"SPLIT_K": split_k})
    assert not op.not_supported_reasons(fmha.Inputs(q, k, v, bias))
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k.float().cpu(), v.float().cpu(), bias.float().cpu())
    assert_o_lse(out, lse, ro, rl, dtype, f"decode with a tensor bias, {layout}")
    assert fmha.b200_splitk.decode_device_status() == 0


@gpu
@pytest.mark.parametrize("Mq,window", [(2, 4), (5, 3), (4, 1), (16, 40)])
def test_local_window_several_queries_small(Mq, window):
    """Windows shorter than, equal to and longer than the number of queries of a sequence, sequences shorter than
    the window: every row's lower limit lies in the first sub-tile of the first chunk."""
    require_cuda()
    g = torch.Generator().manual_seed(Mq * 100 + window)
    lens = [Mq, 64, Mq + window - 1, 37]
    B, pad = len(lens), 64
    q = torch.randn(1, B * Mq, 2, 128, generator=g).bfloat16().cuda()
    k = torch.randn(1, B * pad, 2, 128, generator=g).bfloat16().cuda()
    v = torch.randn(1, B * pad, 2, 128, generator=g).bfloat16().cuda()
    bias = ab.BlockDiagonalCausalLocalAttentionPaddedKeysMask.from_seqlens_local([Mq] * B, pad, lens, window, device="cuda")
    assert not S.FwOp.not_supported_reasons(fmha.Inputs(q, k, v, bias))
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=S.FwOp)
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k.float().cpu(), v.float().cpu(), bias.to("cpu"))
    assert_o_lse(out, lse, ro, rl, torch.bfloat16, f"window {window}, {Mq} queries")


@gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,Mkv,H,K", [(1, 2**16, 3, 128), (5, 53, 4, 64), (7, 51, 4, 256), (3, 51, 2, 512)])
@pytest.mark.parametrize("op", [S.FwOp, None])
def test_mqa_decoding(op, dtype, B, Mkv, H, K):
    """tests/test_mem_eff_attention.py:2276-2313: one query, one kv head expanded
    over H query heads, inputs scaled by 3.  An operator that does not take the
    shape says so (the reference skips then); the dispatcher finds one for every
    head size the library covers."""
    require_cuda()
    g = torch.Generator(device="cuda").manual_seed(K + B)
    q = torch.randn(B, 1, H, K, generator=g, device="cuda", dtype=dtype) * 3
    k = (torch.randn(B, Mkv, 1, K, generator=g, device="cuda", dtype=dtype) * 3).expand(-1, -1, H, -1)
    v = (torch.randn(B, Mkv, 1, K, generator=g, device="cuda", dtype=dtype) * 3).expand(-1, -1, H, -1)
    if op is not None:
        reasons = op.not_supported_reasons(fmha.Inputs(q, k, v))
        assert bool(reasons) == (K not in (64, 128)), reasons
        if reasons:
            pytest.skip("; ".join(reasons))
    elif K > 256:
        with pytest.raises(NotImplementedError):
            fmha.memory_efficient_attention_forward(q, k, v)
        return
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, op=op)
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k.float().cpu(), v.float().cpu(), None)
    assert_o_lse(out, lse, ro, rl, dtype, f"mqa decoding K={K}", o_scale=3.0)
