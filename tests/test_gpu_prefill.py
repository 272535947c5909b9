"""Prefill operator on the GPU against the oracle: both kernels (tcgen05 for
head dims 64/128, mma.sync for the rest), every supported bias, BMK / BMHK /
BMGHK layouts, LSE, sharded keys + merge."""

import pytest
import torch

import oracle
from gpu_utils import ATOL_O, assert_o_lse, gpu, rand_qkv, ref, require_cuda
from xformers_b200.ops import fmha
from xformers_b200.ops.fmha import attn_bias as ab

P = fmha.b200
KERNELS = [P.FwOp_Tcgen05_Persistent, P.FwOp_Tcgen05_M256, P.FwOp_Generic]


def _status_ok():
    assert P.prefill_device_status() == 0, "a wait inside the tcgen05 kernel timed out"


@gpu
def test_baseline_config1_on_gpu():
    """B=2, M=128, H=4, D=64, causal, seed 0 (the CPU-runnable baseline
    configuration) -- inputs cast to bf16, compared with the fp32 golden."""
    require_cuda()
    import numpy as np
    import os

    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "cfg1_seed0.npz"))
    gen = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(2, 128, 4, 64, generator=gen) for _ in range(3))
    for dtype in (torch.bfloat16, torch.float16):
        qd, kd, vd = (t.to(dtype).cuda() for t in (q, k, v))
        ro, rl = ref(qd, kd, vd, ab.LowerTriangularMask())
        for op in KERNELS:
            out, lse = fmha.memory_efficient_attention_forward_requires_grad(qd, kd, vd, ab.LowerTriangularMask(), op=op)
            assert out.shape == (2, 128, 4, 64) and lse.shape == (2, 4, 128)
            assert_o_lse(out, lse, ro, rl, dtype, f"cfg1 {op.NAME}")
            # and against the stored fp32 vectors: only input rounding separates them
            assert np.abs(out.float().cpu().numpy() - g["out"]).max() < 5e-2
    _status_ok()


@gpu
@pytest.mark.parametrize("op", KERNELS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,Mq,Mkv,H", [(1, 128, 128, 1), (2, 256, 256, 3), (1, 384, 640, 2), (3, 32, 1024, 1), (1, 1024, 16, 2),
                                        (2, 3, 15, 1), (1, 31, 33, 2), (1, 132, 136, 1), (1, 90, 72, 5), (1, 2, 2, 1), (1, 257, 511, 1)])
def test_dense_bmhk(op, dtype, D, causal, B, Mq, Mkv, H):
    # shape grid of tests/test_mem_eff_attention.py:143-161 restricted to supported head dims
    require_cuda()
    q, k, v = rand_qkv(B, Mq, Mkv, 1, H, D, dtype, seed=B * Mq + Mkv * D, gqa=False)
    q, k, v = q[:, :, 0], k[:, :, 0], v[:, :, 0]
    bias = ab.LowerTriangularMask() if causal else None
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    ro, rl = ref(q, k, v, bias)
    assert_o_lse(out, lse, ro, rl, dtype, f"{op.NAME} dense")
    out2 = fmha.memory_efficient_attention_forward(q, k, v, bias, op=op)
    assert torch.equal(out, out2), "must be bit-reproducible"
    _status_ok()


@gpu
@pytest.mark.parametrize("D", [8, 16, 32, 40, 72, 96, 120, 160, 256])
@pytest.mark.parametrize("causal", [False, True])
def test_other_head_dims_use_the_mma_kernel(D, causal):
    require_cuda()
    dtype = torch.bfloat16
    q, k, v = rand_qkv(2, 68, 132, 1, 3, D, dtype, seed=D, gqa=False)
    q, k, v = q[:, :, 0], k[:, :, 0], v[:, :, 0]
    bias = ab.LowerTriangularMask() if causal else None
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias)
    ro, rl = ref(q, k, v, bias)
    assert_o_lse(out, lse, ro, rl, dtype, f"D={D}")


@gpu
@pytest.mark.parametrize("op", KERNELS)
def test_bmk_layout_and_packed_qkv(op):
    # tests/test_mem_eff_attention.py:560-585: q/k/v as non-contiguous views of one tensor
    require_cuda()
    dtype = torch.float16
    B, M, H, D = 2, 200, 4, 64
    g = torch.Generator().manual_seed(7)
    qkv = torch.randn(B, M, 3, H, D, generator=g).to(dtype).cuda()
    q, k, v = qkv.unbind(2)
    assert not q.is_contiguous()
    out = fmha.memory_efficient_attention_forward(q, k, v, op=op)
    ro, _ = ref(q, k, v)
    assert_o_lse(out, None, ro, None, dtype, "packed BMHK")
    # BMK: [B*H, M, K]
    q3, k3, v3 = (t.permute(0, 2, 1, 3).reshape(B * H, M, D) for t in (q, k, v))
    out3, lse3 = fmha.memory_efficient_attention_forward_requires_grad(q3, k3, v3, ab.LowerTriangularMask(), op=op)
    assert out3.shape == (B * H, M, D) and lse3.shape == (B * H, M)
    ro3, rl3 = oracle.ref_attention_with_lse(q3.float().cpu(), k3.float().cpu(), v3.float().cpu(), ab.LowerTriangularMask())
    assert_o_lse(out3, lse3, ro3, rl3, dtype, "BMK")
    _status_ok()


@gpu
@pytest.mark.parametrize("op", KERNELS)
@pytest.mark.parametrize("Mq", [1, 13, 512])
@pytest.mark.parametrize("bias_kind", ["none", "causal_br", "causal_tl"])
def test_gqa_bmghk(op, Mq, bias_kind):
    # tests/test_mem_eff_attention.py:2031-2064: B=3, Mkv=512, G=2, H=16, K=128, fp16, stride-0 heads
    require_cuda()
    if bias_kind == "causal_tl" and Mq == 1:
        pytest.skip("top-left causal with one query sees a single key; covered elsewhere")
    dtype = torch.float16
    q, k, v = rand_qkv(3, Mq, 512, 2, 16, 128, dtype, seed=Mq, gqa=True)
    assert k.stride(3) == 0
    bias = {"none": None, "causal_br": ab.LowerTriangularFromBottomRightMask(), "causal_tl": ab.LowerTriangularMask()}[bias_kind]
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    assert out.shape == q.shape and lse.shape == (3, 2, 16, Mq)
    ro, rl = ref(q, k, v, bias)
    assert_o_lse(out, lse, ro, rl, dtype, "GQA")
    _status_ok()


def _varlen_case(lens_q, lens_k, G, H, D, dtype, seed, gqa):
    q, k, v = rand_qkv(1, sum(lens_q), sum(lens_k), G, H, D, dtype, seed=seed, gqa=gqa)
    return q, k, v


@gpu
@pytest.mark.parametrize("op", KERNELS)
@pytest.mark.parametrize("kind", ["plain", "causal", "bottomright", "local", "local_br"])
def test_block_diagonal_varlen(op, kind):
    require_cuda()
    dtype = torch.bfloat16
    lens_q = [3, 130, 1, 256, 77, 128]
    lens_k = [5, 130, 9, 300, 77, 129] if kind in ("plain", "bottomright", "local_br") else lens_q
    q, k, v = _varlen_case(lens_q, lens_k, 2, 2, 128, dtype, seed=11, gqa=True)
    base = ab.BlockDiagonalMask.from_seqlens(lens_q, lens_k, device="cuda")
    bias = {
        "plain": base,
        "causal": base.make_causal(),
        "bottomright": base.make_causal_from_bottomright(),
        "local": base.make_local_attention(37),
        "local_br": base.make_local_attention_from_bottomright(150),
    }[kind]
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    assert lse.shape == (1, 2, 2, sum(lens_q)), "varlen LSE is packed"
    ro, rl = ref(q, k, v, bias)
    assert_o_lse(out, lse, ro, rl, dtype, f"varlen {kind}")
    _status_ok()


@gpu
@pytest.mark.parametrize("op", KERNELS)
def test_padded_keys_prefill_and_nan_padding(op):
    """tests/test_mem_eff_attention.py:1590-1646 (q lengths 4,1,1,...; keys in
    padded slots; bottom-right causal) and :3036-3163 (NaN beyond kv_seqlen)."""
    require_cuda()
    dtype = torch.float16
    bsize, n_heads, d, padding = 8, 3, 64, 160
    k_seqlen = [5, 8, 7, 1, 9, 3, 140, 160]
    q_seqlen = [4] + [1] * 7
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, sum(q_seqlen), n_heads, d, generator=g).to(dtype).cuda()
    k = torch.randn(1, bsize * padding, n_heads, d, generator=g).to(dtype).cuda()
    v = torch.randn(1, bsize * padding, n_heads, d, generator=g).to(dtype).cuda()
    for cls in (ab.BlockDiagonalCausalWithOffsetPaddedKeysMask, ab.BlockDiagonalPaddedKeysMask):
        bias = cls.from_seqlens(q_seqlen=q_seqlen, kv_seqlen=k_seqlen, kv_padding=padding, device="cuda")
        out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, scale=1.0 / 8, op=op)
        ro, rl = ref(q, k, v, bias, scale=1.0 / 8)
        assert_o_lse(out, lse, ro, rl, dtype, "padded keys")
        kn, vn = k.clone(), v.clone()
        for b, n in enumerate(k_seqlen):
            kn[0, b * padding + n : (b + 1) * padding] = float("nan")
            vn[0, b * padding + n : (b + 1) * padding] = float("nan")
        out_n, lse_n = fmha.memory_efficient_attention_forward_requires_grad(q, kn, vn, bias, scale=1.0 / 8, op=op)
        assert not out_n.isnan().any() and not lse_n.isnan().any(), "NaN in padding leaked"
        assert torch.equal(out, out_n) and torch.equal(lse, lse_n)
    _status_ok()

@gpu
@pytest.mark.parametrize("window", [1, 3, 64, 200])
@pytest.mark.parametrize("op", KERNELS)
def test_causal_local_padded_keys_and_bottom_right_local(op, window):
    """The window forms of the bottom-right causal masks
    (BlockDiagonalCausalLocalAttentionPaddedKeysMask,
    LowerTriangularFromBottomRightLocalAttentionMask; bias list of
    tests/test_mem_eff_attention.py:283,389): every query sees at most `window` keys."""
    require_cuda()
    dtype = torch.bfloat16
    n_heads, d, padding = 2, 128, 384
    k_seqlen = [5, 300, 131, 1, 384, 64]
    q_seqlen = [4, 130, 131, 1, 7, 64]
    g = torch.Generator().manual_seed(window)
    q = torch.randn(1, sum(q_seqlen), n_heads, d, generator=g).to(dtype).cuda()
    k = torch.randn(1, len(k_seqlen) * padding, n_heads, d, generator=g).to(dtype).cuda()
    v = torch.randn(1, len(k_seqlen) * padding, n_heads, d, generator=g).to(dtype).cuda()
    bias = ab.BlockDiagonalCausalLocalAttentionPaddedKeysMask.from_seqlens_local(q_seqlen, padding, k_seqlen, window, device="cuda")
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    ro, rl = ref(q, k, v, bias)
    assert_o_lse(out, lse, ro, rl, dtype, "causal local padded keys")
    # NaN beyond the sequences must not leak
    kn, vn = k.clone(), v.clone()
    for b, n in enumerate(k_seqlen):
        kn[0, b * padding + n : (b + 1) * padding] = float("nan")
        vn[0, b * padding + n : (b + 1) * padding] = float("nan")
    out_n, lse_n = fmha.memory_efficient_attention_forward_requires_grad(q, kn, vn, bias, op=op)
    assert torch.equal(out, out_n) and torch.equal(lse, lse_n)

    qd = torch.randn(2, 200, n_heads, d, generator=g).to(dtype).cuda()
    kd = torch.randn(2, 333, n_heads, d, generator=g).to(dtype).cuda()
    vd = torch.randn(2, 333, n_heads, d, generator=g).to(dtype).cuda()
    b2 = ab.LowerTriangularFromBottomRightLocalAttentionMask(window)
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(qd, kd, vd, b2, op=op)
    ro, rl = ref(qd, kd, vd, b2)
    assert_o_lse(out, lse, ro, rl, dtype, "bottom-right local")
    _status_ok()


@gpu
@pytest.mark.parametrize("op", KERNELS)
def test_no_out_of_bounds_reads(op):
    # tests/test_mem_eff_attention.py:499-506,591-598: inputs re-homed in NaN-padded storage
    require_cuda()
    dtype = torch.bfloat16
    B, Mq, Mkv, H, D = 2, 90, 200, 2, 128

    def nan_padded(shape):
        big = torch.full((shape[0], 256 * ((shape[1] + 255) // 256), shape[2], shape[3]), float("nan"), dtype=dtype, device="cuda")
        view = big[:, : shape[1]]
        view.copy_(torch.randn(shape, device="cuda").to(dtype))
        return view

    q, k, v = nan_padded((B, Mq, H, D)), nan_padded((B, Mkv, H, D)), nan_padded((B, Mkv, H, D))
    for bias in (None, ab.LowerTriangularMask()):
        out = fmha.memory_efficient_attention_forward(q, k, v, bias, op=op)
        assert not out.isnan().any()
        ro, _ = ref(q, k, v, bias)
        assert_o_lse(out, None, ro, None, dtype, "NaN-padded storage")
    _status_ok()


@gpu
@pytest.mark.parametrize("op", KERNELS)
@pytest.mark.parametrize("shards", [2, 4])
def test_sharded_keys_merge_to_full_causal(op, shards):
    """Long-context algebra: each shard of the key axis gives a partial
    (O, LSE) with the causal diagonal offset by the shard start; the merge
    equals the full result.  Rows that see nothing in a shard have lse = -inf."""
    require_cuda()
    dtype = torch.bfloat16
    B, S, G, H, D = 1, 1024, 2, 4, 128
    q, k, v = rand_qkv(B, S, S, G, H, D, dtype, seed=5, gqa=True)
    full, lse_full = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, ab.LowerTriangularMask(), op=op)
    outs, lses = [], []
    n = S // shards
    for r in range(shards):
        inp = fmha.Inputs(q, k[:, r * n : (r + 1) * n], v[:, r * n : (r + 1) * n], ab.LowerTriangularMask(), output_dtype=torch.float32, is_partial=True)
        o, ctx = op._apply(inp, want_lse=True, kv_offset=r * n)
        outs.append(o)
        lses.append(ctx.lse)
        if r > 0:
            assert torch.isneginf(ctx.lse[..., : r * n]).all() and (o[:, : r * n] == 0).all()
    merged, lse_m = fmha.merge_attentions(outs, lses, output_dtype=dtype)
    ro, rl = ref(q, k, v, ab.LowerTriangularMask())
    assert_o_lse(merged, lse_m, ro, rl, dtype, "sharded+merged")
    assert (merged.float() - full.float()).abs().max() <= ATOL_O[dtype]
    _status_ok()


@gpu
@pytest.mark.parametrize("world", [1, 2, 4])
def test_zigzag_key_ranges_merge_to_full_causal(world):
    """The balanced layout of the long-context path on one GPU: every emulated
    rank runs sharded_kv_attention_forward on its two key ranges (which merges
    them locally; no process group, so no exchange), and the merge of the ranks'
    results equals the full causal attention."""
    from xformers_b200.ops.fmha.sharded import sharded_kv_attention_forward, zigzag_bounds

    require_cuda()
    dtype = torch.bfloat16
    B, S, G, H, D = 1, 1536, 2, 4, 128
    q, k, v = rand_qkv(B, S, S, G, H, D, dtype, seed=6, gqa=True)
    outs, lses = [], []
    for r in range(world):
        spans = zigzag_bounds(S, world, r)
        o, l = sharded_kv_attention_forward(q, [k[:, a:b] for a, b in spans], [v[:, a:b] for a, b in spans],
                                            kv_offset=[a for a, _ in spans], causal=True, partial_dtype=torch.float32)
        outs.append(o.float())
        lses.append(l)
    merged, lse_m = fmha.merge_attentions(outs, lses, output_dtype=dtype)
    ro, rl = ref(q, k, v, ab.LowerTriangularMask())
    assert_o_lse(merged, lse_m, ro, rl, dtype, f"zigzag world={world}")
    _status_ok()


@gpu
def test_partial_chunks_merge_to_full_decode():
    # tests/test_fmha_merge_attentions.py:234-363: chunked attention + merge == full (1e-3 there)
    require_cuda()
    dtype = torch.bfloat16
    B, max_t, H, D = 16, 2048, 8, 128
    g = torch.Generator().manual_seed(1)
    q = torch.randn(1, B, 1, H, D, generator=g).to(dtype).cuda()
    k = torch.randn(1, B * max_t, 1, 1, D, generator=g).to(dtype).cuda().expand(-1, -1, -1, H, -1)
    v = torch.randn(1, B * max_t, 1, 1, D, generator=g).to(dtype).cuda().expand(-1, -1, -1, H, -1)
    lens = torch.randint(1, max_t + 1, (B,), generator=g).tolist()
    bias = ab.BlockDiagonalPaddedKeysMask.from_seqlens([1] * B, max_t, lens, device="cuda")
    full, lse_full = fmha.memory_efficient_attention_partial(q, k, v, bias, output_dtype=torch.float32)
    bounds = [0, 100, 101, 900, max_t]
    outs, lses = [], []
    for lo, hi in zip(bounds, bounds[1:]):
        # chunk [lo, hi) of every sequence: a padded-keys bias over a strided view of the cache
        kk = k.view(1, B, max_t, 1, H, D)[:, :, lo:hi].reshape(1, B * (hi - lo), 1, H, D)
        vv = v.view(1, B, max_t, 1, H, D)[:, :, lo:hi].reshape(1, B * (hi - lo), 1, H, D)
        kk = kk[:, :, :, :1].expand(-1, -1, -1, H, -1)
        vv = vv[:, :, :, :1].expand(-1, -1, -1, H, -1)
        clens = [max(0, min(n, hi) - lo) for n in lens]
        cb = ab.BlockDiagonalPaddedKeysMask.from_seqlens([1] * B, hi - lo, clens, device="cuda")
        o, l = fmha.memory_efficient_attention_partial(q, kk, vv, cb, output_dtype=torch.float32)
        outs.append(o)
        lses.append(l)
    merged, lse_m = fmha.merge_attentions(outs, lses)
    torch.testing.assert_close(merged, full, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(lse_m, lse_full, rtol=1e-3, atol=1e-3)


@gpu
def test_empty_tensors():
    # tests/test_mem_eff_attention.py:2316-2386
    require_cuda()
    dtype = torch.bfloat16
    q = torch.randn(2, 0, 4, 64, device="cuda").to(dtype)
    k = torch.randn(2, 16, 4, 64, device="cuda").to(dtype)
    assert fmha.memory_efficient_attention_forward(q, k, k).shape == (2, 0, 4, 64)
    q = torch.randn(2, 8, 4, 64, device="cuda").to(dtype)
    k = torch.randn(2, 0, 4, 64, device="cuda").to(dtype)
    out = fmha.memory_efficient_attention_forward(q, k, k, op=P.FwOp)
    assert out.shape == q.shape and (out == 0).all()
    q = torch.randn(0, 8, 4, 64, device="cuda").to(dtype)
    assert fmha.memory_efficient_attention_forward(q, q, q).shape == (0, 8, 4, 64)


@gpu
def test_custom_stream_and_output_dtype():
    # tests/test_mem_eff_attention.py:1153-1216: work is enqueued on the current stream
    require_cuda()
    dtype = torch.bfloat16
    q, k, v = rand_qkv(1, 256, 256, 1, 2, 128, dtype, seed=2, gqa=False)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        out = fmha.memory_efficient_attention_forward(q, k, v, ab.LowerTriangularMask(), output_dtype=torch.float32)
    s.synchronize()
    assert out.dtype == torch.float32
    ro, _ = ref(q, k, v, ab.LowerTriangularMask())
    assert (out.cpu() - ro).abs().max() <= ATOL_O[dtype]
    _status_ok()


@gpu
@pytest.mark.parametrize("bias_dtype", [None, torch.float32])
@pytest.mark.parametrize("layout", ["BMHK", "BMGHK", "BMK"])
@pytest.mark.parametrize("Mq,Mkv,D", [(64, 64, 64), (100, 300, 128), (257, 129, 32)])
@pytest.mark.parametrize("op", [P.FwOp, P.FwOp_Generic, P.FwOp_Tcgen05_Persistent])
def test_additive_tensor_bias(op, Mq, Mkv, D, layout, bias_dtype):
    """A plain tensor as attn_bias is added to q k^T * scale before the softmax
    (tests/test_mem_eff_attention.py:420-440, 664-682)."""
    require_cuda()
    if op is P.FwOp_Tcgen05_Persistent and D not in (64, 128):
        pytest.skip("tcgen05 kernels: head dim 64 or 128")
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(31)
    B, G, H = 2, 2, 3
    if layout == "BMHK":
        qs, ks, bs = (B, Mq, H, D), (B, Mkv, H, D), (B, H, Mq, Mkv)
    elif layout == "BMGHK":
        qs, ks, bs = (B, Mq, G, H, D), (B, Mkv, G, H, D), (B, G, H, Mq, Mkv)
    else:
        qs, ks, bs = (B * H, Mq, D), (B * H, Mkv, D), (B * H, Mq, Mkv)
    q, k, v = (torch.randn(s, generator=g).to(dtype).cuda() for s in (qs, ks, ks))
    bias = (torch.randn(bs, generator=g) * 2).to(bias_dtype or dtype)
    bias[..., 0, : Mkv // 2] = float("-inf")  # -inf entries mask keys like any mask
    bias = bias.cuda()
    assert not op.not_supported_reasons(fmha.Inputs(q, k, v, bias))
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k.float().cpu(), v.float().cpu(), bias.float().cpu())
    assert_o_lse(out, lse, ro, rl, dtype, f"tensor bias {layout}")


@gpu
@pytest.mark.parametrize("Mq,Mkv", [(128, 128), (70, 200)])
def test_causal_with_tensor_bias(Mq, Mkv):
    """LowerTriangularMaskWithTensorBias (tests/test_mem_eff_attention.py:1440-1449);
    the tensor is broadcast over the heads with stride 0."""
    require_cuda()
    dtype, B, H, D = torch.float16, 2, 4, 64
    g = torch.Generator().manual_seed(32)
    q = torch.randn(B, Mq, H, D, generator=g).to(dtype).cuda()
    k = torch.randn(B, Mkv, H, D, generator=g).to(dtype).cuda()
    v = torch.randn(B, Mkv, H, D, generator=g).to(dtype).cuda()
    t = torch.randn(B, 1, Mq, Mkv, generator=g).to(dtype).cuda().expand(B, H, Mq, Mkv)
    bias = ab.LowerTriangularMaskWithTensorBias(t)
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=P.FwOp)
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k.float().cpu(), v.float().cpu(), ab.LowerTriangularMaskWithTensorBias(t.float().cpu()))
    assert_o_lse(out, lse, ro, rl, dtype, "causal + tensor bias")
    # head dim 64: the persistent tcgen05 kernel takes it (and is what the automatic choice ran); the other tcgen05 kernel does not
    assert not P.FwOp_Tcgen05_Persistent.not_supported_reasons(fmha.Inputs(q, k, v, bias))
    assert P.FwOp_Tcgen05_M256.not_supported_reasons(fmha.Inputs(q, k, v, bias))
    out2, lse2 = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=P.FwOp_Generic)
    assert_o_lse(out2, lse2, ro, rl, dtype, "causal + tensor bias, mma.sync kernel")


@gpu
@pytest.mark.parametrize("op", KERNELS)
@pytest.mark.parametrize("wl,wr", [(1, 2), (0, 0), (5, 0), (0, 7), (130, 40), (300, 300)])
@pytest.mark.parametrize("Mq,Mkv", [(4, 4), (200, 200), (129, 520), (520, 129), (1030, 1030)])
def test_local_band_from_bottom_right(op, wl, wr, Mq, Mkv):
    """``LocalAttentionFromBottomRightMask`` (tests/test_mem_eff_attention.py:2389-2399):
    query i sees keys within [i + (Mkv - Mq) - window_left, i + (Mkv - Mq) + window_right]."""
    require_cuda()
    dtype = torch.bfloat16
    q, k, v = rand_qkv(2, Mq, Mkv, 2, 2, 128, dtype, seed=Mq + Mkv + wl, gqa=True)
    bias = ab.LocalAttentionFromBottomRightMask(window_left=wl, window_right=wr)
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    mask = oracle.local_mask(Mq, Mkv, wl, wr)
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k.float().cpu(), v.float().cpu(), mask.expand(2, 2, 2, Mq, Mkv))
    assert_o_lse(out, lse, ro, rl, dtype, f"{op.NAME} local band ({wl},{wr})")
    # rows that see no key at all: zeros and -inf
    dead = torch.isneginf(mask).all(-1)
    if dead.any():
        assert (out[:, dead].float() == 0).all() and torch.isneginf(lse[..., dead]).all()
    _status_ok()


@gpu
@pytest.mark.parametrize("op", KERNELS)
@pytest.mark.parametrize("gappy", [False, True])
def test_block_diagonal_local_padded_and_gappy_keys(op, gappy):
    """``BlockDiagonalLocalAttentionPaddedKeysMask`` and
    ``BlockDiagonalLocalAttentionFromBottomRightGappyKeysMask`` (xformers/ops/fmha/attn_bias.py:34-35):
    the band of the test above inside every block of a padded / gappy key cache."""
    require_cuda()
    dtype = torch.float16
    q_lens, kv_lens, pad = [5, 300, 64, 1], [40, 310, 64, 200], 384
    wl, wr = 33, 4
    g = torch.Generator().manual_seed(11)
    q = torch.randn(1, sum(q_lens), 2, 3, 64, generator=g).to(dtype).cuda()
    k = torch.randn(1, len(q_lens) * pad, 2, 1, 64, generator=g).to(dtype).cuda().expand(-1, -1, -1, 3, -1)
    v = torch.randn(1, len(q_lens) * pad, 2, 1, 64, generator=g).to(dtype).cuda().expand(-1, -1, -1, 3, -1)
    if gappy:
        starts = [7, 400, 800, 1200, len(q_lens) * pad]
        bias = ab.BlockDiagonalLocalAttentionFromBottomRightGappyKeysMask.from_seqlens_local(q_lens, starts, kv_lens, wl, wr, device="cuda")
    else:
        starts = [i * pad for i in range(len(q_lens) + 1)]
        bias = ab.BlockDiagonalLocalAttentionPaddedKeysMask.from_seqlens_local(q_lens, pad, kv_lens, wl, wr, device="cuda")
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    # the mask from plain integer lists: block b couples its queries with the keys [starts[b], starts[b] + kv_lens[b])
    mask = torch.full((sum(q_lens), len(q_lens) * pad), float("-inf"))
    qs = 0
    for b, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        mask[qs : qs + ql, starts[b] : starts[b] + kl] = oracle.local_mask(ql, kl, wl, wr)
        qs += ql
    assert torch.equal(bias.to("cpu").materialize(mask.shape), mask)
    ro, rl = oracle.ref_attention_with_lse(q.float().cpu(), k.float().cpu(), v.float().cpu(), mask.expand(1, 2, 3, *mask.shape))
    assert_o_lse(out, lse, ro, rl, dtype, f"{op.NAME} block-diagonal local, gappy={gappy}")
    _status_ok()


@gpu
def test_memory_efficient_attention_is_the_forward_without_grad():
    """xformers/ops/__init__.py:16: with nothing to differentiate the main entry
    point is the forward pass (examples/llama_inference/model.py:142 calls it so)."""
    require_cuda()
    import xformers_b200.ops as xops

    q, k, v = rand_qkv(1, 300, 300, 2, 4, 128, torch.bfloat16, seed=5, gqa=True)
    bias = ab.LowerTriangularMask()
    out = xops.memory_efficient_attention(q, k, v, attn_bias=bias)
    assert torch.equal(out, xops.memory_efficient_attention_forward(q, k, v, bias))
    out2 = xops.memory_efficient_attention(q, k, v, bias, op=(P.FwOp_Generic, None), scale=0.05, output_dtype=torch.float32)
    ro, _ = ref(q, k, v, bias, scale=0.05)
    assert out2.dtype == torch.float32 and (out2.cpu() - ro).abs().max() <= ATOL_O[torch.bfloat16]
    qg = q.clone().requires_grad_(True)
    with pytest.raises(NotImplementedError):
        xops.memory_efficient_attention(qg, k, v, bias)
    with torch.no_grad():
        assert torch.equal(xops.memory_efficient_attention(qg, k, v, bias), out)


@gpu
@pytest.mark.parametrize("op", KERNELS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("growth,jump_at", [(2.5, 512), (4.0, 600), (40.0, 600), (40.0, 130), (0.05, 384), (12.0, 1000)])
@pytest.mark.parametrize("causal", [False, True])
def test_scores_that_jump_along_the_keys(op, dtype, growth, jump_at, causal):
    """Keys from position ``jump_at`` on are ``growth`` times larger: the row maxima move by a few
    powers of two (re-based one step late), by more than 2^14 (the one-pass softmax has to stop in
    the middle of a tile and rescale what it already stored) or not at all (shrinking scores)."""
    require_cuda()
    B, M, H, D = 2, 1152, 2, 128
    q, k, v = rand_qkv(B, M, M, 1, H, D, dtype, seed=int(growth * 10) + jump_at, gqa=False)
    q, k, v = q[:, :, 0], k[:, :, 0].clone(), v[:, :, 0]
    k[:, jump_at:] *= growth
    bias = ab.LowerTriangularMask() if causal else None
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=op)
    ro, rl = ref(q, k, v, bias)
    assert_o_lse(out, lse, ro, rl, dtype, f"{op.NAME} growth {growth} at {jump_at}")
    _status_ok()


@gpu
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("q0,Mq,L0,o0,L1,o1", [(0, 1000, 256, 0, 300, 700), (0, 1000, 128, 128, 77, 900), (512, 300, 384, 0, 200, 640),
                                              (0, 515, 256, 600, 128, 2000), (100, 400, 128, 0, 256, 128)])
def test_two_key_ranges_in_one_launch(D, q0, Mq, L0, o0, L1, o1):
    """``kv_split``: a rank of a sharded causal sequence holds the key ranges [o0, o0 + L0) and [o1, o1 + L1) back to
    back; query rows are the global rows q0 .. q0 + Mq.  One launch equals the oracle on the visible keys."""
    require_cuda()
    dtype = torch.bfloat16
    S = max(o1 + L1, q0 + Mq)
    q, k, v = rand_qkv(1, S, S, 2, 2, D, dtype, seed=L0 + L1 + o1, gqa=True)
    qs = q[:, q0 : q0 + Mq]
    kc = torch.cat([k[:, o0 : o0 + L0, :, :1], k[:, o1 : o1 + L1, :, :1]], dim=1).expand(-1, -1, -1, 2, -1)
    vc = torch.cat([v[:, o0 : o0 + L0, :, :1], v[:, o1 : o1 + L1, :, :1]], dim=1).expand(-1, -1, -1, 2, -1)
    inp = fmha.Inputs(qs, kc, vc, ab.LowerTriangularMask(), output_dtype=torch.float32, is_partial=True)
    out, ctx = P.FwOp._apply(inp, want_lse=True, kv_offset=o0 - q0, kv_split=L0, kv_offset2=o1 - q0)
    # oracle: the same keys with the mask built from global positions
    key_pos = torch.cat([torch.arange(o0, o0 + L0), torch.arange(o1, o1 + L1)])
    vis = key_pos.view(1, -1) <= (q0 + torch.arange(Mq)).view(-1, 1)
    mask = torch.zeros(Mq, L0 + L1).masked_fill_(~vis, float("-inf"))
    ro, rl = oracle.ref_attention_with_lse(qs.float().cpu(), kc.float().cpu(), vc.float().cpu(), mask.expand(1, 2, 2, Mq, L0 + L1))
    assert_o_lse(out, ctx.lse, ro, rl, dtype, "two key ranges")
    dead = ~vis.any(-1)
    if dead.any():
        assert (out[:, dead] == 0).all() and torch.isneginf(ctx.lse[..., dead]).all()
    _status_ok()
    with pytest.raises(ValueError):
        P.FwOp._apply(inp, want_lse=True, kv_offset=0, kv_split=100, kv_offset2=o1)  # not a multiple of 128
    with pytest.raises(NotImplementedError):
        P.FwOp_Tcgen05_M256._apply(inp, want_lse=True, kv_offset=o0 - q0, kv_split=L0, kv_offset2=o1 - q0)
