"""rope_padded on the GPU against the CPU oracle, in the shape of the
reference's own tests (tests/test_rope_padded.py:155-344): ragged batches in a
padded cache, 4-D and 5-D inputs, odd head sizes, both pair layouts, linear and
wavelength-dependent scaling, shifted and explicit positions, and untouched
cache rows staying bit-identical."""

import pytest
import torch

import oracle
from xformers_b200.ops import fmha, rope_padded

pytestmark = pytest.mark.gpu

# tolerances of tests/test_rope_padded.py:148-152, plus f16 (same mantissa class as its f32 atol)
ATOL_RTOL = {torch.bfloat16: (5e-3, 8e-3), torch.float16: (5e-3, 1e-3), torch.float32: (5e-3, 1e-5)}


def _case(q_seqlen, kv_seqlen, padding, *, heads=10, kv_heads=2, dim=128, groups=None, dtype=torch.bfloat16, seed=0,
          expand_kv=False, cache_noise=True):
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(seed)
    M, B = sum(q_seqlen), len(q_seqlen)
    mid = () if groups is None else (groups,)
    xq = torch.randn((1, M) + mid + (heads, dim), generator=g).to(dtype)
    if expand_kv:
        xk = torch.randn((1, M) + mid + (1, dim), generator=g).to(dtype).expand((1, M) + mid + (kv_heads, dim))
        xv = torch.randn((1, M) + mid + (1, dim), generator=g).to(dtype).expand((1, M) + mid + (kv_heads, dim))
        ck = torch.randn((1, B * padding) + mid + (1, dim), generator=g).to(dtype).expand((1, B * padding) + mid + (kv_heads, dim))
        cv = torch.randn((1, B * padding) + mid + (1, dim), generator=g).to(dtype).expand((1, B * padding) + mid + (kv_heads, dim))
    else:
        xk = torch.randn((1, M) + mid + (kv_heads, dim), generator=g).to(dtype)
        xv = torch.randn((1, M) + mid + (kv_heads, dim), generator=g).to(dtype)
        shape = (1, B * padding) + mid + (kv_heads, dim)
        ck = torch.randn(shape, generator=g).to(dtype) if cache_noise else torch.zeros(shape, dtype=dtype)
        cv = torch.randn(shape, generator=g).to(dtype) if cache_noise else torch.zeros(shape, dtype=dtype)
    bias = fmha.attn_bias.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(
        q_seqlen=list(q_seqlen), kv_padding=padding, kv_seqlen=list(kv_seqlen))
    return dict(xq=xq, xk=xk, xv=xv, ck=ck, cv=cv, bias=bias.to(dev), starts=[b * padding for b in range(B)], dev=dev)


def _run_and_check(c, q_seqlen, kv_seqlen, *, first_seqpos=None, seqpos=None, internal_dtype="", tol=None, **kw):
    dev = c["dev"]

    def put(t):  # an expanded (stride 0) head axis stays expanded on the device
        if t.stride(-2) == 0 and t.shape[-2] > 1:
            return t[..., :1, :].to(dev).expand(t.shape)
        return t.to(dev)

    xq, xk, xv, ck, cv = (put(c[n]) for n in ("xq", "xk", "xv", "ck", "cv"))
    fs = None if first_seqpos is None else torch.tensor(first_seqpos, device=dev)
    sp = None if seqpos is None else torch.tensor(seqpos, device=dev)
    out = rope_padded(xq, xk, xv, ck, cv, c["bias"], first_seqpos=fs, seqpos=sp, internal_dtype=internal_dtype, **kw)
    want_q, want_k, want_v = oracle.rope_padded_ref(
        c["xq"], c["xk"], c["xv"], c["ck"], c["cv"], q_seqlen, c["starts"], kv_seqlen, first_seqpos=first_seqpos, seqpos=seqpos, **kw)
    atol, rtol = tol or ATOL_RTOL[xq.dtype]
    torch.testing.assert_close(out.cpu().float(), want_q.float(), atol=atol, rtol=rtol)
    torch.testing.assert_close(ck.cpu().float(), want_k.float(), atol=atol, rtol=rtol)
    assert torch.equal(cv.cpu(), want_v)  # values are copied, untouched rows keep their bits
    # rows that no token writes are bit-identical in cache_k as well
    written = torch.zeros(c["ck"].shape[1], dtype=torch.bool)
    for b, (ql, kl) in enumerate(zip(q_seqlen, kv_seqlen)):
        written[c["starts"][b] + kl - ql: c["starts"][b] + kl] = True
    assert torch.equal(ck.cpu()[0, ~written], c["ck"][0, ~written])
    return out


@pytest.mark.parametrize("adjacents", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("dim,padding", [(100, 87), (4098, 87), (128, 18300), (96, 87), (4096, 40)])
@pytest.mark.parametrize("groups", [None, 1, 3])
def test_consistency(adjacents, dtype, dim, padding, groups):
    # tests/test_rope_padded.py:155-283
    nq = [2, 1, 1]
    cache_lens = [27, padding - 5, padding // 2]
    c = _case(nq, cache_lens, padding, dim=dim, groups=groups, dtype=dtype, seed=dim + padding)
    _run_and_check(c, nq, cache_lens, adjacents=adjacents)


@pytest.mark.parametrize("adjacents", [True, False])
@pytest.mark.parametrize("kw", [
    dict(linear_scale=4.0),
    dict(theta=500000.0),
    dict(use_dynamic_scaling=True),
    dict(use_dynamic_scaling=True, theta=500000.0, dynamic_old_context_len=4096.0, dynamic_scale_factor=8.0,
         dynamic_low_freq_factor=2.0, dynamic_high_freq_factor=16.0, linear_scale=2.0),
])
def test_scalings(adjacents, kw):
    nq, cache_lens, padding = [2, 1, 1, 5], [27, 9000, 4500, 8192], 9001
    c = _case(nq, cache_lens, padding, dim=128, dtype=torch.bfloat16, seed=7)
    _run_and_check(c, nq, cache_lens, adjacents=adjacents, **kw)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("internal_dtype", ["", "f32", "f64"])
def test_internal_dtype(dtype, internal_dtype):
    nq, cache_lens, padding = [3, 1], [100000, 77777], 100000
    c = _case(nq, cache_lens, padding, heads=4, kv_heads=1, dim=64, dtype=dtype, seed=3)
    # float64 angles: only the final rounding differs; float32 angles at position 1e5 carry ~4e-3 of angle error
    tol = ((1e-6, 1e-6) if dtype == torch.float32 else (1e-6, 8e-3)) if internal_dtype == "f64" else (2e-2, 8e-3)
    _run_and_check(c, nq, cache_lens, internal_dtype=internal_dtype, tol=tol)


@pytest.mark.parametrize("adjacents", [True, False])
@pytest.mark.parametrize("seqlen", [1, 511, 2049])
def test_prefill(adjacents, seqlen):
    # tests/test_rope_padded.py:286-299: one sequence, cache length == query length
    c = _case([seqlen], [seqlen], seqlen + 1, heads=4, kv_heads=2, dim=256, dtype=torch.float32, seed=seqlen)
    _run_and_check(c, [seqlen], [seqlen], adjacents=adjacents)


def test_positions():
    # tests/test_rope_padded.py:302-344
    seqlen = 512
    c = _case([seqlen], [seqlen], seqlen, heads=2, kv_heads=2, dim=32, dtype=torch.float32, seed=1)
    _run_and_check(c, [seqlen], [seqlen], first_seqpos=[4])
    custom = list(range(seqlen))
    custom[231], custom[423] = 934, 134
    _run_and_check(c, [seqlen], [seqlen], seqpos=custom)
    # int32 positions are accepted as well
    dev = c["dev"]
    ck, cv = c["ck"].to(dev), c["cv"].to(dev)
    a = rope_padded(c["xq"].to(dev), c["xk"].to(dev), c["xv"].to(dev), ck, cv, c["bias"], seqpos=torch.tensor(custom, device=dev, dtype=torch.int32))
    b = rope_padded(c["xq"].to(dev), c["xk"].to(dev), c["xv"].to(dev), ck, cv, c["bias"], seqpos=torch.tensor(custom, device=dev))
    assert torch.equal(a, b)


def test_ragged_batch_with_empty_sequence_and_out_q():
    nq, cache_lens, padding = [4, 0, 1, 7], [4, 10, 33, 64], 64
    c = _case(nq, cache_lens, padding, heads=8, kv_heads=8, dim=64, dtype=torch.bfloat16, seed=11)
    out = _run_and_check(c, nq, cache_lens)
    # out_q given (no-grad mode), with room between tokens: strided rows
    dev = c["dev"]
    wide = torch.zeros(1, sum(nq), 8, 96, dtype=torch.bfloat16, device=dev)
    with torch.no_grad():
        got = rope_padded(c["xq"].to(dev), c["xk"].to(dev), c["xv"].to(dev), c["ck"].to(dev), c["cv"].to(dev), c["bias"], out_q=wide[..., :64])
    assert got.data_ptr() == wide.data_ptr() and torch.equal(got, out) and not wide[..., 64:].any()


def test_unaligned_rows_take_the_scalar_path():
    nq, cache_lens, padding = [2, 3], [9, 3], 16
    c = _case(nq, cache_lens, padding, heads=3, kv_heads=1, dim=64, dtype=torch.bfloat16, seed=5)
    dev = c["dev"]
    # rows that start one element off a 16-byte boundary
    pad = torch.zeros(1, 5, 3, 65, dtype=torch.bfloat16, device=dev)
    pad[..., 1:] = c["xq"].to(dev)
    ck, cv = c["ck"].to(dev), c["cv"].to(dev)
    got = rope_padded(pad[..., 1:], c["xk"].to(dev), c["xv"].to(dev), ck, cv, c["bias"])
    want_q, want_k, _ = oracle.rope_padded_ref(c["xq"], c["xk"], c["xv"], c["ck"], c["cv"], nq, c["starts"], cache_lens)
    torch.testing.assert_close(got.cpu().float(), want_q.float(), atol=5e-3, rtol=8e-3)
    torch.testing.assert_close(ck.cpu().float(), want_k.float(), atol=5e-3, rtol=8e-3)


def test_single_kv_head_given_expanded():
    # xformers/ops/rope_padded.py:121-129: stride 0 over the kv heads means one real head
    nq, cache_lens, padding = [1, 1, 2], [5, 40, 17], 40
    c = _case(nq, cache_lens, padding, heads=8, kv_heads=4, dim=128, groups=2, dtype=torch.bfloat16, seed=13, expand_kv=True)
    _run_and_check(c, nq, cache_lens)


def test_feeds_decode_attention():
    # the stated purpose (xformers/ops/rope_padded.py:47-53): out_q, cache_k, cache_v go straight into attention
    nq, cache_lens, padding = [1, 1, 1], [100, 257, 31], 512
    c = _case(nq, cache_lens, padding, heads=8, kv_heads=1, dim=128, dtype=torch.bfloat16, seed=17)
    dev = c["dev"]
    ck, cv = c["ck"].to(dev), c["cv"].to(dev)
    out_q = rope_padded(c["xq"].to(dev), c["xk"].to(dev), c["xv"].to(dev), ck, cv, c["bias"])
    attn = fmha.memory_efficient_attention_forward(out_q, ck.expand(-1, -1, 8, -1), cv.expand(-1, -1, 8, -1), c["bias"])
    want_q, want_k, want_v = oracle.rope_padded_ref(c["xq"], c["xk"], c["xv"], c["ck"], c["cv"], nq, c["starts"], cache_lens)
    for b in range(3):
        kk = want_k[0, b * padding: b * padding + cache_lens[b], 0].float()
        vv = want_v[0, b * padding: b * padding + cache_lens[b], 0].float()
        p = torch.softmax(want_q[0, b].float() @ kk.T * 128**-0.5, -1)
        torch.testing.assert_close(attn[0, b].cpu().float(), p @ vv, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("page_size", [16, 256])
@pytest.mark.parametrize("groups", [None, 2])
def test_paged_cache(page_size, groups):
    # beyond the reference: the caches are page pools reached through block_tables
    nq, cache_lens = [5, 1, 40, 1], [21, 300, 40, 1]
    max_pages = (max(cache_lens) + page_size - 1) // page_size
    B = len(nq)
    g = torch.Generator().manual_seed(page_size)
    tables = torch.randperm(B * max_pages + 3, generator=g)[: B * max_pages].int().view(B, max_pages)
    pool_rows = (B * max_pages + 3) * page_size
    dev = torch.device("cuda")
    mid = () if groups is None else (groups,)
    M, Hq, Hkv, D = sum(nq), 8, 2, 128
    xq = torch.randn((1, M) + mid + (Hq, D), generator=g).bfloat16()
    xk = torch.randn((1, M) + mid + (Hkv, D), generator=g).bfloat16()
    xv = torch.randn((1, M) + mid + (Hkv, D), generator=g).bfloat16()
    ck = torch.randn((1, pool_rows) + mid + (Hkv, D), generator=g).bfloat16()
    cv = torch.randn((1, pool_rows) + mid + (Hkv, D), generator=g).bfloat16()
    bias = fmha.attn_bias.PagedBlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(nq, cache_lens, tables, page_size).to(dev)
    ckd, cvd = ck.to(dev), cv.to(dev)
    out = rope_padded(xq.to(dev), xk.to(dev), xv.to(dev), ckd, cvd, bias)
    want_q, want_k, want_v = oracle.rope_padded_ref(xq, xk, xv, ck, cv, nq, [0] * B, cache_lens, block_tables=tables.tolist(), page_size=page_size)
    torch.testing.assert_close(out.cpu().float(), want_q.float(), atol=5e-3, rtol=8e-3)
    torch.testing.assert_close(ckd.cpu().float(), want_k.float(), atol=5e-3, rtol=8e-3)
    assert torch.equal(cvd.cpu(), want_v)
    changed = (ckd.cpu() != ck).flatten(2).any(-1)[0]
    assert int(changed.sum()) <= M  # only the rows of the new tokens were touched
    if groups is None:
        # and the paged decode operator reads what was written: last query of each sequence
        qlast = out[:, [4, 5, 45, 46]].reshape(1, B, Hkv, Hq // Hkv, D)
        dbias = fmha.attn_bias.PagedBlockDiagonalPaddedKeysMask.from_seqlens([1] * B, cache_lens, tables, page_size).to(dev)
        attn = fmha.memory_efficient_attention_forward(
            qlast, ckd.unsqueeze(3).expand(-1, -1, -1, Hq // Hkv, -1), cvd.unsqueeze(3).expand(-1, -1, -1, Hq // Hkv, -1), dbias,
            op=fmha.triton_splitk.FwOp)
        ref, _ = oracle.ref_attention_with_lse(
            qlast.float().cpu(), want_k.float().unsqueeze(3).expand(-1, -1, -1, Hq // Hkv, -1),
            want_v.float().unsqueeze(3).expand(-1, -1, -1, Hq // Hkv, -1), dbias.to("cpu"))
        torch.testing.assert_close(attn.float().cpu(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("adjacents", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("dim", [64, 128, 256])
@pytest.mark.parametrize("paged", [False, True])
def test_int4_cache_quantised_on_write(paged, dim, dtype, adjacents):
    """Beyond the reference: cache_k / cache_v are int4 row-wise caches
    (benchmarks/benchmark_attn_decoding.py:38-72).  Values are copies, so their
    rows must equal the oracle's quantiser bit for bit; rotated keys may differ
    from the float64 oracle by one rounding of the 16-bit value, i.e. by at most
    one quantisation step after dequantising.  Untouched rows keep their bits."""
    nq, cache_lens, page = [3, 1, 17], [40, 300, 17], 64
    B, Hq, Hkv = len(nq), 8, 2
    g = torch.Generator().manual_seed(dim + int(paged))
    M = sum(nq)
    xq = torch.randn(1, M, Hq, dim, generator=g).to(dtype)
    xk = torch.randn(1, M, Hkv, dim, generator=g).to(dtype)
    xv = torch.randn(1, M, Hkv, dim, generator=g).to(dtype)
    dev = torch.device("cuda")
    if paged:
        max_pages = 5
        tables = torch.randperm(B * max_pages, generator=g).int().view(B, max_pages)
        rows_total, starts = B * max_pages * page, [0] * B
        bias = fmha.attn_bias.PagedBlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(nq, cache_lens, tables, page).to(dev)
        extra = dict(block_tables=tables.tolist(), page_size=page)
    else:
        padding = 320
        rows_total, starts = B * padding, [b * padding for b in range(B)]
        bias = fmha.attn_bias.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=nq, kv_padding=padding, kv_seqlen=cache_lens).to(dev)
        extra = {}
    old_k = torch.randint(-2**31, 2**31 - 1, (1, rows_total, Hkv, 1 + dim // 8), generator=g, dtype=torch.int64).to(torch.int32)
    old_v = torch.randint(-2**31, 2**31 - 1, (1, rows_total, Hkv, 1 + dim // 8), generator=g, dtype=torch.int64).to(torch.int32)
    ck, cv = old_k.to(dev), old_v.to(dev)
    out = rope_padded(xq.to(dev), xk.to(dev), xv.to(dev), ck, cv, bias, adjacents=adjacents)
    # the oracle's pipeline: rope into a 16-bit cache, then quantise the written rows
    z = torch.zeros(1, rows_total, Hkv, dim, dtype=dtype)
    want_q, want_k, want_v = oracle.rope_padded_ref(xq, xk, xv, z, z, nq, starts, cache_lens, adjacents=adjacents, **extra)
    torch.testing.assert_close(out.cpu().float(), want_q.float(), atol=5e-3, rtol=8e-3)
    written = (want_v[0] != 0).flatten(1).any(-1) | (want_k[0] != 0).flatten(1).any(-1)
    assert int(written.sum()) == M
    assert torch.equal(ck.cpu()[0, ~written], old_k[0, ~written]) and torch.equal(cv.cpu()[0, ~written], old_v[0, ~written])
    assert torch.equal(cv.cpu()[0, written], oracle.quantize_kv_int4(want_v[0, written]))
    got_k = oracle.dequantize_kv_int4(ck.cpu()[0, written])
    ref_rows = want_k[0, written].float()
    step = (ref_rows.amax(-1, keepdim=True) - ref_rows.amin(-1, keepdim=True)) / 15
    # half a step of quantisation error, plus one step where the 16-bit rounding of the rotated value fell the other way
    assert ((got_k - ref_rows).abs() <= 1.6 * step + 1e-2).all()
    assert ((got_k - ref_rows).abs() <= 0.51 * step + 1e-2).float().mean() > 0.97


def test_int4_cache_feeds_decode():
    """rope_padded -> int4 paged cache -> split-K decode, against attention on the
    dequantised oracle cache."""
    nq, cache_lens, page, D, Hkv, G = [1, 1, 1], [100, 257, 31], 64, 128, 2, 4
    B = 3
    g = torch.Generator().manual_seed(5)
    dev = torch.device("cuda")
    tables = torch.randperm(B * 5, generator=g).int().view(B, 5)
    rows_total = B * 5 * page
    # a cache whose earlier keys are already there (quantised), then one new token per sequence
    base_k, base_v = torch.randn(1, rows_total, Hkv, D, generator=g).bfloat16(), torch.randn(1, rows_total, Hkv, D, generator=g).bfloat16()
    ck, cv = oracle.quantize_kv_int4(base_k).to(dev), oracle.quantize_kv_int4(base_v).to(dev)
    xq = torch.randn(1, B, Hkv * G, D, generator=g).bfloat16()
    xk, xv = torch.randn(1, B, Hkv, D, generator=g).bfloat16(), torch.randn(1, B, Hkv, D, generator=g).bfloat16()
    bias = fmha.attn_bias.PagedBlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(nq, cache_lens, tables, page).to(dev)
    out_q = rope_padded(xq.to(dev), xk.to(dev), xv.to(dev), ck, cv, bias)
    q5 = out_q.view(1, B, Hkv, G, D)
    attn = fmha.memory_efficient_attention_forward(q5, ck.unsqueeze(3).expand(-1, -1, -1, G, -1), cv.unsqueeze(3).expand(-1, -1, -1, G, -1), bias,
                                                   op=fmha.triton_splitk.FwOp)
    k_deq, v_deq = oracle.dequantize_kv_int4(ck.cpu()), oracle.dequantize_kv_int4(cv.cpu())
    ref, _ = oracle.ref_attention_with_lse(q5.float().cpu(), k_deq.unsqueeze(3).expand(-1, -1, -1, G, -1), v_deq.unsqueeze(3).expand(-1, -1, -1, G, -1), bias.to("cpu"))
    torch.testing.assert_close(attn.float().cpu(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("adjacents", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("paged", [False, True])
def test_fp8_cache_quantised_on_write(paged, dim, dtype, adjacents):
    """Beyond the reference: cache_k / cache_v are fp8 row-wise caches (InputsFp8,
    tests/utils.py:134-222).  The format is defined by its dequantiser, x = fp8 *
    scale + shift: the written rows must dequantise to the oracle's rotated keys
    and to the values within the e4m3 rounding of x - shift (3 mantissa bits) plus
    the fp16 rounding of the shift; other rows and scale words keep their bits."""
    from oracle import fp8 as ofp8

    nq, cache_lens, page = [3, 1, 17], [40, 300, 17], 64
    B, Hq, Hkv = len(nq), 8, 2
    g = torch.Generator().manual_seed(dim + int(paged))
    M = sum(nq)
    xq = torch.randn(1, M, Hq, dim, generator=g).to(dtype)
    xk = (torch.randn(1, M, Hkv, dim, generator=g) + 0.5).to(dtype)
    xv = (torch.randn(1, M, Hkv, dim, generator=g) * 2 - 1).to(dtype)
    dev = torch.device("cuda")
    if paged:
        tables = torch.randperm(B * 5, generator=g).int().view(B, 5)
        rows_total, starts = B * 5 * page, [0] * B
        bias = fmha.attn_bias.PagedBlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(nq, cache_lens, tables, page).to(dev)
        extra = dict(block_tables=tables.tolist(), page_size=page)
    else:
        padding = 320
        rows_total, starts = B * padding, [b * padding for b in range(B)]
        bias = fmha.attn_bias.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=nq, kv_padding=padding, kv_seqlen=cache_lens).to(dev)
        extra = {}
    rnd = lambda *shape: torch.randint(-2**31, 2**31 - 1, shape, generator=g, dtype=torch.int64).to(torch.int32)
    old_k, old_v = rnd(1, rows_total, Hkv, dim // 4), rnd(1, rows_total, Hkv, dim // 4)
    old_ks, old_vs = rnd(1, rows_total, Hkv), rnd(1, rows_total, Hkv)
    ck, cv, ks, vs = old_k.to(dev), old_v.to(dev), old_ks.to(dev), old_vs.to(dev)
    out = rope_padded(xq.to(dev), xk.to(dev), xv.to(dev), ck, cv, bias, adjacents=adjacents, cache_k_scale_shift=ks, cache_v_scale_shift=vs)
    z = torch.zeros(1, rows_total, Hkv, dim, dtype=dtype)
    want_q, want_k, want_v = oracle.rope_padded_ref(xq, xk, xv, z, z, nq, starts, cache_lens, adjacents=adjacents, **extra)
    torch.testing.assert_close(out.cpu().float(), want_q.float(), atol=5e-3, rtol=8e-3)
    written = (want_v[0] != 0).flatten(1).any(-1)
    assert int(written.sum()) == M
    for got, got_ss, old, old_ss, want in ((ck, ks, old_k, old_ks, want_k), (cv, vs, old_v, old_vs, want_v)):
        got, got_ss = got.cpu(), got_ss.cpu()
        assert torch.equal(got[0, ~written], old[0, ~written]) and torch.equal(got_ss[0, ~written], old_ss[0, ~written])
        scale, shift = ofp8.split_scale_shift(got_ss[0, written])
        vals = ofp8.unpack_fp8_words(got[0, written]).float()
        deq = vals * scale.float()[..., None] + shift.float()[..., None]
        ref = want[0, written].float()
        # the stored shift is the row mean up to its fp16 rounding, the scale maps the largest |x - shift| to about 448
        assert ((shift.float() - ref.mean(-1)).abs() <= 2e-3 * ref.mean(-1).abs() + 1e-2).all()
        assert (vals.abs().amax(-1) >= 416).all() and (vals.abs().amax(-1) <= 448).all()
        c = ref - shift.float()[..., None]
        assert ((deq - ref).abs() <= c.abs() * 2**-4 + 2e-2).all()
        assert ((deq - ref).abs().mean() <= 0.03 * c.abs().mean() + 2e-3)


def test_fp8_cache_feeds_decode():
    """rope_padded -> fp8 cache -> split-K decode, against attention on the
    dequantised cache."""
    from oracle import fp8 as ofp8

    nq, cache_lens, padding, D, Hkv, G = [1, 1, 1], [100, 257, 31], 320, 128, 2, 4
    B = 3
    g = torch.Generator().manual_seed(6)
    dev = torch.device("cuda")
    rows_total = B * padding
    # earlier keys written by an earlier call (a prefill of the whole slots), then one new token per sequence
    pre = fmha.attn_bias.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=[padding] * B, kv_padding=padding, kv_seqlen=[padding] * B).to(dev)
    ck = torch.zeros(1, rows_total, Hkv, D // 4, dtype=torch.int32, device=dev)
    cv, ks, vs = torch.zeros_like(ck), torch.zeros(1, rows_total, Hkv, dtype=torch.int32, device=dev), torch.zeros(1, rows_total, Hkv, dtype=torch.int32, device=dev)
    big = lambda h: torch.randn(1, rows_total, h, D, generator=g).bfloat16().to(dev)
    rope_padded(big(Hkv * G), big(Hkv), big(Hkv), ck, cv, pre, cache_k_scale_shift=ks, cache_v_scale_shift=vs)
    xq = torch.randn(1, B, Hkv * G, D, generator=g).bfloat16()
    xk, xv = torch.randn(1, B, Hkv, D, generator=g).bfloat16(), torch.randn(1, B, Hkv, D, generator=g).bfloat16()
    bias = fmha.attn_bias.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=nq, kv_padding=padding, kv_seqlen=cache_lens).to(dev)
    out_q = rope_padded(xq.to(dev), xk.to(dev), xv.to(dev), ck, cv, bias, cache_k_scale_shift=ks, cache_v_scale_shift=vs)
    q5 = out_q.view(1, B, Hkv, G, D)
    ex = lambda t: t.unsqueeze(3).expand(-1, -1, -1, G, -1)
    inp = fmha.triton_splitk.InputsFp8(query=q5, key=ex(ck), value=ex(cv), attn_bias=bias,
                                       k_fp8_scale_shift=ks.unsqueeze(3).expand(-1, -1, -1, G), v_fp8_scale_shift=vs.unsqueeze(3).expand(-1, -1, -1, G))
    attn = fmha._memory_efficient_attention_forward(inp, op=fmha.triton_splitk.FwOp)

    def deq(words, ss):
        scale, shift = ofp8.split_scale_shift(ss.cpu())
        return ofp8.unpack_fp8_words(words.cpu()).float() * scale.float()[..., None] + shift.float()[..., None]

    ref, _ = oracle.ref_attention_with_lse(q5.float().cpu(), ex(deq(ck, ks)), ex(deq(cv, vs)), bias.to("cpu"))
    torch.testing.assert_close(attn.float().cpu(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("paged", [False, True])
def test_lengths_that_do_not_fit_write_nothing_outside_the_slot(paged):
    """The lengths live on the device and may be updated in place between calls
    (examples/llama_inference/generate.py:144-187).  If they stop fitting the
    layout -- fewer keys than new queries, or more keys than the slot holds -- the
    positions outside the slot are skipped instead of landing in a neighbour's
    rows; the positions inside it are written as usual."""
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(2)
    nq, page, D, H = [4, 4, 4], 16, 64, 2
    B, M = 3, 12
    xq = torch.randn(1, M, H, D, generator=g).bfloat16().to(dev)
    xk, xv = torch.randn(1, M, H, D, generator=g).bfloat16().to(dev), torch.randn(1, M, H, D, generator=g).bfloat16().to(dev)
    if paged:
        tables = torch.tensor([[2, 5], [0, 3], [4, 1]], dtype=torch.int32)
        bias = fmha.attn_bias.PagedBlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(nq, [10, 10, 10], tables, page).to(dev)
        row_of = lambda b, t: int(tables[b, t // page]) * page + t % page
    else:
        bias = fmha.attn_bias.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=nq, kv_padding=2 * page, kv_seqlen=[10, 10, 10]).to(dev)
        row_of = lambda b, t: b * 2 * page + t
    # sequence 0: 2 keys for 4 queries (positions -2, -1, 0, 1); sequence 1 fits; sequence 2: 34 keys in a slot of 32 (positions 30 .. 33)
    bias.k_seqinfo.seqlen.copy_(torch.tensor([2, 10, 34], dtype=torch.int32))
    ck = torch.zeros(1, 6 * page, H, D, dtype=torch.bfloat16, device=dev)
    cv = torch.zeros_like(ck)
    rope_padded(xq, xk, xv, ck, cv, bias)
    written = set(torch.nonzero(cv[0].float().abs().flatten(1).sum(-1)).flatten().tolist())
    want = {row_of(0, 0), row_of(0, 1)} | {row_of(1, t) for t in range(6, 10)} | {row_of(2, 30), row_of(2, 31)}
    assert written == want
    assert torch.equal(cv[0, row_of(0, 0)], xv[0, 2]) and torch.equal(cv[0, row_of(2, 31)], xv[0, 9])
