"""The allocation-free decode entry point, called through the C ABI.

``xfb200_decode_forward_static_scratch`` serves callers that cannot allocate
device memory around the attention call (a serving loop pinned to a fixed
memory budget, a plugin whose host application owns the allocator): the
split-K partials go to a 16 MiB array inside the library instead of scratch
from the caller.  It must give exactly what ``xfb200_decode_forward`` gives with
caller-provided scratch -- on two calls in a row, because every call reuses the
same array and finds the previous call's contents in it.

This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""

import ctypes as C

import pytest
import torch

from xformers_b200 import _lib

gpu = pytest.mark.gpu


def _params(q, k, v, out, lse, seqlen, split_k, padding, scratch=None):
    """q [B, Hkv, G, D], k/v [B*padding, Hkv, D], out like q, lse [Hkv, G, B]."""
    B, Hkv, G, D = q.shape
    p = _lib.DecodeParams()
    p.q, p.k, p.v, p.out, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    p.scratch = scratch.data_ptr() if scratch is not None else None
    p.seqlen_k = seqlen.data_ptr()
    p.block_tables = None
    p.dtype = p.out_dtype = _lib.BF16
    p.kv_format, p.num_quant_groups = _lib.KV_PLAIN, 0
    p.batch, p.mq, p.kv_heads, p.q_per_kv, p.head_dim = B, 1, Hkv, G, D
    p.kv_padding, p.page_size, p.block_table_stride, p.split_k = padding, 0, 0, split_k
    p.q_stride_m, p.q_stride_g, p.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    p.k_stride_m, p.k_stride_g = k.stride(0), k.stride(1)
    p.v_stride_m, p.v_stride_g = v.stride(0), v.stride(1)
    p.o_stride_m, p.o_stride_g, p.o_stride_h = out.stride(0), out.stride(1), out.stride(2)
    p.lse_stride_g, p.lse_stride_h = lse.stride(0), lse.stride(1)
    p.mask_type = _lib.MASK_NONE
    p.scale = D**-0.5
    return p


def _run_both(seed, lens, split_k, padding=1024, Hkv=8, G=8, D=128):
    lib = _lib.load()
    dev = torch.device("cuda:0")
    B = len(lens)
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hkv, G, D, generator=g).bfloat16().to(dev)
    k = torch.randn(B * padding, Hkv, D, generator=g).bfloat16().to(dev)
    v = torch.randn(B * padding, Hkv, D, generator=g).bfloat16().to(dev)
    seqlen = torch.tensor(lens, dtype=torch.int32, device=dev)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    need = lib.xfb200_decode_scratch_bytes(B, 1, Hkv, G, D, split_k)
    assert 0 < need <= _lib.DECODE_STATIC_SCRATCH_BYTES
    scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    out_ref = torch.full((B, Hkv, G, D), float("nan"), dtype=torch.bfloat16, device=dev)
    lse_ref = torch.full((Hkv, G, B), float("nan"), dtype=torch.float32, device=dev)
    rc = lib.xfb200_decode_forward(C.byref(_params(q, k, v, out_ref, lse_ref, seqlen, split_k, padding, scratch)), stream)
    _lib.check(rc, "xfb200_decode_forward")

    out_new = torch.full_like(out_ref, float("nan"))
    lse_new = torch.full_like(lse_ref, float("nan"))
    rc = lib.xfb200_decode_forward_static_scratch(C.byref(_params(q, k, v, out_new, lse_new, seqlen, split_k, padding)), stream)
    _lib.check(rc, "xfb200_decode_forward_static_scratch")
    torch.cuda.synchronize(dev)
    return (q, k, v), (out_ref, lse_ref), (out_new, lse_new)


@gpu
def test_static_scratch_entry_point_matches_on_two_calls_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import oracle

    torch.cuda.set_device(0)
    # first call: four chunks per sequence; second call: other lengths and a
    # different split, so it meets the partials the first call left behind
    for seed, lens, split_k in ((0, [1024, 17, 513, 300], 4), (1, [5, 1000, 128, 129, 0, 640], 2)):
        (q, k, v), (out_ref, lse_ref), (out_new, lse_new) = _run_both(seed, lens, split_k)
        assert not out_new.isnan().any() and not lse_new.isnan().any()
        # same kernels, same order of operations: the tolerance of the other decode tests (O 2e-2, LSE 1e-3) is met exactly
        assert torch.equal(out_new, out_ref) and torch.equal(lse_new, lse_ref)
        # and both are right: the fp32 oracle on the same inputs
        B, Hkv, G, D = q.shape
        for b, n in enumerate(lens):
            if n == 0:
                assert (out_new[b] == 0).all() and torch.isneginf(lse_new[:, :, b]).all()
                continue
            kb = k[b * 1024 : b * 1024 + n].float().cpu()  # [n, Hkv, D]
            vb = v[b * 1024 : b * 1024 + n].float().cpu()
            qb = q[b].float().cpu()  # [Hkv, G, D]
            ro, rl = oracle.ref_attention_with_lse(qb, kb.permute(1, 0, 2), vb.permute(1, 0, 2))  # BMK with batch = Hkv
            assert (out_new[b].float().cpu() - ro).abs().max() <= 2e-2
            assert (lse_new[:, :, b].cpu() - rl).abs().max() <= 1e-3


@gpu
def test_static_scratch_entry_point_rejects_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    lib = _lib.load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    B, Hkv, G, D, padding, split_k = 64, 8, 8, 128, 256, 64
    assert lib.xfb200_decode_scratch_bytes(B, 1, Hkv, G, D, split_k) > _lib.DECODE_STATIC_SCRATCH_BYTES
    q = torch.zeros(B, Hkv, G, D, dtype=torch.bfloat16, device=dev)
    k = torch.zeros(B * padding, Hkv, D, dtype=torch.bfloat16, device=dev)
    out = torch.zeros_like(q)
    lse = torch.zeros(Hkv, G, B, device=dev)
    seqlen = torch.full((B,), padding, dtype=torch.int32, device=dev)
    rc = lib.xfb200_decode_forward_static_scratch(
        C.byref(_params(q, k, k, out, lse, seqlen, split_k, padding)), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    )
    assert rc == _lib.XFB200_E_INVALID
    msg = lib.xfb200_last_error().decode()
    assert str(_lib.DECODE_STATIC_SCRATCH_BYTES) in msg and "split" in msg
    with pytest.raises(ValueError):
        _lib.check(rc, "static scratch")
