"""Device status words, bounded waits and use of a second device.

Nothing here faults or hangs a GPU: the one deliberate failure is a wait that
runs out of its (shortened) budget, after which the kernel records a code and
returns normally.
"""

import ctypes as C

import pytest
import torch

from gpu_utils import assert_o_lse, gpu, rand_qkv, ref, require_cuda
from xformers_b200 import _lib
from xformers_b200.ops import fmha
from xformers_b200.ops.fmha import attn_bias as ab

P = fmha.b200


def _withheld(base):
    """``base`` with a wait budget of 2M clocks (about a millisecond) and the testing aid that
    makes the first CTA leave out its last key-tile copy."""
    return type(base.__name__ + "_Withheld", (base,), {"_WAIT_BUDGET_KCYCLES": 2000, "_DEBUG_FLAGS": 1, "NAME": base.NAME + "-withheld"})


@gpu
@pytest.mark.parametrize("base", [P.FwOp_Tcgen05_Persistent, P.FwOp_Tcgen05_M256])
def test_a_wait_that_runs_out_is_reported_cleared_and_harmless(base):
    """One block of query rows, one CTA: the key tile it waits for never comes, the wait
    gives up after its budget, the kernel returns; the host sees XFB200_E_DEVICE once, the
    word is clear afterwards and the next launch on the device is correct."""
    require_cuda()
    dtype = torch.bfloat16
    q, k, v = rand_qkv(1, 256, 256, 1, 1, 128, dtype, seed=1, gqa=False)
    bias = ab.LowerTriangularMask()
    assert P.prefill_device_status() == 0
    fmha.memory_efficient_attention_forward(q, k, v, bias, op=_withheld(base))
    with pytest.raises(RuntimeError, match="gave up a bounded wait"):
        P.check_device_status()
    assert P.prefill_device_status() == 0, "reading the status clears it"
    out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, bias, op=base)
    ro, rl = ref(q, k, v, bias)
    assert_o_lse(out, lse, ro, rl, dtype, "launch after a reported time-out")
    assert P.prefill_device_status() == 0


@gpu
def test_status_calls_through_the_c_abi():
    require_cuda()
    lib = _lib.load()
    st = C.c_int32(-1)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.xfb200_prefill_device_status(stream, C.byref(st)) == _lib.XFB200_OK and st.value == 0
    st = C.c_int32(-1)
    assert lib.xfb200_decode_device_status(stream, C.byref(st)) == _lib.XFB200_OK and st.value == 0
    assert lib.xfb200_decode_device_status(stream, None) == _lib.XFB200_E_INVALID


@gpu
def test_check_status_after_every_call(monkeypatch):
    """XFB200_CHECK_STATUS=1: the operators read the status word after each launch."""
    require_cuda()
    monkeypatch.setenv("XFB200_CHECK_STATUS", "1")
    monkeypatch.setenv("XFB200_DEBUG_CHECKS", "1")
    q, k, v = rand_qkv(1, 256, 256, 1, 2, 128, torch.bfloat16, seed=2, gqa=False)
    with pytest.raises(RuntimeError, match="gave up a bounded wait"):
        fmha.memory_efficient_attention_forward(q, k, v, ab.LowerTriangularMask(), op=_withheld(P.FwOp_Tcgen05_Persistent))
    out = fmha.memory_efficient_attention_forward(q, k, v, ab.LowerTriangularMask(), op=P.FwOp)
    ro, _ = ref(q, k, v, ab.LowerTriangularMask())
    assert_o_lse(out, None, ro, None, torch.bfloat16, "after a raised time-out")


@gpu
def test_debug_checks_catch_bad_page_tables_and_lengths(monkeypatch):
    """XFB200_DEBUG_CHECKS=1: a page id outside the pool, a length beyond its slot and a
    non-monotone seqstart are refused on the host before any launch."""
    require_cuda()
    monkeypatch.setenv("XFB200_DEBUG_CHECKS", "1")
    dtype, page, B = torch.bfloat16, 64, 2
    q = torch.randn(1, B, 2, 4, 128, dtype=dtype, device="cuda")
    # (the pool is a view of a larger allocation: the bad page id below stays inside memory this test owns)
    k = torch.randn(1, 16 * page, 2, 1, 128, dtype=dtype, device="cuda")[:, : 4 * page].expand(-1, -1, -1, 4, -1)
    table = torch.tensor([[0, 1], [2, 9]], dtype=torch.int32, device="cuda")  # the pool has pages 0..3
    bias = ab.PagedBlockDiagonalPaddedKeysMask.from_seqlens([1, 1], [100, 100], table, page)
    with pytest.raises(ValueError, match="outside the pool"):
        fmha.memory_efficient_attention_forward(q, k, k, bias, op=fmha.b200_splitk.FwOp)
    # without the check the tiled copies are still bounded by the pool's rows: what lies past them reads as zeros
    monkeypatch.setenv("XFB200_DEBUG_CHECKS", "0")
    out = fmha.memory_efficient_attention_forward(q, k, k, bias, op=fmha.b200_splitk.FwOp)
    assert torch.isfinite(out.float()).all()
    monkeypatch.setenv("XFB200_DEBUG_CHECKS", "1")
    pbias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens([1, 1], 128, [100, 100], device="cuda")
    pbias.k_seqinfo.seqlen.fill_(500)  # longer than the slot of 128 rows
    with pytest.raises(ValueError, match="does not fit"):
        fmha.memory_efficient_attention_forward(q, k, k, pbias, op=fmha.b200_splitk.FwOp)
    vb = ab.BlockDiagonalCausalMask.from_seqlens([100, 156], device="cuda")
    vb.q_seqinfo.seqstart.copy_(torch.tensor([0, 200, 150], dtype=torch.int32))
    qq = torch.randn(1, 256, 2, 4, 128, dtype=dtype, device="cuda")
    with pytest.raises(ValueError, match="monotone"):
        fmha.memory_efficient_attention_forward(qq, qq, qq, vb, op=P.FwOp)


@gpu
def test_second_device_in_one_process():
    """Function attributes (the dynamic shared-memory limit) and the status words are per
    device: every kernel family runs on cuda:1 after it ran on cuda:0, with cuda:0 current."""
    require_cuda()
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import oracle

    dtype = torch.bfloat16
    for dev in ("cuda:0", "cuda:1"):
        torch.cuda.set_device(0)
        q, k, v = rand_qkv(1, 300, 300, 2, 4, 128, dtype, seed=3, gqa=True, device=dev)
        for op in (P.FwOp_Tcgen05_Persistent, P.FwOp_Tcgen05_M256, P.FwOp_Generic):
            out, lse = fmha.memory_efficient_attention_forward_requires_grad(q, k, v, ab.LowerTriangularMask(), op=op)
            ro, rl = ref(q, k, v, ab.LowerTriangularMask())
            assert_o_lse(out, lse, ro, rl, dtype, f"{op.NAME} on {dev}")
        assert P.prefill_device_status(dev) == 0
        qd = torch.randn(1, 3, 2, 4, 128, dtype=dtype, device=dev)
        kd = torch.randn(1, 3 * 512, 2, 1, 128, dtype=dtype, device=dev).expand(-1, -1, -1, 4, -1)
        vd = torch.randn(1, 3 * 512, 2, 1, 128, dtype=dtype, device=dev).expand(-1, -1, -1, 4, -1)
        bias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens([1, 1, 1], 512, [500, 17, 512], device=dev)
        od, ld = fmha.memory_efficient_attention_forward_requires_grad(qd, kd, vd, bias, op=fmha.b200_splitk.FwOp_S4)
        ro, rl = ref(qd, kd, vd, bias)
        assert_o_lse(od, ld, ro, rl, dtype, f"decode on {dev}")
        assert fmha.b200_splitk.decode_device_status(dev) == 0
        a = torch.randn(3, 2, 5, 4, 128, device=dev)
        l = torch.randn(3, 2, 4, 5, device=dev)
        mo, ml = fmha.merge_attentions(a, l)
        ro, rl = oracle.merge_attentions_ref(a, l)
        assert (mo.cpu() - ro).abs().max() <= 1e-4 and (ml.cpu() - rl).abs().max() <= 1e-4
