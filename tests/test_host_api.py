"""Host-side logic that needs no GPU: bias classes, argument validation,
dispatch rules, the C-ABI library's exports."""

import ctypes
import os
import re

import pytest
import torch

import xformers_b200.ops as xops
from xformers_b200 import _lib
from xformers_b200.ops import fmha
from xformers_b200.ops.fmha import attn_bias as ab

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "xfb200.h")).read()
    declared = re.findall(r"XFB200_API\s+[\w\s\*]+?\b(xfb200_\w+)\s*\(", header)
    assert len(declared) >= 8
    assert _lib.is_built(), "build the library first: python -m xformers_b200.build"
    lib = ctypes.CDLL(str(_lib.library_path()))
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/xfb200.h but not exported"
    assert set(declared) == set(_lib.EXPORTED_SYMBOLS)
    assert _lib.load().xfb200_abi_version() == _lib.ABI_VERSION == 4


def test_struct_sizes_match_header():
    # sizes computed by hand from include/xfb200.h (LP64)
    assert ctypes.sizeof(_lib.Strides) == 32
    assert ctypes.sizeof(_lib.PrefillParams) == 8 * 8 + 8 * 4 + 4 * 32 + 3 * 8 + 6 * 4 + 8 + 2 * 4 + 4 * 8 + 6 * 4
    assert ctypes.sizeof(_lib.DecodeParams) == 8 * 8 + 12 * 4 + 12 * 8 + 4 * 4 + 2 * 8 + 4 * 8 + 8 + 8 + 2 * 4 + 8 + 2 * 4 + 4 * 8
    assert ctypes.sizeof(_lib.MergeParams) == 16 + 8 + 16 + 32 + 24 + 16 + 32 + 24 + 8 * 4


def test_c_abi_rejects_bad_arguments_without_a_gpu():
    lib = _lib.load()
    assert lib.xfb200_prefill_forward(None, None) == _lib.XFB200_E_INVALID
    assert b"null" in lib.xfb200_last_error()
    p = _lib.PrefillParams()
    p.dtype, p.out_dtype, p.batch, p.mq, p.groups, p.heads_per_group, p.head_dim = 7, 0, 1, 1, 1, 1, 64
    assert lib.xfb200_prefill_forward(ctypes.byref(p), None) == _lib.XFB200_E_INVALID
    p.dtype, p.head_dim = _lib.BF16, 12
    assert lib.xfb200_prefill_forward(ctypes.byref(p), None) == _lib.XFB200_E_UNSUPPORTED
    d = _lib.DecodeParams()
    d.batch, d.mq, d.kv_heads, d.q_per_kv, d.head_dim = 1, 1, 1, 1, 96
    d.q = d.k = d.v = d.out = 16
    assert lib.xfb200_decode_forward(ctypes.byref(d), None) == _lib.XFB200_E_UNSUPPORTED
    m = _lib.MergeParams()
    assert lib.xfb200_merge_attentions(ctypes.byref(m), None) == _lib.XFB200_E_INVALID
    with pytest.raises(ValueError):
        _lib.check(_lib.XFB200_E_INVALID, "x")
    with pytest.raises(NotImplementedError):
        _lib.check(_lib.XFB200_E_UNSUPPORTED, "x")
    assert lib.xfb200_decode_scratch_bytes(2, 1, 8, 8, 128, 1) == 0
    assert lib.xfb200_decode_scratch_bytes(2, 1, 8, 8, 128, 4) == 2 * 4 * 64 * 128 * 4 + 2 * 4 * 64 * 4


def test_public_names_exist():
    for name in (
        "memory_efficient_attention_forward",
        "memory_efficient_attention_forward_requires_grad",
        "memory_efficient_attention_partial",
        "merge_attentions",
        "Inputs",
        "AttentionFwOpBase",
        "AttentionOpBase",
        "AttentionBias",
        "LowerTriangularMask",
        "BlockDiagonalMask",
        "ALL_FW_OPS",
        "_dispatch_fw",
    ):
        assert hasattr(fmha, name), name
    for name in (
        "LowerTriangularMask",
        "BlockDiagonalMask",
        "BlockDiagonalCausalMask",
        "BlockDiagonalPaddedKeysMask",
        "BlockDiagonalCausalWithOffsetPaddedKeysMask",
        "PagedBlockDiagonalPaddedKeysMask",
        "PagedBlockDiagonalCausalWithOffsetPaddedKeysMask",
        "_SeqLenInfo",
        "_PaddedSeqLenInfo",
        "VARLEN_BIASES",
    ):
        assert hasattr(fmha.attn_bias, name), name
    for name in ("Inputs", "Context", "AttentionFwOpBase", "bmk2bmhk", "check_lastdim_alignment_stride1"):
        assert hasattr(fmha.common, name), name
    assert hasattr(fmha.dispatch, "_dispatch_fw_priority_list")
    assert issubclass(fmha.triton_splitk.FwOp_S4, fmha.b200_splitk.FwOp) and fmha.triton_splitk.FwOp_S4.SPLIT_K == 4
    assert xops.memory_efficient_attention_forward is fmha.memory_efficient_attention_forward
    for op in fmha.ALL_FW_OPS:
        for attr in ("NAME", "OPERATOR", "SUPPORTED_DEVICES", "CUDA_MINIMUM_COMPUTE_CAPABILITY", "SUPPORTED_DTYPES", "SUPPORTED_MAX_K",
                     "SUPPORTED_MIN_K", "SUPPORTS_DIFFERENT_VALUE_EMBED", "SUPPORTED_ATTN_BIAS_TYPES", "SUPPORTS_BMGHK",
                     "SUPPORTS_OUTPUT_DTYPE", "SUPPORTS_CUSTOM_SCALE", "VARLEN_LSE_PACKED", "ERROR_ATOL", "ERROR_RTOL", "_TEST_BATCH_SIZES", "_TEST_K"):
            assert hasattr(op, attr), (op, attr)
        assert fmha._unserialize_op(fmha._serialize_op(op)) is op


def test_seqleninfo_and_split():
    # tests/test_mem_eff_attention.py:1452-1538
    qs = [torch.randn(1, 3, 1, 8), torch.randn(3, 2, 1, 8), torch.randn(1, 5, 1, 8)]
    bias, q = ab.BlockDiagonalMask.from_tensor_list(qs)
    assert q.shape == (1, 14, 1, 8)
    assert bias.q_seqinfo.seqstart.dtype == torch.int32 and bias.q_seqinfo.seqstart.tolist() == [0, 3, 5, 7, 9, 14]
    assert bias.q_seqinfo.max_seqlen == 5 and bias.q_seqinfo.min_seqlen == 2
    back = bias.split(q)
    assert len(back) == 3 and all(torch.equal(a, b) for a, b in zip(qs, back))
    lq = [torch.randn(1, 3, 1, 8), torch.randn(2, 1, 1, 8)]
    lk = [torch.randn(1, 2, 1, 8), torch.randn(2, 3, 1, 8)]
    bias, q, k, _ = ab.BlockDiagonalMask.from_tensor_lists_qkv(lq, lk)
    assert all(torch.equal(a, b) for a, b in zip(lq, bias.split_queries(q)))
    assert all(torch.equal(a, b) for a, b in zip(lk, bias.split_kv(k)))
    with pytest.raises(ValueError):
        bias.split_queries(k)
    assert list(bias.q_seqinfo.intervals()) == [(0, 3), (3, 4), (4, 5)]


def test_padded_and_paged_bias_records():
    bias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=[1, 1], kv_padding=16, kv_seqlen=[3, 16])
    assert isinstance(bias.k_seqinfo, ab._PaddedSeqLenInfo)
    assert bias.k_seqinfo.seqstart.tolist() == [0, 16, 32] and bias.k_seqinfo.seqlen.tolist() == [3, 16] and bias.k_seqinfo.padding == 16
    assert bias.k_seqinfo.seqlen.dtype == torch.int32
    with pytest.raises(ValueError):
        ab.BlockDiagonalPaddedKeysMask.from_seqlens(q_seqlen=[1], kv_padding=4, kv_seqlen=[5])
    bt = torch.tensor([[1, 0], [2, 3]], dtype=torch.int32)
    paged = bias.make_paged(bt, 8, ab.PagedBlockDiagonalCausalWithOffsetPaddedKeysMask)
    assert isinstance(paged, ab.PagedBlockDiagonalPaddedKeysMask) and paged.page_size == 8
    assert paged.k_seqinfo.seqlen is bias.k_seqinfo.seqlen  # in-place length updates stay visible
    assert isinstance(bias, ab.VARLEN_BIASES) and isinstance(paged, ab.VARLEN_BIASES)
    assert type(ab.LowerTriangularMask().to("cpu")) is ab.LowerTriangularMask


def test_cpu_tensors_and_bad_inputs_raise_value_error():
    # tests/test_mem_eff_attention.py:1371-1407: never a CUDA error for a checkable input
    q = torch.randn(1, 8, 2, 64)
    with pytest.raises(ValueError):
        xops.memory_efficient_attention_forward(q, q, q)
    with pytest.raises(ValueError):
        xops.memory_efficient_attention_forward(q, q[:, :4], q)  # k/v length mismatch
    with pytest.raises(ValueError):
        xops.memory_efficient_attention_forward(q, q.double(), q)  # dtype mismatch
    with pytest.raises(ValueError):
        xops.memory_efficient_attention_forward(torch.randn(8, 64), torch.randn(8, 64), torch.randn(8, 64))
    bias = ab.BlockDiagonalMask.from_seqlens([4, 4])
    with pytest.raises(ValueError):
        xops.memory_efficient_attention_forward(torch.randn(2, 8, 2, 64), torch.randn(2, 8, 2, 64), torch.randn(2, 8, 2, 64), bias)
    # the reference's main entry point: forward when nothing asks for a gradient (CPU tensors: ValueError as above),
    # NotImplementedError only when autograd would have to record the call
    with pytest.raises(ValueError):
        xops.memory_efficient_attention(q, q, q)
    qg = q.clone().requires_grad_(True)
    with pytest.raises(NotImplementedError):
        xops.memory_efficient_attention(qg, q, q)
    with torch.no_grad(), pytest.raises(ValueError):
        xops.memory_efficient_attention(qg, q, q)


def test_not_supported_reasons_strings():
    q = torch.randn(1, 16, 2, 64, dtype=torch.bfloat16)
    r = fmha.b200.FwOp.not_supported_reasons(fmha.Inputs(q, q, q))
    assert any("device=cpu" in s for s in r)
    r = fmha.b200.FwOp.not_supported_reasons(fmha.Inputs(q.float(), q.float(), q.float()))
    assert any("dtype=torch.float32" in s for s in r)
    qo = torch.randn(1, 16, 2, 72, dtype=torch.bfloat16)[..., :65]  # K+1 slice: misaligned
    r = fmha.b200.FwOp.not_supported_reasons(fmha.Inputs(qo, qo, qo))
    assert any("% 8 != 0" in s for s in r)
    qs = torch.randn(1, 16, 2, 128, dtype=torch.bfloat16)[..., ::2]  # last-dim stride 2
    r = fmha.b200.FwOp.not_supported_reasons(fmha.Inputs(qs, qs, qs))
    assert any("stride(-1) == 1" in s for s in r)
    assert fmha.b200.FwOp.shape_not_supported_reasons(16, 16, 512, 512)
    assert fmha.b200.FwOp.shape_not_supported_reasons(16, 16, 64, 32)
    assert not fmha.b200.FwOp.shape_not_supported_reasons(16, 16, 64, 64)
    assert fmha.b200_splitk.FwOp.shape_not_supported_reasons(1, 16, 32, 32)
    r = fmha.b200_splitk.FwOp.not_supported_reasons(fmha.Inputs(torch.randn(1, 128, 1, 32, 128).bfloat16(), torch.randn(1, 64, 1, 1, 128).bfloat16().expand(-1, -1, -1, 32, -1), torch.randn(1, 64, 1, 1, 128).bfloat16().expand(-1, -1, -1, 32, -1)))
    assert any("this is a prefill" in s for s in r)


def test_tensor_bias_and_window_rules_of_the_operators():
    """Which operator takes an additive tensor bias or a window, judged from the records alone (no GPU)."""
    from xformers_b200.ops.fmha import attn_bias as ab

    only_device = lambda reasons: [r for r in reasons if "device=" not in r]
    q = torch.randn(2, 4, 2, 128, dtype=torch.bfloat16)
    k = torch.randn(2, 40, 2, 128, dtype=torch.bfloat16)
    bias = torch.randn(2, 2, 4, 40, dtype=torch.bfloat16)
    # prefill: the automatic choice, the persistent tcgen05 kernel and the mma.sync kernel take it; the other tcgen05 kernel does not
    for op in (fmha.b200.FwOp, fmha.b200.FwOp_Tcgen05_Persistent, fmha.b200.FwOp_Generic):
        assert not only_device(op.not_supported_reasons(fmha.Inputs(q, k, k, bias))), op.NAME
    assert any("additive biases" in r for r in fmha.b200.FwOp_Tcgen05_M256.not_supported_reasons(fmha.Inputs(q, k, k, bias)))
    # decode: 16-bit caches only, shape and stride rules
    S = fmha.b200_splitk.FwOp
    assert not only_device(S.not_supported_reasons(fmha.Inputs(q, k, k, bias)))
    assert any("expected [B, (G,) H, Mq, Mkv]" in r for r in S.not_supported_reasons(fmha.Inputs(q, k, k, bias[..., :39])))
    assert any("unit stride" in r for r in S.not_supported_reasons(fmha.Inputs(q, k, k, torch.randn(2, 2, 4, 80, dtype=torch.bfloat16)[..., ::2])))
    ki = torch.zeros(2, 40, 2, 17, dtype=torch.int32)
    assert any("16-bit cache" in r for r in S.not_supported_reasons(fmha.Inputs(q, ki, ki, bias)))
    # windows with several queries per sequence: the decode operator on 16-bit caches, not on quantised ones
    q1 = torch.randn(1, 2 * 3, 2, 128, dtype=torch.bfloat16)
    k1 = torch.randn(1, 2 * 64, 2, 128, dtype=torch.bfloat16)
    local = ab.BlockDiagonalCausalLocalAttentionPaddedKeysMask.from_seqlens_local([3, 3], 64, [10, 20], 4)
    assert not only_device(S.not_supported_reasons(fmha.Inputs(q1, k1, k1, local)))
    k1i = torch.zeros(1, 2 * 64, 2, 17, dtype=torch.int32)
    assert any("one query per sequence" in r for r in S.not_supported_reasons(fmha.Inputs(q1, k1i, k1i, local)))


def _first(q, kv):
    return fmha._dispatch_fw_priority_list(fmha.Inputs(q, kv, kv), False)[0]


def test_dispatch_rules_bmhk():
    # tests/test_mem_eff_attention.py:2189-2211
    S = fmha.b200_splitk.FwOp
    assert not issubclass(_first(torch.empty([1, 8, 1, 128]), torch.empty([1, 2048, 1, 128])), S)
    assert issubclass(_first(torch.empty([1, 8, 32, 128]), torch.empty([1, 2048, 1, 128]).expand(-1, -1, 32, -1)), S)
    assert not issubclass(_first(torch.empty([1, 8, 32, 128]), torch.empty([1, 2048, 32, 128])), S)
    assert not issubclass(_first(torch.empty([1, 128, 32, 128]), torch.empty([1, 2048, 1, 128]).expand(-1, -1, 32, -1)), S)
    assert not issubclass(_first(torch.empty([128, 8, 32, 128]), torch.empty([128, 2048, 1, 128]).expand(-1, -1, 32, -1)), S)


def test_dispatch_rules_bmghk():
    # tests/test_mem_eff_attention.py:2214-2236
    S = fmha.b200_splitk.FwOp
    assert not issubclass(_first(torch.empty([1, 8, 1, 1, 128]), torch.empty([1, 2048, 1, 1, 128])), S)
    assert issubclass(_first(torch.empty([1, 8, 1, 32, 128]), torch.empty([1, 2048, 1, 1, 128]).expand(-1, -1, -1, 32, -1)), S)
    assert issubclass(_first(torch.empty([1, 8, 4, 32, 128]), torch.empty([1, 2048, 4, 1, 128]).expand(-1, -1, -1, 32, -1)), S)
    assert not issubclass(_first(torch.empty([1, 8, 1, 32, 128]), torch.empty([1, 2048, 1, 32, 128])), S)
    assert not issubclass(_first(torch.empty([1, 128, 1, 32, 128]), torch.empty([1, 2048, 1, 1, 128]).expand(-1, -1, -1, 32, -1)), S)
    assert not issubclass(_first(torch.empty([128, 8, 1, 32, 128]), torch.empty([128, 2048, 1, 1, 128]).expand(-1, -1, -1, 32, -1)), S)


def test_dispatch_raises_not_implemented_with_reasons():
    q = torch.randn(1, 8, 2, 64)
    inp = fmha.Inputs(q, q, q)
    with pytest.raises(NotImplementedError) as e:
        fmha._dispatch_fw(inp, False)
    assert "is not supported because" in str(e.value)


def test_split_k_heuristic_is_static():
    f = fmha.b200_splitk.FwOp.get_split_k
    # BASELINE decode config: 64 sequences, 32768-token bound, 8 KV heads, bf16 rows of 256 B
    s = f(64, 32768, 8, 256)
    assert 16 <= s <= 256 and f(64, 32768, 8, 256) == s
    assert f(1, 128, 1, 256) == 1
    assert fmha.b200_splitk.FwOp_S8.get_split_k(64, 32768, 8, 256) == 8
