"""merge_attentions on the GPU against the oracle (tests/test_fmha_merge_attentions.py)."""

import math

import pytest
import torch

import oracle
from gpu_utils import gpu, require_cuda
from xformers_b200.ops import fmha


@gpu
@pytest.mark.parametrize("bmghk", [False, True])
@pytest.mark.parametrize("stacked", [True, False])
def test_merge_against_ref(bmghk, stacked):
    # tests/test_fmha_merge_attentions.py:488-510: split_k=16, B=12, M=137, H=8, D=128, fp32, 1e-4
    require_cuda()
    torch.manual_seed(0)
    S, B, M, G, H, D = 16, 12, 137, 2 if bmghk else 1, 8, 128
    attn = torch.randn(S, B, M, G, H, D, device="cuda")
    lse = torch.randn(S, B, G, H, M, device="cuda")
    if not bmghk:
        attn, lse = attn[:, :, :, 0], lse[:, :, 0]
    ro, rl = oracle.merge_attentions_ref(attn, lse)
    if stacked:
        out, lo = fmha.merge_attentions(attn, lse)
    else:
        out, lo = fmha.merge_attentions(list(attn.unbind(0)), list(lse.unbind(0)))
    torch.testing.assert_close(out.cpu(), ro, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(lo.cpu(), rl, rtol=1e-4, atol=1e-4)
    out2, _ = fmha.merge_attentions(attn, lse, write_lse=False)
    assert _ is None and torch.equal(out, out2), "merge must be bit-reproducible"


@gpu
@pytest.mark.parametrize("G,H", [(1, 11), (7, 1), (1, 1), (7, 11), (None, 11)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_merge_with_self(G, H, dtype):
    # tests/test_fmha_merge_attentions.py:80-138: same output, lse + ln 2
    require_cuda()
    torch.manual_seed(1)
    B, M, D = 13, 3, 128
    shape_a = (B, M, H, D) if G is None else (B, M, G, H, D)
    shape_l = (B, H, M) if G is None else (B, G, H, M)
    a = torch.randn(shape_a, device="cuda").to(dtype)
    l = torch.randn(shape_l, device="cuda")
    out, lo = fmha.merge_attentions([a, a], [l, l], output_dtype=torch.float32)
    assert out.dtype == torch.float32
    torch.testing.assert_close(out, a.float(), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(lo, l + math.log(2), rtol=1e-5, atol=1e-5)


@gpu
def test_merge_empty_partials_and_odd_dims():
    require_cuda()
    torch.manual_seed(2)
    S, B, M, H, D = 5, 2, 9, 3, 72  # D not a multiple of 128; rows still 16-B aligned
    attn = torch.randn(S, B, M, H, D, device="cuda")
    lse = torch.randn(S, B, H, M, device="cuda")
    attn[1] = float("nan")
    lse[1] = float("-inf")
    lse[:, 0, 0, 0] = float("-inf")  # a row that no partial covers
    ro, rl = oracle.merge_attentions_ref(attn, lse)
    out, lo = fmha.merge_attentions(attn, lse)
    assert not out.isnan().any()
    torch.testing.assert_close(out.cpu(), ro, rtol=1e-4, atol=1e-4)
    assert torch.isneginf(lo[0, 0, 0]) and (out[0, 0, 0] == 0).all()
    torch.testing.assert_close(lo.cpu(), rl, rtol=1e-4, atol=1e-4)
    # unaligned head dim -> scalar path
    a3 = torch.randn(3, 1, 4, 2, 13, device="cuda")
    l3 = torch.randn(3, 1, 2, 4, device="cuda")
    o3, ll3 = fmha.merge_attentions(a3, l3, output_dtype=torch.bfloat16)
    r3, rl3 = oracle.merge_attentions_ref(a3, l3)
    torch.testing.assert_close(o3.float().cpu(), r3, rtol=2e-2, atol=2e-2)
    # more separate partials than the kernel takes by pointer -> stacked internally
    many_a = [torch.randn(1, 2, 2, 16, device="cuda") for _ in range(40)]
    many_l = [torch.randn(1, 2, 2, device="cuda") for _ in range(40)]
    o, l = fmha.merge_attentions(many_a, many_l)
    r, rl = oracle.merge_attentions_ref(torch.stack(many_a), torch.stack(many_l))
    torch.testing.assert_close(o.cpu(), r, rtol=1e-4, atol=1e-4)
    with pytest.raises(ValueError):
        fmha.merge_attentions(attn.cpu(), lse.cpu())
    with pytest.raises(ValueError):
        fmha.merge_attentions(attn, lse[:, :, :, :4])
