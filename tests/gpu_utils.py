"""Helpers shared by the GPU parity tests."""

import pytest
import torch

import oracle

gpu = pytest.mark.gpu

# Tolerances of the north-star statement: O max-abs error, LSE max-abs error.
ATOL_O = {torch.bfloat16: 2e-2, torch.float16: 4e-3}
ATOL_LSE = 1e-3


def require_cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def assert_o_lse(out, lse, ref_out, ref_lse, dtype, what="", o_scale=1.0):
    assert not out.isnan().any(), f"{what}: NaN in output"
    err = (out.float().cpu() - ref_out).abs().max().item() if out.numel() else 0.0
    assert err <= ATOL_O[dtype] * o_scale, f"{what}: O max-abs error {err:.3e} > {ATOL_O[dtype] * o_scale:.1e}"
    if lse is not None:
        l, r = lse.float().cpu(), ref_lse
        both_inf = torch.isneginf(l) & torch.isneginf(r)
        diff = torch.where(both_inf, torch.zeros_like(l), (l - r).abs())
        lerr = diff.max().item() if diff.numel() else 0.0
        assert lerr <= ATOL_LSE, f"{what}: LSE max-abs error {lerr:.3e} > {ATOL_LSE:.0e}"


def rand_qkv(B, Mq, Mkv, G, H, D, dtype, seed, gqa=True, scale=1.0, device="cuda"):
    """BMGHK tensors; K/V shared by the H heads of a group when ``gqa``."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = (torch.randn(B, Mq, G, H, D, generator=g) * scale).to(dtype).to(device)
    hk = 1 if gqa else H
    k = (torch.randn(B, Mkv, G, hk, D, generator=g) * scale).to(dtype).to(device)
    v = (torch.randn(B, Mkv, G, hk, D, generator=g) * scale).to(dtype).to(device)
    if gqa:
        k = k.expand(B, Mkv, G, H, D)
        v = v.expand(B, Mkv, G, H, D)
    return q, k, v


def ref(q, k, v, bias=None, scale=None):
    cpu_bias = bias.to("cpu") if hasattr(bias, "to") else bias
    return oracle.ref_attention_with_lse(q.float().cpu(), k.float().cpu(), v.float().cpu(), cpu_bias, scale)
