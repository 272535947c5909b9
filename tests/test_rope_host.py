"""Host-side validation of rope_padded: the errors the reference raises for
malformed inputs (xformers/ops/rope_padded.py:97-233), checked without a GPU."""

import pytest
import torch

from xformers_b200.ops import fmha, rope_padded


def _inputs(M=4, H=4, Hkv=2, D=8, rows=32, groups=None):
    mid = () if groups is None else (groups,)
    xq = torch.zeros((1, M) + mid + (H, D))
    xk = torch.zeros((1, M) + mid + (Hkv, D))
    xv = torch.zeros((1, M) + mid + (Hkv, D))
    ck = torch.zeros((1, rows) + mid + (Hkv, D))
    cv = torch.zeros((1, rows) + mid + (Hkv, D))
    bias = fmha.attn_bias.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=[3, 1], kv_padding=16, kv_seqlen=[5, 9])
    return xq, xk, xv, ck, cv, bias


def test_shape_errors():
    xq, xk, xv, ck, cv, bias = _inputs()
    with pytest.raises(ValueError, match="Unexpected xq dimension"):
        rope_padded(xq[0], xk, xv, ck, cv, bias)
    with pytest.raises(ValueError, match="unexpected k shape"):
        rope_padded(xq, xk[:, :3], xv, ck, cv, bias)
    with pytest.raises(ValueError, match="unexpected v shape"):
        rope_padded(xq, xk, xv[..., :4], ck, cv, bias)
    with pytest.raises(ValueError, match="unexpected cache_k shape"):
        rope_padded(xq, xk, xv, ck[:, :31], cv, bias)
    with pytest.raises(ValueError, match="unexpected cache_v shape"):
        rope_padded(xq, xk, xv, ck, cv[:, :, :1], bias)
    with pytest.raises(ValueError, match="Each q head must be contiguous"):
        rope_padded(torch.zeros(1, 4, 4, 16)[..., ::2], xk, xv, ck, cv, bias)
    with pytest.raises(ValueError, match="Unexpected shape of out_q"):
        with torch.no_grad():
            rope_padded(xq, xk, xv, ck, cv, bias, out_q=torch.zeros(1, 4, 4, 4))


def test_batch_dimension_must_be_one():
    xq, xk, xv, ck, cv, bias = _inputs()
    with pytest.raises(ValueError, match="batch size dimension to be 1"):
        rope_padded(xq.expand(2, -1, -1, -1), xk, xv, ck, cv, bias)


def test_position_errors():
    xq, xk, xv, ck, cv, bias = _inputs()
    with pytest.raises(ValueError, match="may not both be provided"):
        rope_padded(xq, xk, xv, ck, cv, bias, first_seqpos=torch.zeros(2, dtype=torch.long), seqpos=torch.zeros(4, dtype=torch.long))
    with pytest.raises(ValueError, match=r"first_seqpos.shape \(3,\) but \(2,\) expected"):
        rope_padded(xq, xk, xv, ck, cv, bias, first_seqpos=torch.zeros(3, dtype=torch.long))
    with pytest.raises(ValueError, match=r"seqpos.shape \(5,\) but \(4,\) expected"):
        rope_padded(xq, xk, xv, ck, cv, bias, seqpos=torch.zeros(5, dtype=torch.long))


def test_gradients_and_out_q_in_grad_mode():
    xq, xk, xv, ck, cv, bias = _inputs()
    with pytest.raises(ValueError, match="Gradients not supported"):
        rope_padded(xq.requires_grad_(), xk, xv, ck, cv, bias)
    with pytest.raises(ValueError, match="Gradients not supported"):
        rope_padded(xq.detach(), xk, xv, ck, cv, bias, out_q=torch.zeros(1, 4, 4, 8))


def test_no_cpu_path():
    xq, xk, xv, ck, cv, bias = _inputs(groups=2)
    with pytest.raises(ValueError, match="needs CUDA tensors"):
        rope_padded(xq, xk, xv, ck, cv, bias)
