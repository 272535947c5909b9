"""Generates tests/golden/cfg1_seed0.npz: O and LSE of the CPU-runnable
baseline configuration (B=2, Mq=Mkv=128, H=4, D=64, fp32, BMHK,
LowerTriangularMask, N(0,1) inputs from seed 0, scale 1/sqrt(D)).

The reference's own ``ref_attention`` cannot be imported (it lives in the
un-vendored ``mslk`` package), so the vectors come from two independent
implementations that must agree before the file is written: the oracle
(``oracle.ref_attention_with_lse``) and PyTorch's
``scaled_dot_product_attention`` in float64.  Only a checksum-sized slice of the
inputs is stored; the inputs are regenerated from the seed.

    python tests/golden/make_cfg1_golden.py
"""

import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import oracle  # noqa: E402


def cfg1_inputs():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(2, 128, 4, 64, generator=g)
    k = torch.randn(2, 128, 4, 64, generator=g)
    v = torch.randn(2, 128, 4, 64, generator=g)
    return q, k, v


def main():
    q, k, v = cfg1_inputs()
    out, lse = oracle.ref_attention_with_lse(q, k, v, oracle.causal_mask(128, 128), scale=64**-0.5)
    qd, kd, vd = (t.transpose(1, 2).double() for t in (q, k, v))
    sdpa = torch.nn.functional.scaled_dot_product_attention(qd, kd, vd, is_causal=True).transpose(1, 2)
    s = (qd * 64**-0.5) @ kd.transpose(-1, -2)
    s = s.masked_fill(torch.triu(torch.ones(128, 128, dtype=torch.bool), 1), float("-inf"))
    lse64 = torch.logsumexp(s, -1)
    assert (out.double() - sdpa).abs().max() < 1e-5
    assert (lse.double() - lse64).abs().max() < 1e-5
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cfg1_seed0.npz")
    np.savez_compressed(
        path,
        out=sdpa.float().numpy(),
        lse=lse64.float().numpy(),
        q_head=q[0, :4, 0, :8].numpy(),  # guards against a changed RNG stream
    )
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
