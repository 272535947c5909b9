"""The rope oracle against independent statements of the same definition:
complex multiplication by e^{i * position * freq} (the published RoPE formula,
as tests/test_rope_padded.py:88-100 does it), closed-form angles, and the
cache-row bookkeeping of the padded-keys layout."""

import math

import pytest
import torch

import oracle
from oracle.rope import rope_frequencies, rope_rotate


def _complex_rope(x, positions, freqs, adjacents, linear_scale=1.0):
    ang = torch.outer(positions.double() / linear_scale, freqs)
    cis = torch.polar(torch.ones_like(ang), ang)
    for _ in range(x.ndim - 2):
        cis = cis[:, None]
    if adjacents:
        xc = torch.view_as_complex(x.double().unflatten(-1, (-1, 2)).contiguous())
        return torch.view_as_real(xc * cis).flatten(-2)
    xc = torch.view_as_complex(x.double().unflatten(-1, (2, -1)).transpose(-1, -2).contiguous())
    return torch.view_as_real(xc * cis).transpose(-1, -2).flatten(-2)


@pytest.mark.parametrize("adjacents", [True, False])
@pytest.mark.parametrize("dim", [2, 100, 128])
def test_rotation_is_complex_multiplication(adjacents, dim):
    g = torch.Generator().manual_seed(dim)
    x = torch.randn(7, 3, dim, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 1, 5, 1000, 17, 99999, 3])
    freqs = rope_frequencies(dim)
    got = rope_rotate(x, pos, freqs, adjacents=adjacents, linear_scale=2.0)
    want = _complex_rope(x, pos, freqs, adjacents, linear_scale=2.0)
    torch.testing.assert_close(got, want, atol=1e-12, rtol=1e-12)
    # position 0 is the identity; a rotation keeps the norm of every pair
    torch.testing.assert_close(got[0], x[0])
    torch.testing.assert_close(got.square().sum(-1), x.square().sum(-1))


def test_known_angles():
    # dim 2: one pair, frequency theta^0 = 1, angle = position
    x = torch.tensor([[[1.0, 0.0]]], dtype=torch.float64)
    out = rope_rotate(x, torch.tensor([1]), rope_frequencies(2))
    torch.testing.assert_close(out[0, 0], torch.tensor([math.cos(1.0), math.sin(1.0)], dtype=torch.float64))
    # dim 4, theta 10000: frequencies 1 and 1/100
    f = rope_frequencies(4)
    torch.testing.assert_close(f, torch.tensor([1.0, 0.01], dtype=torch.float64))


def test_dynamic_scaling_bands():
    # tests/test_rope_padded.py:24-50: long wavelengths are divided by the factor, short ones kept, the middle band interpolated
    dim, old, factor, lo_f, hi_f = 128, 8192.0, 16.0, 1.0, 32.0
    base = rope_frequencies(dim, theta=500000.0)
    scaled = rope_frequencies(dim, theta=500000.0, use_dynamic_scaling=True, dynamic_old_context_len=old,
                              dynamic_scale_factor=factor, dynamic_low_freq_factor=lo_f, dynamic_high_freq_factor=hi_f)
    wavelen = 2 * math.pi / base
    low, high = wavelen > old / lo_f, wavelen <= old / hi_f
    assert low.any() and high.any() and (~low & ~high).any()
    torch.testing.assert_close(scaled[low], base[low] / factor)
    torch.testing.assert_close(scaled[high], base[high])
    mid = ~low & ~high
    assert ((scaled[mid] > base[mid] / factor) & (scaled[mid] < base[mid])).all()
    assert (scaled[:-1] >= scaled[1:]).all()  # still monotone


def test_cache_rows_and_positions():
    # three sequences in slots of 16 rows; the queries are the last keys (xformers/ops/_triton/rope_padded_kernels.py:103-121)
    q_seqlen, kv_seqlen, starts = [2, 1, 3], [5, 16, 3], [0, 16, 32]
    G, Hq, Hkv, D = 1, 4, 2, 8
    g = torch.Generator().manual_seed(0)
    M = sum(q_seqlen)
    xq, xk, xv = (torch.randn(1, M, h, D, generator=g) for h in (Hq, Hkv, Hkv))
    ck, cv = torch.randn(1, 48, Hkv, D, generator=g), torch.randn(1, 48, Hkv, D, generator=g)
    oq, nk, nv = oracle.rope_padded_ref(xq, xk, xv, ck, cv, q_seqlen, starts, kv_seqlen)
    rows = [3, 4, 31, 32, 33, 34]
    pos = torch.tensor([3, 4, 15, 0, 1, 2])
    untouched = [r for r in range(48) if r not in rows]
    assert torch.equal(nk[0, untouched], ck[0, untouched]) and torch.equal(nv[0, untouched], cv[0, untouched])
    assert torch.equal(nv[0, rows], xv[0])
    f = rope_frequencies(D)
    torch.testing.assert_close(nk[0, rows], rope_rotate(xk[0], pos, f))
    torch.testing.assert_close(oq[0], rope_rotate(xq[0], pos, f))
    # first_seqpos shifts the positions of a sequence, explicit seqpos replaces them; the rows stay
    oq2, nk2, _ = oracle.rope_padded_ref(xq, xk, xv, ck, cv, q_seqlen, starts, kv_seqlen, first_seqpos=[10, 0, 7])
    torch.testing.assert_close(oq2[0], rope_rotate(xq[0], pos + torch.tensor([10, 10, 0, 7, 7, 7]), f))
    assert torch.equal(nk2[0, untouched], ck[0, untouched])
    oq3, _, _ = oracle.rope_padded_ref(xq, xk, xv, ck, cv, q_seqlen, starts, kv_seqlen, seqpos=[9, 8, 7, 6, 5, 4])
    torch.testing.assert_close(oq3[0], rope_rotate(xq[0], torch.tensor([9, 8, 7, 6, 5, 4]), f))


def test_paged_rows():
    # key t of sequence b -> row block_tables[b][t // page] * page + t % page
    q_seqlen, kv_seqlen, page = [3, 1], [6, 9], 4
    tables = [[5, 2, 0], [1, 3, 4]]
    g = torch.Generator().manual_seed(1)
    xq, xk, xv = (torch.randn(1, 4, 2, 8, generator=g) for _ in range(3))
    ck, cv = torch.randn(1, 24, 2, 8, generator=g), torch.randn(1, 24, 2, 8, generator=g)
    oq, nk, nv = oracle.rope_padded_ref(xq, xk, xv, ck, cv, q_seqlen, [0, 0], kv_seqlen, block_tables=tables, page_size=page)
    rows = [5 * 4 + 3, 2 * 4 + 0, 2 * 4 + 1, 4 * 4 + 0]  # keys 3, 4, 5 of sequence 0; key 8 of sequence 1
    pos = torch.tensor([3, 4, 5, 8])
    f = rope_frequencies(8)
    torch.testing.assert_close(nk[0, rows], rope_rotate(xk[0], pos, f))
    assert torch.equal(nv[0, rows], xv[0])
    untouched = [r for r in range(24) if r not in rows]
    assert torch.equal(nk[0, untouched], ck[0, untouched]) and torch.equal(nv[0, untouched], cv[0, untouched])
    torch.testing.assert_close(oq[0], rope_rotate(xq[0], pos, f))
