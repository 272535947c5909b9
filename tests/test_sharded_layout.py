"""Host-side arithmetic of the key sharding and of the query stripes.

``zigzag_bounds`` gives rank r the chunks r and 2R-1-r of 2R (equal causal work
over the whole sequence); ``mirror_stripes`` pairs a block of query rows with its
mirror image so that the work is also equal in every stripe (a row at x and the
row at S-x see, of a mirror pair of key ranges, the length of one range).
"""

import pytest

from xformers_b200.ops.fmha.sharded import shard_bounds, zigzag_bounds


def _visible(bounds, row):
    """Keys of the ranges ``bounds`` that the causal query ``row`` sees."""
    return sum(max(0, min(hi, row + 1) - lo) for lo, hi in bounds)


@pytest.mark.parametrize("S,R", [(4096, 2), (4096, 4), (8192, 8)])
def test_zigzag_ranges_cover_the_keys_and_balance_the_causal_work(S, R):
    ranges = [zigzag_bounds(S, R, r) for r in range(R)]
    covered = sorted(x for b in ranges for x in b)
    assert covered[0][0] == 0 and covered[-1][1] == S
    assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
    work = [sum(_visible(b, x) for x in range(0, S, 7)) for b in ranges]
    assert max(work) - min(work) <= 0.01 * max(work)
    # contiguous shards are not balanced: the last rank sees the most
    contiguous = [sum(_visible([shard_bounds(S, R, r)], x) for x in range(0, S, 7)) for r in range(R)]
    assert contiguous[0] > 2 * contiguous[-1]


@pytest.mark.parametrize("S,R,stripes", [(4096, 2, 4), (4096, 4, 8), (8192, 8, 8)])
def test_mirrored_stripes_give_every_rank_the_same_work_in_every_stripe(S, R, stripes):
    w = S // (2 * stripes)
    for s in range(stripes):
        rows = list(range(s * w, (s + 1) * w)) + list(range(S - (s + 1) * w, S - s * w))
        work = [sum(_visible(zigzag_bounds(S, R, r), x) for x in rows) for r in range(R)]
        assert max(work) - min(work) <= 2 * w, (s, work)
    # plain stripes of consecutive rows are not: the first stripe is the first rank's alone
    first = [sum(_visible(zigzag_bounds(S, R, r), x) for x in range(0, 2 * w)) for r in range(R)]
    assert first[0] > 0 and first[-1] == 0
