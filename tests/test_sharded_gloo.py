"""Host-side logic of the key-sharded long-context path with two CPU ranks
(gloo): shard bounds, offsets, gather order and the merge must reproduce the
un-sharded result.  The kernels are replaced by the oracle here; the GPU
version of the same check is tests/test_gpu_prefill.py::test_sharded_keys_merge_to_full_causal."""

import os
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cpu_partial(q, k, v, causal, kv_offset, scale, partial_dtype):
    import oracle

    bias = oracle.causal_mask(q.shape[1], k.shape[1], kv_offset=kv_offset) if causal else None
    return oracle.ref_attention_with_lse(q, k, v, bias, scale)


def _cpu_merge(outs, lses, out_dtype):
    import oracle

    if isinstance(outs, (list, tuple)):
        outs, lses = torch.stack(outs), torch.stack(lses)
    return oracle.merge_attentions_ref(outs, lses)


def _worker(rank, world, init_file, fail_rank, result_file, zigzag=False):
    sys.path.insert(0, ROOT)
    import oracle
    from xformers_b200.ops.fmha.sharded import shard_bounds, sharded_kv_attention_forward, zigzag_bounds

    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        S, G, H, D = 300, 2, 2, 16
        q = torch.randn(1, S, G, H, D, generator=g)
        k = torch.randn(1, S, G, 1, D, generator=g).expand(-1, -1, -1, H, -1)
        v = torch.randn(1, S, G, 1, D, generator=g).expand(-1, -1, -1, H, -1)
        lo, hi = shard_bounds(S, world, rank)
        if rank == fail_rank:
            raise RuntimeError("injected host-side failure before the collective")
        if zigzag:
            spans = zigzag_bounds(S, world, rank)
            out, lse = sharded_kv_attention_forward(
                q, [k[:, a:b] for a, b in spans], [v[:, a:b] for a, b in spans], kv_offset=[a for a, _ in spans],
                causal=True, partial_fn=_cpu_partial, merge_fn=_cpu_merge,
            )
            # both exchanges give the same answer
            out_g, lse_g = sharded_kv_attention_forward(
                q, [k[:, a:b] for a, b in spans], [v[:, a:b] for a, b in spans], kv_offset=[a for a, _ in spans],
                causal=True, partial_fn=_cpu_partial, merge_fn=_cpu_merge, exchange="all_gather",
            )
            assert (out - out_g).abs().max() < 1e-5 and (lse - lse_g).abs().max() < 1e-5
            # query stripes, plain and as mirrored row blocks: the same rows end up in the same places
            for extra in (dict(stripes=3), dict(stripes=3, mirror_stripes=True), dict(stripes=5, mirror_stripes=True)):
                out_s, lse_s = sharded_kv_attention_forward(
                    q, [k[:, a:b] for a, b in spans], [v[:, a:b] for a, b in spans], kv_offset=[a for a, _ in spans],
                    causal=True, partial_fn=_cpu_partial, merge_fn=_cpu_merge, **extra,
                )
                assert (out - out_s).abs().max() < 1e-5 and (lse - lse_s).abs().max() < 1e-5, extra
        else:
            out, lse = sharded_kv_attention_forward(
                q, k[:, lo:hi], v[:, lo:hi], kv_offset=lo, causal=True, partial_fn=_cpu_partial, merge_fn=_cpu_merge
            )
        ro, rl = oracle.ref_attention_with_lse(q, k, v, oracle.causal_mask(S, S))
        ok = bool((out - ro).abs().max() < 1e-5 and (lse - rl).abs().max() < 1e-5)
        with open(f"{result_file}.{rank}", "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


def test_shard_bounds_cover_the_sequence():
    from xformers_b200.ops.fmha.sharded import shard_bounds

    for total in (1, 127, 128, 300, 131072):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b
            assert all(a % 128 == 0 for a, _ in spans if a < total)


def test_zigzag_bounds_cover_the_sequence_and_balance_causal_work():
    from xformers_b200.ops.fmha.sharded import zigzag_bounds

    for total in (1, 127, 300, 1024, 131072):
        for world in (1, 2, 3, 4, 8):
            spans = sorted(sp for r in range(world) for sp in zigzag_bounds(total, world, r))
            assert spans[0][0] == 0 and max(b for _, b in spans) == total
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and a <= b  # the 2 * world chunks tile the sequence in order
    # visible (query, key) pairs per rank under a causal mask: equal up to the chunk granularity
    total, world = 131072, 8
    work = [sum((total - a) * (b - a) - (b - a) * (b - a - 1) // 2 for a, b in zigzag_bounds(total, world, r)) for r in range(world)]
    assert max(work) / min(work) < 1.001


def test_two_rank_zigzag_shards_match_full():
    with tempfile.TemporaryDirectory() as tmp:
        init, res = os.path.join(tmp, "init"), os.path.join(tmp, "res")
        mp.spawn(_worker, args=(2, init, -1, res, True), nprocs=2, join=True)
        assert [open(f"{res}.{r}").read() for r in range(2)] == ["ok", "ok"]


def test_two_rank_gather_and_merge_matches_full():
    with tempfile.TemporaryDirectory() as tmp:
        init, res = os.path.join(tmp, "init"), os.path.join(tmp, "res")
        mp.spawn(_worker, args=(2, init, -1, res), nprocs=2, join=True)
        assert [open(f"{res}.{r}").read() for r in range(2)] == ["ok", "ok"]


def test_rank_failing_on_the_host_is_reported():
    """A rank that raises before the collective must surface as an error of the
    job (the other rank's all-gather ends with an error or is torn down), never
    as a silent wrong answer."""
    with tempfile.TemporaryDirectory() as tmp:
        init, res = os.path.join(tmp, "init"), os.path.join(tmp, "res")
        with pytest.raises(Exception):
            mp.spawn(_worker, args=(2, init, 1, res), nprocs=2, join=True)
        assert not os.path.exists(f"{res}.1")
