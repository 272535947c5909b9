"""Long-context attention with the key/value sequence sharded across ranks.

The reference has no ring or context-parallel attention; its long-context
primitive is algebraic: attention over parts of the keys
(``memory_efficient_attention_partial``) followed by ``merge_attentions``
(tests/test_fmha_merge_attentions.py:234-363).  Here the parts live on
different GPUs of one NVSwitch box: rank r holds one or two ranges of the keys,
runs the prefill kernel over the queries against them with the causal diagonal
shifted by the ranges' positions, and the per-rank ``(O_r, LSE_r)`` are
exchanged over NCCL/NVLink and combined by the same LSE-merge kernel.  Query
rows that lie before a range see none of its keys and arrive with ``LSE =
-inf`` (weight 0).

For balanced causal work a rank holds the two key ranges of
:func:`zigzag_bounds`; they are laid back to back once (keys and values are
small next to the partial outputs) and one kernel launch covers both, so no
local merge is needed.  The queries are processed in stripes: the exchange of
a stripe -- all-to-all of the partials by query slice, LSE merge of the slice,
all-gather of the merged slices -- runs on a side stream while the next stripe
is computed.  Remote data is always landed in local memory by NCCL before a
kernel reads it.
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from .attn_bias import LowerTriangularMask
from .common import Inputs


def shard_bounds(total: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous, 128-aligned shards of ``total`` keys (the last may be short)."""
    per = -(-total // world_size)
    per = -(-per // 128) * 128
    lo = min(total, rank * per)
    return lo, min(total, lo + per)


def zigzag_bounds(total: int, world_size: int, rank: int) -> List[Tuple[int, int]]:
    """Two 128-aligned key ranges per rank: chunks ``rank`` and ``2 * world_size -
    1 - rank`` of ``2 * world_size``.  Under a causal mask every query sees all of
    an early chunk and little of a late one; pairing them gives every rank the
    same number of visible (query, key) pairs, which contiguous shards do not
    (their slowest rank does about twice the average)."""
    per = -(-total // (2 * world_size))
    per = -(-per // 128) * 128

    def span(c: int) -> Tuple[int, int]:
        lo = min(total, c * per)
        return lo, min(total, lo + per)

    return [span(rank), span(2 * world_size - 1 - rank)]


def _partial_on_gpu(q, k, v, causal: bool, kv_offset: int, scale, partial_dtype, kv_split: int = 0, kv_offset2: int = 0, sm_margin: int = 0):
    from . import b200

    inp = Inputs(q, k, v, LowerTriangularMask() if causal else None, scale=scale, output_dtype=partial_dtype, is_partial=True)
    inp.validate_inputs()
    reasons = b200.FwOp.not_supported_reasons(inp)
    if reasons:
        raise ValueError("sharded attention: " + "; ".join(reasons))
    out, ctx = b200.FwOp._apply(inp, want_lse=True, kv_offset=kv_offset if causal else 0, kv_split=kv_split, kv_offset2=kv_offset2, sm_margin=sm_margin)
    return out, ctx.lse


def _merge_on_gpu(outs, lses, out_dtype):
    from .merge import merge_attentions

    return merge_attentions(outs, lses, write_lse=True, output_dtype=out_dtype)


def _cat_keeping_broadcast(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``torch.cat`` along the sequence axis that keeps a broadcast head axis (stride 0) broadcast."""
    if a.ndim == 5 and a.stride(3) == 0 and b.stride(3) == 0:
        return torch.cat([a[:, :, :, :1], b[:, :, :, :1]], dim=1).expand(-1, -1, -1, a.shape[3], -1)
    if a.ndim == 4 and a.stride(2) == 0 and b.stride(2) == 0:
        return torch.cat([a[:, :, :1], b[:, :, :1]], dim=1).expand(-1, -1, a.shape[2], -1)
    return torch.cat([a, b], dim=1)


def exchange_group(ranks=None, max_ctas: int = 8):
    """A process group over ``ranks`` (default: all) for the striped exchange: its NCCL kernels use at most
    ``max_ctas`` CTAs, which fit the SMs the attention kernel leaves free (``sm_margin``), and run on a
    high-priority stream."""
    opts = dist.ProcessGroupNCCL.Options()
    opts.is_high_priority_stream = True
    opts.config.max_ctas = int(max_ctas)
    opts.config.min_ctas = 1
    return dist.new_group(ranks=ranks, backend="nccl", pg_options=opts)


_COMM_STREAMS: Dict[int, "torch.cuda.Stream"] = {}


def _comm_stream(device: torch.device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _COMM_STREAMS:
        _COMM_STREAMS[idx] = torch.cuda.Stream(device=device, priority=-1)
    return _COMM_STREAMS[idx]


def sharded_kv_attention_forward(
    query: torch.Tensor,
    key_shard: Union[torch.Tensor, Sequence[torch.Tensor]],
    value_shard: Union[torch.Tensor, Sequence[torch.Tensor]],
    *,
    kv_offset: Union[int, Sequence[int]],
    causal: bool = True,
    scale: Optional[float] = None,
    group: Optional[dist.ProcessGroup] = None,
    partial_dtype: Optional[torch.dtype] = None,
    partial_fn: Callable = _partial_on_gpu,
    merge_fn: Callable = _merge_on_gpu,
    exchange: str = "all_to_all",
    stripes: int = 1,
    sm_margin: int = 0,
    last_group: Optional[dist.ProcessGroup] = None,
    mirror_stripes: bool = False,
    timings: Optional[dict] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Every rank passes the full ``query`` ``[B, Mq, (G,) H, D]`` and its own
    key/value shard ``[B, len_r, (G,) H, D]`` starting at global key index
    ``kv_offset``.  Returns the full ``(out, lse)`` on every rank.  Several key
    ranges per rank are passed as sequences of shards and offsets (empty ranges
    are skipped).

    ``exchange="all_to_all"`` (when the queries of a stripe divide by the number
    of ranks): every rank receives the partials of its slice of the queries,
    merges them and the merged slices are all-gathered; ``"all_gather"``: every
    rank receives every partial and merges all queries itself.  ``stripes`` cuts
    the queries into that many stripes whose exchanges overlap the attention of
    the following stripe (CUDA tensors, all-to-all exchange).  ``timings``, a
    dict, receives CUDA events (``start``, ``attention_done``, ``done``) for a
    break-down; if it holds a list under ``"stripes"``, one list of events per
    unit of rows is appended to it (start, partials laid out, all-to-all done,
    merge done, all-gather done).

    ``partial_fn`` / ``merge_fn`` exist so that the exchange logic can be
    exercised with CPU stand-ins under the gloo backend.

    The attention kernel is persistent: it holds every SM it is given until it
    ends, and the next stripe's kernel is queued right behind it, so a collective
    of another stream would find no SM before the last stripe is done.  With
    stripes, pass ``sm_margin`` (SMs the attention leaves free) and a ``group``
    whose NCCL kernels fit into them (:func:`exchange_group`).  The exchange of
    the last stripe has the GPU to itself: ``last_group`` (same ranks; e.g. the
    default group, whose kernels use as many SMs as NCCL likes) is used for it
    when given.

    ``mirror_stripes``: a stripe is the query rows ``[i w, (i + 1) w)`` together
    with their mirror image ``[Mq - (i + 1) w, Mq - i w)``.  With causal masks and
    keys sharded in mirror-symmetric ranges (:func:`zigzag_bounds`) every rank
    then has the same amount of work in every stripe (a row at x and the row at
    Mq - x see, of any mirror pair of key ranges, the length of one range), so no
    rank's exchange waits for another rank's attention.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if isinstance(key_shard, torch.Tensor):
        key_shard, value_shard, kv_offset = [key_shard], [value_shard], [kv_offset]
    if not (len(key_shard) == len(value_shard) == len(kv_offset)) or not len(key_shard):
        raise ValueError("sharded attention: key shards, value shards and offsets must pair up")
    ranges = [(k, v, int(off)) for k, v, off in zip(key_shard, value_shard, kv_offset) if k.shape[1] > 0]
    mq = query.shape[1]
    on_gpu = query.is_cuda

    # Two ranges that one launch can cover: causal, the first one a whole number of key tiles, the second one later.
    fused = None
    if (partial_fn is _partial_on_gpu and causal and len(ranges) == 2 and ranges[0][0].shape[1] % 128 == 0
            and ranges[1][2] >= ranges[0][2] + ranges[0][0].shape[1] and query.shape[-1] in (64, 128)):
        (k0, v0, o0), (k1, v1, o1) = ranges
        fused = (_cat_keeping_broadcast(k0, k1), _cat_keeping_broadcast(v0, v1), k0.shape[1], o0, o1)

    margin = 0  # set below, once it is known whether an exchange runs beside the attention

    def local_partial(a: int, b: int):
        """(out, lse) of this rank's keys for the query rows [a, b)."""
        q = query[:, a:b]
        if fused is not None:
            kc, vc, split, o0, o1 = fused
            return partial_fn(q, kc, vc, True, o0 - a, scale, partial_dtype, kv_split=split, kv_offset2=o1 - a, sm_margin=margin)
        extra = {"sm_margin": margin} if (margin and partial_fn is _partial_on_gpu) else {}
        parts = [partial_fn(q, k, v, causal, off - a, scale, partial_dtype, **extra) for k, v, off in ranges]
        if not parts:
            # this rank holds no keys at all: a partial of weight 0, shaped like a neighbour's (one key, then discarded)
            k0, v0 = key_shard[0], value_shard[0]
            one = lambda t: t.new_zeros((t.shape[0], 1) + tuple(t.shape[2:]))
            o, l = partial_fn(q, one(k0), one(v0), False, 0, scale, partial_dtype)
            return torch.zeros_like(o), torch.full_like(l, float("-inf"))
        if len(parts) == 1:
            return parts[0]
        return merge_fn([p[0] for p in parts], [p[1] for p in parts], parts[0][0].dtype)

    if timings is not None and on_gpu:
        timings["start"] = torch.cuda.Event(enable_timing=True)
        timings["start"].record()

    if world == 1:
        out_r, lse_r = local_partial(0, mq)
        res = merge_fn([out_r], [lse_r], query.dtype)
        if timings is not None and on_gpu:
            for name in ("attention_done", "done"):
                timings[name] = torch.cuda.Event(enable_timing=True)
                timings[name].record()
        return res

    use_a2a = exchange == "all_to_all" and mq % world == 0
    # (without CUDA streams the stripes simply run one after the other: the bookkeeping is the same)
    n_stripes = max(1, int(stripes)) if use_a2a else 1
    while n_stripes > 1 and (mq % n_stripes or (mq // n_stripes) % world):
        n_stripes -= 1
    margin = 0

    if not use_a2a:
        out_r, lse_r = local_partial(0, mq)
        out_r, lse_r = out_r.contiguous(), lse_r.contiguous()
        if timings is not None and on_gpu:
            timings["attention_done"] = torch.cuda.Event(enable_timing=True)
            timings["attention_done"].record()
        outs = torch.empty((world,) + tuple(out_r.shape), dtype=out_r.dtype, device=out_r.device)
        lses = torch.empty((world,) + tuple(lse_r.shape), dtype=lse_r.dtype, device=lse_r.device)
        # the flat form (ranks concatenated along dim 0) is the one every backend takes
        dist.all_gather_into_tensor(outs.view(-1, *out_r.shape[1:]), out_r, group=group)
        dist.all_gather_into_tensor(lses.view(-1, *lse_r.shape[1:]), lse_r, group=group)
        res = merge_fn(outs, lses, query.dtype)
        if timings is not None and on_gpu:
            timings["done"] = torch.cuda.Event(enable_timing=True)
            timings["done"].record()
        return res

    # ---- all-to-all by query slice, stripe by stripe
    mirrored = bool(mirror_stripes) and n_stripes > 1 and mq % (2 * n_stripes) == 0 and (mq // (2 * n_stripes)) % world == 0
    ms = mq // (2 * n_stripes) if mirrored else mq // n_stripes  # rows that are exchanged as a unit
    msw = ms // world                                            # rows of a unit that one rank merges
    # the result is allocated by the calling stream; the side stream fills it stripe by stripe
    out = torch.empty(query.shape, dtype=query.dtype, device=query.device)
    lse = torch.empty((query.shape[0],) + tuple(query.shape[2:-1]) + (mq,), dtype=torch.float32, device=query.device)
    main = torch.cuda.current_stream(query.device) if on_gpu else None
    comm = _comm_stream(query.device) if (on_gpu and n_stripes > 1) else main

    detail = timings.get("stripes") if (timings is not None and on_gpu) else None

    def mark(tag_list):
        if detail is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            tag_list.append(e)

    # The exchange of a unit (ms query rows) has three parts: the all-to-all of the partials by query slice, the merge of
    # this rank's slice, the all-gather of the merged slices.  With a side stream the collectives run there and the
    # merge runs on the calling stream, between two attention launches: a merge that had to share the few SMs the
    # attention leaves free with the collectives took longer than both of them together.
    def scatter(a: int, out_s: torch.Tensor, lse_s: torch.Tensor, grp):
        B = out_s.shape[0]
        ev = []
        if detail is not None:
            detail.append(ev)
        mark(ev)
        # partials of query slice w go to rank w: [world, B, msw, ...] (no copy for B == 1) and [world, B, .., msw]
        send_o = out_s.reshape(B, world, msw, *out_s.shape[2:]).transpose(0, 1).contiguous()
        send_l = lse_s.reshape(*lse_s.shape[:-1], world, msw).movedim(-2, 0).contiguous()
        recv_o, recv_l = torch.empty_like(send_o), torch.empty_like(send_l)
        mark(ev)
        dist.all_to_all_single(recv_o, send_o, group=grp)
        dist.all_to_all_single(recv_l, send_l, group=grp)
        mark(ev)
        return a, recv_o, recv_l, grp, ev

    def merge_unit(unit):
        a, recv_o, recv_l, grp, ev = unit
        m_o, m_l = merge_fn(recv_o, recv_l, query.dtype)                       # [B, msw, ...], [B, .., msw]
        m_o, m_l = m_o.contiguous(), m_l.contiguous()
        mark(ev)
        return a, m_o, m_l, grp, ev

    def gather(unit):
        a, m_o, m_l, grp, ev = unit
        B = m_o.shape[0]
        if B == 1:
            # the merged slices of a unit are consecutive rows of the result: gather them in place
            dist.all_gather_into_tensor(out[0, a : a + ms], m_o[0], group=grp)
        else:
            all_o = torch.empty((world,) + tuple(m_o.shape), dtype=m_o.dtype, device=m_o.device)
            dist.all_gather_into_tensor(all_o.view(-1, *m_o.shape[1:]), m_o, group=grp)
            out[:, a : a + ms] = all_o.transpose(0, 1).reshape(B, ms, *m_o.shape[2:])
        all_l = torch.empty((world,) + tuple(m_l.shape), dtype=m_l.dtype, device=m_l.device)
        dist.all_gather_into_tensor(all_l.view(-1, *m_l.shape[1:]), m_l, group=grp)
        lse[..., a : a + ms] = all_l.movedim(0, -2).reshape(*m_l.shape[:-1], ms)
        mark(ev)

    def finish(pending):
        """Merge (calling stream) and all-gather (side stream) of the units whose all-to-all was queued earlier."""
        units, scattered = pending
        main.wait_event(scattered)
        merged = []
        for unit in units:
            unit[1].record_stream(main)  # (allocated by the side stream, read by the calling stream)
            unit[2].record_stream(main)
            merged.append(merge_unit(unit))
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(comm):
            comm.wait_event(done)
            for unit in merged:
                unit[1].record_stream(comm)
                unit[2].record_stream(comm)
                gather(unit)

    pending = None
    for s in range(n_stripes):
        # the row ranges of this stripe, each exchanged as a unit of ms rows
        if mirrored:
            starts = [s * ms, mq - (s + 1) * ms]
        else:
            starts = [s * ms]
        # (no collective runs beside the first stripe's attention: it may have every SM)
        margin = int(sm_margin) if (n_stripes > 1 and s > 0) else 0
        parts = [(a,) + tuple(local_partial(a, a + ms)) for a in starts]
        grp = last_group if (s == n_stripes - 1 and last_group is not None and comm is not main) else group
        if comm is main:
            for a, out_s, lse_s in parts:
                gather(merge_unit(scatter(a, out_s, lse_s, grp)))
            continue
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(comm):
            comm.wait_event(ready)
            units = []
            for a, out_s, lse_s in parts:
                # (allocated by the calling stream, consumed by the side stream: their memory must not be reused before that)
                out_s.record_stream(comm)
                lse_s.record_stream(comm)
                units.append(scatter(a, out_s, lse_s, grp))
            scattered = torch.cuda.Event()
            scattered.record(comm)
        # the stripe before this one: its all-to-all had this stripe's attention to finish behind
        if pending is not None:
            finish(pending)
        pending = (units, scattered)
    if pending is not None:
        finish(pending)
    if timings is not None and on_gpu:
        timings["attention_done"] = torch.cuda.Event(enable_timing=True)
        timings["attention_done"].record(main)
    if comm is not main:
        out.record_stream(comm)
        lse.record_stream(comm)
        main.wait_stream(comm)
    if timings is not None and on_gpu:
        timings["done"] = torch.cuda.Event(enable_timing=True)
        timings["done"].record(main)
    return out, lse
