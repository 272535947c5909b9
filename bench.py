#!/usr/bin/env python
"""Benchmark of the attention-forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout (rank 0).  A step is one pass of the hot path over one
batch of synthetic input:

* headline (`value`): forward attention TFLOP/s of the causal prefill
  configuration B=4, Mq=Mkv=4096, Hq=Hkv=32, D=128, bf16 (FLOP convention of
  the reference: 4*Mq*Mkv*D per head, halved for causal).  With N > 1 every
  rank runs the same configuration on its own batch shard (batch x head work is
  sharded without communication: weak scaling).
* `e2e`: the same metric through the public API with HOST (pinned) q/k/v and a
  host copy of the output inside the timed region.
* `roofline`: tensor-pipe roofline of the prefill kernel against the measured
  cuBLAS bf16 peak of this pool (MEASURED_PEAKS.json); `sustained`: the same
  kernel over a timed region of at least a second, against the sustained peak.
  `decode_bf16` / `decode_int4` / `decode_fp8`: KV-read GB/s of the split-K
  decode configuration (64 sequences, lengths U[1024,32768], paged 256,
  Hq=64/Hkv=8) with their HBM rooflines, `rope_padded`, `varlen_gqa`: the packed
  varlen GQA prefill configuration; these legs are medians of CUDA-graph replays.
  `long_context`: one 131072-token causal sequence with the key axis sharded
  over the N ranks in two ranges each (equal causal work), partials exchanged by
  NCCL all-to-all per query slice, LSE merge, all-gather of the merged slices;
  `long_context_contiguous`: the same sequence with one contiguous key shard per
  rank and an all-gather of the partials.
* every leg carries `parity`: a slice of that leg's own output compared with
  the CPU oracle outside the timed region (max-abs error of O and of the LSE).
* `cpu_baseline`: the CPU oracle timed on a bounded slice of the headline
  configuration on this box's host cores (a reported baseline only).

`--impl reference` times the reference algorithm's CPU restatement (the oracle;
the reference's own kernels live in the un-vendored `mslk` package) on the same
slice, on the host cores.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "fwd attn TFLOP/s (prefill) & KV-read GB/s (split-K decode), 1-8 B200"
UNIT = "TFLOP/s"
WORKLOAD = "causal prefill B=4 Mq=Mkv=4096 Hq=Hkv=32 D=128 bf16 BMHK LowerTriangularMask"
CFG2 = dict(B=4, M=4096, H=32, D=128)
CPU_SAMPLE = dict(B=1, H=4)  # slice of CFG2 timed on the host


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one launch: constants taken from the ncu captures
# summarised under profiles/ (a run of this script does not measure them): bytes for the B=1 prefill case (every batch element adds the same), and traffic per algorithmic
# byte for the decode kernels (measured on 16 sequences; traffic grows with the tokens streamed).
NCU_TRAFFIC = {"prefill": 546.44e6 + 114.17e6, "decode_bf16": (980.12e6 + 14.07e6) / 979.88e6, "decode_int4": (261.43e6 + 4.82e6) / 260.67e6,
               "decode_fp8": (505.73e6 + 12.46e6) / 505.51e6, "rope": (100.70e6 + 55.24e6) / 201.33e6}


def causal_flops(B, M, H, D):
    return 4.0 * M * M * D * B * H / 2.0


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed regions."""

    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.samples = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self, windows):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        for t, line in self.samples:
            if not any(a <= t <= b for a, b in windows):
                continue
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


# ---------------------------------------------------------------------------
# CPU arm (reference algorithm restated by the oracle)
# ---------------------------------------------------------------------------
def cpu_sample_inputs():
    g = torch.Generator().manual_seed(0)
    B, H, M, D = CPU_SAMPLE["B"], CPU_SAMPLE["H"], CFG2["M"], CFG2["D"]
    q, k, v = (torch.randn(B, M, H, D, generator=g).bfloat16().float() for _ in range(3))
    return q, k, v


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1 to every rank; the CPU arm runs on
    rank 0 alone and may use every core the process is allowed on."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_step(q, k, v):
    # (the CPU arm imports the oracle only: nothing of the product package is loaded into its process)
    import oracle

    return oracle.ref_attention_with_lse(q, k, v, oracle.causal_mask(q.shape[1], k.shape[1]))


def time_cpu(budget_s: float, max_reps: int, warmup: int = 1):
    use_all_host_threads()
    q, k, v = cpu_sample_inputs()
    for _ in range(warmup):
        cpu_step(q, k, v)
    times = []
    t_start = time.perf_counter()
    while len(times) < max_reps and (time.perf_counter() - t_start < budget_s or len(times) < 3):
        t0 = time.perf_counter()
        cpu_step(q, k, v)
        times.append(time.perf_counter() - t0)
    flops = causal_flops(CPU_SAMPLE["B"], CFG2["M"], CPU_SAMPLE["H"], CFG2["D"])
    return flops, times


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    use_all_host_threads()
    q, k, v = cpu_sample_inputs()
    for _ in range(max(args.warmup, 1)):
        cpu_step(q, k, v)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(q, k, v)
    dt = time.perf_counter() - t0
    flops = causal_flops(CPU_SAMPLE["B"], CFG2["M"], CPU_SAMPLE["H"], CFG2["D"])
    val = flops * args.steps / dt / 1e12
    sample = f"B={CPU_SAMPLE['B']} x H={CPU_SAMPLE['H']} heads of the headline configuration per step (fp32 dense softmax(QK^T)V with LSE)"
    line = {
        "impl": "reference",
        "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "per_gpu_batch": CFG2["B"], "l2": "inputs (512 MiB per step) exceed the 126 MB L2",
                   "parallelism": f"batch-sharded x{args.gpus}, no communication", "peaks": load_peaks()["source"],
                   "sample": f"each step computes B={CPU_SAMPLE['B']} x H={CPU_SAMPLE['H']} heads of the workload (1/{CFG2['B'] * CFG2['H'] // (CPU_SAMPLE['B'] * CPU_SAMPLE['H'])} of it); value = FLOPs of the sample / time",
                   "note": "CPU restatement of the reference attention (oracle); mslk, which holds the reference kernels, is not installable offline"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def event_time_ms(fn, steps, warmup, barrier=None):
    for _ in range(warmup):
        fn()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    if barrier is not None:
        barrier()
    return e0.elapsed_time(e1), (t0, t1)


def graph_time_ms(fn, reps, warmup=3):
    """Median device time of ``reps`` replays of a CUDA graph holding one call of ``fn`` (the reference's
    harness times its decode operators the same way, xformers/benchmarks/utils.py:733-750).  The eager
    warm-up calls come first: whatever a first call sets up happens outside the capture."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    times = []
    t0 = time.time()
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        times.append((e0, e1))
    torch.cuda.synchronize()
    t1 = time.time()
    ms = sorted(a.elapsed_time(b) for a, b in times)
    return statistics.median(ms), ms[0], (t0, t1)


def parity_block(out, lse, ref_out, ref_lse, rows):
    """max-abs error of a slice of a leg's output against the oracle (tolerances: O 2e-2 for bf16, LSE 1e-3)."""
    eo = float((out.float().cpu() - ref_out).abs().max()) if out is not None else None
    el = None
    if lse is not None:
        l, r = lse.float().cpu(), ref_lse
        el = float(torch.where(torch.isneginf(l) & torch.isneginf(r), torch.zeros_like(l), (l - r).abs()).max())
    ok = (eo is None or eo <= 2e-2) and (el is None or el <= 1e-3)
    return {"max_abs_o": eo, "max_abs_lse": el, "rows": rows, "ok": bool(ok), "tolerance": "O 2e-2, LSE 1e-3"}


def decode_parity(q, k, v, bias, out, lse, quant, kss=None, vss=None, n_seqs=4):
    """Oracle check of a few sequences of a paged decode leg: their pages are gathered, dequantised on the host."""
    import oracle

    lens = bias.k_seqinfo.seqlen_py
    order = sorted(range(len(lens)), key=lambda i: lens[i])
    picks = sorted(set([order[0], order[-1]] + order[len(order) // 3 :: max(1, len(order) // 3)][: n_seqs - 2]))
    eo = el = 0.0
    for b in picks:
        rows = torch.from_numpy(oracle.physical_rows(bias.block_tables, bias.page_size, b, lens[b])).to(k.device)
        kb, vb = k[0, rows, :, 0].cpu(), v[0, rows, :, 0].cpu()
        if quant == "fp8":
            ksc, ksh = oracle.split_scale_shift(kss[0, rows, :, 0].cpu())
            vsc, vsh = oracle.split_scale_shift(vss[0, rows, :, 0].cpu())
            kr = oracle.dequantize_fp8_asymmetric(oracle.unpack_fp8_words(kb), ksc, ksh)
            vr = oracle.dequantize_fp8_asymmetric(oracle.unpack_fp8_words(vb), vsc, vsh)
        elif quant:
            kr, vr = oracle.dequantize_kv_int4(kb), oracle.dequantize_kv_int4(vb)
        else:
            kr, vr = kb.float(), vb.float()
        G = q.shape[3]
        qb = q[0, b].float().cpu()[None, None]
        ro, rl = oracle.ref_attention_with_lse(qb, kr[None, :, :, None].expand(-1, -1, -1, G, -1), vr[None, :, :, None].expand(-1, -1, -1, G, -1))
        eo = max(eo, float((out[:, b : b + 1].float().cpu() - ro).abs().max()))
        el = max(el, float((lse[:, :, :, b : b + 1].cpu() - rl).abs().max()))
    return {"max_abs_o": eo, "max_abs_lse": el, "rows": f"sequences {picks} of {len(lens)}", "ok": bool(eo <= 2e-2 and el <= 1e-3),
            "tolerance": "O 2e-2, LSE 1e-3"}


def gpu_quantize_int4(x):
    """Device-side restatement of the int4 row quantiser, used only to prepare
    synthetic caches (benchmarks/benchmark_attn_decoding.py:38-72)."""
    xf = x.float()
    mx, mn = xf.max(-1, keepdim=True).values, xf.min(-1, keepdim=True).values
    scale = ((mx - mn) / 15).half()
    shift = mn.half()
    qv = ((xf - shift.float()) / scale.float() + 0.5).to(torch.uint8) & 0xF
    packed = qv[..., ::2] + (qv[..., 1::2] << 4)
    ss = torch.cat([scale.view(torch.uint8), shift.view(torch.uint8)], dim=-1)
    return torch.cat([ss, packed], dim=-1).contiguous().view(torch.int32)


def gpu_quantize_fp8(x):
    """Device-side restatement of the row-wise fp8 quantiser of the reference's
    tests (tests/utils.py:311-333), used only to prepare synthetic caches:
    returns (int32 words of four e4m3 values, int32 [scale | shift << 16])."""
    xf = x.float()
    shift = xf.mean(-1, keepdim=True)
    c = xf - shift
    scale = torch.nan_to_num(448.0 / c.abs().amax(-1, keepdim=True), posinf=1.0)
    q8 = (c / scale).to(torch.float8_e4m3fn)
    ss = torch.cat([scale.half().view(torch.uint8), shift.half().view(torch.uint8)], dim=-1).contiguous().view(torch.int32)
    return q8.contiguous().view(torch.int32), ss.squeeze(-1)


def decode_workload(dev, quant, seed: int = 0, B: int = 64):
    from xformers_b200.ops.fmha import attn_bias as ab

    g = torch.Generator().manual_seed(seed)
    page, Hkv, G, D = 256, 8, 8, 128
    lens = torch.randint(1024, 32769, (B,), generator=g)
    pages = (lens + page - 1) // page
    pool = int(pages.sum())
    max_pages = 32768 // page
    perm = torch.randperm(pool, generator=g).int()
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    s = 0
    for b in range(B):
        n = int(pages[b])
        table[b, :n] = perm[s : s + n]
        s += n
    gd = torch.Generator(device=dev).manual_seed(seed)
    q = torch.randn(1, B, Hkv, G, D, generator=gd, device=dev, dtype=torch.bfloat16)
    shape = (1, pool * page, Hkv, 1, D)
    k = torch.randn(shape, generator=gd, device=dev, dtype=torch.bfloat16)
    v = torch.randn(shape, generator=gd, device=dev, dtype=torch.bfloat16)
    kss = vss = None
    if quant == "fp8":
        kq = torch.empty(shape[:-1] + (D // 4,), dtype=torch.int32, device=dev)
        vq = torch.empty_like(kq)
        kss = torch.empty(shape[:-1], dtype=torch.int32, device=dev)
        vss = torch.empty_like(kss)
        step = 64 * page
        for lo in range(0, pool * page, step):
            kq[:, lo : lo + step], kss[:, lo : lo + step] = gpu_quantize_fp8(k[:, lo : lo + step])
            vq[:, lo : lo + step], vss[:, lo : lo + step] = gpu_quantize_fp8(v[:, lo : lo + step])
        k, v = kq, vq
        row_bytes = D + 4
        # one scale/shift word per token and kv head, expanded over the query heads of the group like K and V themselves
        kss, vss = kss.expand(-1, -1, -1, G), vss.expand(-1, -1, -1, G)
    elif quant:
        kq = torch.empty(shape[:-1] + (D // 8 + 1,), dtype=torch.int32, device=dev)
        vq = torch.empty_like(kq)
        step = 64 * page
        for lo in range(0, pool * page, step):
            kq[:, lo : lo + step] = gpu_quantize_int4(k[:, lo : lo + step])
            vq[:, lo : lo + step] = gpu_quantize_int4(v[:, lo : lo + step])
        k, v = kq, vq
        row_bytes = (D // 8 + 1) * 4
    else:
        row_bytes = D * 2
    k = k.expand(-1, -1, -1, G, -1)
    v = v.expand(-1, -1, -1, G, -1)
    bias = ab.PagedBlockDiagonalPaddedKeysMask.from_seqlens([1] * B, lens.tolist(), table.to(dev), page)
    kv_bytes = float(lens.sum()) * Hkv * 2 * row_bytes
    qo_bytes = 2.0 * B * Hkv * G * D * 2
    if quant == "fp8":
        return q, k, v, bias, kv_bytes + qo_bytes + table.numel() * 4, kss, vss
    return q, k, v, bias, kv_bytes + qo_bytes + table.numel() * 4


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-extras", action="store_true", help="headline only (no decode / varlen / long-context / CPU legs)")
    ap.add_argument("--e2e-mode", default="pipelined", choices=["pipelined", "serial"],
                    help="e2e leg: overlap upload / kernel / read-back of neighbouring steps, or run them back to back")
    ap.add_argument("--only", default="", help="comma list of legs to run: prefill,e2e,decode_bf16,decode_int4,decode_fp8,rope,varlen,long,cpu")
    ap.add_argument("--small", action="store_true",
                    help="profiling case: one batch of the headline configuration (128 MB of tensors, still larger than L2) and 16 decode sequences; not a bench value")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch.distributed as dist

    import xformers_b200.ops as xops
    from xformers_b200.ops import fmha
    from xformers_b200.ops.fmha import attn_bias as ab
    from xformers_b200.ops.fmha.sharded import sharded_kv_attention_forward, zigzag_bounds

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the operators")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    # stdout carries the one JSON line: whatever a library prints there meanwhile (NCCL's version banner) goes to stderr
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    legs = set(args.only.split(",")) if args.only else {"prefill", "e2e", "decode_bf16", "decode_int4", "decode_fp8", "rope", "varlen", "long", "cpu"}
    if args.skip_extras:
        legs &= {"prefill", "e2e"}
    peaks = load_peaks()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    windows = []

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out_line = {
        "metric": METRIC, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "per_gpu_batch": CFG2["B"], "l2": "inputs (512 MiB per step) exceed the 126 MB L2",
                   "parallelism": f"batch-sharded x{world}, no communication", "peaks": peaks["source"]},
    }

    # ------------------------------------------------------------- headline
    B, M, H, D = (1 if args.small else CFG2["B"]), CFG2["M"], CFG2["H"], CFG2["D"]
    if args.small:
        out_line["config"]["small"] = "profiling case, not a bench value"
    gd = torch.Generator(device=dev).manual_seed(rank)
    q, k, v = (torch.randn(B, M, H, D, generator=gd, device=dev, dtype=torch.bfloat16) for _ in range(3))
    causal = ab.LowerTriangularMask()
    flops = causal_flops(B, M, H, D)
    launches = 0
    if "prefill" in legs:
        import oracle

        fn = lambda: xops.memory_efficient_attention_forward(q, k, v, causal, op=fmha.b200.FwOp)
        ms, win = event_time_ms(fn, args.steps, args.warmup, barrier)
        windows.append(win)
        ms = max_over_ranks(ms)
        per_step = ms / args.steps
        tfs = flops / (per_step * 1e-3) / 1e12
        launches = args.steps
        out_line.update({"value": tfs * world, "ms_per_step": per_step, "gpu_launches": launches})
        # the same launch over a timed region of at least a second: what the kernel holds once the part is power-capped
        s_steps = args.steps if args.small else max(args.steps, int(math.ceil(1000.0 / max(per_step, 1e-3))))
        s_ms, win = event_time_ms(fn, s_steps, 0, barrier)
        windows.append(win)
        s_ms = max_over_ranks(s_ms)
        s_tfs = flops / (s_ms / s_steps * 1e-3) / 1e12
        status = fmha.b200.prefill_device_status()
        # parity of this leg's own output: two heads of the first batch element against the oracle
        po, pl = xops.memory_efficient_attention_forward_requires_grad(q, k, v, causal, op=fmha.b200.FwOp)
        hs = [0, H - 1]
        ro, rl = oracle.ref_attention_with_lse(q[:1, :, hs].float().cpu(), k[:1, :, hs].float().cpu(), v[:1, :, hs].float().cpu(), oracle.causal_mask(M, M))
        out_line["parity"] = parity_block(po[:1, :, hs], pl[:1, hs], ro, rl, f"batch 0, heads {hs}, all {M} rows (rank {rank})")
        del po, pl
        out_line["roofline"] = {"bound": "tensor", "achieved": tfs, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                "frac": tfs / peaks["bf16_tflops"], "traffic": NCU_TRAFFIC["prefill"] * (B / 4),
                                "traffic_unit": "bytes per launch (constant from profiles/: ncu on the full-size B=4 launch, scaled by B)",
                                "kernel": "prefill_sm100_persist_kernel<128, bf16>",
                                "of": peaks["source"], "frac_of_nominal_2250": tfs / 2250.0, "device_status": status}
        out_line["sustained"] = {"value": s_tfs * world, "unit": UNIT, "steps": s_steps, "timed_region_s": s_ms * 1e-3, "ms_per_step": s_ms / s_steps,
                                 "peak": peaks["bf16_tflops_sustained"], "frac": s_tfs / peaks["bf16_tflops_sustained"], "of": peaks["source"],
                                 "note": "same launch repeated for at least a second; the peak is cuBLAS bf16 held for seconds under the power cap"}
        launches += s_steps + 1
        out_line["gpu_launches"] = launches
    # ------------------------------------------------------------------ e2e
    if "e2e" in legs:
        hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
        ho = torch.empty((B, M, H, D), dtype=torch.bfloat16).pin_memory()

        # Three streams, two sets of device buffers: the upload of step i+1 and
        # the read-back of step i-1 overlap the kernel of step i, as a serving
        # loop would run it.  Every step still moves its own inputs and result.
        s_in, s_out, s_cmp = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        slots = [tuple(torch.empty_like(q) for _ in range(3)) for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_cmp = [torch.cuda.Event() for _ in range(2)]
        ev_out = torch.cuda.Event()
        counter = [0]

        def e2e_step_serial():
            for dst, src in zip(slots[0], (hq, hk, hv)):
                dst.copy_(src, non_blocking=True)
            o = xops.memory_efficient_attention_forward(*slots[0], causal)
            ho.copy_(o, non_blocking=True)

        def e2e_step():
            if args.e2e_mode == "serial":
                return e2e_step_serial()
            i = counter[0] % 2
            counter[0] += 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_cmp[i])  # the kernel that last read this slot is done
                for dst, src in zip(slots[i], (hq, hk, hv)):
                    dst.copy_(src, non_blocking=True)
                ev_in[i].record(s_in)
            s_cmp.wait_event(ev_in[i])
            o = xops.memory_efficient_attention_forward(*slots[i], causal)
            ev_cmp[i].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[i])
                ho.copy_(o, non_blocking=True)
                o.record_stream(s_out)
                ev_out.record(s_out)

        def e2e_drain():
            if args.e2e_mode != "serial":
                s_cmp.wait_event(ev_out)  # the timed region ends when the last result is on the host

        e_steps = max(3, min(args.steps, 20))
        s_in.wait_stream(s_cmp)
        for _ in range(3):
            e2e_step()
        e2e_drain()
        barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        s_in.wait_event(e0)
        for _ in range(e_steps):
            e2e_step()
        e2e_drain()
        e1.record()
        torch.cuda.synchronize()
        win = (t0, time.time())
        barrier()
        ms = e0.elapsed_time(e1)
        windows.append(win)
        ms = max_over_ranks(ms)
        nbytes = q.numel() * 2
        out_line["e2e"] = {"value": world * flops / (ms / e_steps * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": 3 * nbytes,
                           "d2h_bytes_per_step": nbytes, "ms_per_step": ms / e_steps, "steps": e_steps, "mode": args.e2e_mode}
        del hq, hk, hv, ho, slots
    del q, k, v
    torch.cuda.empty_cache()

    # --------------------------------------------------- decode (rank 0 only)
    for name, quant in (("decode_bf16", False), ("decode_int4", True), ("decode_fp8", "fp8")):
        if name in legs and rank == 0:
            wl = decode_workload(dev, quant, B=16 if args.small else 64)
            dq, dk, dv, dbias, nbytes = wl[:5]
            kss = vss = None
            if quant == "fp8":
                kss, vss = wl[5], wl[6]
                inp = fmha.triton_splitk.InputsFp8(query=dq, key=dk, value=dv, attn_bias=dbias, k_fp8_scale_shift=kss, v_fp8_scale_shift=vss)
                fn = lambda: fmha._memory_efficient_attention_forward(inp, op=fmha.b200_splitk.FwOp)
                fn_lse = lambda: fmha._memory_efficient_attention_forward_requires_grad(inp, op=fmha.b200_splitk.FwOp)
            else:
                fn = lambda: xops.memory_efficient_attention_forward(dq, dk, dv, dbias, op=fmha.b200_splitk.FwOp)
                fn_lse = lambda: xops.memory_efficient_attention_forward_requires_grad(dq, dk, dv, dbias, op=fmha.b200_splitk.FwOp)
            d_reps = max(20, min(args.steps, 50))
            med, best, win = graph_time_ms(fn, d_reps)
            windows.append(win)
            gbs = nbytes / (med * 1e-3) / 1e9
            o_, l_ = fn_lse()
            l_ = l_.lse if hasattr(l_, "lse") else l_
            par = decode_parity(dq, dk, dv, dbias, o_, l_, quant, kss, vss)
            par["device_status"] = fmha.b200_splitk.decode_device_status()
            row_bytes = 132 if quant == "fp8" else 68 if quant else 256
            split = fmha.b200_splitk.FwOp.get_split_k(16 if args.small else 64, 32768, 8, row_bytes)
            out_line[name] = {"value": gbs, "unit": "GB/s", "ms_per_step": med, "ms_best": best, "replays": d_reps, "timing": "median of CUDA-graph replays",
                              "bytes_per_step": nbytes, "split_k": split, "parity": par,
                              "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                           "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC[name] * nbytes,
                                           "traffic_unit": "bytes per launch (constant from profiles/: ncu ratio to algorithmic bytes on the 16-sequence case)",
                                           "of": peaks["source"]},
                              "workload": "64 seqs, kv len U[1024,32768], paged 256, Hq=64 Hkv=8 D=128, 1 query each; cache far larger than L2"
                                          + ("; row-wise fp8 cache (128 B + one scale/shift word per token and head)" if quant == "fp8" else "; int4 row-wise cache (68 B per token and head)" if quant else "")}
            launches += 2 * (d_reps + 7)
            del dq, dk, dv, dbias, wl, kss, vss, o_, l_
            if quant == "fp8":
                del inp
            torch.cuda.empty_cache()
        barrier()

    # ------------------------------ rope_padded: prefill into a padded cache (rank 0)
    if "rope" in legs and rank == 0:
        r_seqs, r_len, r_hq, r_hkv, r_pad = (2, 4096, 32, 8, 4160) if args.small else (8, 4096, 32, 8, 4160)
        gd = torch.Generator(device=dev).manual_seed(0)
        rq = torch.randn(1, r_seqs * r_len, r_hq, 128, generator=gd, device=dev, dtype=torch.bfloat16)
        rk = torch.randn(1, r_seqs * r_len, r_hkv, 128, generator=gd, device=dev, dtype=torch.bfloat16)
        rv = torch.randn(1, r_seqs * r_len, r_hkv, 128, generator=gd, device=dev, dtype=torch.bfloat16)
        rck = torch.zeros(1, r_seqs * r_pad, r_hkv, 128, device=dev, dtype=torch.bfloat16)
        rcv = torch.zeros_like(rck)
        rout = torch.empty_like(rq)
        rbias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=[r_len] * r_seqs, kv_padding=r_pad, kv_seqlen=[r_len + 17] * r_seqs).to(dev)

        def rope_step():
            with torch.no_grad():
                xops.rope_padded(rq, rk, rv, rck, rcv, rbias, out_q=rout)

        r_reps = max(20, min(args.steps, 50))
        med, best, win = graph_time_ms(rope_step, r_reps)
        windows.append(win)
        rbytes = 2 * rq.numel() * 2 + 2 * (rk.numel() + rv.numel()) * 2  # every row read once and written once
        gbs = rbytes / (med * 1e-3) / 1e9
        launches += r_reps + 6
        out_line["rope_padded"] = {"value": gbs, "unit": "GB/s", "ms_per_step": med, "ms_best": best, "replays": r_reps, "timing": "median of CUDA-graph replays", "bytes_per_step": rbytes,
                                   "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                                                "traffic": NCU_TRAFFIC["rope"] * rbytes, "traffic_unit": "bytes per launch (constant from profiles/: ncu ratio to algorithmic bytes on the 2-sequence case)", "of": peaks["source"]},
                                   "workload": f"{r_seqs} seqs x {r_len} new tokens into slots of {r_pad} rows, Hq={r_hq} Hkv={r_hkv} D=128 bf16, adjacent pairs; {rbytes >> 20} MiB per step, larger than L2"}
        del rq, rk, rv, rck, rcv, rout
        torch.cuda.empty_cache()
    barrier()

    # ------------------------------------------- packed varlen GQA (rank 0)
    if "varlen" in legs and rank == 0:
        import oracle

        g = torch.Generator().manual_seed(0)
        lens = torch.randint(256, 4097, (16,), generator=g).tolist()
        total = sum(lens)
        gd = torch.Generator(device=dev).manual_seed(0)
        vq = torch.randn(1, total, 8, 4, 128, generator=gd, device=dev, dtype=torch.bfloat16)
        vk = torch.randn(1, total, 8, 1, 128, generator=gd, device=dev, dtype=torch.bfloat16).expand(-1, -1, -1, 4, -1)
        vv = torch.randn(1, total, 8, 1, 128, generator=gd, device=dev, dtype=torch.bfloat16).expand(-1, -1, -1, 4, -1)
        vbias = ab.BlockDiagonalCausalMask.from_seqlens(lens, device=dev)
        fn = lambda: xops.memory_efficient_attention_forward(vq, vk, vv, vbias, op=fmha.b200.FwOp)
        v_reps = max(20, min(args.steps, 50))
        med, best, win = graph_time_ms(fn, v_reps)
        windows.append(win)
        vflops = 8192.0 * sum(l * l for l in lens)
        vt = vflops / (med * 1e-3) / 1e12
        # parity: the shortest and the longest sequence, one KV group each
        vo, vl = xops.memory_efficient_attention_forward_requires_grad(vq, vk, vv, vbias, op=fmha.b200.FwOp)
        starts = [0]
        for n in lens:
            starts.append(starts[-1] + n)
        eo = el = 0.0
        picks = [min(range(16), key=lambda i: lens[i]), max(range(16), key=lambda i: lens[i])]
        for i, grp in zip(picks, (0, 7)):
            a_, b_ = starts[i], starts[i + 1]
            ro, rl = oracle.ref_attention_with_lse(vq[:, a_:b_, grp].float().cpu(), vk[:, a_:b_, grp].float().cpu(), vv[:, a_:b_, grp].float().cpu(),
                                                   oracle.causal_mask(b_ - a_, b_ - a_))
            eo = max(eo, float((vo[:, a_:b_, grp].float().cpu() - ro).abs().max()))
            el = max(el, float((vl[:, grp, :, a_:b_].cpu() - rl).abs().max()))
        out_line["varlen_gqa"] = {"value": vt, "unit": UNIT, "ms_per_step": med, "ms_best": best, "replays": v_reps, "timing": "median of CUDA-graph replays",
                                  "frac_of_peak": vt / peaks["bf16_tflops"],
                                  "parity": {"max_abs_o": eo, "max_abs_lse": el, "rows": f"sequences {picks} (lengths {[lens[i] for i in picks]}), groups 0 and 7",
                                             "ok": bool(eo <= 2e-2 and el <= 1e-3), "tolerance": "O 2e-2, LSE 1e-3"},
                                  "workload": f"16 seqs U[256,4096] (total {total}), BlockDiagonalCausalMask, Hq=32 Hkv=8 D=128 bf16"}
        launches += v_reps + 6
        del vq, vk, vv, vo, vl
        torch.cuda.empty_cache()
    barrier()

    # ------------------------------------------------ long context (all ranks)
    if "long" in legs:
        import oracle

        S, Hkv, G, D = (32768 if args.small else 131072), 8, 8, 128
        gd = torch.Generator(device=dev).manual_seed(1234)  # the same tensors on every rank; a rank uses its key ranges only
        lq = torch.randn(1, S, Hkv, G, D, generator=gd, device=dev, dtype=torch.bfloat16)
        lk_full = torch.randn(1, S, Hkv, 1, D, generator=gd, device=dev, dtype=torch.bfloat16)
        lv_full = torch.randn(1, S, Hkv, 1, D, generator=gd, device=dev, dtype=torch.bfloat16)
        lflops = 4.0 * S * S * D * Hkv * G / 2.0
        hp_group = None
        # SMs the attention leaves to the collectives that run beside it: the exchange of a stripe has one stripe of attention to
        # finish behind, and that shrinks with the number of ranks while the exchange does not
        sm_margin = int(os.environ.get("XFB200_BENCH_SM_MARGIN", "8" if world <= 4 else "12"))
        n_str_default = int(os.environ.get("XFB200_BENCH_STRIPES", "8"))
        if world > 1:
            from xformers_b200.ops.fmha.sharded import exchange_group

            hp_group = exchange_group(max_ctas=sm_margin)

        def long_leg(spans, exchange, stripes, l_steps, l_warm, group, sm_margin, last_group=None):
            lk = [lk_full[:, a:b].expand(-1, -1, -1, G, -1) for a, b in spans]
            lv = [lv_full[:, a:b].expand(-1, -1, -1, G, -1) for a, b in spans]
            res = {}

            def fn():
                res["out"], res["lse"] = sharded_kv_attention_forward(lq, lk, lv, kv_offset=[a for a, _ in spans], causal=True,
                                                                      exchange=exchange, stripes=stripes, group=group, sm_margin=sm_margin,
                                                                      last_group=last_group, mirror_stripes=stripes > 1)

            ms, win = event_time_ms(fn, l_steps, l_warm, barrier)
            windows.append(win)
            ms = max_over_ranks(ms) / l_steps
            # break-down of one more step: attention of this rank's keys / what the exchange adds after it
            tm = {}
            sharded_kv_attention_forward(lq, lk, lv, kv_offset=[a for a, _ in spans], causal=True, exchange=exchange, stripes=stripes, timings=tm,
                                         group=group, sm_margin=sm_margin, last_group=last_group, mirror_stripes=stripes > 1)
            torch.cuda.synchronize()
            att = max_over_ranks(tm["start"].elapsed_time(tm["attention_done"]))
            tot = max_over_ranks(tm["start"].elapsed_time(tm["done"]))
            # parity of the leg's own output: rows at the start, the middle and the end of this rank's share of the queries
            lo_r, hi_r = rank * (S // world), (rank + 1) * (S // world)
            rows = sorted({lo_r, lo_r + 1, (lo_r + hi_r) // 2, hi_r - 2, hi_r - 1})
            heads = [0, G - 1]
            mask = torch.stack([oracle.causal_mask(1, S, kv_offset=-r)[0] for r in rows])
            ro, rl = oracle.ref_attention_with_lse(lq[:, rows, 0][:, :, heads].float().cpu(), lk_full[:, :, 0].expand(-1, -1, len(heads), -1).float().cpu(),
                                                   lv_full[:, :, 0].expand(-1, -1, len(heads), -1).float().cpu(), mask.expand(1, len(heads), len(rows), S))
            eo = float((res["out"][:, rows, 0][:, :, heads].float().cpu() - ro).abs().max())
            el = float((res["lse"][:, 0][:, heads][..., rows].cpu() - rl).abs().max())
            if world > 1:
                t = torch.tensor([eo, el], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                eo, el = float(t[0]), float(t[1])
            del res
            return ms, {"attention_ms": att, "step_ms": tot, "exchange_after_attention_ms": tot - att}, \
                {"max_abs_o": eo, "max_abs_lse": el, "rows": f"5 rows of every rank's share of the queries, KV group 0, heads {heads} (max over ranks)",
                 "ok": bool(eo <= 2e-2 and el <= 1e-3), "tolerance": "O 2e-2, LSE 1e-3"}

        l_steps, l_warm = (10, 2) if not args.small else (3, 1)
        spans = zigzag_bounds(S, world, rank) if world > 1 else [(0, S)]
        n_str = n_str_default if world > 1 else 1
        # (the last stripe's exchange has the GPU to itself: the default group, whose kernels are not limited to the margin)
        use_last = world > 1 and os.environ.get("XFB200_BENCH_LAST_GROUP", "1") == "1"
        ms, brk, par = long_leg(spans, "all_to_all", n_str, l_steps, l_warm, hp_group, sm_margin if world > 1 else 0,
                                last_group=torch.distributed.group.WORLD if use_last else None)
        lt = lflops / (ms * 1e-3) / 1e12
        out_line["long_context"] = {"value": lt, "unit": UNIT, "ms_per_step": ms, "steps": l_steps, "warmup": l_warm, "scaling": "strong",
                                    "ideal_speedup": float(world), "breakdown": brk, "parity": par, "query_stripes": n_str, "sm_margin": sm_margin if world > 1 else 0,
                                    "workload": f"1 x {S} causal, Hq=64 Hkv=8 D=128 bf16; keys sharded over ranks in two ranges each (chunks r and 2N-1-r of 2N: equal causal work) covered by one launch per query stripe; a stripe is a block of query rows and its mirror image (equal work on every rank); per stripe NCCL all-to-all of the partials (input dtype, LSE fp32) by query slice on a side stream, LSE merge of the slice on the main stream, all-gather of the merged slices on the side stream, behind the next stripe's attention"}
        launches += (l_steps + l_warm + 1) * n_str
        if world > 1:
            # the literal form of the baseline configuration: one contiguous key shard per rank, all-gather of the partials, one merge
            from xformers_b200.ops.fmha.sharded import shard_bounds

            c_steps, c_warm = (5, 1)
            ms, brk, par = long_leg([shard_bounds(S, world, rank)], "all_gather", 1, c_steps, c_warm, None, 0)
            ct = lflops / (ms * 1e-3) / 1e12
            r2 = world * world / (2.0 * world - 1.0)
            out_line["long_context_contiguous"] = {"value": ct, "unit": UNIT, "ms_per_step": ms, "steps": c_steps, "warmup": c_warm, "scaling": "strong",
                                                   "ideal_speedup": r2, "breakdown": brk, "parity": par,
                                                   "workload": f"1 x {S} causal, contiguous key shards, NCCL all-gather of the partials (input dtype, LSE fp32), one LSE merge; causal work is imbalanced by construction: ideal speed-up R^2/(2R-1) = {r2:.2f}"}
        del lq, lk_full, lv_full
        torch.cuda.empty_cache()

    if rank == 0:
        out_line["clocks"] = sampler.stop(windows) if sampler is not None else None
        if "cpu" in legs:
            cflops, times = time_cpu(budget_s=12.0, max_reps=20)
            best = min(times)
            out_line["cpu_baseline"] = {
                "value": cflops / best / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                "sample": f"B={CPU_SAMPLE['B']} x H={CPU_SAMPLE['H']} heads of the headline configuration, best of {len(times)} runs (median {statistics.median(times):.3f} s); fp32 oracle",
            }
        out_line["gpu_launches_all_legs"] = launches
        json_out.write(json.dumps(out_line) + "\n")
        json_out.flush()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
