"""KV-sharded long-context attention on real ranks: one process per GPU, NCCL.

Needs two GPUs (skipped otherwise).  Every rank holds its key ranges only, the
result of the exchange is compared with the oracle on a few rows and with the
single-GPU operator on all of them, for both exchanges, with and without query
stripes, and for contiguous shards.  Ranks leave only after a final barrier.
"""

import os
import tempfile

import pytest
import torch

from gpu_utils import ATOL_LSE, ATOL_O, gpu


def _worker(rank, world, init_file, out_file):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist

    import oracle
    from xformers_b200.ops import fmha
    from xformers_b200.ops.fmha import attn_bias as ab
    from xformers_b200.ops.fmha.sharded import exchange_group, shard_bounds, sharded_kv_attention_forward, zigzag_bounds

    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world, device_id=dev)
    ok, msg = True, []
    try:
        S, Hkv, G, D = 4096, 2, 4, 128
        g = torch.Generator().manual_seed(7)  # the same tensors on every rank
        q = torch.randn(1, S, Hkv, G, D, generator=g).bfloat16().to(dev)
        k = torch.randn(1, S, Hkv, 1, D, generator=g).bfloat16().to(dev)
        v = torch.randn(1, S, Hkv, 1, D, generator=g).bfloat16().to(dev)
        ke, ve = k.expand(-1, -1, -1, G, -1), v.expand(-1, -1, -1, G, -1)
        full_o, full_l = fmha.memory_efficient_attention_forward_requires_grad(q, ke, ve, ab.LowerTriangularMask())
        rows = [0, 1, 127, 128, S // 2 - 1, S // 2, S - 2, S - 1]
        ro, rl = oracle.ref_attention_with_lse(q[:, rows].float().cpu(), ke.float().cpu(), ve.float().cpu(),
                                               torch.stack([oracle.causal_mask(1, S, kv_offset=-r)[0] for r in rows]).expand(1, Hkv, G, len(rows), S))
        cases = [("zigzag a2a", zigzag_bounds(S, world, rank), dict(exchange="all_to_all", stripes=1)),
                 ("zigzag a2a 4 stripes", zigzag_bounds(S, world, rank), dict(exchange="all_to_all", stripes=4)),
                 ("zigzag a2a 4 stripes, SMs left free, a narrow group and the default group for the last stripe", zigzag_bounds(S, world, rank),
                  dict(exchange="all_to_all", stripes=4, sm_margin=8, group=exchange_group(max_ctas=8), last_group=dist.group.WORLD)),
                 ("zigzag a2a, 4 stripes of mirrored row blocks", zigzag_bounds(S, world, rank),
                  dict(exchange="all_to_all", stripes=4, mirror_stripes=True, sm_margin=8, group=exchange_group(max_ctas=8), last_group=dist.group.WORLD)),
                 ("zigzag gather", zigzag_bounds(S, world, rank), dict(exchange="all_gather")),
                 ("contiguous gather", [shard_bounds(S, world, rank)], dict(exchange="all_gather")),
                 ("contiguous a2a 2 stripes", [shard_bounds(S, world, rank)], dict(exchange="all_to_all", stripes=2))]
        for name, spans, kw in cases:
            ks = [ke[:, a:b] for a, b in spans]
            vs = [ve[:, a:b] for a, b in spans]
            out, lse = sharded_kv_attention_forward(q, ks, vs, kv_offset=[a for a, _ in spans], causal=True, **kw)
            torch.cuda.synchronize()
            eo = (out[:, rows].float().cpu() - ro).abs().max().item()
            el = (lse[..., rows].cpu() - rl).abs().max().item()
            do = (out.float() - full_o.float()).abs().max().item()
            dl = (lse - full_l).abs().max().item()
            if not (eo <= ATOL_O[torch.bfloat16] and el <= ATOL_LSE and do <= ATOL_O[torch.bfloat16] and dl <= ATOL_LSE):
                ok = False
            msg.append(f"{name}: oracle O {eo:.2e} LSE {el:.2e}; single-GPU O {do:.2e} LSE {dl:.2e}")
        st = fmha.b200.prefill_device_status()
        if st != 0:
            ok = False
            msg.append(f"device status {st}")
    except Exception as e:  # reported by the parent
        ok = False
        msg.append(repr(e))
    with open(f"{out_file}.{rank}", "w") as f:
        f.write(("OK\n" if ok else "FAIL\n") + "\n".join(msg))
    dist.barrier()
    dist.destroy_process_group()


@gpu
def test_sharded_long_context_on_two_nccl_ranks():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world = 2
    with tempfile.TemporaryDirectory() as d:
        init_file, out_file = os.path.join(d, "init"), os.path.join(d, "out")
        mp.spawn(_worker, args=(world, init_file, out_file), nprocs=world, join=True)
        for r in range(world):
            text = open(f"{out_file}.{r}").read()
            assert text.startswith("OK"), f"rank {r}:\n{text}"
