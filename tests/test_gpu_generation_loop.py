"""The caller of the hot path: a LLaMA-style generation loop.

Follows examples/llama_inference/generate.py:100-187 and model.py:100-151 with a
toy model (random weights: neither checkpoint nor tokenizer is involved in the
contract): ONE ``BlockDiagonalCausalWithOffsetPaddedKeysMask`` for prompts of
unequal length, ``rope_padded`` + ``memory_efficient_attention_forward`` on 5-D
GQA views in every layer for the prefill, then the decode step captured in a
CUDA graph and replayed, with ``q_seqstart.copy_``, ``kv_seqlen.add_`` and
``max_seqlen = 1`` applied to the same bias object between replays.  Every
step's attention output of every layer is compared with the oracle on a host
copy of the rotated queries and of the caches.  A second run keeps the cache
paged and in the int4 row-wise format, written by ``rope_padded`` itself.
"""

import pytest
import torch

import oracle
from gpu_utils import ATOL_LSE, ATOL_O, gpu, require_cuda
import xformers_b200.ops as xops
from xformers_b200.ops import fmha
from xformers_b200.ops.fmha import attn_bias as ab

N_LAYERS, N_KV, HPG, HD, VOCAB = 2, 2, 4, 128, 64
DIM = N_KV * HPG * HD
GRAPH_WARMUPS = 1


class ToyModel:
    """Embedding -> N_LAYERS x (wqkv, rope + cache write, attention, wo, residual) -> logits."""

    def __init__(self, dev, dtype, seed=0):
        g = torch.Generator().manual_seed(seed)
        mk = lambda *s: (torch.randn(*s, generator=g) * s[-1] ** -0.5).to(dtype).to(dev)
        self.emb = (torch.randn(VOCAB, DIM, generator=g)).to(dtype).to(dev)
        self.wqkv = [mk((N_KV * HPG + 2 * N_KV) * HD, DIM) for _ in range(N_LAYERS)]
        self.wo = [mk(DIM, DIM) for _ in range(N_LAYERS)]
        self.head = mk(VOCAB, DIM)
        self.trace = []  # per layer: (rotated queries, attention output) of the latest forward

    def forward(self, tokens, bias, caches):
        self.trace = []
        x = self.emb[tokens.long()]
        for layer in range(N_LAYERS):
            xqkv = x @ self.wqkv[layer].t()
            xq = xqkv[:, : N_KV * HPG * HD]
            xk, xv = xqkv[:, N_KV * HPG * HD :].chunk(2, 1)
            shape = xq.shape
            xq = xq.view(1, xq.shape[0], N_KV, HPG, HD)
            xk = xk.view(1, xk.shape[0], N_KV, 1, HD)
            xv = xv.view(1, xv.shape[0], N_KV, 1, HD)
            cache_k, cache_v = caches[layer]
            xq = xops.rope_padded(xq=xq, xk=xk, xv=xv, cache_k=cache_k, cache_v=cache_v, attn_bias=bias, theta=10000.0)
            # rope_padded() updated the caches: attention reads them
            ck = cache_k.expand(-1, -1, -1, HPG, -1)
            cv = cache_v.expand(-1, -1, -1, HPG, -1)
            out = xops.memory_efficient_attention_forward(xq, ck, cv, bias)
            self.trace.append((xq, out))
            x = x + out.reshape(shape) @ self.wo[layer].t()
        return x @ self.head.t()


def _check_layers(model, caches, q_lens, kv_lens, padding, dtype, what, dequant=None, table=None, page=None):
    """Attention of every layer of the latest forward against the oracle on host copies."""
    bias = ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=q_lens, kv_padding=padding, kv_seqlen=kv_lens)
    for layer, (xq, out) in enumerate(model.trace):
        ck, cv = caches[layer]
        if table is not None:
            ck = oracle.gather_paged(ck, table, page, kv_lens, padding)
            cv = oracle.gather_paged(cv, table, page, kv_lens, padding)
        ck, cv = ck.cpu(), cv.cpu()
        if dequant is not None:
            ck, cv = dequant(ck), dequant(cv)
        ck = ck.float().expand(-1, -1, -1, HPG, -1)
        cv = cv.float().expand(-1, -1, -1, HPG, -1)
        ro, _ = oracle.ref_attention_with_lse(xq.float().cpu(), ck, cv, bias)
        err = (out.float().cpu() - ro).abs().max().item()
        assert err <= ATOL_O[dtype], f"{what}, layer {layer}: attention error {err:.3e}"
        assert torch.isfinite(out.float()).all()


def _run_loop(dev, dtype, prompts, gen_length, make_caches, make_bias, checker):
    """generate.py:100-187 with the toy model; returns the generated tokens [gen_length, bs]."""
    bs = len(prompts)
    prompt_lens = [len(p) for p in prompts]
    max_seq_length = max(prompt_lens) + gen_length
    model = ToyModel(dev, dtype)
    caches = make_caches(bs, max_seq_length)
    bias = make_bias(prompt_lens, max_seq_length)
    graph = torch.cuda.CUDAGraph()
    q_seqstart = bias.q_seqinfo.seqstart
    kv_seqlen = bias.k_seqinfo.seqlen
    tokens = torch.tensor(sum(prompts, []), dtype=torch.int32, device=dev)
    out_tokens = torch.zeros((gen_length, bs), dtype=torch.int32)
    q_lens, kv_lens = list(prompt_lens), list(prompt_lens)
    replays = 0
    output = None
    for niter in range(gen_length):
        if niter <= GRAPH_WARMUPS:
            output = model.forward(tokens, bias, caches)
        elif niter == GRAPH_WARMUPS + 1:
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                output = model.forward(tokens, bias, caches)
            graph.replay()
        else:
            graph.replay()
            replays += 1
        torch.cuda.synchronize()
        checker(model, caches, q_lens, kv_lens, max_seq_length, f"step {niter}")
        if niter == 0:
            last = torch.tensor([sum(prompt_lens[: i + 1]) - 1 for i in range(bs)], device=dev)
            logits = output[last]
        else:
            logits = output.view(bs, VOCAB)
        next_token = torch.argmax(logits.float(), dim=-1).int().reshape(bs)
        out_tokens[niter] = next_token.cpu()
        # the bias object is updated in place for the decoding rounds (generate.py:174-185)
        if niter == 0:
            q_seqstart.copy_(torch.arange(bs + 1, dtype=torch.int32))
            bias.q_seqinfo.min_seqlen = 1
            bias.q_seqinfo.max_seqlen = 1
            bias.q_seqinfo.seqstart_py = q_seqstart.tolist()
            tokens = tokens[:bs]
            q_lens = [1] * bs
        kv_seqlen.add_((kv_seqlen < max_seq_length).int())
        kv_lens = [min(n + 1, max_seq_length) for n in kv_lens]
        tokens.copy_(next_token)
    assert replays >= 8
    assert fmha.b200.prefill_device_status() == 0 and fmha.b200_splitk.decode_device_status() == 0
    return out_tokens


@gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_generation_loop_padded_cache_under_cuda_graph(dtype):
    require_cuda()
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, VOCAB, (n,), generator=g).tolist() for n in (17, 5, 300)]

    def make_caches(bs, max_len):
        return [tuple(torch.zeros(1, bs * max_len, N_KV, 1, HD, dtype=dtype, device=dev) for _ in range(2)) for _ in range(N_LAYERS)]

    def make_bias(prompt_lens, max_len):
        return ab.BlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(q_seqlen=prompt_lens, kv_seqlen=prompt_lens, kv_padding=max_len, device=dev)

    def checker(model, caches, q_lens, kv_lens, padding, what):
        _check_layers(model, caches, q_lens, kv_lens, padding, dtype, what)

    toks = _run_loop(dev, dtype, prompts, 12, make_caches, make_bias, checker)
    # the loop is deterministic: a second run generates the same tokens
    assert torch.equal(toks, _run_loop(dev, dtype, prompts, 12, make_caches, make_bias, checker))


@gpu
def test_generation_loop_paged_int4_cache_under_cuda_graph():
    """Same loop over a paged pool in the int4 row-wise format that rope_padded
    writes itself; quantised caches are read by the split-K operator, which takes
    the same number of queries for every sequence, so the prompts are equally long."""
    require_cuda()
    dev, dtype = torch.device("cuda"), torch.bfloat16
    g = torch.Generator().manual_seed(4)
    bs, plen, gen, page = 4, 6, 12, 16
    prompts = [torch.randint(0, VOCAB, (plen,), generator=g).tolist() for _ in range(bs)]
    pages_per_seq = -(-(plen + gen) // page)
    table = torch.randperm(bs * pages_per_seq, generator=g).int().view(bs, pages_per_seq).to(dev)

    def make_caches(bs_, max_len):
        return [tuple(torch.zeros(1, bs_ * pages_per_seq * page, N_KV, 1, 1 + HD // 8, dtype=torch.int32, device=dev) for _ in range(2))
                for _ in range(N_LAYERS)]

    def make_bias(prompt_lens, max_len):
        return ab.PagedBlockDiagonalCausalWithOffsetPaddedKeysMask.from_seqlens(prompt_lens, prompt_lens, table, page)

    def checker(model, caches, q_lens, kv_lens, padding, what):
        _check_layers(model, caches, q_lens, kv_lens, pages_per_seq * page, dtype, what, dequant=oracle.dequantize_kv_int4, table=table, page=page)

    toks = _run_loop(dev, dtype, prompts, gen, make_caches, make_bias, checker)
    assert toks.shape == (gen, bs)
