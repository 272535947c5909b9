"""The forward operator as a ``torch.library`` op (schemas of
xformers/ops/fmha/__init__.py:72-103): shapes through the Meta implementation,
fake tensors, the FLOP formula (in the manner of tests/test_fmha_flop_formula.py)
and, on a GPU, equality with the Python entry point and capture by torch.compile
without graph breaks."""

import pytest
import torch
from torch.utils.flop_counter import FlopCounterMode

import xformers_b200.ops as xops  # noqa: F401  (registers the ops)
from xformers_b200.ops import fmha
from xformers_b200.ops.fmha import torch_library


def test_namespaces_and_schemas():
    assert "xformers_b200" in torch_library.NAMESPACES
    for ns in torch_library.NAMESPACES:
        ops = getattr(torch.ops, ns)
        s = str(ops.memory_efficient_attention_forward.default._schema)
        assert "Tensor q, Tensor k, Tensor v, Tensor? b=None, float? p=0., float? scale=None" in s
        s = str(ops.memory_efficient_attention_forward_with_bias.default._schema)
        assert "Tensor q, Tensor k, Tensor v, Tensor b," in s


@pytest.mark.parametrize("shape_q,shape_kv,kv", [
    ((2, 128, 4, 64), (2, 256, 4, 64), 32),
    ((3, 13, 2, 7, 128), (3, 17, 2, 7, 128), 128),
    ((6, 40, 64), (6, 24, 64), 64),
])
def test_meta_and_flops(shape_q, shape_kv, kv):
    q = torch.empty(shape_q, device="meta", dtype=torch.bfloat16)
    k = torch.empty(shape_kv, device="meta", dtype=torch.bfloat16)
    v = torch.empty(shape_kv[:-1] + (kv,), device="meta", dtype=torch.bfloat16)
    with FlopCounterMode(display=False) as fc:
        out = torch.ops.xformers_b200.memory_efficient_attention_forward(q, k, v)
    assert out.shape == shape_q[:-1] + (kv,) and out.dtype == torch.bfloat16
    heads = 1
    for n in shape_q[2:-1]:
        heads *= n
    assert fc.get_total_flops() == 2 * shape_q[0] * heads * shape_q[1] * shape_kv[1] * (shape_q[-1] + kv)


def test_no_cpu_kernel():
    q = torch.zeros(1, 8, 1, 64)
    with pytest.raises(NotImplementedError):
        torch.ops.xformers_b200.memory_efficient_attention_forward(q, q, q)


@pytest.mark.gpu
def test_matches_python_entry_point_and_compiles():
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(2, 256, 4, 128, generator=g, device=dev, dtype=torch.bfloat16)
    k = torch.randn(2, 384, 4, 128, generator=g, device=dev, dtype=torch.bfloat16)
    v = torch.randn(2, 384, 4, 128, generator=g, device=dev, dtype=torch.bfloat16)
    want = fmha.memory_efficient_attention_forward(q, k, v, scale=0.1)
    got = torch.ops.xformers_b200.memory_efficient_attention_forward(q, k, v, None, 0.0, 0.1)
    assert torch.equal(got, want)
    bias = torch.randn(2, 4, 256, 384, generator=g, device=dev, dtype=torch.bfloat16)
    want_b = fmha.memory_efficient_attention_forward(q, k, v, bias)
    got_b = torch.ops.xformers_b200.memory_efficient_attention_forward_with_bias(q, k, v, bias)
    assert torch.equal(got_b, want_b)

    def f(q, k, v):
        return torch.ops.xformers_b200.memory_efficient_attention_forward(q, k, v, None, 0.0, 0.1).float() * 2

    compiled = torch.compile(f, fullgraph=True, backend="aot_eager")
    torch.testing.assert_close(compiled(q, k, v), want.float() * 2)


def test_merge_varargs_custom_op_is_registered_with_a_fake():
    s = str(torch.ops.xformers_b200.fmha_merge_attentions_varargs.default._schema)
    assert "Tensor[] attn_split, Tensor[] lse_split, bool write_lse=True, ScalarType? output_dtype=None" in s
    a = [torch.empty(2, 5, 3, 4, 64, device="meta") for _ in range(3)]
    l = [torch.empty(2, 3, 4, 5, device="meta") for _ in range(3)]
    out, lse = torch.ops.xformers_b200.fmha_merge_attentions_varargs(a, l, True, torch.bfloat16)
    assert out.shape == (2, 5, 3, 4, 64) and out.dtype == torch.bfloat16 and lse.shape == (2, 3, 4, 5)


@pytest.mark.gpu
def test_merge_varargs_compiles_without_graph_break():
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    a = [torch.randn(2, 5, 3, 4, 64, generator=g, device=dev) for _ in range(3)]
    l = [torch.randn(2, 3, 4, 5, generator=g, device=dev) for _ in range(3)]
    want_o, want_l = fmha.merge_attentions(a, l)

    def f(a0, a1, a2, l0, l1, l2):
        o, lse = fmha.merge_attentions_varargs([a0, a1, a2], [l0, l1, l2])
        return o * 2, lse

    compiled = torch.compile(f, fullgraph=True, backend="aot_eager")
    o, lse = compiled(*a, *l)
    torch.testing.assert_close(o, want_o * 2)
    torch.testing.assert_close(lse, want_l)
    o2, none = fmha.merge_attentions_varargs(a, l, write_lse=False)
    assert none is None and torch.equal(o2, want_o)
