"""IR-level known answers for the immut:: operators: graphs written as IR text must parse against the registered schema
strings and compute what ATen's view + copy_ compute.

The five cases restate test/test_immut_tensorexpr.py:11-95 of the reference (same operators, shapes and argument
values: select / select_rev / slice / slice_rev / unsqueeze on [10,20] and [3000,4] fp32).  The reference checks its NNC
kernel against the NNC fallback; here the graph runs through the registered operators (CPU test kernels here, the CUDA
kernels in the gpu-marked twin) and is compared with the aten:: formulation."""
import pytest
import torch

import oracle.immut_cpu  # noqa: F401  (test-only CPU kernels)
from functs_b200 import _C

CASES = [
    # name, tensor inputs (name, shape), int inputs, constants, op line, result shape, args, aten reference
    ("select", [("x", (10, 20))], ["i"], {"d": 0}, "immut::select(%x, %d, %i)", (20,), (0,),
     lambda x, i: x.select(0, i).clone()),
    ("select_rev", [("x", (3000, 4)), ("s", (3000,))], ["i"], {"d": 1}, "immut::select_rev(%x, %s, %d, %i)", (3000, 4), (0,),
     lambda x, s, i: _assign(x, lambda v: v.select(1, i), s)),
    ("slice", [("x", (3000, 4))], ["a", "b", "c"], {"d": 1}, "immut::slice(%x, %d, %a, %b, %c)", (3000, 1), (0, 3, 4),
     lambda x, a, b, c: x[:, a:b:c].clone()),
    ("slice_rev", [("x", (3000, 4)), ("s", (3000, 1))], ["a", "b", "c"], {"d": 1},
     "immut::slice_rev(%x, %s, %d, %a, %b, %c)", (3000, 4), (0, 3, 4),
     lambda x, s, a, b, c: _assign(x, lambda v: v[:, a:b:c], s)),
    ("unsqueeze", [("x", (3000, 4))], [], {"d": 0}, "immut::unsqueeze(%x, %d)", (1, 3000, 4), (),
     lambda x: x.unsqueeze(0).clone()),
]


def _assign(x, view, src):
    out = x.clone()
    view(out).copy_(src)
    return out


def _strides(shape):
    st, acc = [], 1
    for n in reversed(shape):
        st.append(acc)
        acc *= n
    return list(reversed(st))


def _ttype(shape, device):
    return f"Float({', '.join(map(str, shape))}, strides=[{', '.join(map(str, _strides(shape)))}], device={device})"


def build_ir(case, device):
    name, tensors, ints, consts, op, rshape, _, _ = case
    params = [f"%{n} : {_ttype(s, device)}" for n, s in tensors] + [f"%{n} : int" for n in ints]
    lines = [f"graph({', '.join(params)}):"]
    for k, v in consts.items():
        lines.append(f"  %{k} : int = prim::Constant[value={v}]()")
    lines.append(f"  %r : {_ttype(rshape, device)} = {op}")
    lines.append("  return (%r)")
    return "\n".join(lines)


def run_case(case, device):
    name, tensors, ints, consts, op, rshape, args, ref = case
    g = torch.parse_ir(build_ir(case, "cpu" if device == "cpu" else "cuda:0"))
    assert any(n.kind().startswith("immut::") for n in g.nodes())
    fn = _C._create_function_from_graph(f"immut_ir_{name}", g)
    gen = torch.Generator().manual_seed(11)
    xs = [torch.rand(*s, generator=gen).to(device) for _, s in tensors]
    before = [x.clone() for x in xs]
    got = fn(*xs, *args)
    want = ref(*xs, *args)
    assert got.shape == torch.Size(rshape)
    assert torch.equal(got, want), name
    for a, b in zip(xs, before):
        assert torch.equal(a, b), "immut:: operators never write into their inputs"


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_immut_ir_known_answers_cpu(case):
    run_case(case, "cpu")


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_immut_ir_known_answers_cuda(case, cuda_device):
    run_case(case, "cuda")
