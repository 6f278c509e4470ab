"""TensorSSA functionalization passes (functs_b200._C) on CPU.

Programs restate the reference's functionalization tests (test/test_basic.py:6-38: dataflow, loop, branch,
branch_loop) and examples/get_started.py:10-27; as there, the functionalized graph must compute what the eager
program computes.  The graphs run on CPU through test-only kernels for the immut:: operators (oracle/immut_cpu.py);
the product registers CUDA kernels only.  IR known answers follow the reference README's printed graphs
(README.md:284-299: clone -> Loop{ immut::select -> add -> immut::select_rev } with the tensor loop-carried).
"""
import pytest
import torch

from functs_b200 import _C, jit as fjit
import oracle.immut_cpu  # noqa: F401  (CPU kernels for immut::*, test infrastructure)


def kinds(block):
    out = []
    for n in block.nodes():
        out.append(n.kind())
        for b in n.blocks():
            out.extend(kinds(b))
    return out


def fresh_graph(fn):
    """torch.jit.script caches the compiled function per Python function: work on a copy of its graph."""
    return torch.jit.script(fn).graph.copy()


def functionalize(fn, **kw):
    g = fresh_graph(fn)
    fjit.functionalize_graph(g, **kw)
    return torch._C._create_function_from_graph(fn.__name__, g)


def get_started(a: torch.Tensor, b: torch.Tensor, n: int):
    a = a.clone()
    b = b.clone()
    for i in range(n):
        b[i] = b[i] + 1
    return b


def data_control_flow(a: torch.Tensor, b: torch.Tensor, idx: int):
    a = a.clone()
    b = b.clone()
    if idx >= 0:
        a = a + 1
        b[idx].copy_(a[idx])
    else:
        a = a - 1
        b[-idx].copy_(a[-idx])
    return a + b


def dataflow(a: torch.Tensor, b: torch.Tensor):
    a = a.clone()
    a[0].copy_(b[0])
    a[1].copy_(b[1])
    a[0:1] = b[0:1]
    return a + a[0:1]


def loop(a: torch.Tensor, b: torch.Tensor):
    a = a.clone()
    for i in range(10):
        a[i].copy_(b[i + 1])
    return a


def branch(a: torch.Tensor, b: torch.Tensor, cond: int):
    a = a.clone()
    tmp_1 = a[1]
    if cond > 0:
        tmp_1.copy_(b[0])
    else:
        tmp_1.copy_(b[1] * 2)
    return a


def branch_loop(a: torch.Tensor, c: torch.Tensor, d: torch.Tensor):
    tmp_0 = d.clone()
    tmp_1 = tmp_0[1]
    if a.nonzero().sum():
        tmp_0 = tmp_0 + 1
        for i in range(10):
            tmp_1.copy_(tmp_0[i + 1])
    else:
        tmp_0 = tmp_0 + tmp_1
        tmp_1.copy_(tmp_0[2])
    return tmp_1 + tmp_0


def inplace_ops(x: torch.Tensor, y: torch.Tensor):
    t = x.clone()
    t[..., 0:2].sigmoid_()
    t[:, 1::2].clamp_(min=0.1, max=0.6)
    t[2].add_(y[2])
    u = t.permute(1, 0)
    u[0] = u[0] * 3
    return t, u


def nested_views(x: torch.Tensor):
    t = x.clone()
    row = t[1]
    cell = row[2:5]
    cell[1] = 7.0
    v = t.unsqueeze(0)
    v[0, 3] = row * 2
    return t + row.sum() + v.squeeze(0)


def untouched_input_mutation(a: torch.Tensor, b: torch.Tensor):
    # graph inputs alias memory the caller owns: like the reference, the passes leave such writes alone
    a[0].copy_(b[0])
    return a * 2


def rnd(*shape, seed=0):
    return torch.rand(*shape, generator=torch.Generator().manual_seed(seed + sum(shape)))


CASES = [
    (get_started, lambda: (rnd(8, 16), rnd(8, 16, seed=1), 5)),
    (data_control_flow, lambda: (rnd(6, 4), rnd(6, 4, seed=1), 2)),
    (data_control_flow, lambda: (rnd(6, 4), rnd(6, 4, seed=1), -3)),
    (dataflow, lambda: (rnd(32, 8), rnd(32, 8, seed=1))),
    (loop, lambda: (rnd(16, 8), rnd(16, 8, seed=1))),
    (branch, lambda: (rnd(4, 8), rnd(4, 8, seed=1), 1)),
    (branch, lambda: (rnd(4, 8), rnd(4, 8, seed=1), -1)),
    (branch_loop, lambda: (torch.ones(3), rnd(2, 2), rnd(12, 5, seed=2))),
    (branch_loop, lambda: (torch.zeros(3), rnd(2, 2), rnd(12, 5, seed=2))),
    (inplace_ops, lambda: (rnd(6, 8), rnd(6, 8, seed=3))),
    (nested_views, lambda: (rnd(5, 6),)),
    (untouched_input_mutation, lambda: (rnd(4, 4), rnd(4, 4, seed=1))),
]


@pytest.mark.parametrize("fn,make", CASES, ids=[f"{c[0].__name__}-{i}" for i, c in enumerate(CASES)])
def test_functionalized_graph_equals_eager(fn, make):
    f = functionalize(fn)
    want = fn(*make())
    got = f(*make())
    if isinstance(want, tuple):
        assert all(torch.equal(g, w) for g, w in zip(got, want))
    else:
        assert torch.equal(got, want)


def test_no_mutation_left_in_owned_memory():
    for fn in (get_started, data_control_flow, dataflow, loop, branch, branch_loop, inplace_ops, nested_views):
        ks = kinds(functionalize(fn).graph)
        assert "aten::copy_" not in ks, fn.__name__
        assert not any(k.endswith("_") and k.startswith("aten::") for k in ks), (fn.__name__, ks)
        assert "tssa::update" not in ks and "immut::assign" not in ks


def test_get_started_known_answer():
    g = functionalize(get_started).graph
    assert kinds(g) == ["prim::Constant"] * 4 + ["aten::clone", "prim::Loop", "immut::select", "aten::add", "immut::select_rev"]
    loop_node = [n for n in g.nodes() if n.kind() == "prim::Loop"][0]
    assert len(list(loop_node.inputs())) == 3 and len(list(loop_node.outputs())) == 1  # b became loop-carried
    body = list(loop_node.blocks())[0]
    assert [v.type().kind() for v in body.inputs()] == ["IntType", "TensorType"]


def test_step_by_step_api_and_mutate_info():
    g = fresh_graph(get_started)
    torch._C._jit_pass_inline(g)
    info = _C.TensorSSAMutateInfo()
    _C._jit_pass_rewrite_mutation(g, info)
    assert len(info.mutValues) == 3          # b and its two select views
    assert sum(len(v) for v in info.mutNodes.values()) == 3
    assert kinds(g).count("tssa::update") == 3 and "immut::assign" in kinds(g)
    _C._jit_pass_block_propagation(g, info)
    assert kinds(g).count("tssa::update") == 5   # + loop parameter and loop result markers
    _C._jit_pass_rename(g)
    _C._jit_pass_tensorssa_remove_update(g)
    torch._C._jit_pass_dce(g)
    f = torch._C._create_function_from_graph("get_started", g)
    a, b = rnd(8, 16), rnd(8, 16, seed=1)
    assert torch.equal(f(a, b, 3), get_started(a, b, 3))


def test_graph_inputs_are_left_alone_unless_cloned():
    ks = kinds(functionalize(untouched_input_mutation).graph)
    assert "aten::copy_" in ks and "immut::select_rev" not in ks
    f = functionalize(untouched_input_mutation, add_clone=True)
    ks = kinds(f.graph)
    assert "aten::copy_" not in ks and "immut::select_rev" in ks
    a, b = rnd(4, 4), rnd(4, 4, seed=1)
    a_before = a.clone()
    assert torch.equal(f(a, b), untouched_input_mutation(a.clone(), b))
    assert torch.equal(a, a_before)  # with add_clone the caller's tensor is no longer written


def test_unsupported_alias_poisons_the_tree():
    def fn(x: torch.Tensor):
        t = x.clone()
        e = t[0:1].expand(3, 4)    # writing through an expanded view is ill posed: the tree is left alone
        t[0] = 1.0
        return e + t
    f = functionalize(fn)
    assert "aten::copy_" in kinds(f.graph)
    assert torch.equal(f(rnd(3, 4)), fn(rnd(3, 4)))


def test_schema_strings_match_the_reference():
    want = {
        "immut::select_rev": "immut::select_rev(Tensor self, Tensor src, int dim, int index) -> Tensor",
        "immut::slice_rev": "immut::slice_rev(Tensor self, Tensor src, int dim=0, SymInt? start=None, SymInt? end=None, SymInt step=1) -> Tensor",
        "immut::assign": "immut::assign(Tensor self, Tensor src, bool? n=None) -> Tensor",
        "immut::index": "immut::index.Tensor(Tensor self, Tensor?[] indices) -> Tensor",
        "immut::expand": "immut::expand(Tensor self, int[] size, *, bool implicit) -> Tensor",
    }
    for name, schema in want.items():
        got = [str(s) for s in torch._C._jit_get_schemas_for_operator(name)]
        assert schema in got, (name, got)
    g = torch.parse_ir("""
graph(%self : Float(3000, 4, strides=[4, 1], device=cpu),
      %src : Float(3000, strides=[1], device=cpu),
      %idx : int):
      %dim : int = prim::Constant[value=1]()
      %res : Float(3000, 4, strides=[4, 1], device=cpu) = immut::select_rev(%self, %src, %dim, %idx)
      return (%res)
""")
    fn = torch._C._create_function_from_graph("f", g)
    x, s = rnd(3000, 4), rnd(3000, seed=1)
    want_t = x.clone()
    want_t[:, 0] = s
    assert torch.equal(fn(x, s, 0), want_t)


def test_whole_tensor_copy_keeps_shape_and_dtype():
    """x.copy_(row) broadcasts and converts: after functionalization the value that replaces x must still have x's shape
    and dtype (a cast and an expand_as are inserted when the static types do not prove that src already has them)."""
    def bcast(x: torch.Tensor, row: torch.Tensor):
        x = x.clone()
        x.copy_(row)
        return x * 2

    def cast(x: torch.Tensor, i: torch.Tensor):
        x = x.clone()
        x.copy_(i)
        return x + 0.5
    for fn, args in ((bcast, (torch.rand(3, 4), torch.rand(4))), (cast, (torch.rand(2, 3), torch.arange(6).reshape(2, 3)))):
        g = torch.jit.script(fn).graph.copy()
        fjit.functionalize_graph(g)
        assert "aten::copy_" not in [n.kind() for n in g.nodes()]
        f = torch._C._create_function_from_graph(fn.__name__, g)
        got, want = f(*args), fn(*args)
        assert got.shape == want.shape and got.dtype == want.dtype and torch.equal(got, want)


def test_metadata_inplace_ops_are_left_alone():
    """unsqueeze_ / squeeze_ / t_ change the tensor's shape, not its values: RemoveInplace must not turn them into
    "view, then copy_ back"."""
    def f(x: torch.Tensor):
        y = x.clone()
        y.unsqueeze_(0)
        return y + 1
    g = torch.jit.script(f).graph.copy()
    _C._jit_pass_remove_inplace(g)
    kinds = [n.kind() for n in g.nodes()]
    assert "aten::unsqueeze_" in kinds and "aten::copy_" not in kinds
