"""ParallelizeLoops / FuseOps / functor lowering and the tssa::ParallelFunctor operator, on CPU graphs.

The passes only rewrite graphs; the functor operator interprets its subgraph through a GraphExecutor, for which the
test-only CPU kernels of the immut:: operators (oracle/immut_cpu.py) are enough.  Results are compared with eager
execution of the same Python function."""
from typing import List

import pytest
import torch

import oracle.immut_cpu  # noqa: F401  (test-only CPU implementations of immut::)

fjit = pytest.importorskip("functs_b200.jit")
from functs_b200 import _C  # noqa: E402


def kinds(g, recursive=True):
    out = []

    def walk(block):
        for n in block.nodes():
            out.append(n.kind())
            if recursive:
                for b in n.blocks():
                    walk(b)
    walk(g)
    return out


def scales_decode(feats: List[torch.Tensor], offs: List[torch.Tensor]):
    outs: List[torch.Tensor] = []
    for i in range(3):
        x = feats[i].clone()
        x[:, 0:2] = torch.sigmoid(x[:, 0:2]) + offs[i]
        x[:, 2:4] = torch.exp(x[:, 2:4]) * 2.0
        outs.append(x * 8.0)  # the mutated tensor itself does not escape into the list
    return outs


def carried(b: torch.Tensor, n: int):
    b = b.clone()
    for i in range(n):
        b[i] = b[i] + 1
    return b


def dependent(xs: List[torch.Tensor]):
    outs: List[torch.Tensor] = []
    acc = torch.zeros_like(xs[0])
    for i in range(len(xs)):
        acc = acc + xs[i]
        outs.append(acc * 2.0)
    return outs


def reads_own_output(xs: List[torch.Tensor]):
    outs: List[torch.Tensor] = [xs[0]]
    for i in range(1, len(xs)):
        outs.append(outs[i - 1] + xs[i])
    return outs


def make_lists():
    g = torch.Generator().manual_seed(3)
    feats = [torch.randn(5 + i, 6, generator=g) for i in range(3)]
    offs = [torch.randn(5 + i, 2, generator=g) for i in range(3)]
    return feats, offs


def test_independent_loop_becomes_one_parallel_functor():
    feats, offs = make_lists()
    want = scales_decode(feats, offs)
    fn = fjit.build(scales_decode, (feats, offs))
    ks = kinds(fn.graph)
    assert "prim::Loop" not in ks and "tssa::ParallelMap" not in ks
    assert ks.count("tssa::ParallelFunctor") == 1 and fjit.count_groups(fn.graph) == 1
    node = [n for n in fn.graph.nodes() if n.kind() == "tssa::ParallelFunctor"][0]
    assert node.i("is_parallel_map") == 1 and node.i("parallel_degree") == 3
    assert list(getattr(node, "is")("is_parallel_args")) == [1, 1]
    sub = node.g("Subgraph")
    assert str(list(sub.inputs())[0].type()) == "int"
    sub_kinds = [n.kind() for n in sub.nodes()]
    assert "immut::slice_rev" in sub_kinds and "aten::sigmoid" in sub_kinds and "aten::copy_" not in sub_kinds
    got = fn(feats, offs)
    assert len(got) == 3
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    # inputs are not modified (the clone inside the loop is part of the group)
    feats2, _ = make_lists()
    for a, b in zip(feats, feats2):
        assert torch.equal(a, b)


def test_parallelize_loops_alone_and_back():
    g = torch.jit.script(scales_decode).graph.copy()  # torch.jit.script caches: never edit the cached graph
    torch._C._jit_pass_inline(g)
    _C._jit_pass_convert_to_tensorssa(g)
    _C._jit_pass_tensorssa_remove_update(g)
    _C._jit_pass_parallelize_loops(g)
    ks = kinds(g, recursive=False)
    assert "tssa::ParallelMap" in ks and "prim::Loop" not in ks
    m = [n for n in g.nodes() if n.kind() == "tssa::ParallelMap"][0]
    assert len(list(m.inputs())) == 3 and len(list(m.outputs())) == 1  # trip count + two lists -> one list
    body = list(m.blocks())[0]
    assert len(list(body.inputs())) == 3 and len(list(body.outputs())) == 1
    assert "aten::__getitem__" not in kinds(g) and "aten::append" not in kinds(g)
    # without grouping, lowering turns the map back into an equivalent loop
    _C._jit_pass_lower_to_parallel_functors(g)
    ks = kinds(g)
    assert "tssa::ParallelMap" not in ks and "prim::Loop" in ks and "aten::append" in ks
    feats, offs = make_lists()
    want = scales_decode(feats, offs)
    got = _C._create_function_from_graph("lowered", g)(feats, offs)
    for a, b in zip(got, want):
        assert torch.equal(a, b)


@pytest.mark.parametrize("fn", [dependent, reads_own_output])
def test_loops_with_dependences_stay_loops(fn):
    g = torch.Generator().manual_seed(4)
    xs = [torch.randn(4, 3, generator=g) for _ in range(4)]
    want = fn(xs)
    built = fjit.build(fn, (xs,))
    ks = kinds(built.graph)
    assert "prim::Loop" in ks and "tssa::ParallelMap" not in ks
    got = built(xs)
    for a, b in zip(got, want):
        assert torch.equal(a, b)


def test_carried_row_loop_is_matched_to_the_precompiled_group():
    b = torch.randn(6, 5)
    fn = fjit.build(carried, (b, 6))
    nodes = [n for n in fn.graph.nodes() if n.kind() == "tssa::ParallelFunctor"]
    assert len(nodes) == 1 and "prim::Loop" not in kinds(fn.graph, recursive=False)
    assert nodes[0].s("kernel_signature") == "loop[i<n]{immut::select(b,0,i)->aten::add(.,c)->immut::select_rev(b,.,0,i)}"
    assert nodes[0].i("is_parallel_map") == 0
    # CPU tensors: the operator interprets the subgraph (the precompiled kernel only takes CUDA fp32 matrices)
    assert torch.equal(fn(b, 6), carried(b, 6))
    assert torch.equal(fn(b, 4), carried(b, 4))


def test_plain_group_outside_loops():
    def f(x: torch.Tensor, y: torch.Tensor):
        z = x.clone()
        z[1] = torch.sigmoid(y[0]) * 3.0
        return z + 1.0

    x, y = torch.randn(4, 3), torch.randn(2, 3)
    fn = fjit.build(f, (x, y))
    nodes = [n for n in fn.graph.nodes() if n.kind() == "tssa::ParallelFunctor"]
    assert len(nodes) == 1 and nodes[0].i("is_parallel_map") == 0
    assert str(list(nodes[0].g("Subgraph").inputs())[0].type()) == "NoneType"
    assert torch.equal(fn(x, y), f(x, y))


def test_pass_api_names():
    for name in ("_jit_pass_fait_pipeline", "_jit_pass_fait_fuse_ops", "_jit_pass_fait_shape_infer", "_jit_pass_freeze",
                 "_jit_pass_clone", "_create_function_from_graph", "_jit_pass_parallelize_loops"):
        assert hasattr(_C, name), name
    g = torch.jit.script(carried).graph.copy()
    f = _C._create_function_from_graph("roundtrip", g)
    assert torch.equal(f(torch.ones(3, 2), 2), carried(torch.ones(3, 2), 2))


def test_shape_inference_through_immut_ops():
    """_jit_pass_fait_shape_infer: type hints on the inputs, TorchScript's propagation for aten:: ops and the immut::
    table for the Access / Assign family; the inferred sizes must be those of an actual run."""
    def f(x: torch.Tensor, y: torch.Tensor):
        z = x.clone()
        z[:, 1:7:2] = torch.sigmoid(y).unsqueeze(1).expand(-1, 3)
        w = z.permute(1, 0)[2:5]
        return w * 2.0, z[3] + 1.0  # only values of pure ops leave the graph

    x, y = torch.randn(10, 8), torch.randn(10)
    g = torch.jit.script(f).graph.copy()
    torch._C._jit_pass_inline(g)
    _C._jit_pass_convert_to_tensorssa(g)
    _C._jit_pass_tensorssa_remove_update(g)
    torch._C._jit_pass_dce(g)
    torch._C._jit_pass_constant_propagation(g)
    hints = [torch._C.TensorType.create_from_tensor(t) for t in (x, y)]
    _C._jit_pass_fait_shape_infer(g, hints)
    seen = {}
    for n in g.nodes():
        if n.kind().startswith("immut::"):
            sizes = n.output().type().sizes()
            assert sizes is not None, f"{n.kind()} has no static shape"
            seen.setdefault(n.kind(), []).append(tuple(sizes))
    assert "immut::slice_rev" in seen and all(s == (10, 8) for s in seen["immut::slice_rev"])
    assert (8, 10) in seen.get("immut::permute", [])
    assert (3, 10) in seen.get("immut::slice", [])
    assert (8,) in seen.get("immut::select", [])
    out_sizes = [tuple(o.type().sizes()) for o in g.outputs()] if len(list(g.outputs())) > 1 else None
    fn = _C._create_function_from_graph("shapes", g)
    got = fn(x, y)
    want = f(x, y)
    for a, b in zip(got, want):
        assert torch.equal(a, b) and a.shape == b.shape


def test_constant_trip_loop_with_carried_tensor_is_unrolled_into_one_group():
    def f(x: torch.Tensor, w: torch.Tensor):
        acc = x.clone()
        for i in range(4):
            acc[i] = torch.tanh(acc[i] * w[i]) + 1.0
        return acc * 0.5

    x, w = torch.randn(6, 5), torch.randn(4, 5)
    fn = fjit.build(f, (x, w))
    ks = kinds(fn.graph)
    assert "prim::Loop" not in ks
    assert fjit.count_groups(fn.graph) == 1  # all four iterations and the epilogue in one fusion group
    assert torch.equal(fn(x, w), f(x, w))


def split_body(feats: List[torch.Tensor]):
    outs: List[torch.Tensor] = []
    for i in range(len(feats)):
        x = feats[i].clone()
        x[:, 0:2] = torch.sigmoid(x[:, 0:2]) * 2.0   # first group
        s = x.sum()                                    # a reduction: not fusable, stays between the groups
        y = x * 3.0 + s                                # second group, reads the per-iteration value s
        outs.append(torch.tanh(y))
    return outs


def test_map_with_two_groups_is_split():
    """SplitParallelMaps: the map body [group, sum, group] becomes map{group} -> loop{sum} -> map{group}; the two group maps
    turn into functors with is_parallel_map = 1, the values between them travel as lists."""
    feats, _ = make_lists()
    want = split_body(feats)
    fn = fjit.build(split_body, (feats,))
    functors = [n for n in fn.graph.nodes() if n.kind() == "tssa::ParallelFunctor"]
    assert len(functors) == 2 and all(n.i("is_parallel_map") == 1 for n in functors)
    ks = kinds(fn.graph, recursive=False)
    assert ks.count("prim::Loop") == 1 and "tssa::ParallelMap" not in ks
    loop = [n for n in fn.graph.nodes() if n.kind() == "prim::Loop"][0]
    assert "aten::sum" in [n.kind() for n in list(loop.blocks())[0].nodes()]
    got = fn(feats)
    assert len(got) == len(want)
    for a, b in zip(got, want):
        assert torch.allclose(a, b, rtol=1e-6, atol=1e-6)


def test_fuse_tensorexpr_entry_point_groups_a_functionalized_graph():
    """_jit_pass_fuse_tensorexpr (the reference binds this name, functs/csrc/jit/python/init.cpp:40-42): groups of a
    functionalized graph become tssa::ParallelFunctor nodes."""
    def f(x: torch.Tensor):
        t = x.clone()
        t[0] = torch.sigmoid(t[0]) * 2.0
        return t + 1.0
    g = torch.jit.script(f).graph.copy()
    fjit.functionalize_graph(g)
    _C._jit_pass_fuse_tensorexpr(g)
    assert "tssa::ParallelFunctor" in kinds(g) and "aten::sigmoid" not in kinds(g, recursive=False)
    fn = torch._C._create_function_from_graph("f", g)
    x = torch.randn(4, 5, generator=torch.Generator().manual_seed(1))
    assert torch.allclose(fn(x), f(x))


def test_shape_inference_refines_lists_of_tensors():
    """Tuple type hints describe the elements of List[Tensor] inputs; list[i] with a constant index, the element
    parameters of a map and cat / stack over a list take their types from there (the reference's refined list types)."""
    def heads(feats: List[torch.Tensor]):
        a = feats[0] * 2.0
        b = torch.cat(feats, dim=0)
        return a, b
    feats, _ = make_lists()
    g = torch.jit.script(heads).graph.copy()
    refined = fjit.shape_infer(g, (feats,))
    assert any(t.kind() == "TupleType" for t in refined.values())
    by_kind = {n.kind(): n for n in g.nodes()}
    assert by_kind["aten::__getitem__"].output().type().sizes() == [5, 6]
    assert by_kind["aten::mul"].output().type().sizes() == [5, 6]
    assert by_kind["aten::cat"].output().type().sizes() == [5 + 6 + 7, 6]
    # inside the pipeline: the element parameters of the map over scales get the unified element type (rank and dtype known,
    # the row count differs per scale)
    g2 = torch.jit.script(scales_decode).graph.copy()
    fjit.functionalize_graph(g2)
    _C._jit_pass_parallelize_loops(g2)
    fjit.shape_infer(g2, make_lists())
    m = [n for n in g2.nodes() if n.kind() == "tssa::ParallelMap"][0]
    params = list(list(m.blocks())[0].inputs())
    assert params[1].type().dim() == 2 and params[1].type().scalarType() == "Float"
    assert params[1].type().sizes() is None or params[1].type().sizes()[1] == 6


def captures_outer(feats: List[torch.Tensor], w: torch.Tensor):
    outs: List[torch.Tensor] = []
    for i in range(3):
        outs.append(feats[i] * w)
    return outs


def test_unroll_simple_maps():
    """A map with a constant trip count and a self-contained body is written out per index (list[i] reads, one
    ListConstruct); a map that captures an outer tensor is not simple and stays (fait/passes/parallelize_loops.cpp:372-392)."""
    g = torch.jit.script(scales_decode).graph.copy()
    torch._C._jit_pass_inline(g)
    _C._jit_pass_convert_to_tensorssa(g)
    _C._jit_pass_tensorssa_remove_update(g)
    _C._jit_pass_parallelize_loops(g)
    assert "tssa::ParallelMap" in kinds(g, recursive=False)
    _C._jit_pass_unroll_simple_maps(g)
    ks = kinds(g)
    assert "tssa::ParallelMap" not in ks and "prim::Loop" not in ks
    assert ks.count("aten::__getitem__") == 6 and ks.count("aten::sigmoid") == 3 and ks.count("prim::ListConstruct") >= 1
    torch._C._jit_pass_lint(g)
    feats, offs = make_lists()
    want = scales_decode(feats, offs)
    got = _C._create_function_from_graph("unrolled", g)(feats, offs)
    for a, b in zip(got, want):
        assert torch.equal(a, b)

    g2 = torch.jit.script(captures_outer).graph.copy()
    torch._C._jit_pass_inline(g2)
    _C._jit_pass_convert_to_tensorssa(g2)
    _C._jit_pass_parallelize_loops(g2)
    assert "tssa::ParallelMap" in kinds(g2, recursive=False)
    _C._jit_pass_unroll_simple_maps(g2)
    assert "tssa::ParallelMap" in kinds(g2, recursive=False)


def test_json_input_type_specs():
    """The reference's JSON type specs (fait/models/*.json format) become the type hints the pipeline takes."""
    from functs_b200 import jit as J
    spec = """[
      {"kind": "TupleType", "elements": [
        {"kind": "TensorType", "shape": [5, 6], "dtype": "Float"},
        {"kind": "TensorType", "shape": [6, 6], "dtype": "Float"},
        {"kind": "TensorType", "shape": [7, 6], "dtype": "Float"}]},
      {"kind": "ListType", "element": {"kind": "TensorType", "shape": [5, 2], "dtype": "Float"}},
      {"kind": "IntType"}, {"kind": "BoolType"}, {"kind": "FloatType"},
      {"kind": "TensorType", "shape": [3, 4], "dtype": "Long"}
    ]"""
    hints = J.parse_input_types(spec, device="cpu")
    assert len(hints) == 6
    assert isinstance(hints[0], torch._C.TupleType) and [e.sizes() for e in hints[0].elements()] == [[5, 6], [6, 6], [7, 6]]
    assert hints[0].elements()[0].dtype() == torch.float32
    assert isinstance(hints[1], torch._C.ListType) and hints[1].getElementType().sizes() == [5, 2]
    assert str(hints[2]) == "int" and str(hints[3]) == "bool" and str(hints[4]) == "float"
    assert hints[5].dtype() == torch.int64 and hints[5].sizes() == [3, 4]
    # the tuple hint refines a list input: shapes flow into the map's element parameters
    g = torch.jit.script(scales_decode).graph.copy()
    torch._C._jit_pass_inline(g)
    _C._jit_pass_convert_to_tensorssa(g)
    _C._jit_pass_tensorssa_remove_update(g)
    offs = J.parse_input_types('[{"kind": "TupleType", "elements": [{"kind": "TensorType", "shape": [5, 2], "dtype": "Float"},'
                               '{"kind": "TensorType", "shape": [6, 2], "dtype": "Float"},'
                               '{"kind": "TensorType", "shape": [7, 2], "dtype": "Float"}]}]', device="cpu")
    refined = _C._jit_pass_fait_shape_infer(g, [hints[0], offs[0]])
    assert any(isinstance(t, torch._C.TupleType) for t in refined.values())
    with pytest.raises(ValueError):
        J.parse_input_types('[{"kind": "DictType"}]')
