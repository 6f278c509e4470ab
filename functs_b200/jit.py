"""Python front door, mirroring the reference's functs.jit (functs/jit/_script.py:71-108).

    script(fn, remove_update=True, enable_dce_cse=True, add_clone=False) -> torch.jit.ScriptFunction / ScriptModule

scripts `fn`, inlines, runs the TensorSSA functionalization passes of functs_b200._C on the graph in place and
(optionally) cleans up with TorchScript's own DCE / CSE / constant propagation.  The resulting graph contains
immut:: operators, which execute as CUDA launches of libfuncts_b200.so.
"""
import inspect

import torch

from . import _C  # noqa: F401  (registers the immut:: operators and exposes the passes)


def functionalize_graph(g: torch.Graph, remove_update: bool = True, enable_dce_cse: bool = True,
                        add_clone: bool = False) -> None:
    if add_clone:
        _C._jit_pass_dumb_remove_inter_precedure_mutation(g)
    torch._C._jit_pass_inline(g)
    _C._jit_pass_convert_to_tensorssa(g)
    if remove_update:
        _C._jit_pass_tensorssa_remove_update(g)
    if enable_dce_cse:
        torch._C._jit_pass_dce(g)
        torch._C._jit_pass_cse(g)
        torch._C._jit_pass_constant_propagation(g)


def script(fn, backend: str = "jit", remove_update: bool = True, enable_dce_cse: bool = True, add_clone: bool = False):
    if backend not in ("jit", "aot"):
        raise AttributeError("No backend named {}".format(backend))
    jit_fn = torch.jit.script(fn)
    if not inspect.isfunction(fn):
        jit_fn = torch.jit.freeze(jit_fn.cuda().eval())
    functionalize_graph(jit_fn.graph, remove_update, enable_dce_cse, add_clone)
    return jit_fn


def fait_pipeline(g: torch.Graph, type_hint=()) -> None:
    """Functionalize `g` (already inlined), turn independent loops into maps, group fusable ops and lower everything to
    tssa::ParallelFunctor nodes: the counterpart of the reference's _jit_pass_fait_pipeline (fait/fait.cpp pipeline
    order: TensorSSA -> ParallelizeLoops -> FuseOps -> functor nodes)."""
    torch._C._jit_pass_inline(g)
    _C._jit_pass_fait_pipeline(g, list(type_hint))


def type_hint_of(value):
    """Type hint of one example input, as the reference's extract_type_hint_from_tensor builds it (functs/jit/_script.py:
    26-45): dtype + sizes + device for a tensor, a tuple of those for a list / tuple of tensors, None otherwise."""
    if isinstance(value, torch.Tensor):
        return torch._C.TensorType.create_from_tensor(value)
    if isinstance(value, (list, tuple)) and value and all(isinstance(v, torch.Tensor) for v in value):
        return torch._C.TupleType([torch._C.TensorType.create_from_tensor(v) for v in value])
    return None


_JSON_DTYPES = {"Float": torch.float32, "Double": torch.float64, "Half": torch.float16, "BFloat16": torch.bfloat16,
                "Long": torch.int64, "Int": torch.int32, "Short": torch.int16, "Char": torch.int8, "Byte": torch.uint8,
                "Bool": torch.bool}


def parse_input_types(spec, device="cuda") -> list:
    """Type hints from the reference's JSON input-type specs (fait/models/*.json, read there by parseInputTypes,
    fait/passes/refine_types.cpp:131-177): a list of {"kind": "TensorType", "shape": [...], "dtype": "Float"} /
    {"kind": "TupleType", "elements": [...]} / {"kind": "ListType", "element": {...}} / BoolType / IntType / FloatType
    records, one per graph input.  `spec` is the JSON text, a path to such a file, or the parsed list.  Tensors are
    contiguous and live on `device`, as in the reference."""
    import json
    import os
    if isinstance(spec, (str, bytes, os.PathLike)):
        text = spec
        if not str(spec).lstrip().startswith("["):
            with open(spec) as f:
                text = f.read()
        spec = json.loads(text)

    def one(rec):
        kind = rec["kind"]
        if kind == "TensorType":
            if rec["dtype"] not in _JSON_DTYPES:
                raise ValueError(f"unknown dtype {rec['dtype']!r} in a TensorType record")
            return (torch._C.TensorType.get().with_dtype(_JSON_DTYPES[rec["dtype"]])
                    .with_sizes([int(v) for v in rec["shape"]]).with_device(torch.device(device)))
        if kind == "TupleType":
            return torch._C.TupleType([one(e) for e in rec["elements"]])
        if kind == "ListType":
            return torch._C.ListType(one(rec["element"]))
        if kind in ("BoolType", "IntType", "FloatType"):
            return getattr(torch._C, kind).get()
        raise ValueError(f"cannot parse type record of kind {kind!r}")

    return [one(rec) for rec in spec]


def shape_infer(g: torch.Graph, example_inputs=(), has_self: bool = False) -> dict:
    """Counterpart of the reference's functs.jit.shape_infer (functs/jit/_script.py:48-51): refines the graph's value types
    from example inputs in place and returns {debug name of a list value: tuple type of its elements}."""
    hints = ([None] if has_self else []) + [type_hint_of(v) for v in example_inputs]
    return dict(_C._jit_pass_fait_shape_infer(g, hints))


def build(fn, example_inputs=(), add_clone: bool = False):
    """Counterpart of the reference's functs.jit.build(fn, example_inputs) (functs/jit/_build.py): script, optionally
    clone tensor inputs, run the pipeline with the example inputs' types as hints.  Returns the scripted function; its
    graph holds tssa::ParallelFunctor nodes, which launch a precompiled kernel of libfuncts_b200.so when their signature
    names one and otherwise run their subgraph on the immut:: kernels."""
    jit_fn = torch.jit.script(fn)
    if not inspect.isfunction(fn):
        jit_fn = torch.jit.freeze(jit_fn.eval())
    else:
        # torch.jit.script caches per Python function: work on a private copy of the graph
        jit_fn = _C._create_function_from_graph(jit_fn.qualified_name.split(".")[-1], jit_fn.graph.copy())
    g = jit_fn.graph
    if add_clone:
        _C._jit_pass_dumb_remove_inter_precedure_mutation(g)
    hints = [type_hint_of(v) for v in example_inputs]
    if not inspect.isfunction(fn):
        hints = [None] + hints  # self
    from . import patterns
    patterns.register_all()  # the programs that the precompiled kernel sequences stand for (once per process)
    fait_pipeline(g, hints)
    return jit_fn


def functor_regions(g: torch.Graph):
    """Kernel adapter bound to each tssa::ParallelFunctor node of `g`, in graph order ("" = its subgraph is interpreted)."""
    return list(_C._functor_regions(g))


def generic_group_runs() -> int:
    """How many functor executions of this process ran as one launch of the generic program kernel."""
    return int(_C._generic_group_runs())


def last_generic_refusal() -> str:
    """Why the most recent group that could not be expressed as a program was refused ("" if none was)."""
    return str(_C._last_generic_refusal())


def interpreted_functor_runs() -> int:
    """How many functor executions of this process went through the subgraph interpreter instead of a precompiled kernel."""
    return int(_C._interpreted_functor_runs())


def count_groups(g: torch.Graph) -> int:
    """Number of tssa::ParallelFunctor nodes: the unit the kernels-per-call metric counts."""
    return int(_C._count_parallel_functors(g))
