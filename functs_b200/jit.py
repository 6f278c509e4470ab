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
