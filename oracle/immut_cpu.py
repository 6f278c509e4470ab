"""CPU kernels for the immut:: operators, built from ATen view ops.  TEST INFRASTRUCTURE ONLY.

The product registers CUDA kernels only (functs_b200/csrc/torch_ext/immut_ops.cpp).  Tests that want to RUN a
functionalized graph on a machine without a GPU import this module, which adds a CPU implementation of every
operator with the meaning the reference's eager kernels give them (functs/csrc/jit/ir/symbol_ext.cpp:9-117), made
pure: a `*_rev` op returns a new tensor instead of writing into `self`.
"""
import torch

_lib = torch.library.Library("immut", "IMPL", "CPU")


def _rev(view_fn):
    def impl(self, src, *args):
        out = self.clone()
        view_fn(out, *args).copy_(src)
        return out
    return impl


_lib.impl("access", lambda src: src.clone())
_lib.impl("assign", lambda self, src, n=None: src.clone())
_lib.impl("select", lambda src, dim, index: src.select(dim, index).clone())
_lib.impl("select_rev", _rev(lambda t, dim, index: t.select(dim, index)))
_lib.impl("slice", lambda src, dim=0, start=None, end=None, step=1: torch.ops.aten.slice(src, dim, start, end, step).clone())
_lib.impl("slice_rev", _rev(lambda t, dim=0, start=None, end=None, step=1: torch.ops.aten.slice(t, dim, start, end, step)))
_lib.impl("squeeze", lambda self, dim: self.squeeze(dim).clone())
_lib.impl("unsqueeze", lambda self, dim: self.unsqueeze(dim).clone())
_lib.impl("view", lambda self, size: self.reshape(size).clone())
_lib.impl("reshape", lambda self, size: self.reshape(size).clone())
_lib.impl("permute", lambda self, sizes: self.permute(sizes).contiguous())
_lib.impl("permute_rev", lambda self, size: self.permute([list(size).index(i) for i in range(len(size))]).contiguous())
_lib.impl("expand", lambda self, size, implicit=False: self.expand(size).contiguous())
_lib.impl("expand_rev", lambda self, size, implicit=False: self.expand(size).contiguous())
_lib.impl("repeat", lambda self, size: self.repeat(size))
_lib.impl("repeat_rev", lambda self, src, size: self.clone())
_lib.impl("expand_as", lambda self, other: self.expand_as(other).contiguous())
_lib.impl("expand_as_rev", lambda self, src, other: src.clone())
_lib.impl("index.Tensor", lambda self, indices: self[indices[0]])
