"""The immut:: Access / Assign operators as stand-alone CUDA launches.

Names, argument order and defaults follow the reference's operator schemas
(functs/csrc/jit/ir/symbol_ext.cpp:121-199), e.g.
  immut::select_rev(Tensor self, Tensor src, int dim, int index) -> Tensor
  immut::slice_rev(Tensor self, Tensor src, int dim=0, SymInt? start=None, SymInt? end=None, SymInt step=1) -> Tensor
Unlike the reference's eager kernels, which return views (access ops) or write into ``self`` in place
(``*_rev``, symbol_ext.cpp:21-29, 40-50), every function here is pure: it returns a fresh contiguous tensor, which is
the meaning the functionalized graph gives these ops.  Error behaviour follows ATen (IndexError for out-of-range
dims / indices, ValueError/RuntimeError for shape mismatches).
"""
import ctypes
from typing import List, Optional, Sequence

import torch

from . import access_desc as ad
from ._lib import AccessDesc, check, lib

_ELEM = {1, 2, 4, 8}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _prep(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (functs_b200 has no CPU path)")
    if t.element_size() not in _ELEM:
        raise TypeError(f"{name}: unsupported element size {t.element_size()}")
    return t.contiguous()


def _run_access(src: torch.Tensor, a: ad.Access) -> torch.Tensor:
    ad.compose_check(a)
    out = torch.empty(a.out_shape, dtype=src.dtype, device=src.device)
    if a.numel == 0:
        return out
    d = AccessDesc()
    d.rank = len(a.out_shape)
    for i in range(d.rank):
        d.out_shape[i] = a.out_shape[i]
        d.src_stride[i] = a.src_stride[i]
        d.src_mod[i] = a.src_mod[i]
    d.src_offset = a.src_offset
    check(lib.functs_b200_access(src.data_ptr(), out.data_ptr(), ctypes.byref(d), src.element_size(), _stream()), "access")
    return out


def access(src: torch.Tensor) -> torch.Tensor:
    src = _prep(src, "src")
    return _run_access(src, ad.identity(src.shape))


def assign(self: torch.Tensor, src: torch.Tensor, n: Optional[bool] = None) -> torch.Tensor:
    """immut::assign(self, src, n) = src (self is ignored; the op is erased before execution in the reference,
    functs/csrc/jit/passes/convert_to_tensorssa.cpp:409-413)."""
    return access(src)


def select(src: torch.Tensor, dim: int, index: int) -> torch.Tensor:
    src = _prep(src, "src")
    return _run_access(src, ad.select(src.shape, dim, index))


def slice(src: torch.Tensor, dim: int = 0, start: Optional[int] = None, end: Optional[int] = None,  # noqa: A001
          step: int = 1) -> torch.Tensor:
    src = _prep(src, "src")
    return _run_access(src, ad.slice_(src.shape, dim, start, end, step))


def squeeze(src: torch.Tensor, dim: int) -> torch.Tensor:
    src = _prep(src, "src")
    return _run_access(src, ad.squeeze(src.shape, dim))


def unsqueeze(src: torch.Tensor, dim: int) -> torch.Tensor:
    src = _prep(src, "src")
    return _run_access(src, ad.unsqueeze(src.shape, dim))


def view(src: torch.Tensor, size: Sequence[int]) -> torch.Tensor:
    src = _prep(src, "src")
    return _run_access(src, ad.view(src.shape, size))


reshape = view


def permute(src: torch.Tensor, dims: Sequence[int]) -> torch.Tensor:
    src = _prep(src, "src")
    return _run_access(src, ad.permute(src.shape, dims))


def expand(src: torch.Tensor, size: Sequence[int], implicit: bool = False) -> torch.Tensor:
    src = _prep(src, "src")
    return _run_access(src, ad.expand(src.shape, size))


def expand_as(src: torch.Tensor, other: torch.Tensor) -> torch.Tensor:
    return expand(src, list(other.shape))


def repeat(src: torch.Tensor, repeats: Sequence[int]) -> torch.Tensor:
    src = _prep(src, "src")
    return _run_access(src, ad.repeat(src.shape, repeats))


def index(src: torch.Tensor, indices: List[Optional[torch.Tensor]]) -> torch.Tensor:
    """immut::index.Tensor: first index tensor only, dimension 0, int64 indices
    (functs/csrc/jit/tensorexpr/nnc_ext.cpp:372-392); bool masks are not an immut op
    (convert_to_tensorssa.cpp:422-443 sends them back to aten::index)."""
    src = _prep(src, "src")
    if len(indices) < 1 or indices[0] is None or any(i is not None for i in indices[1:]):
        raise ValueError("immut::index supports exactly one index tensor, on dimension 0")
    idx = indices[0]
    if idx.dtype != torch.int64:
        raise TypeError("immut::index needs int64 indices (bool masks go through aten::index)")
    idx = idx.contiguous()
    rows = src.size(0)
    row_elems = src[0].numel() if src.dim() > 1 else 1
    out = torch.empty(list(idx.shape) + list(src.shape[1:]), dtype=src.dtype, device=src.device)
    status = torch.zeros(1, dtype=torch.int32, device=src.device)
    check(lib.functs_b200_index_rows(src.data_ptr(), idx.data_ptr(), out.data_ptr(), rows, idx.numel(), row_elems,
                                     src.element_size(), status.data_ptr(), _stream()), "index")
    if int(status.item()) != 0:
        raise IndexError("index out of range in immut::index")
    return out


# ---- reverse ("assign") forms --------------------------------------------------------------------------------


def _shape_arr(shape):
    return (ctypes.c_int64 * len(shape))(*shape)


def select_rev(self: torch.Tensor, src: torch.Tensor, dim: int, index: int) -> torch.Tensor:
    self = _prep(self, "self")
    src = _prep(src, "src").to(self.dtype)
    rank = self.dim()
    dim = ad._norm_dim(dim, rank, "select_rev")
    size = self.size(dim)
    if index < -size or index >= size:
        raise IndexError(f"select_rev: index {index} out of range for dimension {dim} with size {size}")
    if index < 0:
        index += size
    want = [s for d, s in enumerate(self.shape) if d != dim]
    src = src.expand(want).contiguous() if list(src.shape) != want else src
    out = torch.empty_like(self)
    check(lib.functs_b200_select_rev(self.data_ptr(), src.data_ptr(), out.data_ptr(), _shape_arr(list(self.shape)), rank,
                                     dim, index, self.element_size(), _stream()), "select_rev")
    return out


def slice_rev(self: torch.Tensor, src: torch.Tensor, dim: int = 0, start: Optional[int] = None,
              end: Optional[int] = None, step: int = 1) -> torch.Tensor:
    self = _prep(self, "self")
    src = _prep(src, "src").to(self.dtype)
    rank = self.dim()
    dim = ad._norm_dim(dim, rank, "slice_rev")
    s, e, length = ad.normalize_slice(self.size(dim), start, end, step)
    want = list(self.shape)
    want[dim] = length
    src = src.expand(want).contiguous() if list(src.shape) != want else src
    out = torch.empty_like(self)
    check(lib.functs_b200_slice_rev(self.data_ptr(), src.data_ptr(), out.data_ptr(), _shape_arr(list(self.shape)), rank,
                                    dim, s, e, step, self.element_size(), _stream()), "slice_rev")
    return out


def squeeze_rev(self: torch.Tensor, src: torch.Tensor, dim: int) -> torch.Tensor:
    """The whole tensor is replaced: src, given back the squeezed axis."""
    return view(src.to(self.dtype), list(self.shape))


def unsqueeze_rev(self: torch.Tensor, src: torch.Tensor, dim: int) -> torch.Tensor:
    return view(src.to(self.dtype), list(self.shape))


def view_rev(self: torch.Tensor, src: torch.Tensor, size: Sequence[int]) -> torch.Tensor:
    """Inverse of view/reshape: src relabelled with self's shape (the reference maps the reverse of
    view/reshape to immut::view, functs/csrc/jit/ir/symbol_ext.h:72-85)."""
    return view(src.to(self.dtype), list(self.shape))


reshape_rev = view_rev


def permute_rev(self: torch.Tensor, src: torch.Tensor, dims: Sequence[int]) -> torch.Tensor:
    """Inverse permutation applied to src (src has self.permute(dims)'s shape)."""
    rank = self.dim()
    dims = [ad._norm_dim(d, rank, "permute_rev") for d in dims]
    inv = [0] * rank
    for i, d in enumerate(dims):
        inv[d] = i
    return permute(src.to(self.dtype), inv)


def expand_rev(self: torch.Tensor, src: torch.Tensor, size: Sequence[int], implicit: bool = False) -> torch.Tensor:
    """Well-posed only when no element of self is expanded into several destinations (all expanded extents are 1,
    i.e. expand was a relabelling); otherwise writing through the expanded view is ambiguous and is rejected,
    as torch rejects copy_ into an overlapping view."""
    a = ad.expand(self.shape, size)
    if a.numel != self.numel():
        raise RuntimeError("expand_rev: destinations overlap (an extent of 1 was expanded); the assignment is ill-posed")
    return view(src.to(self.dtype), list(self.shape))


def expand_as_rev(self: torch.Tensor, src: torch.Tensor, other: torch.Tensor) -> torch.Tensor:
    return expand_rev(self, src, list(other.shape))


def repeat_rev(self: torch.Tensor, src: torch.Tensor, repeats: Sequence[int]) -> torch.Tensor:
    """self.repeat(r) is a copy, not a view, so assigning to it never reaches self
    (the reference's eager kernel returns self unchanged, symbol_ext.cpp:94-101)."""
    return access(self)


def index_rev(self: torch.Tensor, src: torch.Tensor, indices: List[Optional[torch.Tensor]]) -> torch.Tensor:
    """Row scatter: out = self; out[idx[i]] = src[i].  With duplicate indices the winner is unspecified."""
    self = _prep(self, "self")
    src = _prep(src, "src").to(self.dtype)
    if len(indices) < 1 or indices[0] is None or any(i is not None for i in indices[1:]):
        raise ValueError("immut::index_rev supports exactly one index tensor, on dimension 0")
    idx = indices[0]
    if idx.dtype != torch.int64:
        raise TypeError("immut::index_rev needs int64 indices")
    idx = idx.contiguous()
    rows = self.size(0)
    row_elems = self[0].numel() if self.dim() > 1 else 1
    want = list(idx.shape) + list(self.shape[1:])
    src = src.expand(want).contiguous() if list(src.shape) != want else src
    out = torch.empty_like(self)
    status = torch.zeros(1, dtype=torch.int32, device=self.device)
    check(lib.functs_b200_index_rows_rev(self.data_ptr(), src.data_ptr(), idx.data_ptr(), out.data_ptr(), rows, idx.numel(),
                                         row_elems, self.element_size(), status.data_ptr(), _stream()), "index_rev")
    if int(status.item()) != 0:
        raise IndexError("index out of range in immut::index_rev")
    return out
