"""Index descriptions of the immut:: Access family (host-side integer logic, no device work).

An access op on a contiguous source is described by, per OUTPUT axis d, a source stride and an optional modulus,
plus a source offset:  out[ax] = src.flat[offset + sum_d (ax_d % mod_d) * stride_d].
The rules restate the reference's lowerings (functs/csrc/jit/tensorexpr/nnc_ext.cpp:82-110 slice, :166-185 select,
:214-229 unsqueeze, :231-295 view/reshape, :297-318 expand/expand_as/repeat, :320-358 permute) with ATen's
normalisation of negative dims, indices and slice bounds (functs/csrc/jit/ir/symbol_ext.cpp:17-117 defines the eager
meaning of every op as the ATen view op of the same name).
"""
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

MAX_RANK = 8


@dataclass
class Access:
    out_shape: List[int]
    src_stride: List[int]
    src_mod: List[int]  # 0 = no modulus
    src_offset: int = 0

    @property
    def numel(self) -> int:
        n = 1
        for s in self.out_shape:
            n *= s
        return n


def contiguous_strides(shape: Sequence[int]) -> List[int]:
    st, acc = [0] * len(shape), 1
    for d in range(len(shape) - 1, -1, -1):
        st[d] = acc
        acc *= shape[d]
    return st


def _norm_dim(dim: int, rank: int, what: str) -> int:
    if dim < -rank or dim >= rank:
        raise IndexError(f"{what}: dimension {dim} out of range for rank {rank}")
    return dim + rank if dim < 0 else dim


def identity(shape: Sequence[int]) -> Access:
    return Access(list(shape), contiguous_strides(shape), [0] * len(shape), 0)


def select(shape: Sequence[int], dim: int, index: int) -> Access:
    rank = len(shape)
    dim = _norm_dim(dim, rank, "select")
    size = shape[dim]
    if index < -size or index >= size:
        raise IndexError(f"select: index {index} out of range for dimension {dim} with size {size}")
    if index < 0:
        index += size
    st = contiguous_strides(shape)
    return Access([s for d, s in enumerate(shape) if d != dim], [s for d, s in enumerate(st) if d != dim],
                  [0] * (rank - 1), index * st[dim])


def normalize_slice(size: int, start: Optional[int], end: Optional[int], step: int) -> Tuple[int, int, int]:
    """ATen slice normalisation: None -> 0 / size, negative -> + size, then clamp to [0, size]; returns (start, end, len)."""
    if step <= 0:
        raise ValueError("slice step must be positive")
    start = 0 if start is None else start
    end = size if end is None else end
    if start < 0:
        start += size
    if end < 0:
        end += size
    start = min(max(start, 0), size)
    end = min(max(end, start), size)
    return start, end, (end - start + step - 1) // step


def slice_(shape: Sequence[int], dim: int = 0, start: Optional[int] = None, end: Optional[int] = None,
           step: int = 1) -> Access:
    rank = len(shape)
    dim = _norm_dim(dim, rank, "slice")
    start, _, length = normalize_slice(shape[dim], start, end, step)
    st = contiguous_strides(shape)
    out_shape = list(shape)
    out_shape[dim] = length
    strides = list(st)
    strides[dim] = st[dim] * step
    return Access(out_shape, strides, [0] * rank, start * st[dim])


def squeeze(shape: Sequence[int], dim: int) -> Access:
    rank = len(shape)
    dim = _norm_dim(dim, max(rank, 1), "squeeze")
    if rank == 0 or shape[dim] != 1:
        return identity(shape)
    st = contiguous_strides(shape)
    return Access([s for d, s in enumerate(shape) if d != dim], [s for d, s in enumerate(st) if d != dim],
                  [0] * (rank - 1), 0)


def unsqueeze(shape: Sequence[int], dim: int) -> Access:
    rank = len(shape)
    dim = _norm_dim(dim, rank + 1, "unsqueeze")
    st = contiguous_strides(shape)
    out_shape = list(shape[:dim]) + [1] + list(shape[dim:])
    strides = st[:dim] + [0] + st[dim:]
    return Access(out_shape, strides, [0] * (rank + 1), 0)


def infer_view_shape(numel: int, size: Sequence[int]) -> List[int]:
    size = list(size)
    neg = [i for i, s in enumerate(size) if s == -1]
    if len(neg) > 1:
        raise ValueError("only one dimension can be inferred")
    known = 1
    for s in size:
        if s != -1:
            if s < 0:
                raise ValueError(f"invalid shape dimension {s}")
            known *= s
    if neg:
        if known == 0 or numel % known != 0:
            raise ValueError(f"shape {size} is invalid for input of size {numel}")
        size[neg[0]] = numel // known
    elif known != numel:
        raise ValueError(f"shape {size} is invalid for input of size {numel}")
    return size


def view(shape: Sequence[int], size: Sequence[int]) -> Access:
    """view / reshape of a contiguous source: a pure relabelling of the flat index."""
    numel = 1
    for s in shape:
        numel *= s
    return identity(infer_view_shape(numel, size))


def permute(shape: Sequence[int], dims: Sequence[int]) -> Access:
    rank = len(shape)
    dims = [_norm_dim(d, rank, "permute") for d in dims]
    if sorted(dims) != list(range(rank)):
        raise ValueError("permute: dims must be a permutation")
    st = contiguous_strides(shape)
    return Access([shape[d] for d in dims], [st[d] for d in dims], [0] * rank, 0)


def expand(shape: Sequence[int], size: Sequence[int]) -> Access:
    rank, orank = len(shape), len(size)
    if orank < rank:
        raise ValueError("expand: the number of sizes must be >= the tensor rank")
    st = contiguous_strides(shape)
    lead = orank - rank
    out_shape, strides = [], []
    for d in range(orank):
        if d < lead:
            if size[d] < 0:
                raise ValueError("expand: -1 is not allowed in a leading, non-existing dimension")
            out_shape.append(size[d])
            strides.append(0)
        else:
            in_sz = shape[d - lead]
            want = in_sz if size[d] == -1 else size[d]
            if want != in_sz and in_sz != 1:
                raise ValueError(f"expand: size {want} must match the existing size {in_sz} at dimension {d}")
            out_shape.append(want)
            strides.append(0 if (in_sz == 1 and want != 1) else st[d - lead])
    return Access(out_shape, strides, [0] * orank, 0)


def repeat(shape: Sequence[int], repeats: Sequence[int]) -> Access:
    rank, orank = len(shape), len(repeats)
    if orank < rank:
        raise ValueError("repeat: the number of repeats must be >= the tensor rank")
    st = contiguous_strides(shape)
    lead = orank - rank
    out_shape, strides, mods = [], [], []
    for d in range(orank):
        if repeats[d] < 0:
            raise ValueError("repeat: negative repeat")
        if d < lead:
            out_shape.append(repeats[d])
            strides.append(0)
            mods.append(0)
        else:
            in_sz = shape[d - lead]
            out_shape.append(in_sz * repeats[d])
            strides.append(st[d - lead])
            mods.append(in_sz if repeats[d] != 1 else 0)
    return Access(out_shape, strides, mods, 0)


def compose_check(a: Access) -> None:
    if len(a.out_shape) > MAX_RANK:
        raise ValueError(f"rank {len(a.out_shape)} exceeds the supported maximum of {MAX_RANK}")
