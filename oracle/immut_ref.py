"""numpy restatement of the Access / Assign index semantics.  TEST INFRASTRUCTURE ONLY.

``eval_access`` evaluates an index description exactly as the device kernel does
(out[ax] = src.flat[offset + sum_d (ax_d % mod_d) * stride_d]); the ``*_rev`` functions state the
"self with the accessed region replaced by src" rule of the reference's lowerings
(functs/csrc/jit/tensorexpr/nnc_ext.cpp:112-164 slice_rev, :187-212 select_rev).
"""
import numpy as np


def eval_access(src: np.ndarray, out_shape, src_stride, src_mod, src_offset) -> np.ndarray:
    flat = np.ascontiguousarray(src).reshape(-1)
    out_shape = list(out_shape)
    if len(out_shape) == 0:
        return flat[src_offset].reshape(())
    grids = np.indices(out_shape, dtype=np.int64)
    off = np.full(out_shape, src_offset, dtype=np.int64)
    for d in range(len(out_shape)):
        ax = grids[d]
        if src_mod[d] > 0:
            ax = ax % src_mod[d]
        off = off + ax * src_stride[d]
    return flat[off]


def select_rev(self_: np.ndarray, src: np.ndarray, dim: int, index: int) -> np.ndarray:
    out = self_.copy()
    ax = np.indices(self_.shape)[dim]
    sel = ax == (index if index >= 0 else index + self_.shape[dim])
    out[sel] = np.broadcast_to(np.expand_dims(src, dim), self_.shape)[sel]
    return out


def slice_rev(self_: np.ndarray, src: np.ndarray, dim: int, start: int, end: int, step: int) -> np.ndarray:
    """start/end already normalised to [0, size]."""
    out = self_.copy()
    ax = np.indices(self_.shape)[dim]
    not_set = (ax < start) | (ax >= end) | (((ax - start) % step) != 0)
    src_idx = np.where(not_set, 0, (ax - start) // step)
    gathered = np.take_along_axis(src, src_idx, axis=dim) if src.shape[dim] > 0 else out
    return np.where(not_set, out, gathered)
