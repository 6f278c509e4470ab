"""Tensor-level wrappers over the C ABI: torch owns device memory and streams, the library launches.

Every function takes CUDA tensors, allocates the outputs (and scratch) with torch, and calls one or more
entry points of libfuncts_b200.so on the current CUDA stream.  Nothing here computes with torch ops.
"""
from typing import List, Optional, Tuple

import torch

from . import _lib
from ._lib import check, lib


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _req(t: torch.Tensor, dtype: torch.dtype, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (functs_b200 has no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    return t.contiguous()


def new_status(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def raise_on_status(status: torch.Tensor, what: str) -> None:
    """Reads the device status word (synchronises) and raises if a kernel reported a problem."""
    bits = int(status.item())
    if bits == 0:
        return
    msgs = []
    if bits & _lib.FB_STATUS_CAND_OVERFLOW:
        msgs.append("a candidate list overflowed its capacity")
    if bits & _lib.FB_STATUS_WAIT_TIMEOUT:
        msgs.append("a bounded device-side wait ran out")
    if bits & _lib.FB_STATUS_INDEX_RANGE:
        msgs.append("an index was out of range")
    raise _lib.FunctsB200Error(f"{what}: " + "; ".join(msgs) + f" (status={bits})")


# ---- C1 ------------------------------------------------------------------------------------------------------


def rows_select_add_select_rev(b: torch.Tensor, n: int, addend: float = 1.0) -> torch.Tensor:
    b = _req(b, torch.float32, "b")
    if b.dim() != 2:
        raise ValueError("b must be 2-D")
    out = torch.empty_like(b)
    check(lib.functs_b200_rows_select_add_select_rev(_ptr(b), _ptr(out), b.size(0), b.size(1), int(n), float(addend),
                                                     _stream()), "rows_select_add_select_rev")
    return out


# ---- masked index / top-k / NMS --------------------------------------------------------------------------------


def threshold_compact(scores: torch.Tensor, thr: float, capacity: Optional[int] = None,
                      status: Optional[torch.Tensor] = None, with_hist: bool = False):
    """scores [G, n] -> (keys uint64-as-int64 [G, capacity], counts int32 [G][, hist int32 [G, bins]])."""
    scores = _req(scores, torch.float32, "scores")
    g, n = scores.shape
    capacity = int(capacity or n)
    keys = torch.empty(g, capacity, dtype=torch.int64, device=scores.device)
    counts = torch.empty(g, dtype=torch.int32, device=scores.device)
    hist = torch.empty(g, int(lib.functs_b200_hist_bins()), dtype=torch.int32, device=scores.device) if with_hist else None
    check(lib.functs_b200_threshold_compact(_ptr(scores), g, n, float(thr), _ptr(keys), _ptr(counts), capacity, 1,
                                            _ptr(hist), _ptr(status), _stream()), "threshold_compact")
    return (keys, counts, hist) if with_hist else (keys, counts)


def select_topk_binned(keys: torch.Tensor, counts: torch.Tensor, hist: torch.Tensor, thr: float, topk: int,
                       return_fallbacks: bool = False):
    """Wide variant of select_topk driven by the producer's score histogram (same thr as the producer).
    return_fallbacks adds an int32 [G] tensor: 1 where the group was finished by the generic selection."""
    keys = _req(keys, torch.int64, "keys")
    counts = _req(counts, torch.int32, "counts")
    hist = _req(hist, torch.int32, "hist")
    g, capacity = keys.shape
    out_keys = torch.empty(g, topk, dtype=torch.int64, device=keys.device)
    out_counts = torch.empty(g, dtype=torch.int32, device=keys.device)
    scratch = torch.empty(int(lib.functs_b200_select_binned_scratch_bytes(g)), dtype=torch.uint8, device=keys.device)
    check(lib.functs_b200_select_topk_binned(_ptr(keys), _ptr(counts), capacity, _ptr(hist), float(thr), g, int(topk),
                                             _ptr(out_keys), _ptr(out_counts), _ptr(scratch), _stream()),
          "select_topk_binned")
    if return_fallbacks:
        return out_keys, out_counts, scratch[: g * 16].view(torch.int32).reshape(g, 4)[:, 3].clone()
    return out_keys, out_counts


def select_topk(keys: torch.Tensor, counts: torch.Tensor, topk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    keys = _req(keys, torch.int64, "keys")
    counts = _req(counts, torch.int32, "counts")
    g, capacity = keys.shape
    out_keys = torch.empty(g, topk, dtype=torch.int64, device=keys.device)
    out_counts = torch.empty(g, dtype=torch.int32, device=keys.device)
    check(lib.functs_b200_select_topk(_ptr(keys), _ptr(counts), capacity, g, int(topk), _ptr(out_keys),
                                      _ptr(out_counts), _stream()), "select_topk")
    return out_keys, out_counts


def batched_nms(boxes: torch.Tensor, num_classes: int, sel_keys: torch.Tensor, sel_counts: torch.Tensor,
                iou_thr: float, class_offset: bool, status: Optional[torch.Tensor] = None):
    """boxes [G, N, 4]; sel_keys [G, K] -> (dets [G,K,5], labels [G,K], flat_ids [G,K], keep [G,K], counts [G])."""
    boxes = _req(boxes, torch.float32, "boxes")
    sel_keys = _req(sel_keys, torch.int64, "sel_keys")
    sel_counts = _req(sel_counts, torch.int32, "sel_counts")
    g, k = sel_keys.shape
    dev = boxes.device
    dets = torch.empty(g, k, 5, dtype=torch.float32, device=dev)
    labels = torch.empty(g, k, dtype=torch.int64, device=dev)
    flat_ids = torch.empty(g, k, dtype=torch.int64, device=dev)
    keep = torch.empty(g, k, dtype=torch.int64, device=dev)
    counts = torch.empty(g, dtype=torch.int32, device=dev)
    scratch = torch.empty(int(lib.functs_b200_nms_scratch_bytes(g, k)), dtype=torch.uint8, device=dev)
    check(lib.functs_b200_batched_nms(_ptr(boxes), boxes.size(1), int(num_classes), _ptr(sel_keys), _ptr(sel_counts), g, k,
                                      float(iou_thr), 1 if class_offset else 0, _ptr(dets), _ptr(labels), _ptr(flat_ids),
                                      _ptr(keep), _ptr(counts), _ptr(status), _ptr(scratch), _stream()), "batched_nms")
    return dets, labels, flat_ids, keep, counts


# ---- C2 ------------------------------------------------------------------------------------------------------


def yolo_decode(maps: List[torch.Tensor], score_thr: float, capacity: Optional[int] = None, dense: bool = False,
                status: Optional[torch.Tensor] = None, with_hist: bool = False):
    """-> (boxes [B,N,4], obj [B,N] | None, cls [B,N,80] | None, cand_keys [B,cap], cand_counts [B][, hist])."""
    maps = [_req(m, torch.float32, "pred map") for m in maps]
    if len(maps) != 3 or any(m.dim() != 4 or m.size(1) != 255 or m.size(2) != m.size(3) for m in maps):
        raise ValueError("expected three [B, 255, S, S] maps")
    b = maps[0].size(0)
    s = [m.size(2) for m in maps]
    n = 3 * sum(x * x for x in s)
    capacity = int(capacity or n * 80)
    dev = maps[0].device
    boxes = torch.empty(b, n, 4, dtype=torch.float32, device=dev)
    obj = torch.empty(b, n, dtype=torch.float32, device=dev) if dense else None
    cls = torch.empty(b, n, 80, dtype=torch.float32, device=dev) if dense else None
    keys = torch.empty(b, capacity, dtype=torch.int64, device=dev)
    counts = torch.empty(b, dtype=torch.int32, device=dev)
    hist = torch.empty(b, int(lib.functs_b200_hist_bins()), dtype=torch.int32, device=dev) if with_hist else None
    check(lib.functs_b200_yolo_decode(_ptr(maps[0]), _ptr(maps[1]), _ptr(maps[2]), b, s[0], s[1], s[2], float(score_thr),
                                      _ptr(boxes), _ptr(obj), _ptr(cls), _ptr(keys), _ptr(counts), capacity, _ptr(hist),
                                      _ptr(status), _stream()), "yolo_decode")
    if with_hist:
        return boxes, obj, cls, keys, counts, hist
    return boxes, obj, cls, keys, counts


class YoloPostprocessPlan:
    """Pre-allocated outputs + scratch for repeated calls at one batch size (no allocation per call)."""

    def __init__(self, batch: int, sizes=(13, 26, 52), topk: int = 1000, capacity: Optional[int] = None,
                 device="cuda"):
        self.batch, self.sizes, self.topk = batch, tuple(sizes), topk
        self.num_boxes = 3 * sum(s * s for s in sizes)
        self.capacity = int(capacity or self.num_boxes * 80)
        dev = torch.device(device)
        self.boxes = torch.empty(batch, self.num_boxes, 4, dtype=torch.float32, device=dev)
        self.dets = torch.empty(batch, topk, 5, dtype=torch.float32, device=dev)
        self.labels = torch.empty(batch, topk, dtype=torch.int64, device=dev)
        self.flat_ids = torch.empty(batch, topk, dtype=torch.int64, device=dev)
        self.counts = torch.empty(batch, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        nbytes = int(lib.functs_b200_yolo_scratch_bytes(batch, *self.sizes, self.capacity, topk))
        self.scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)

    def select_fallbacks(self) -> int:
        """Number of images of the last call whose top-k was finished by the generic (slow, exact) selection."""
        counts_bytes = (self.batch * 4 + 255) // 256 * 256
        hist_bytes = (self.batch * int(lib.functs_b200_hist_bins()) * 4 + 255) // 256 * 256
        ctr = self.scratch[counts_bytes + hist_bytes: counts_bytes + hist_bytes + self.batch * 16].view(torch.int32)
        return int(ctr.reshape(self.batch, 4)[:, 3].sum())

    def run(self, maps: List[torch.Tensor], score_thr: float = 0.5, iou_thr: float = 0.45,
            records: Optional[torch.Tensor] = None) -> None:
        """records (optional, int32 [batch, topk, 8]): the NMS kernel also writes the gather records (no pack launch)."""
        s = self.sizes
        if records is not None and (records.dtype != torch.int32 or not records.is_contiguous()
                                    or records.numel() != self.batch * self.topk * 8):
            raise ValueError("records must be a contiguous int32 [batch, topk, 8] tensor")
        check(lib.functs_b200_yolo_postprocess_dense(maps[0].data_ptr(), maps[1].data_ptr(), maps[2].data_ptr(), self.batch,
                                                     s[0], s[1], s[2], float(score_thr), self.topk, float(iou_thr),
                                                     self.capacity, _ptr(self.boxes), None, None, _ptr(self.dets),
                                                     _ptr(self.labels), _ptr(self.flat_ids), _ptr(self.counts),
                                                     _ptr(records), _ptr(self.status), _ptr(self.scratch), _stream()),
              "yolo_postprocess")


# ---- C3 ------------------------------------------------------------------------------------------------------


def ssd_softmax_decode(loc: torch.Tensor, conf: torch.Tensor, priors: torch.Tensor, clamp_max: float = 300.0,
                       out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    loc = _req(loc, torch.float32, "loc")
    conf = _req(conf, torch.float32, "conf")
    priors = _req(priors, torch.float32, "priors")
    b, p, _ = loc.shape
    c = conf.size(2) - 1
    if out is None:
        boxes = torch.empty(b, p, 4, dtype=torch.float32, device=loc.device)
        scores_cm = torch.empty(b, c, p, dtype=torch.float32, device=loc.device)
    else:
        boxes, scores_cm = out
    check(lib.functs_b200_ssd_softmax_decode(_ptr(loc), _ptr(conf), _ptr(priors), b, p, c, float(clamp_max), _ptr(boxes),
                                             _ptr(scores_cm), _stream()), "ssd_softmax_decode")
    return boxes, scores_cm


def ssd_class_nms(boxes: torch.Tensor, scores_cm: torch.Tensor, score_thr: float = 0.01, topk: int = 200,
                  iou_thr: float = 0.45, out=None):
    boxes = _req(boxes, torch.float32, "boxes")
    scores_cm = _req(scores_cm, torch.float32, "scores_cm")
    b, c, p = scores_cm.shape
    dev = boxes.device
    if out is None:
        dets = torch.empty(b, c, topk, 5, dtype=torch.float32, device=dev)
        ids = torch.empty(b, c, topk, dtype=torch.int64, device=dev)
        counts = torch.empty(b, c, dtype=torch.int32, device=dev)
    else:
        dets, ids, counts = out
    check(lib.functs_b200_ssd_class_nms(_ptr(boxes), _ptr(scores_cm), b, p, c, float(score_thr), int(topk), float(iou_thr),
                                        _ptr(dets), _ptr(ids), _ptr(counts), _stream()), "ssd_class_nms")
    return dets, ids, counts


# ---- C4 ------------------------------------------------------------------------------------------------------


def lstm_forward(x: torch.Tensor, w_ih: torch.Tensor, w_hh: torch.Tensor, b_ih: torch.Tensor, b_hh: torch.Tensor,
                 mode: int = 0, scratch: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                 out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    x = _req(x, torch.float32, "x")
    w_ih = _req(w_ih, torch.float32, "w_ih")
    w_hh = _req(w_hh, torch.float32, "w_hh")
    b_ih = _req(b_ih, torch.float32, "b_ih")
    b_hh = _req(b_hh, torch.float32, "b_hh")
    t, b, i = x.shape
    h = w_hh.size(2)
    if tuple(w_ih.shape) != (4, i, h) or tuple(w_hh.shape) != (4, h, h):
        raise ValueError("weights must be gate-leading: w_ih [4, I, H], w_hh [4, H, H]")
    if b_ih.numel() != 4 * h or b_hh.numel() != 4 * h:
        raise ValueError("biases must have 4*H elements")
    dev = x.device
    if out is None:
        hs = torch.empty(t, b, h, dtype=torch.float32, device=dev)
        cs = torch.empty(t, b, h, dtype=torch.float32, device=dev)
    else:
        hs, cs = out
    if scratch is None:
        scratch = torch.empty(int(lib.functs_b200_lstm_scratch_bytes(t, b, i, h)), dtype=torch.uint8, device=dev)
    own_status = status is None
    if own_status:
        status = new_status(dev)
    check(lib.functs_b200_lstm_forward_mode(_ptr(x), _ptr(w_ih), _ptr(w_hh), _ptr(b_ih), _ptr(b_hh), t, b, i, h, _ptr(hs),
                                            _ptr(cs), _ptr(status), _ptr(scratch), _stream(), int(mode)), "lstm_forward")
    if own_status:
        raise_on_status(status, "lstm_forward")
    return hs, cs


# ---- C5 ------------------------------------------------------------------------------------------------------


def yolact_masks(proto: torch.Tensor, coef: torch.Tensor, boxes: torch.Tensor, thr: float = 0.5,
                 with_logits: bool = False, out: Optional[torch.Tensor] = None):
    proto = _req(proto, torch.float32, "proto")
    coef = _req(coef, torch.float32, "coef")
    boxes = _req(boxes, torch.float32, "boxes")
    b, h, w, k = proto.shape
    if k != 32:
        raise ValueError("prototype depth must be 32")
    n = coef.size(1)
    masks = out if out is not None else torch.empty(b, n, h, w, dtype=torch.uint8, device=proto.device)
    logits = torch.empty(b, n, h, w, dtype=torch.float32, device=proto.device) if with_logits else None
    check(lib.functs_b200_yolact_masks(_ptr(proto), _ptr(coef), _ptr(boxes), b, h, w, n, float(thr), _ptr(masks),
                                       _ptr(logits), _stream()), "yolact_masks")
    return (masks, logits) if with_logits else masks
