"""Host-side mirrors of the reference's post-processing modules, executed by the sm_100a kernels.

Class names and call conventions follow the reference's benchmark modules
(functs/benchmark/ai_model/{yolov3/yolov3_bbox.py:184-243, ssd/ssd_bbox.py:217-290, lstm/lstm.py:100-133,
yolact/yolact_mask.py:150-264}) and examples/get_started.py:10-15: a module is called with the same tensors and
returns the same Python structure (lists of (dets, labels) tuples, masks per image ...).  Inputs may live on the host:
they are copied to the module's device first.  There is no CPU execution path.
"""
from typing import List, Optional, Tuple

import torch

from . import ops
from ._lib import launch_count


def _dev(device) -> torch.device:
    d = torch.device(device)
    if d.type != "cuda":
        raise ValueError("functs_b200 modules run on CUDA devices only")
    return d


def get_started(a: torch.Tensor, b: torch.Tensor, n: int, device="cuda") -> torch.Tensor:
    """examples/get_started.py:10-15: b = b.clone(); for i in range(n): b[i] = b[i] + 1; return b."""
    if n > b.size(0):
        raise IndexError(f"index {b.size(0)} is out of bounds for dimension 0 with size {b.size(0)}")
    return ops.rows_select_add_select_rev(b.to(_dev(device)), n, 1.0)


class YOLOV3BBox:
    """Decode three [B, 255, S, S] maps, score mask, top-k, class-wise NMS.  3 kernel launches (+1 memset) per call."""

    def __init__(self, sizes=(13, 26, 52), score_thr: float = 0.5, topk: int = 1000, iou_thr: float = 0.45,
                 device="cuda"):
        self.sizes, self.score_thr, self.topk, self.iou_thr = tuple(sizes), score_thr, topk, iou_thr
        self.device = _dev(device)
        self._plan: Optional[ops.YoloPostprocessPlan] = None
        self.kernels_last_call = 0

    def _plan_for(self, batch: int) -> ops.YoloPostprocessPlan:
        if self._plan is None or self._plan.batch != batch:
            self._plan = ops.YoloPostprocessPlan(batch, self.sizes, self.topk, device=self.device)
        return self._plan

    def forward_padded(self, pred_maps: List[torch.Tensor]):
        """-> (dets [B,K,5], labels [B,K], flat_ids [B,K], counts [B]) on the device, rows past counts[b] are padding.
        The tensors belong to the module and are overwritten by the next call."""
        maps = [m.to(self.device, non_blocking=True).contiguous() for m in pred_maps]
        if len(maps) != 3 or any(m.dim() != 4 or m.size(1) != 255 for m in maps):
            raise ValueError("expected three [B, 255, S, S] maps")
        if tuple(m.size(2) for m in maps) != self.sizes:
            raise ValueError(f"map sizes {[m.size(2) for m in maps]} differ from the configured {self.sizes}")
        plan = self._plan_for(maps[0].size(0))
        before = launch_count()
        plan.run(maps, self.score_thr, self.iou_thr)
        self.kernels_last_call = launch_count() - before
        return plan.dets, plan.labels, plan.flat_ids, plan.counts

    def __call__(self, pred_maps: List[torch.Tensor]) -> List[Tuple[torch.Tensor, torch.Tensor]]:
        dets, labels, _, counts = self.forward_padded(pred_maps)
        cnt = counts.tolist()
        ops.raise_on_status(self._plan.status, "YOLOV3BBox")
        return [(dets[b, :cnt[b]].clone(), labels[b, :cnt[b]].clone()) for b in range(len(cnt))]


class SSDBBox:
    """softmax + decode, then the per-class loop (mask, top-k, NMS) with one CTA per (image, class).  2 launches."""

    def __init__(self, priors: torch.Tensor, score_thr: float = 0.01, topk: int = 200, iou_thr: float = 0.45,
                 clamp_max: float = 300.0, device="cuda"):
        self.device = _dev(device)
        self.priors = priors.to(self.device, torch.float32).contiguous()
        self.score_thr, self.topk, self.iou_thr, self.clamp_max = score_thr, topk, iou_thr, clamp_max
        self._bufs = None
        self.kernels_last_call = 0

    def forward_padded(self, loc: torch.Tensor, conf: torch.Tensor):
        """-> (boxes [B,P,4], dets [B,C,K,5], prior_ids [B,C,K], counts [B,C]); buffers are reused across calls."""
        loc = loc.to(self.device, non_blocking=True).contiguous()
        conf = conf.to(self.device, non_blocking=True).contiguous()
        b, p, _ = loc.shape
        c = conf.size(2) - 1
        key = (b, p, c)
        if self._bufs is None or self._bufs[0] != key:
            dev = self.device
            self._bufs = (key,
                          torch.empty(b, p, 4, dtype=torch.float32, device=dev),
                          torch.empty(b, c, p, dtype=torch.float32, device=dev),
                          torch.empty(b, c, self.topk, 5, dtype=torch.float32, device=dev),
                          torch.empty(b, c, self.topk, dtype=torch.int64, device=dev),
                          torch.empty(b, c, dtype=torch.int32, device=dev))
        _, boxes, scores_cm, dets, ids, counts = self._bufs
        before = launch_count()
        ops.ssd_softmax_decode(loc, conf, self.priors, self.clamp_max, out=(boxes, scores_cm))
        ops.ssd_class_nms(boxes, scores_cm, self.score_thr, self.topk, self.iou_thr, out=(dets, ids, counts))
        self.kernels_last_call = launch_count() - before
        return boxes, dets, ids, counts

    def __call__(self, loc: torch.Tensor, conf: torch.Tensor) -> List[Tuple[torch.Tensor, torch.Tensor]]:
        _, dets, ids, counts = self.forward_padded(loc, conf)
        return [(d, l) for d, l, _ in self.unpad(dets, ids, counts)]

    @staticmethod
    def unpad(dets: torch.Tensor, ids: torch.Tensor, counts: torch.Tensor):
        """Padded per-class outputs -> per image (dets [m,5], labels [m], prior_ids [m]) concatenated in class order."""
        b, c, k, _ = dets.shape
        valid = torch.arange(k, device=dets.device)[None, None, :] < counts[:, :, None]
        labels = torch.arange(c, device=dets.device)[None, :, None].expand(b, c, k)
        out = []
        for i in range(b):
            m = valid[i]
            out.append((dets[i][m], labels[i][m], ids[i][m]))
        return out


class LSTM:
    """One-layer LSTM with per-step outputs written by slice assignment (hs[t] = h, cs[t] = c).  2 launches (3 when the tensor-core projection runs: operand split, GEMM, recurrence)."""

    def __init__(self, w_ih: torch.Tensor, w_hh: torch.Tensor, b_ih: torch.Tensor, b_hh: torch.Tensor, device="cuda"):
        self.device = _dev(device)
        self.w_ih = w_ih.to(self.device, torch.float32).contiguous()
        self.w_hh = w_hh.to(self.device, torch.float32).contiguous()
        self.b_ih = b_ih.to(self.device, torch.float32).reshape(4, -1).contiguous()
        self.b_hh = b_hh.to(self.device, torch.float32).reshape(4, -1).contiguous()
        self._scratch = None
        self._out = None
        self._status = ops.new_status(self.device)
        self.kernels_last_call = 0

    @staticmethod
    def expected_launches(seq_len: int, batch: int, hidden: int, mode: int = 0) -> int:
        """Kernel launches of one call: operand split + tensor-core projection + recurrence, or (mode 1, or a shape the
        tensor-core projection does not take) CUDA-core projection + recurrence.  The recurrence is one launch in every
        mode."""
        return 3 if (mode != 1 and (seq_len * batch) % 128 == 0 and hidden % 128 == 0) else 2

    def forward_device(self, x: torch.Tensor, mode: int = 0):
        """x on the device; outputs and scratch are reused across calls; no synchronisation."""
        t, b, i = x.shape
        h = self.w_hh.size(2)
        if self._out is None or self._out[0].shape != (t, b, h):
            self._out = (torch.empty(t, b, h, dtype=torch.float32, device=self.device),
                         torch.empty(t, b, h, dtype=torch.float32, device=self.device))
            from ._lib import lib
            self._scratch = torch.empty(int(lib.functs_b200_lstm_scratch_bytes(t, b, i, h)), dtype=torch.uint8,
                                        device=self.device)
        before = launch_count()
        ops.lstm_forward(x, self.w_ih, self.w_hh, self.b_ih, self.b_hh, mode=mode, scratch=self._scratch,
                         status=self._status, out=self._out)
        self.kernels_last_call = launch_count() - before
        return self._out

    def __call__(self, x: torch.Tensor, mode: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
        hs, cs = self.forward_device(x.to(self.device, non_blocking=True).contiguous(), mode)
        ops.raise_on_status(self._status, "LSTM")
        return hs, cs


class YolactBBoxMask:
    """Mask assembly: sigmoid(proto @ coef) cropped per detection and thresholded.  1 launch."""

    def __init__(self, thr: float = 0.5, device="cuda"):
        self.device = _dev(device)
        self.thr = thr
        self._out = None
        self.kernels_last_call = 0

    def __call__(self, proto: torch.Tensor, coef: torch.Tensor, boxes: torch.Tensor) -> torch.Tensor:
        proto = proto.to(self.device, non_blocking=True).contiguous()
        coef = coef.to(self.device, non_blocking=True).contiguous()
        boxes = boxes.to(self.device, non_blocking=True).contiguous()
        b, h, w, _ = proto.shape
        n = coef.size(1)
        if self._out is None or self._out.shape != (b, n, h, w):
            self._out = torch.empty(b, n, h, w, dtype=torch.uint8, device=self.device)
        before = launch_count()
        ops.yolact_masks(proto, coef, boxes, self.thr, out=self._out)
        self.kernels_last_call = launch_count() - before
        return self._out
