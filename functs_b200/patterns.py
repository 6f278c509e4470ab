"""Pattern programs: the imperative programs that the precompiled kernel sequences of libfuncts_b200.so replace.

The reference compiles whatever subgraph a ``tssa::ParallelFunctor`` carries (fait/fuser/graph_builder.cpp:259-712).
Here the kernels are written by hand, so each of them is described by the program it stands for, written the way the
reference's benchmark modules are written (views + in-place slice / select assignment + Python loops):

  YOLOV3Post   functs/benchmark/ai_model/yolov3/yolov3_bbox.py:195-243 (+ multiclass_nms :104-136, batched_nms :139-179)
  SSDPost      functs/benchmark/ai_model/ssd/ssd_bbox.py:254-290 (+ delta2bbox :121-154, filter_scores_and_topk :163-172)
  LSTMSeq      functs/benchmark/ai_model/lstm/lstm.py:79-133
  YolactMasks  functs/benchmark/ai_model/yolact/yolact_mask.py:250-264, 306-333

``register_all()`` scripts every pattern, runs it through the same functionalization as a user's program
(``_C._jit_pass_prepare_for_matching``) and registers its canonical signature with the kernel adapter that executes it.
A user's program whose functionalized graph contains a region with the same signature — same operations, same structural
constants; thresholds, top-k and the frozen tensors (priors, weights) are free — is then lowered by
``functs_b200.jit.build`` to one ``tssa::ParallelFunctor`` bound to those kernels.

The free scalars are found by value: a pattern is instantiated with values that occur nowhere else in it, and every
constant slot that holds such a value becomes a named wildcard.
"""
import math
import threading
from typing import List, Tuple

import torch
import torchvision  # noqa: F401  (registers torchvision::nms for TorchScript)
from torch import Tensor

from . import _C

# ---- shared pieces -------------------------------------------------------------------------------------------------


def batched_nms(boxes: Tensor, scores: Tensor, idxs: Tensor, iou_threshold: float) -> Tuple[Tensor, Tensor]:
    max_coordinate = boxes.max()
    offsets = idxs.to(boxes) * (max_coordinate + 1)
    boxes_for_nms = boxes + offsets[:, None]
    keep = torchvision.ops.nms(boxes_for_nms, scores, iou_threshold)
    dets = torch.cat([boxes[keep], scores[keep].reshape(-1, 1)], dim=1)
    return dets, keep


def select_topk(scores: Tensor, score_thr: float, topk: int) -> Tuple[Tensor, Tensor]:
    valid_mask = scores > score_thr
    cand = scores[valid_mask]
    valid_idxs = torch.nonzero(valid_mask)
    num_topk = min(topk, valid_idxs.size(0))
    sorted_scores, order = cand.sort(descending=True, stable=True)
    sorted_scores = sorted_scores[:num_topk]
    topk_idxs = valid_idxs[order[:num_topk]]
    return sorted_scores, topk_idxs


# ---- YOLOv3 ----------------------------------------------------------------------------------------------------------

YOLO_STRIDES = (32, 16, 8)
YOLO_ANCHORS = (((116, 90), (156, 198), (373, 326)),
                ((30, 61), (62, 45), (59, 119)),
                ((10, 13), (16, 30), (33, 23)))


def yolo_grid(size: int) -> Tensor:
    xs = torch.arange(size, dtype=torch.float32).repeat(size)
    ys = torch.arange(size, dtype=torch.float32).reshape(-1, 1).repeat(1, size).reshape(-1)
    g = torch.stack([xs, ys], dim=-1)
    return g[:, None, :].expand(size * size, 3, 2).reshape(-1, 2).clone()


def yolo_anchor_wh(level: int, size: int) -> Tensor:
    a = torch.tensor(YOLO_ANCHORS[level], dtype=torch.float32)
    return a[None, :, :].expand(size * size, 3, 2).reshape(-1, 2).clone()


class YOLOV3Post(torch.nn.Module):
    """forward(pred_maps) -> (bboxes, obj, cls, per-image (dets, labels, flat_ids)); see YOLOV3Det for results only."""

    def __init__(self, sizes: Tuple[int, int, int] = (13, 26, 52), score_thr: float = 0.5, topk: int = 1000,
                 iou_thr: float = 0.45):
        super().__init__()
        self.score_thr = score_thr
        self.topk = topk
        self.iou_thr = iou_thr
        self.num_attrib = 85
        self.grids = [yolo_grid(s) for s in sizes]
        self.anchor_whs = [yolo_anchor_wh(i, s) for i, s in enumerate(sizes)]
        self.strides = [float(s) for s in YOLO_STRIDES]
        self.num_classes = 80

    def decode(self, pred_maps: List[Tensor]) -> Tuple[Tensor, Tensor, Tensor]:
        num_imgs = pred_maps[0].size(0)
        flatten_preds = []
        for lvl in range(3):
            pred = pred_maps[lvl].permute(0, 2, 3, 1).reshape(num_imgs, -1, self.num_attrib).clone()
            pred[..., 0:2].sigmoid_()
            pred[..., 4:].sigmoid_()
            pred[..., 0:2] = (pred[..., 0:2] + self.grids[lvl]) * self.strides[lvl]
            pred[..., 2:4] = pred[..., 2:4].exp() * self.anchor_whs[lvl]
            flatten_preds.append(pred.clone())
        flat = torch.cat(flatten_preds, dim=1)
        xy = flat[..., 0:2]
        half = flat[..., 2:4] * 0.5
        bboxes = torch.cat([xy - half, xy + half], dim=-1)
        obj = flat[..., 4].clone()
        cls = flat[..., 5:].clone()
        return bboxes, obj, cls

    def post_single(self, bboxes: Tensor, obj: Tensor, cls: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
        scores = obj.unsqueeze(-1) * cls
        s, idx = select_topk(scores, self.score_thr, self.topk)
        box_idx = idx[:, 0]
        labels = idx[:, 1]
        if s.size(0) == 0:
            return (torch.zeros([0, 5], dtype=bboxes.dtype), torch.zeros([0], dtype=torch.long),
                    torch.zeros([0], dtype=torch.long))
        dets, keep = batched_nms(bboxes[box_idx], s, labels, self.iou_thr)
        flat_ids = box_idx * self.num_classes + labels
        return dets, labels[keep], flat_ids[keep]

    def forward(self, pred_maps: List[Tensor]):
        bboxes, obj, cls = self.decode(pred_maps)
        results: List[Tuple[Tensor, Tensor, Tensor]] = []
        for b in range(bboxes.size(0)):
            results.append(self.post_single(bboxes[b], obj[b], cls[b]))
        return bboxes, obj, cls, results


class YOLOV3Det(YOLOV3Post):
    """The same program returning only the per-image detections (what the reference's module returns)."""

    def forward(self, pred_maps: List[Tensor]):
        bboxes, obj, cls = self.decode(pred_maps)
        results: List[Tuple[Tensor, Tensor, Tensor]] = []
        for b in range(bboxes.size(0)):
            results.append(self.post_single(bboxes[b], obj[b], cls[b]))
        return results


# ---- SSD -------------------------------------------------------------------------------------------------------------


def ssd_delta2bbox(priors: Tensor, loc: Tensor, clamp_max: float = 300.0) -> Tensor:
    pxy = priors[:, 0:2]
    pwh = priors[:, 2:4]
    gxy = pxy + pwh * (loc[:, 0:2] * 0.1)
    gwh = pwh * (loc[:, 2:4] * 0.2).exp()
    x1y1 = gxy - gwh * 0.5
    x2y2 = gxy + gwh * 0.5
    bboxes = torch.cat([x1y1, x2y2], dim=-1)
    bboxes[..., 0::2].clamp_(min=0.0, max=clamp_max)
    bboxes[..., 1::2].clamp_(min=0.0, max=clamp_max)
    return bboxes.clone()


class SSDPost(torch.nn.Module):
    """forward(loc [B,P,4], conf [B,P,C+1]) -> (bboxes, scores, per-image (dets, labels, prior_ids))."""

    def __init__(self, priors: Tensor, score_thr: float = 0.01, topk: int = 200, iou_thr: float = 0.45,
                 clamp_max: float = 300.0):
        super().__init__()
        self.priors = priors
        self.score_thr = score_thr
        self.topk = topk
        self.iou_thr = iou_thr
        self.clamp_max = clamp_max

    def class_single(self, bboxes: Tensor, scores_c: Tensor) -> Tuple[Tensor, Tensor]:
        mask = scores_c > self.score_thr
        idx = torch.nonzero(mask)[:, 0]
        cand = scores_c[mask]
        k = min(self.topk, idx.size(0))
        s, order = cand.sort(descending=True, stable=True)
        s = s[:k]
        idx = idx[order[:k]]
        bx = bboxes[idx]
        keep = torchvision.ops.nms(bx, s, self.iou_thr)
        dets = torch.cat([bx[keep], s[keep].reshape(-1, 1)], dim=1)
        return dets, idx[keep]

    def post_single(self, bboxes: Tensor, scores: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
        dets_l = []
        labels_l = []
        ids_l = []
        for c in range(scores.size(1)):
            dets, ids = self.class_single(bboxes, scores[:, c])
            dets_l.append(dets)
            ids_l.append(ids)
            labels_l.append(torch.full([ids.size(0)], c, dtype=torch.long))
        return torch.cat(dets_l), torch.cat(labels_l), torch.cat(ids_l)

    def forward(self, loc: Tensor, conf: Tensor):
        num_imgs = loc.size(0)
        scores = conf.softmax(-1)[..., :-1]
        bboxes = torch.zeros_like(loc)
        results: List[Tuple[Tensor, Tensor, Tensor]] = []
        for b in range(num_imgs):
            bboxes[b] = ssd_delta2bbox(self.priors, loc[b], self.clamp_max)
            results.append(self.post_single(bboxes[b], scores[b]))
        return bboxes, scores, results


# ---- LSTM ------------------------------------------------------------------------------------------------------------


def lstm_cell(x: Tensor, h: Tensor, c: Tensor, w_ih: Tensor, w_hh: Tensor, b_ih: Tensor,
              b_hh: Tensor) -> Tuple[Tensor, Tensor]:
    ih = torch.matmul(x, w_ih) + b_ih
    hh = torch.matmul(h, w_hh) + b_hh
    ingate = torch.sigmoid(ih[0] + hh[0])
    forgetgate = torch.sigmoid(ih[1] + hh[1])
    cellgate = torch.tanh(ih[2] + hh[2])
    outgate = torch.sigmoid(ih[3] + hh[3])
    c = (forgetgate * c) + (ingate * cellgate)
    h = outgate * torch.tanh(c)
    return h, c


class LSTMSeq(torch.nn.Module):
    def __init__(self, w_ih: Tensor, w_hh: Tensor, b_ih: Tensor, b_hh: Tensor):
        super().__init__()
        self.w_ih = w_ih
        self.w_hh = w_hh
        self.b_ih = b_ih
        self.b_hh = b_hh

    def forward(self, x: Tensor) -> Tuple[Tensor, Tensor]:
        seq_len, batch, _ = x.shape
        hidden = self.w_hh.size(2)
        hs = torch.zeros(seq_len, batch, hidden, dtype=x.dtype)
        cs = torch.zeros(seq_len, batch, hidden, dtype=x.dtype)
        h = torch.zeros(batch, hidden, dtype=x.dtype)
        c = torch.zeros(batch, hidden, dtype=x.dtype)
        for t in range(seq_len):
            h, c = lstm_cell(x[t], h, c, self.w_ih, self.w_hh, self.b_ih, self.b_hh)
            hs[t] = h
            cs[t] = c
        return hs, cs


# ---- YOLACT ----------------------------------------------------------------------------------------------------------


def sanitize_coordinates(x1: Tensor, x2: Tensor, img_size: int) -> Tuple[Tensor, Tensor]:
    padding = 1
    x1 = torch.min(x1, x2)
    x2 = torch.max(x1, x2)
    x1 = torch.clamp(x1 - padding, min=0)
    x2 = torch.clamp(x2 + padding, max=img_size)
    return x1, x2


def crop_bounds(boxes: Tensor, h: int, w: int) -> Tensor:
    x1, x2 = sanitize_coordinates(boxes[:, 0], boxes[:, 2], w)
    y1, y2 = sanitize_coordinates(boxes[:, 1], boxes[:, 3], h)
    return torch.stack([torch.ceil(x1), torch.ceil(x2), torch.ceil(y1), torch.ceil(y2)], dim=1).to(torch.long)


def crop_by_slice_assign(mask_pred: Tensor, boxes: Tensor) -> Tensor:
    h, w, n = mask_pred.shape
    bounds = crop_bounds(boxes, h, w)
    cropped = torch.zeros(n, h, w, dtype=mask_pred.dtype)
    for d in range(n):
        xs = int(bounds[d, 0])
        xe = int(bounds[d, 1])
        ys = int(bounds[d, 2])
        ye = int(bounds[d, 3])
        cropped[d, ys:ye, xs:xe] = mask_pred[ys:ye, xs:xe, d]
    return cropped


class YolactMasks(torch.nn.Module):
    """forward(proto [B,H,W,K], coef [B,N,K], boxes [B,N,4]) -> (masks uint8 [B,N,H,W], logits [B,H,W,N])."""

    def __init__(self, thr: float = 0.5):
        super().__init__()
        self.thr = thr

    def forward(self, proto: Tensor, coef: Tensor, boxes: Tensor) -> Tuple[Tensor, Tensor]:
        num_imgs, h, w, _ = proto.shape
        n = coef.size(1)
        out = torch.zeros(num_imgs, n, h, w, dtype=torch.uint8)
        logits = torch.zeros(num_imgs, h, w, n, dtype=proto.dtype)
        for b in range(num_imgs):
            mask_pred = proto[b] @ coef[b].t()
            logits[b] = mask_pred
            mask_pred = torch.sigmoid(mask_pred)
            cropped = crop_by_slice_assign(mask_pred, boxes[b])
            out[b] = (cropped > self.thr).to(torch.uint8)
        return out, logits


class YolactMasksOnly(torch.nn.Module):
    """The same program without the dense logits output: forward(...) -> masks uint8 [B,N,H,W]."""

    def __init__(self, thr: float = 0.5):
        super().__init__()
        self.thr = thr

    def forward(self, proto: Tensor, coef: Tensor, boxes: Tensor) -> Tensor:
        num_imgs, h, w, _ = proto.shape
        n = coef.size(1)
        out = torch.zeros(num_imgs, n, h, w, dtype=torch.uint8)
        for b in range(num_imgs):
            mask_pred = torch.sigmoid(proto[b] @ coef[b].t())
            cropped = crop_by_slice_assign(mask_pred, boxes[b])
            out[b] = (cropped > self.thr).to(torch.uint8)
        return out


# ---- registration ----------------------------------------------------------------------------------------------------

# values that occur nowhere else in the programs: the constant slots that hold them become the named wildcards
_F = {"score_thr": 0.515625, "iou_thr": 0.4375, "clamp_max": 301.5, "thr": 0.53125}
_I = {"topk": 777, "hidden": 48}


def _prepared_graph(module: torch.nn.Module) -> torch.Graph:
    frozen = torch.jit.freeze(torch.jit.script(module).eval())
    g = frozen.graph
    torch._C._jit_pass_inline(g)
    _C._jit_pass_prepare_for_matching(g)
    return g


def _register(adapter: str, module: torch.nn.Module, float_roles=(), int_roles=()) -> dict:
    g = _prepared_graph(module)
    d = _C._describe_region(g)
    froles, iroles = [], []
    for name in float_roles:
        slots = [i for i, v in enumerate(d["fconsts"]) if v == _F[name]]
        if not slots:
            raise RuntimeError(f"pattern '{adapter}': no constant slot holds {name}")
        froles += [(name, i) for i in slots]
    for name in int_roles:
        slots = [i for i, v in enumerate(d["iconsts"]) if v == _I[name]]
        if not slots:
            raise RuntimeError(f"pattern '{adapter}': no constant slot holds {name}")
        iroles += [(name, i) for i in slots]
    _C._register_region_pattern(adapter, g, froles, iroles)
    return _C._describe_region(g, [i for _, i in froles], [i for _, i in iroles])


_lock = threading.Lock()
_registered = {}


def register_all() -> dict:
    """Registers every pattern once per process; returns {adapter: description} (signature, node and constant counts)."""
    with _lock:
        if _registered:
            return _registered
        yolo = dict(sizes=(2, 3, 5), score_thr=_F["score_thr"], topk=_I["topk"], iou_thr=_F["iou_thr"])
        _registered["yolov3_post_dense"] = _register("yolov3_post_dense", YOLOV3Post(**yolo),
                                                     ("score_thr", "iou_thr"), ("topk",))
        _registered["yolov3_post"] = _register("yolov3_post", YOLOV3Det(**yolo), ("score_thr", "iou_thr"), ("topk",))
        g = torch.Generator().manual_seed(1)
        priors = torch.rand(12, 4, generator=g) * 100 + 1
        _registered["ssd_post"] = _register(
            "ssd_post", SSDPost(priors, score_thr=_F["score_thr"], topk=_I["topk"], iou_thr=_F["iou_thr"],
                                clamp_max=_F["clamp_max"]), ("score_thr", "iou_thr", "clamp_max"), ("topk",))
        h = _I["hidden"]
        bound = 1.0 / math.sqrt(h)
        w = [(torch.rand(*shape, generator=g) * 2 - 1) * bound for shape in ((4, h, h), (4, h, h), (4, 1, h), (4, 1, h))]
        _registered["lstm_seq"] = _register("lstm_seq", LSTMSeq(*w), (), ("hidden",))
        _registered["yolact_masks_logits"] = _register("yolact_masks_logits", YolactMasks(_F["thr"]), ("thr",))
        _registered["yolact_masks"] = _register("yolact_masks", YolactMasksOnly(_F["thr"]), ("thr",))
        return _registered
