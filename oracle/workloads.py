"""CPU oracle: the five imperative tensor programs, un-functionalized, for TorchScript.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file; it is the
checker used by the tests, by the smoke run and by the CPU-baseline leg of the benchmark.

Each module below is a restatement, for CPU and for the configured shapes, of one of the
reference's imperative workloads (views + in-place slice/select assignment + Python loops).
Running the un-functionalized program through ``torch.jit.script`` on CPU is what the
reference's own tests use as ground truth (reference ``test/test_basic.py:42-52`` compares
the functionalized graph with the eager program), so these programs define the expected
answers for the CUDA kernels.

Parity pin status:
  * ``get_started``, ``batched_nms``, ``select_topk``, ``ssd_delta2bbox``, ``lstm_cell`` and
    ``crop_by_slice_assign`` are pinned, bit for bit, against outputs of the reference's own Python
    functions (``tests/golden/make_golden.py`` wrote the fixtures; ``tests/test_oracle_golden.py``
    checks them).  The YOLOv3 decode (sigmoid + grid offset, exp * anchor) is pinned to 1e-5 relative, not bit for
    bit, against the reference's ``decode_bboxes`` on the anchors of its ``YOLOAnchorGenerator``
    (yolov3_bbox.py:12-100): the reference forms the centre as anchor centre + (sigmoid - 0.5) * stride, this
    program as (sigmoid + cell) * stride — the same boxes through another operation order.
  * ``torchvision.ops.nms``, ``torch.sort`` and the ATen CPU math kernels are third-party
    arithmetic that the reference's tests do not pin; the installed CPU kernels define the answer.

Reference files followed (paths inside the reference project):
  get_started : examples/get_started.py:10-15
  YOLOv3      : functs/benchmark/ai_model/yolov3/yolov3_bbox.py:12-23, 104-179, 195-243
  SSD         : functs/benchmark/ai_model/ssd/ssd_bbox.py:121-214, 254-290
  LSTM        : functs/benchmark/ai_model/lstm/lstm.py:47-133
  YOLACT      : functs/benchmark/ai_model/yolact/yolact_mask.py:250-264, 306-333
"""
from typing import List, Tuple

import math

import torch
import torchvision  # noqa: F401  (registers torchvision::nms for TorchScript)
from torch import Tensor

# ----------------------------------------------------------------------------------------
# C1: get_started loop  (examples/get_started.py:10-15)
# ----------------------------------------------------------------------------------------


def get_started(a: Tensor, b: Tensor, n: int) -> Tensor:
    a = a.clone()
    b = b.clone()
    for i in range(n):
        b[i] = b[i] + 1
    return b


# ----------------------------------------------------------------------------------------
# shared: class-offset NMS  (yolov3_bbox.py:139-179 == ssd_bbox.py:175-214, small-input branch)
# ----------------------------------------------------------------------------------------


def batched_nms(boxes: Tensor, scores: Tensor, idxs: Tensor, iou_threshold: float) -> Tuple[Tensor, Tensor]:
    """Class-wise NMS by shifting every class into its own coordinate range.

    Returns (dets [m,5] = kept boxes (un-shifted) + score, keep [m] indices into the inputs).
    """
    max_coordinate = boxes.max()
    offsets = idxs.to(boxes) * (max_coordinate + 1)
    boxes_for_nms = boxes + offsets[:, None]
    keep = torchvision.ops.nms(boxes_for_nms, scores, iou_threshold)
    dets = torch.cat([boxes[keep], scores[keep].reshape(-1, 1)], dim=1)
    return dets, keep


def select_topk(scores: Tensor, score_thr: float, topk: int) -> Tuple[Tensor, Tensor]:
    """mask -> nonzero -> stable descending sort -> truncate.

    ``scores`` is [N, C].  Returns (sorted scores [k], idx [k,2] = (row, col) of each survivor).
    Follows ssd_bbox.py:163-172 (filter_scores_and_topk) with the sort made explicitly stable
    so that equal scores keep ascending (row, col) order.
    """
    valid_mask = scores > score_thr
    cand = scores[valid_mask]
    valid_idxs = torch.nonzero(valid_mask)
    num_topk = min(topk, valid_idxs.size(0))
    sorted_scores, order = cand.sort(descending=True, stable=True)
    sorted_scores = sorted_scores[:num_topk]
    topk_idxs = valid_idxs[order[:num_topk]]
    return sorted_scores, topk_idxs


# ----------------------------------------------------------------------------------------
# C2: YOLOv3-style decode + mask + top-k + class-wise NMS
# ----------------------------------------------------------------------------------------

YOLO_STRIDES = (32, 16, 8)
YOLO_ANCHORS = (((116, 90), (156, 198), (373, 326)),
                ((30, 61), (62, 45), (59, 119)),
                ((10, 13), (16, 30), (33, 23)))  # yolov3_bbox.py:191-193
YOLO_NUM_CLASSES = 80


def yolo_grid(size: int) -> Tensor:
    """[size*size*3, 2] (x, y) cell offsets in box order (y, x, anchor)."""
    xs = torch.arange(size, dtype=torch.float32).repeat(size)
    ys = torch.arange(size, dtype=torch.float32).reshape(-1, 1).repeat(1, size).reshape(-1)
    g = torch.stack([xs, ys], dim=-1)  # [S*S, 2]
    return g[:, None, :].expand(size * size, 3, 2).reshape(-1, 2).clone()


def yolo_anchor_wh(level: int, size: int) -> Tensor:
    a = torch.tensor(YOLO_ANCHORS[level], dtype=torch.float32)  # [3,2]
    return a[None, :, :].expand(size * size, 3, 2).reshape(-1, 2).clone()


class YOLOV3Post(torch.nn.Module):
    """Decode three NCHW logit maps and post-process every image.

    forward(pred_maps) -> (bboxes [B,N,4], obj [B,N], cls [B,N,80], per-image results)
    where every result is (dets [m,5], labels [m] int64, flat_ids [m] int64 = box*80+label).
    """

    def __init__(self, sizes: Tuple[int, int, int] = (13, 26, 52), score_thr: float = 0.5,
                 topk: int = 1000, iou_thr: float = 0.45):
        super().__init__()
        self.sizes = list(sizes)
        self.score_thr = score_thr
        self.topk = topk
        self.iou_thr = iou_thr
        self.num_attrib = 5 + YOLO_NUM_CLASSES
        self.grids = [yolo_grid(s) for s in sizes]
        self.anchor_whs = [yolo_anchor_wh(i, s) for i, s in enumerate(sizes)]
        self.strides = [float(s) for s in YOLO_STRIDES]
        self.num_classes = YOLO_NUM_CLASSES

    def decode(self, pred_maps: List[Tensor]) -> Tuple[Tensor, Tensor, Tensor]:
        num_imgs = pred_maps[0].size(0)
        flatten_preds = []
        for lvl in range(3):
            pred = pred_maps[lvl].permute(0, 2, 3, 1).reshape(num_imgs, -1, self.num_attrib).clone()
            pred[..., 0:2].sigmoid_()
            pred[..., 4:].sigmoid_()
            pred[..., 0:2] = (pred[..., 0:2] + self.grids[lvl]) * self.strides[lvl]
            pred[..., 2:4] = pred[..., 2:4].exp() * self.anchor_whs[lvl]
            flatten_preds.append(pred.clone())  # a copy goes into the list, as in yolov3_bbox.py:213
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


# ----------------------------------------------------------------------------------------
# C3: SSD-style post-process
# ----------------------------------------------------------------------------------------

SSD_IMG = 300.0
SSD_FEATS = (38, 19, 10, 5, 3, 1)
SSD_STEPS = (8, 16, 32, 64, 100, 300)
SSD_MIN = (30.0, 60.0, 111.0, 162.0, 213.0, 264.0)
SSD_MAX = (60.0, 111.0, 162.0, 213.0, 264.0, 315.0)
SSD_RATIOS = ((2,), (2, 3), (2, 3), (2, 3), (2,), (2,))
SSD_NUM_CLASSES = 80


def ssd_priors() -> Tensor:
    """[8732,4] (cx, cy, w, h) in pixels of a 300x300 image, fixed SSD300 grid, fp32.

    Box order: level, y, x, shape-within-cell (small square, large square, then w>h / h>w pairs).
    Everything is computed in float64 and rounded once so the table is identical anywhere.
    """
    out = []
    for k in range(6):
        f = SSD_FEATS[k]
        for i in range(f):
            for j in range(f):
                cx = (j + 0.5) * SSD_STEPS[k]
                cy = (i + 0.5) * SSD_STEPS[k]
                s = SSD_MIN[k]
                out.append((cx, cy, s, s))
                sp = math.sqrt(SSD_MIN[k] * SSD_MAX[k])
                out.append((cx, cy, sp, sp))
                for r in SSD_RATIOS[k]:
                    q = math.sqrt(float(r))
                    out.append((cx, cy, s * q, s / q))
                    out.append((cx, cy, s / q, s * q))
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


def ssd_delta2bbox(priors: Tensor, loc: Tensor, clamp_max: float = 300.0) -> Tensor:
    """Variance-scaled centre/size decode with the strided in-place clamp of
    ssd_bbox.py:121-154 (stds 0.1/0.2 play the role of the variances; clamp_ on [..., 0::2] / [..., 1::2])."""
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
    """forward(loc [B,P,4], conf [B,P,81]) -> (bboxes [B,P,4], scores [B,P,80], per-image results).

    Every result is (dets [m,5], labels [m], prior_ids [m]) concatenated over the class loop.
    The last confidence column is background (ssd_bbox.py:268 drops the last column).
    """

    def __init__(self, score_thr: float = 0.01, topk: int = 200, iou_thr: float = 0.45):
        super().__init__()
        self.priors = ssd_priors()
        self.score_thr = score_thr
        self.topk = topk
        self.iou_thr = iou_thr
        self.num_classes = SSD_NUM_CLASSES

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
            bboxes[b] = ssd_delta2bbox(self.priors, loc[b])
            results.append(self.post_single(bboxes[b], scores[b]))
        return bboxes, scores, results


# ----------------------------------------------------------------------------------------
# C4: imperative LSTM with slice-assigned outputs  (lstm.py:79-133; one layer, hs/cs kept per step)
# ----------------------------------------------------------------------------------------


def lstm_cell(x: Tensor, h: Tensor, c: Tensor, w_ih: Tensor, w_hh: Tensor, b_ih: Tensor,
              b_hh: Tensor) -> Tuple[Tensor, Tensor]:
    """One step, lstm.py:79-98: gates picked by select on the leading gate dimension."""
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
    """Weights use the reference's gate-leading layout [4, in, H] (lstm.py:60-77); gate order i,f,g,o."""

    def __init__(self, w_ih: Tensor, w_hh: Tensor, b_ih: Tensor, b_hh: Tensor):
        super().__init__()
        self.w_ih = w_ih  # [4, I, H]
        self.w_hh = w_hh  # [4, H, H]
        self.b_ih = b_ih  # [4, 1, H]
        self.b_hh = b_hh  # [4, 1, H]

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


# ----------------------------------------------------------------------------------------
# C5: YOLACT-style mask assembly  (yolact_mask.py:250-264, 306-333)
# ----------------------------------------------------------------------------------------


def sanitize_coordinates(x1: Tensor, x2: Tensor, img_size: int) -> Tuple[Tensor, Tensor]:
    """yolact_mask.py:327-333 (padding 1; note x2 uses the already-minimised x1, as there)."""
    padding = 1
    x1 = torch.min(x1, x2)
    x2 = torch.max(x1, x2)
    x1 = torch.clamp(x1 - padding, min=0)
    x2 = torch.clamp(x2 + padding, max=img_size)
    return x1, x2


def crop_bounds(boxes: Tensor, h: int, w: int) -> Tensor:
    """Integer [N,4] (xs, xe, ys, ye): pixel column j is inside iff j >= x1 and j < x2
    (yolact_mask.py:318-323), i.e. ceil(x1) <= j < ceil(x2)."""
    x1, x2 = sanitize_coordinates(boxes[:, 0], boxes[:, 2], w)
    y1, y2 = sanitize_coordinates(boxes[:, 1], boxes[:, 3], h)
    return torch.stack([torch.ceil(x1), torch.ceil(x2), torch.ceil(y1), torch.ceil(y2)], dim=1).to(torch.long)


def crop_by_slice_assign(mask_pred: Tensor, boxes: Tensor) -> Tensor:
    """mask_pred [H,W,N] -> [N,H,W]: zero outside each detection's sanitised box, written by slice assignment."""
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


# ----------------------------------------------------------------------------------------
# seeded synthetic inputs (seed = 1000*config + batch index; every image differs)
# ----------------------------------------------------------------------------------------


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def make_get_started_inputs() -> Tuple[Tensor, Tensor, int]:
    g = _gen(1000)
    return torch.randn(64, 1024, generator=g), torch.randn(64, 1024, generator=g), 64


def make_yolo_inputs(batch: int, sizes: Tuple[int, int, int] = (13, 26, 52), first: int = 0) -> List[Tensor]:
    maps = [torch.empty(batch, 255, s, s) for s in sizes]
    for b in range(batch):
        g = _gen(2000 + first + b)
        for lvl, s in enumerate(sizes):
            maps[lvl][b] = torch.randn(255, s, s, generator=g)
    return maps


def make_ssd_inputs(batch: int, first: int = 0) -> Tuple[Tensor, Tensor]:
    loc = torch.empty(batch, 8732, 4)
    conf = torch.empty(batch, 8732, 81)
    for b in range(batch):
        g = _gen(3000 + first + b)
        loc[b] = torch.randn(8732, 4, generator=g)
        conf[b] = torch.randn(8732, 81, generator=g)
    return loc, conf


def make_lstm_inputs(seq_len: int = 64, batch: int = 64, hidden: int = 512, first: int = 0):
    """x is drawn per sequence so that a batch shard [first, first+batch) equals the same rows of the full batch."""
    g = _gen(4000)
    bound = 1.0 / math.sqrt(hidden)
    w_ih = (torch.rand(4, hidden, hidden, generator=g) * 2 - 1) * bound
    w_hh = (torch.rand(4, hidden, hidden, generator=g) * 2 - 1) * bound
    b_ih = (torch.rand(4, 1, hidden, generator=g) * 2 - 1) * bound
    b_hh = (torch.rand(4, 1, hidden, generator=g) * 2 - 1) * bound
    x = torch.empty(seq_len, batch, hidden)
    for b in range(batch):
        gb = _gen(4100 + first + b)
        x[:, b, :] = torch.randn(seq_len, hidden, generator=gb)
    return x, w_ih, w_hh, b_ih, b_hh


def make_yolact_inputs(batch: int, size: int = 138, num_det: int = 100, first: int = 0):
    proto = torch.empty(batch, size, size, 32)
    coef = torch.empty(batch, num_det, 32)
    boxes = torch.empty(batch, num_det, 4)
    for b in range(batch):
        g = _gen(5000 + first + b)
        proto[b] = torch.randn(size, size, 32, generator=g)
        coef[b] = torch.tanh(torch.randn(num_det, 32, generator=g))
        u = torch.rand(num_det, 4, generator=g)
        xs, _ = torch.sort(u[:, 0:2], dim=1)
        ys, _ = torch.sort(u[:, 2:4], dim=1)
        boxes[b] = torch.stack([xs[:, 0], ys[:, 0], xs[:, 1], ys[:, 1]], dim=1) * float(size)
    return proto, coef, boxes
