"""Tie-band audit: when a device result differs from the CPU oracle's own run, prove that the first decision on which
the two runs part lies inside the band where last-ulp differences of fp32 exp / softmax / dot products can flip it.

The integer stages (mask -> stable sort -> top-k -> greedy NMS) are exact functions of their fp32 inputs, and the GPU
tests check separately that the device output IS that function of the device's own floats.  Two runs of an exact
function can therefore only differ because their float inputs differ, and the difference must start at a decision
whose margin is of the size of the input difference.  The audit finds that first decision and measures its margin in
fp64; everything after it is a consequence and is not examined.  A run that differs without such a decision fails.

Stages audited, in pipeline order:
  selection  the two sorted top-k lists are compared position by position: ids that differ at a position must have fp64
             scores within `eps_score` relative of each other (a swap of near-equal scores, or an exchange at the top-k
             boundary); surplus entries of the longer list must have fp64 scores within `eps_score` of the mask threshold;
  nms        only when the selected lists are identical: at the first candidate that one run keeps and the other
             suppresses, some box kept earlier by both must have an fp64 IoU with it within `eps_iou` of the threshold,
             where eps_iou is derived from the measured coordinate difference of the two runs' boxes.
"""
from typing import Optional, Sequence, Tuple

import torch

EPS_SCORE = 1e-6   # relative: a few ulp (6e-8) of an fp32 score that went through exp, divide and one or two products


def audit_selection(ids_a: torch.Tensor, ids_b: torch.Tensor, score64: torch.Tensor, thr: float, topk: int,
                    eps: float = EPS_SCORE) -> int:
    """ids_*: flat candidate ids of the two runs' sorted top-k lists; score64: fp64 score per flat id.
    Returns the number of positions that differ (0 = identical); raises AssertionError on an unexplained difference."""
    na, nb = ids_a.numel(), ids_b.numel()
    n = min(na, nb)
    differ = torch.nonzero(ids_a[:n] != ids_b[:n])[:, 0]
    if differ.numel():
        sa, sb = score64[ids_a[:n][differ]], score64[ids_b[:n][differ]]
        gap = (sa - sb).abs() / torch.maximum(sa.abs(), sb.abs())
        assert bool((gap <= eps).all()), (
            f"selection differs at {differ.numel()} positions; largest fp64 score gap {float(gap.max()):.3e} > {eps}")
    extra = ids_a[n:] if na > nb else ids_b[n:]
    if extra.numel():
        assert max(na, nb) <= topk
        gap = (score64[extra] - thr).abs() / thr
        assert bool((gap <= eps).all()), (
            f"{extra.numel()} surplus candidates are not at the mask threshold: largest gap {float(gap.max()):.3e}")
    return int(differ.numel()) + int(extra.numel())


def offset_boxes(boxes: torch.Tensor, labels: Optional[torch.Tensor]) -> torch.Tensor:
    """fp32 boxes shifted per class exactly as the oracle's batched_nms shifts them (no shift when labels is None)."""
    if labels is None or boxes.numel() == 0:
        return boxes
    max_coordinate = boxes.max()
    offsets = labels.to(boxes) * (max_coordinate + 1)
    return boxes + offsets[:, None]


def iou64(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a [4], b [m,4] (any float dtype) -> fp64 IoU [m] with the torchvision formula."""
    a, b = a.double(), b.double()
    area_a = (a[2] - a[0]) * (a[3] - a[1])
    area_b = (b[:, 2] - b[:, 0]) * (b[:, 3] - b[:, 1])
    w = (torch.minimum(a[2], b[:, 2]) - torch.maximum(a[0], b[:, 0])).clamp(min=0)
    h = (torch.minimum(a[3], b[:, 3]) - torch.maximum(a[1], b[:, 1])).clamp(min=0)
    inter = w * h
    return inter / (area_a + area_b - inter)


def audit_nms(keep_a: torch.Tensor, keep_b: torch.Tensor, boxes_a: torch.Tensor, boxes_b: torch.Tensor,
              labels: Optional[torch.Tensor], iou_thr: float) -> Tuple[int, float]:
    """keep_*: kept positions (ascending) in the SAME selected list; boxes_*: the two runs' fp32 boxes of that list
    [n,4]; labels: class of each candidate for class-offset NMS (None = plain NMS).
    Returns (first differing candidate or -1, its margin).  Raises on an unexplained difference."""
    ka, kb = keep_a.tolist(), keep_b.tolist()
    if ka == kb:
        return -1, 0.0
    p = 0
    while p < min(len(ka), len(kb)) and ka[p] == kb[p]:
        p += 1
    # x: the first candidate on which the runs disagree (kept by exactly one of them)
    cand = [k[p] for k in (ka, kb) if p < len(k)]
    x = min(cand)
    common = torch.tensor(ka[:p], dtype=torch.long)
    assert common.numel() > 0, "the first candidate is always kept: a difference before any kept box is a bug"
    oa, ob = offset_boxes(boxes_a, labels), offset_boxes(boxes_b, labels)
    # coordinate difference of the two runs (after the class shift, whose fp32 rounding dominates it)
    sel = torch.cat([common, torch.tensor([x])])
    delta = float((oa[sel].double() - ob[sel].double()).abs().max())
    mag = float(torch.maximum(oa[sel].abs(), ob[sel].abs()).max())
    assert delta <= 4 * mag * 2.0 ** -23 + 1e-30, f"boxes of the two runs differ by {delta:.3e} at magnitude {mag:.3e}"
    ia, ib = iou64(oa[x], oa[common]), iou64(ob[x], ob[common])
    side = float(torch.minimum(oa[sel, 2] - oa[sel, 0], oa[sel, 3] - oa[sel, 1]).min())
    # an IoU moves by at most ~4 * delta / side when every coordinate moves by delta; fp32 evaluation adds ~1e-6 relative
    eps_iou = 16.0 * delta / max(side, 1e-12) + 4e-6
    margin = torch.minimum((ia - iou_thr).abs(), (ib - iou_thr).abs())
    best = float(margin.min())
    assert best <= eps_iou, (
        f"candidate {x} is kept by one run and suppressed by the other, but no earlier kept box has an IoU within "
        f"{eps_iou:.3e} of {iou_thr}: closest margin {best:.3e}")
    return x, best


def explain_or_fail(sel_ids_a: torch.Tensor, sel_ids_b: torch.Tensor, score64: torch.Tensor, thr: float, topk: int,
                    keep_a: torch.Tensor, keep_b: torch.Tensor, boxes_a: torch.Tensor, boxes_b: torch.Tensor,
                    labels: Optional[torch.Tensor], iou_thr: float) -> str:
    """Full audit of one list.  a = device run, b = oracle run.  Returns a one-line description of the first divergence
    ("identical" when there is none)."""
    ndiff = audit_selection(sel_ids_a, sel_ids_b, score64, thr, topk)
    if ndiff:
        return f"selection: {ndiff} positions inside the {EPS_SCORE} score band"
    x, margin = audit_nms(keep_a, keep_b, boxes_a, boxes_b, labels, iou_thr)
    if x < 0:
        return "identical"
    return f"nms: candidate {x} decided by an IoU {margin:.2e} from the threshold"
