"""The fp64 tie-band audit itself (tests/tieband.py), on CPU: it must accept differences that one-ulp input changes cause
and reject differences that larger input changes cause."""
import pytest
import torch

from oracle import workloads as W
from tests import tieband


def stages(scores, boxes, labels_of, thr, topk, iou):
    """mask -> stable sort -> top-k -> class-offset NMS on [N, C] scores; returns (ids, kept positions, boxes, labels)."""
    s, idx = W.select_topk(scores, thr, topk)
    ids = idx[:, 0] * scores.size(1) + idx[:, 1]
    _, keep = W.batched_nms(boxes[idx[:, 0]], s, idx[:, 1], iou)
    return ids, keep.sort().values, boxes[idx[:, 0]], idx[:, 1]


def make(seed, n=400, c=3):
    g = torch.Generator().manual_seed(seed)
    s64 = torch.rand(n, c, generator=g, dtype=torch.float64) * 0.6 + 0.3
    xy = torch.rand(n, 2, generator=g) * 60
    wh = torch.rand(n, 2, generator=g) * 30 + 4
    return s64, torch.cat([xy, xy + wh], dim=1)


def test_one_ulp_changes_are_explained():
    explained = 0
    for seed in range(40):
        s64, boxes = make(seed)
        # quantise so that many scores are one ulp apart: ulp-level noise then reorders them
        base = (s64 * 4096).round() / 4096
        g = torch.Generator().manual_seed(1000 + seed)
        a = base.float()
        b = torch.nextafter(a, torch.where(torch.rand(a.shape, generator=g) < 0.5, torch.zeros_like(a), torch.ones_like(a)))
        ra = stages(a, boxes, None, 0.5, 100, 0.45)
        rb = stages(b, boxes, None, 0.5, 100, 0.45)
        why = tieband.explain_or_fail(ra[0], rb[0], base.reshape(-1), 0.5, 100, ra[1], rb[1], ra[2], rb[2], ra[3], 0.45)
        explained += why != "identical"
    assert explained > 0, "the construction must produce runs that differ"


def test_large_score_changes_are_rejected():
    s64, boxes = make(7)
    a = s64.float()
    b = a.clone()
    b[5, 1] = a[5, 1] + 0.05 if a[5, 1] < 0.8 else a[5, 1] - 0.05   # a real error, far outside the band
    ra = stages(a, boxes, None, 0.2, 2000, 0.45)
    rb = stages(b, boxes, None, 0.2, 2000, 0.45)
    assert not torch.equal(ra[0], rb[0])
    with pytest.raises(AssertionError):
        tieband.explain_or_fail(ra[0], rb[0], s64.reshape(-1), 0.2, 2000, ra[1], rb[1], ra[2], rb[2], ra[3], 0.45)


def test_wrong_nms_decision_is_rejected():
    s64, boxes = make(11)
    a = s64.float()
    ra = stages(a, boxes, None, 0.5, 200, 0.45)
    kept = ra[1]
    wrong = kept[kept != kept[3]]          # drop one survivor although nothing suppresses it
    with pytest.raises(AssertionError):
        tieband.explain_or_fail(ra[0], ra[0], s64.reshape(-1), 0.5, 200, wrong, kept, ra[2], ra[2], ra[3], 0.45)


def test_near_threshold_iou_is_explained():
    # two boxes whose IoU sits at the threshold: moving one coordinate by an ulp flips the decision
    a = torch.tensor([[0.0, 0.0, 10.0, 10.0], [0.0, 0.0, 10.0, 4.5], [50.0, 50.0, 60.0, 60.0]])
    b = a.clone()
    b[1, 3] = torch.nextafter(a[1, 3], torch.tensor(10.0))
    labels = None
    keep_a = torch.tensor([0, 1, 2])    # IoU 0.45 is not > 0.45: kept
    keep_b = torch.tensor([0, 2])       # a hair larger: suppressed
    x, margin = tieband.audit_nms(keep_a, keep_b, a, b, labels, 0.45)
    assert x == 1 and margin < 1e-5
