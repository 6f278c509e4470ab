"""Pins the oracle against outputs of the reference's own functions (fixtures in tests/golden/, written by
tests/golden/make_golden.py from the reference sources).  CPU only; bit-exact unless stated."""
import os

import torch

from oracle import workloads as W

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return torch.load(os.path.join(G, name + ".pt"))


def test_get_started_matches_reference():
    f = load("get_started")
    assert torch.equal(W.get_started(f["a"], f["b"], f["n"]), f["out"])
    assert torch.equal(torch.jit.script(W.get_started)(f["a"], f["b"], f["n"]), f["out"])


def test_batched_nms_matches_reference():
    f = load("batched_nms")
    dets, keep = W.batched_nms(f["boxes"], f["scores"], f["labels"], f["iou_thr"])
    assert torch.equal(keep, f["keep"])
    assert torch.equal(dets, f["dets"])


def test_select_topk_matches_reference():
    f = load("filter_topk")
    s, idx = W.select_topk(f["scores"], f["thr"], f["topk"])
    assert torch.equal(s, f["out_scores"])
    assert torch.equal(idx[:, 0], f["out_rows"])
    assert torch.equal(idx[:, 1], f["out_labels"])


def test_ssd_decode_matches_reference():
    f = load("delta2bbox")
    out = W.ssd_delta2bbox(f["priors"], f["deltas"], f["clamp_max"])
    assert torch.equal(out, f["out"])


def test_lstm_cell_matches_reference():
    f = load("lstm_cell")
    h1, c1 = W.lstm_cell(f["x"], f["h0"], f["c0"], f["w_ih"], f["w_hh"], f["b_ih"], f["b_hh"])
    assert torch.equal(h1, f["h1"])
    assert torch.equal(c1, f["c1"])


def test_crop_matches_reference():
    f = load("yolact_crop")
    got = W.crop_by_slice_assign(f["masks"], f["boxes"])  # [N,H,W]
    assert torch.equal(got.permute(1, 2, 0), f["out"])


def test_scripted_workloads_run_and_edge_cases():
    # all-negative logits: no candidate survives the mask
    m = torch.jit.script(W.YOLOV3Post(sizes=(2, 4, 8)))
    maps = [torch.full((1, 255, s, s), -3.0) for s in (2, 4, 8)]
    _, _, _, res = m(maps)
    assert res[0][0].shape == (0, 5) and res[0][1].numel() == 0
    # priors table has the SSD300 size and a sane layout
    p = W.ssd_priors()
    assert p.shape == (8732, 4) and float(p.min()) > 0
    # synthetic inputs are reproducible and differ per image
    a = W.make_yolo_inputs(2, sizes=(2, 4, 8))
    b = W.make_yolo_inputs(2, sizes=(2, 4, 8))
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert not torch.equal(a[0][0], a[0][1])
    c = W.make_yolo_inputs(1, sizes=(2, 4, 8), first=1)
    assert torch.equal(c[0][0], a[0][1])


def test_yolo_decode_matches_reference():
    """decode_bboxes on the reference's anchor grid gives the same boxes through another operation order (anchor centre
    + (sigmoid - 0.5) * stride instead of (sigmoid + cell) * stride): 1e-5 relative to the box's own magnitude (centre
    plus extent; a corner is a difference of the two).  Objectness and class scores are the same sigmoid, evaluated in place
    on a strided slice here and out of place there (ATen picks different vector kernels): 1e-6 relative."""
    f = load("yolo_decode")
    o = W.YOLOV3Post(sizes=tuple(f["sizes"]))
    bboxes, obj, cls = o.decode(f["maps"])
    want = f["bboxes"]
    centre = (want[..., 0:2] + want[..., 2:4]).abs() * 0.5
    extent = (want[..., 2:4] - want[..., 0:2]).abs()
    scale = torch.cat([centre + extent, centre + extent], dim=-1)
    err = (bboxes.double() - want.double()).abs()
    assert bool((err <= 1e-5 * scale.double()).all()), float((err / scale.double()).max())
    assert torch.allclose(obj, f["objectness"], rtol=1e-6, atol=0.0)
    assert torch.allclose(cls, f["cls_scores"], rtol=1e-6, atol=0.0)
    sb, sobj, scls = torch.jit.script(o).decode(f["maps"])
    assert torch.equal(sb, bboxes) and torch.equal(sobj, obj) and torch.equal(scls, cls)
