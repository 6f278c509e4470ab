"""GPU parity for C3 (SSD-style softmax + decode, per-class mask / top-k / NMS) against the TorchScript CPU oracle.
Floats within 1e-5 relative; the per-class integer stages bit-exact on the GPU's own floats; end to end against the
oracle's own floats every (image, class) list is identical, or the first decision on which the two runs part is shown
in fp64 to lie inside the last-ulp band (tests/tieband.py); anything else fails."""
import pytest
import torch

from oracle import workloads as W
from tests import tieband
from tests.util import close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fb(cuda_device):
    import functs_b200
    return functs_b200


def run_case(fb, loc, conf, priors, thr=0.01, topk=200, iou=0.45):
    o = W.SSDPost(score_thr=thr, topk=topk, iou_thr=iou)
    o.priors = priors
    obox, oscores, ores = torch.jit.script(o)(loc, conf) if priors.size(0) == 8732 else o(loc, conf)
    mod = fb.workloads.SSDBBox(priors, score_thr=thr, topk=topk, iou_thr=iou)
    boxes, dets, ids, counts = mod.forward_padded(loc, conf)
    assert mod.kernels_last_call == 2
    scores_cm = mod._bufs[2]
    boxes_c, scores_c = boxes.cpu(), scores_cm.cpu().permute(0, 2, 1).contiguous()  # [B,P,C]
    # values
    close(scores_c, oscores, rtol=1e-5, atol=1e-9, what="softmax scores")
    pm = priors[:, 0:2].abs() + priors[:, 2:4].abs() * 4
    close(boxes_c, obox, rtol=1e-5, scale=torch.cat([pm, pm], dim=1)[None].expand_as(obox), what="decoded boxes")
    # integer stages on the GPU's floats: exact
    per_image = mod.unpad(dets, ids, counts)
    exact = total = 0
    b, p, c = scores_c.shape
    for i in range(b):
        gd, gl, gi = [t.cpu() for t in per_image[i]]
        wd, wl, wi = o.post_single(boxes_c[i], scores_c[i])
        assert gi.numel() == wi.numel(), f"image {i}: kept {gi.numel()} vs {wi.numel()}"
        assert torch.equal(gi, wi) and torch.equal(gl, wl) and torch.equal(gd, wd)
        # against the oracle's own floats, class by class
        od, ol, oi = ores[i]
        score64 = None
        for k in range(c):
            total += 1
            a, bb = gi[gl == k], oi[ol == k]
            if a.numel() == bb.numel() and torch.equal(a, bb):
                exact += 1
                continue
            if score64 is None:
                score64 = conf[i].double().softmax(-1)
            ga, gk, gb = class_stages(boxes_c[i], scores_c[i][:, k], thr, topk, iou)
            ca, ck, cb = class_stages(obox[i], oscores[i][:, k], thr, topk, iou)
            why = tieband.explain_or_fail(ga, ca, score64[:, k], thr, topk, gk, ck, gb, cb, None, iou)
            assert why != "identical"
            print(f"[tie-band] image {i} class {k}: {why}")
    print(f"(image, class) lists identical to the oracle's own run: {exact}/{total}; the others were explained by the "
          f"fp64 audit")
    return exact, total


def class_stages(bboxes, scores_c, thr, topk, iou):
    """The oracle's per-class stages (SSDPost.class_single) with the intermediate lists kept: selected prior ids in
    sorted order, kept positions, selected boxes."""
    import torchvision
    mask = scores_c > thr
    idx = torch.nonzero(mask)[:, 0]
    s, order = scores_c[mask].sort(descending=True, stable=True)
    k = min(topk, idx.numel())
    s, idx = s[:k], idx[order[:k]]
    bx = bboxes[idx]
    keep = torchvision.ops.nms(bx, s, iou)
    return idx, keep.sort().values, bx


def test_ssd_config_shapes(fb):
    loc, conf = W.make_ssd_inputs(2)
    run_case(fb, loc, conf, W.ssd_priors())


def test_ssd_full_batch_against_oracle(fb):
    """B = 64 (5120 (image, class) lists) against the oracle's own run."""
    loc, conf = W.make_ssd_inputs(64)
    exact, total = run_case(fb, loc, conf, W.ssd_priors())
    assert total == 64 * 80


def test_ssd_ragged_small(fb):
    """Prior count that is not a multiple of the tile (and of 4): plain-load path, tail tile, short lists."""
    g = torch.Generator().manual_seed(9)
    p, c = 333, 5
    pri = torch.cat([torch.rand(p, 2, generator=g) * 300, torch.rand(p, 2, generator=g) * 80 + 4], dim=1)
    loc = torch.randn(2, p, 4, generator=g)
    conf = torch.randn(2, p, c + 1, generator=g) * 2
    run_case(fb, loc, conf, pri, thr=0.05, topk=50)


def test_ssd_golden_decode(fb):
    """Decode against the fixture written by the reference's delta2bbox (clamp 320)."""
    import os
    f = torch.load(os.path.join(os.path.dirname(__file__), "golden", "delta2bbox.pt"))
    p = f["priors"].size(0)
    conf = torch.zeros(1, p, 3)
    boxes, _ = fb.ops.ssd_softmax_decode(f["deltas"][None].cuda(), conf.cuda(), f["priors"].cuda(), clamp_max=320.0)
    close(boxes[0].cpu(), f["out"], rtol=1e-5, scale=400.0, what="delta2bbox fixture")


def test_ssd_no_candidates_and_all_candidates(fb):
    pri = W.ssd_priors()[:256].contiguous()
    loc = torch.zeros(1, 256, 4)
    conf = torch.zeros(1, 256, 4)
    conf[..., -1] = 20.0  # everything is background: no class passes 0.01
    mod = fb.workloads.SSDBBox(pri)
    _, dets, ids, counts = mod.forward_padded(loc, conf)
    assert int(counts.sum()) == 0 and bool((ids == -1).all())
    conf = torch.zeros(1, 256, 4)  # uniform: every prior is a candidate of every class, all scores tie
    _, dets, ids, counts = mod.forward_padded(loc, conf)
    o = W.SSDPost()
    o.priors = pri
    _, _, res = o(loc, conf)
    got = mod.unpad(dets, ids, counts)[0]
    assert torch.equal(got[2].cpu(), res[0][2])


def _class_nms_case(fb, boxes, scores, thr=0.01, topk=200, iou=0.45):
    """boxes [P,4], scores [P,C] (CPU): the GPU per-class kernel against the oracle's per-class loop, bit for bit."""
    o = W.SSDPost(score_thr=thr, topk=topk, iou_thr=iou)
    wd, wl, wi = o.post_single(boxes, scores)
    dev = torch.device("cuda:0")
    scores_cm = scores.t().contiguous()[None].to(dev)
    dets, ids, counts = fb.ops.ssd_class_nms(boxes[None].contiguous().to(dev), scores_cm, thr, topk, iou)
    torch.cuda.synchronize()
    gd, gl, gi = [], [], []
    for c in range(scores.size(1)):
        k = int(counts[0, c])
        gd.append(dets[0, c, :k].cpu())
        gi.append(ids[0, c, :k].cpu())
        gl.append(torch.full([k], c, dtype=torch.long))
    gd, gl, gi = torch.cat(gd), torch.cat(gl), torch.cat(gi)
    assert torch.equal(gi, wi) and torch.equal(gl, wl) and torch.equal(gd, wd)
    return counts[0].cpu()


def test_ssd_class_nms_suppression_chain(fb):
    """Box k overlaps box k + 1 above the threshold and box k + 2 below it: the greedy result alternates and every
    decision depends on the one before (the deepest dependency chain the parallel resolve can meet)."""
    n = 200
    x0 = torch.arange(n, dtype=torch.float32) * 3.0      # width 10, shift 3: IoU 7/13 = 0.54, shift 6: 4/16 = 0.25
    boxes = torch.stack([x0, torch.zeros(n), x0 + 10.0, torch.full([n], 10.0)], dim=1)
    scores = torch.zeros(n, 2)
    scores[:, 0] = torch.linspace(0.9, 0.1, n)           # class 0: score order = chain order
    scores[:, 1] = torch.linspace(0.1, 0.9, n)           # class 1: the chain runs the other way
    counts = _class_nms_case(fb, boxes, scores)
    assert counts.tolist() == [100, 100]


def test_ssd_class_nms_ties_and_duplicates(fb):
    """Equal scores fill one histogram bucket (order falls back to the prior index), identical boxes are all
    suppressed by the first, and more candidates than top-k tie at the boundary."""
    g = torch.Generator().manual_seed(21)
    p = 600
    xy = torch.rand(p, 2, generator=g) * 250.0
    wh = torch.rand(p, 2, generator=g) * 40.0 + 5.0
    boxes = torch.cat([xy, xy + wh], dim=1)
    boxes[100:140] = boxes[100]                            # forty copies of one box
    scores = torch.zeros(p, 3)
    scores[:, 0] = 0.5                                     # all tie: top-k takes priors 0..199
    scores[:, 1] = (torch.randint(0, 4, (p,), generator=g).float() + 1.0) * 0.125   # four score levels
    scores[:, 2] = torch.rand(p, generator=g)
    scores[100:140, 2] = 0.99
    _class_nms_case(fb, boxes, scores)


def test_ssd_class_nms_wild_boxes(fb):
    """Coordinates far outside the tame range take the guarded IoU path; degenerate boxes never suppress."""
    g = torch.Generator().manual_seed(5)
    p = 300
    xy = torch.rand(p, 2, generator=g) * 100.0
    wh = torch.rand(p, 2, generator=g) * 30.0 + 1.0
    boxes = torch.cat([xy, xy + wh], dim=1)
    boxes[7] = torch.tensor([0.0, 0.0, 3.0e19, 3.0e19])    # area overflows to inf
    boxes[9] = torch.tensor([50.0, 50.0, 40.0, 40.0])      # negative extent
    scores = torch.rand(p, 2, generator=g)
    _class_nms_case(fb, boxes, scores)
