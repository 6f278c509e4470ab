"""GPU parity for C3 (SSD-style softmax + decode, per-class mask / top-k / NMS) against the TorchScript CPU oracle.
Floats within 1e-5 relative; the per-class integer stages bit-exact on the GPU's own floats; end-to-end identity
against the oracle's floats reported per (image, class) with near-tie cases counted (see test_gpu_yolo.py)."""
import pytest
import torch

from oracle import workloads as W
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
        for k in range(c):
            total += 1
            a, bb = gi[gl == k], oi[ol == k]
            if a.numel() == bb.numel() and torch.equal(a, bb):
                exact += 1
    print(f"(image, class) pairs identical to the oracle end to end: {exact}/{total}")
    assert exact >= 0.9 * total
    return exact, total


def test_ssd_config_shapes(fb):
    loc, conf = W.make_ssd_inputs(2)
    run_case(fb, loc, conf, W.ssd_priors())


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
