"""The scratch-free NMS entry point (functs_b200_batched_nms_static), called through the C ABI.

It serves hosts that bind only the C ABI and have no device allocator to take scratch from (all device memory is in
another framework's pool, or an allocation call would stall their loop); the suppression matrix lives in a fixed
1258 KB (about 1.3 MB) array inside the library instead.  The test feeds the same selected candidates to the regular entry point (with
caller-provided scratch) and to the static one, twice in a row with different data — the second call runs on the
array the first one left behind — and requires identical outputs (integer work: exact equality); the static entry
point's survivors are also compared directly with the CPU oracle's class-offset NMS.  This file sorts last on purpose, so that a run that stops at the first failure has already run everything else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def make_case(seed, groups, n, classes, num_boxes=1500):
    from tests.util import make_keys
    g = torch.Generator().manual_seed(seed)
    ctr = torch.rand(groups, num_boxes, 2, generator=g) * 60
    wh = torch.rand(groups, num_boxes, 2, generator=g) * 30 + 1
    boxes = torch.cat([ctr - wh / 2, ctr + wh / 2], dim=2)
    keys = torch.zeros(groups, n, dtype=torch.int64)
    for gi in range(groups):
        scores = (torch.rand(n, generator=g) * 0.5 + 0.5)
        flat = torch.randperm(num_boxes * classes, generator=g)[:n]
        keys[gi] = make_keys(scores, flat).sort(descending=True).values
    counts = torch.full((groups,), n, dtype=torch.int32)
    return boxes.cuda(), keys.cuda(), counts.cuda()


def oracle_nms(boxes, classes, keys, iou, offset):
    """CPU oracle on the same candidates: (dets, labels, flat ids, kept positions) of one group."""
    import torchvision
    from oracle import workloads as W
    from tests.util import key_index, key_scores
    s, fl = key_scores(keys), key_index(keys)
    bi, lab = fl // classes, fl % classes
    if offset:
        dets, keep = W.batched_nms(boxes[bi], s, lab, iou)
    else:
        keep = torchvision.ops.nms(boxes[bi], s, iou)
        dets = torch.cat([boxes[bi][keep], s[keep, None]], dim=1)
    return dets, lab[keep], fl[keep], keep


def call_static(lib, check, boxes, classes, keys, counts, iou, offset):
    g, k = keys.shape
    dev = boxes.device
    dets = torch.empty(g, k, 5, dtype=torch.float32, device=dev)
    labels = torch.empty(g, k, dtype=torch.int64, device=dev)
    flat_ids = torch.empty(g, k, dtype=torch.int64, device=dev)
    keep = torch.empty(g, k, dtype=torch.int64, device=dev)
    out_counts = torch.empty(g, dtype=torch.int32, device=dev)
    rc = lib.functs_b200_batched_nms_static(boxes.data_ptr(), boxes.size(1), classes, keys.data_ptr(), counts.data_ptr(), g, k,
                                            iou, 1 if offset else 0, dets.data_ptr(), labels.data_ptr(), flat_ids.data_ptr(),
                                            keep.data_ptr(), out_counts.data_ptr(), None,
                                            torch.cuda.current_stream().cuda_stream)
    check(rc, "batched_nms_static")
    return dets, labels, flat_ids, keep, out_counts


def test_static_nms_matches_regular_entry_point_twice(cuda_device):
    import functs_b200 as fb
    from functs_b200._lib import check, lib
    assert lib.functs_b200_batched_nms_static_max_groups() == 8
    # first call: large lists; second call: fewer, shorter lists on top of the first call's leftovers
    for seed, groups, n, classes, offset in ((1, 8, 1000, 6, True), (2, 3, 77, 1, False)):
        boxes, keys, counts = make_case(seed, groups, n, classes)
        want = fb.ops.batched_nms(boxes, classes, keys, counts, 0.45, offset)
        got = call_static(lib, check, boxes, classes, keys, counts, 0.45, offset)
        torch.cuda.synchronize()
        for w, g_ in zip(want, got):
            assert torch.equal(w, g_)
        assert int(got[4].min()) > 0
        dets, labels, flat_ids, keep, out_counts = [t.cpu() for t in got]
        for gi in range(groups):
            wd, wl, wf, wk = oracle_nms(boxes[gi].cpu(), classes, keys[gi].cpu(), 0.45, offset)
            m = int(out_counts[gi])
            assert m == wk.numel()
            assert torch.equal(keep[gi, :m], wk) and torch.equal(flat_ids[gi, :m], wf)
            assert torch.equal(labels[gi, :m], wl) and torch.equal(dets[gi, :m], wd)


def test_static_nms_rejects_too_many_groups(cuda_device):
    import functs_b200 as fb
    from functs_b200._lib import check, lib
    boxes, keys, counts = make_case(3, 9, 16, 2)
    with pytest.raises(fb.FunctsB200Error, match="at most 8"):
        call_static(lib, check, boxes, 2, keys, counts, 0.45, True)
