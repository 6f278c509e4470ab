"""GPU parity: C1, masked index, top-k and NMS kernels against the CPU oracle — integer results bit-exact."""
import pytest
import torch

from oracle import workloads as W
from tests.util import key_index, key_scores, make_keys

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fb(cuda_device):
    import functs_b200
    return functs_b200


def gen(seed):
    return torch.Generator().manual_seed(seed)


# ---- C1 ---------------------------------------------------------------------------------------------------


@pytest.mark.parametrize("rows,cols,n", [(64, 1024, 64), (64, 1024, 3), (8, 16, 0), (5, 7, 5), (3, 1023, 2)])
def test_get_started_bit_exact(fb, cuda_device, rows, cols, n):
    g = gen(rows * cols + n)
    a, b = torch.randn(rows, cols, generator=g), torch.randn(rows, cols, generator=g)
    want = torch.jit.script(W.get_started)(a, b, n)
    got = fb.workloads.get_started(a, b, n)
    assert torch.equal(got.cpu(), want)


def test_get_started_config_inputs(fb, cuda_device):
    a, b, n = W.make_get_started_inputs()
    assert torch.equal(fb.workloads.get_started(a, b, n).cpu(), W.get_started(a, b, n))
    with pytest.raises(IndexError):
        fb.workloads.get_started(a, b, 65)


# ---- threshold + compaction -----------------------------------------------------------------------------


@pytest.mark.parametrize("groups,n,thr", [(1, 1, 0.5), (3, 5000, 0.5), (2, 851760, 0.9), (4, 2048, 0.0001), (2, 777, 0.999999)])
def test_threshold_compact_matches_nonzero(fb, cuda_device, groups, n, thr):
    s = torch.rand(groups, n, generator=gen(n)) * 0.999 + 0.0005
    keys, counts = fb.ops.threshold_compact(s.cuda(), thr)
    keys, counts = keys.cpu(), counts.cpu()
    for g in range(groups):
        idx = torch.nonzero(s[g] > thr)[:, 0]
        assert int(counts[g]) == idx.numel()
        got = keys[g, :idx.numel()].sort(descending=True).values
        want = make_keys(s[g][idx], idx).sort(descending=True).values
        assert torch.equal(got, want)


def test_threshold_compact_overflow_is_reported(fb, cuda_device):
    s = torch.rand(1, 4096, generator=gen(5)) * 0.5 + 0.5
    status = fb.ops.new_status(cuda_device)
    keys, counts = fb.ops.threshold_compact(s.cuda(), 0.1, capacity=100, status=status)
    assert int(counts[0]) == 4096
    assert int(status.item()) & 1
    with pytest.raises(fb.FunctsB200Error):
        fb.ops.raise_on_status(status, "compact")


# ---- top-k -----------------------------------------------------------------------------------------------


def oracle_topk(scores_flat, thr, k):
    s, idx = W.select_topk(scores_flat.reshape(-1, 1), thr, k)
    return make_keys(s, idx[:, 0])


@pytest.mark.parametrize("n,k,quant", [
    (1, 1000, 0), (0, 1000, 0), (999, 1000, 0), (1000, 1000, 0), (1001, 1000, 0), (70000, 1000, 0),
    (70000, 1000, 256),      # heavy exact ties: 256 distinct scores
    (5000, 200, 16), (5000, 1, 0), (300000, 1024, 4), (4096, 1000, 1),  # quant=1: every score identical
])
def test_select_topk_matches_stable_sort(fb, cuda_device, n, k, quant):
    g = gen(n + k + quant)
    groups = 3
    u = torch.rand(groups, max(n, 1), generator=g)
    if quant:
        u = (u * quant).floor() / quant
    s = u * 0.4 + 0.55
    thr = 0.5
    if n == 0:
        s = torch.zeros(groups, 1)
    keys, counts, hist = fb.ops.threshold_compact(s.cuda(), thr, with_hist=True)
    assert torch.equal(hist.sum(dim=1), counts)
    for name, (sel, m) in {"generic": fb.ops.select_topk(keys, counts, k),
                           "binned": fb.ops.select_topk_binned(keys, counts, hist, thr, k)}.items():
        sel, m = sel.cpu(), m.cpu()
        for gi in range(groups):
            want = oracle_topk(s[gi], thr, k)
            assert int(m[gi]) == want.numel(), name
            assert torch.equal(sel[gi, :want.numel()], want), f"{name}: group {gi}"
            assert bool((sel[gi, want.numel():] == 0).all()), name


def test_select_topk_varied_exponents(fb, cuda_device):
    # scores across many binades (as softmax outputs are), shuffled candidate order
    g = gen(77)
    s = torch.exp(torch.randn(2, 8732, generator=g) * 2 - 4).clamp(max=0.99)
    keys, counts, hist = fb.ops.threshold_compact(s.cuda(), 0.01, with_hist=True)
    sel, m = fb.ops.select_topk(keys, counts, 200)
    sel_b, m_b = fb.ops.select_topk_binned(keys, counts, hist, 0.01, 200)
    for gi in range(2):
        want = oracle_topk(s[gi], 0.01, 200)
        assert torch.equal(sel[gi].cpu()[:want.numel()], want)
        assert torch.equal(sel_b[gi].cpu()[:want.numel()], want)


def test_select_binned_with_wrong_histogram_falls_back(fb, cuda_device):
    """A histogram that does not describe the list (all zero) must not change the answer: the generic path runs."""
    g = gen(123)
    s = torch.rand(2, 20000, generator=g) * 0.45 + 0.52
    keys, counts, hist = fb.ops.threshold_compact(s.cuda(), 0.5, with_hist=True)
    sel, m, fell = fb.ops.select_topk_binned(keys, counts, torch.zeros_like(hist), 0.5, 1000, return_fallbacks=True)
    assert fell.tolist() == [1, 1]
    _, _, fell = fb.ops.select_topk_binned(keys, counts, hist, 0.5, 1000, return_fallbacks=True)
    assert fell.tolist() == [0, 0], "well-spread scores must be finished by the binned path"
    for gi in range(2):
        want = oracle_topk(s[gi], 0.5, 1000)
        assert torch.equal(sel[gi].cpu(), want)


# ---- NMS -------------------------------------------------------------------------------------------------


def random_boxes(n, g, spread=100.0, size=40.0):
    ctr = torch.rand(n, 2, generator=g) * spread
    wh = torch.rand(n, 2, generator=g) * size + 1
    return torch.cat([ctr - wh / 2, ctr + wh / 2], dim=1)


@pytest.mark.parametrize("n,classes,offset,spread", [
    (1000, 80, True, 100.0), (1000, 1, False, 60.0), (333, 4, True, 50.0), (1, 3, True, 10.0), (64, 2, True, 5.0),
    (1024, 3, True, 30.0), (31, 1, False, 20.0), (33, 1, False, 20.0),
])
def test_batched_nms_bit_exact(fb, cuda_device, n, classes, offset, spread):
    g = gen(n * 7 + classes)
    groups = 2
    num_boxes = 2000
    for iou in (0.45, 0.3):
        boxes = torch.stack([random_boxes(num_boxes, g, spread) for _ in range(groups)])
        sel_keys = torch.zeros(groups, n, dtype=torch.int64)
        want = []
        for gi in range(groups):
            scores = torch.rand(n, generator=g) * 0.5 + 0.5
            scores = (scores * 512).floor() / 512 + 0.0001  # ties on purpose
            flat = torch.randperm(num_boxes * classes, generator=g)[:n]
            keys = make_keys(scores, flat).sort(descending=True).values
            sel_keys[gi] = keys
            s, fl = key_scores(keys), key_index(keys)
            bi, lab = fl // classes, fl % classes
            if offset:
                dets, keep = W.batched_nms(boxes[gi][bi], s, lab, iou)
            else:
                import torchvision
                keep = torchvision.ops.nms(boxes[gi][bi], s, iou)
                dets = torch.cat([boxes[gi][bi][keep], s[keep, None]], dim=1)
            want.append((dets, lab[keep], fl[keep], keep))
        counts = torch.full((groups,), n, dtype=torch.int32)
        dets, labels, flat_ids, keep, out_counts = fb.ops.batched_nms(boxes.cuda(), classes, sel_keys.cuda(), counts.cuda(),
                                                                      iou, offset)
        for gi in range(groups):
            m = int(out_counts[gi])
            wd, wl, wf, wk = want[gi]
            assert m == wk.numel(), f"group {gi}: kept {m}, oracle {wk.numel()}"
            assert torch.equal(keep[gi, :m].cpu(), wk)
            assert torch.equal(flat_ids[gi, :m].cpu(), wf)
            assert torch.equal(labels[gi, :m].cpu(), wl)
            assert torch.equal(dets[gi, :m].cpu(), wd)
            assert bool((labels[gi, m:] == -1).all())


def test_batched_nms_out_of_range_key_is_skipped_and_reported(fb, cuda_device):
    """Keys come from the caller.  One whose box index lies beyond num_boxes (and an all-zero key, whose flat index is
    0xFFFFFFFF) must not be dereferenced: the status word reports it and the other candidates give the oracle's answer."""
    g = gen(4242)
    num_boxes, classes, n = 500, 3, 200
    boxes = random_boxes(num_boxes, g, 40.0)
    scores = torch.rand(n, generator=g) * 0.5 + 0.5
    flat = torch.randperm(num_boxes * classes, generator=g)[:n]
    flat[17] = num_boxes * classes + 5          # box index == num_boxes + 1
    flat[120] = (1 << 31) + 12345               # far outside
    keys = make_keys(scores, flat).sort(descending=True).values
    keys[n - 1] = 0                              # stale row: flat index 0xFFFFFFFF
    fl = key_index(keys)
    valid = (fl // classes) < num_boxes
    assert int((~valid).sum()) == 3
    s, bi, lab = key_scores(keys)[valid], (fl // classes)[valid], (fl % classes)[valid]
    wd, wkeep = W.batched_nms(boxes[bi], s, lab, 0.45)
    pos = torch.nonzero(valid)[:, 0][wkeep]      # positions in the full selected list
    status = fb.ops.new_status(cuda_device)
    dets, labels, flat_ids, keep, cnt = fb.ops.batched_nms(boxes[None].cuda(), classes, keys[None].cuda(),
                                                           torch.tensor([n], dtype=torch.int32).cuda(), 0.45, True,
                                                           status=status)
    assert int(status.item()) == 4               # FB_STATUS_INDEX_RANGE
    m = int(cnt[0])
    assert m == pos.numel()
    assert torch.equal(keep[0, :m].cpu(), pos)
    assert torch.equal(flat_ids[0, :m].cpu(), fl[valid][wkeep])
    assert torch.equal(dets[0, :m].cpu(), wd)
    # a clean call leaves the status word alone
    status.zero_()
    fb.ops.batched_nms(boxes[None].cuda(), classes, keys[valid][None, :50].contiguous().cuda(),
                       torch.tensor([50], dtype=torch.int32).cuda(), 0.45, True, status=status)
    assert int(status.item()) == 0


def test_batched_nms_golden_fixture(fb, cuda_device):
    """The fixture produced by the reference's own batched_nms (tests/golden/batched_nms.pt)."""
    import os
    f = torch.load(os.path.join(os.path.dirname(__file__), "golden", "batched_nms.pt"))
    n = f["scores"].numel()
    classes = 4
    # candidate i is box i with its label: flat = i * classes + label
    flat = torch.arange(n) * classes + f["labels"]
    keys = make_keys(f["scores"], flat)
    assert torch.equal(keys.sort(descending=True, stable=True).values, keys)  # fixture scores are sorted
    dets, labels, flat_ids, keep, cnt = fb.ops.batched_nms(f["boxes"][None].cuda(), classes, keys[None].cuda(),
                                                           torch.tensor([n], dtype=torch.int32).cuda(), f["iou_thr"], True)
    m = int(cnt[0])
    assert m == f["keep"].numel()
    assert torch.equal(keep[0, :m].cpu(), f["keep"])
    assert torch.equal(dets[0, :m].cpu(), f["dets"])


def test_argument_errors(fb, cuda_device):
    with pytest.raises(fb.FunctsB200Error):
        fb.ops.select_topk(torch.zeros(1, 8, dtype=torch.int64, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda"), 2000)
    with pytest.raises(ValueError):
        fb.ops.threshold_compact(torch.zeros(1, 8), 0.5)  # CPU tensor: no CPU path


def test_pack_detections_matches_host_packing(fb, cuda_device):
    """The pack kernel (records for the multi-GPU gather) against the tensor-op packing that the gloo tests use."""
    from functs_b200 import dist as fdist
    g = torch.Generator().manual_seed(5)
    b, k = 3, 37
    dets = torch.randn(b, k, 5, generator=g)
    labels = torch.randint(0, 80, (b, k), generator=g)
    ids = torch.randint(0, 10647 * 80, (b, k), generator=g)
    counts = torch.tensor([0, 17, 37], dtype=torch.int32)
    want = fdist.pack_detections(dets, labels, ids, counts)
    got = fdist.pack_detections(dets.cuda(), labels.cuda(), ids.cuda(), counts.cuda())
    torch.cuda.synchronize()
    assert torch.equal(got.cpu(), want)
    d2, l2, i2, c2 = fdist.unpack_detections(got.cpu())
    assert torch.equal(d2, dets) and torch.equal(l2, labels) and torch.equal(i2, ids) and torch.equal(c2, counts)


def test_postprocess_writes_gather_records(fb, cuda_device):
    """The one-call post-process can write the 32-byte gather records itself (no pack launch): they must equal what the
    pack kernel makes of the padded outputs."""
    from functs_b200 import dist as fdist
    maps = [m.cuda() for m in W.make_yolo_inputs(3)]
    plan = fb.ops.YoloPostprocessPlan(3)
    rec = torch.full((3, 1000, fdist.RECORD_WORDS), 7, dtype=torch.int32, device="cuda")
    before = fb.launch_count()
    plan.run(maps, 0.5, 0.45, records=rec)
    assert fb.launch_count() - before == 3
    want = fdist.pack_detections(plan.dets, plan.labels, plan.flat_ids, plan.counts)
    torch.cuda.synchronize()
    assert torch.equal(rec, want)
