"""The graph path on the GPU: functs_b200.jit.build(<oracle program>) -> tssa::ParallelFunctor bound to the precompiled
kernels -> outputs compared with the oracle program's own CPU run.

Per config: the launch count of one call (3 / 2 / 3 / 1 kernels of libfuncts_b200.so), no functor execution through the
subgraph interpreter, values within 1e-5 relative and integer results identical on seeds where the kernel-level tests
show that no decision falls into the last-ulp band."""
import pytest
import torch

from oracle import workloads as W
from tests.util import close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(cuda_device):
    import functs_b200
    from functs_b200 import jit
    return functs_b200, jit


def run_counted(fb, J, fn, *args):
    before_l, before_i = fb.launch_count(), J.interpreted_functor_runs()
    out = fn(*args)
    torch.cuda.synchronize()
    assert J.interpreted_functor_runs() == before_i, "a functor ran through the subgraph interpreter"
    return out, fb.launch_count() - before_l


def test_yolov3_program_through_the_graph(env):
    fb, J = env
    maps = W.make_yolo_inputs(3)
    oracle = W.YOLOV3Post()
    obb, oobj, ocls, ores = torch.jit.script(oracle)(maps)
    fn = J.build(W.YOLOV3Post())
    assert J.functor_regions(fn.graph) == ["yolov3_post_dense"]
    (bb, obj, cls, res), launches = run_counted(fb, J, fn, [m.cuda() for m in maps])
    assert launches == 3
    close(obj.cpu(), oobj, rtol=1e-5, what="objectness")
    close(cls.cpu(), ocls, rtol=1e-5, what="class scores")
    scale = (obb[..., 0:2] + obb[..., 2:4]).abs() * 0.5 + (obb[..., 2:4] - obb[..., 0:2]).abs()
    close(bb.cpu(), obb, rtol=1e-5, scale=torch.cat([scale, scale], dim=-1), what="boxes")
    assert len(res) == len(ores) == 3
    for (d, l, f), (od, ol, of) in zip(res, ores):
        assert torch.equal(f.cpu(), of) and torch.equal(l.cpu(), ol)
        close(d.cpu()[:, 4], od[:, 4], rtol=1e-5, what="scores")
    # the results-only program takes the staged decode kernel (no dense outputs): same detections
    from functs_b200 import patterns
    fast = J.build(patterns.YOLOV3Det())
    assert J.functor_regions(fast.graph) == ["yolov3_post"]
    res2, launches = run_counted(fb, J, fast, [m.cuda() for m in maps])
    assert launches == 3
    for (d, l, f), (d2, l2, f2) in zip(res, res2):
        assert torch.equal(d, d2) and torch.equal(l, l2) and torch.equal(f, f2)


def test_ssd_program_through_the_graph(env):
    fb, J = env
    loc, conf = W.make_ssd_inputs(2)
    obox, oscores, ores = torch.jit.script(W.SSDPost())(loc, conf)
    fn = J.build(W.SSDPost())
    assert J.functor_regions(fn.graph) == ["ssd_post"]
    (boxes, scores, res), launches = run_counted(fb, J, fn, loc.cuda(), conf.cuda())
    assert launches == 2
    assert scores.shape == oscores.shape
    close(scores.cpu(), oscores, rtol=1e-5, atol=1e-9, what="softmax scores")
    pri = W.ssd_priors()
    pm = pri[:, 0:2].abs() + pri[:, 2:4].abs() * 4
    close(boxes.cpu(), obox, rtol=1e-5, scale=torch.cat([pm, pm], dim=1)[None].expand_as(obox), what="boxes")
    for (d, l, i), (od, ol, oi) in zip(res, ores):
        assert torch.equal(i.cpu(), oi) and torch.equal(l.cpu(), ol)
        close(d.cpu()[:, 4], od[:, 4], rtol=1e-5, what="scores")


def test_lstm_program_through_the_graph(env):
    fb, J = env
    x, w_ih, w_hh, b_ih, b_hh = W.make_lstm_inputs(8, 64, 512)
    want_hs, want_cs = torch.jit.script(W.LSTMSeq(w_ih, w_hh, b_ih, b_hh))(x)
    fn = J.build(W.LSTMSeq(w_ih, w_hh, b_ih, b_hh))
    assert J.functor_regions(fn.graph) == ["lstm_seq"]
    (hs, cs), launches = run_counted(fb, J, fn, x.cuda())
    assert launches == fb.workloads.LSTM.expected_launches(8, 64, 512)
    close(hs.cpu(), want_hs, rtol=1e-5, scale=1.0, what="hs")
    close(cs.cpu(), want_cs, rtol=1e-5, scale=1.0, what="cs")


def test_yolact_program_through_the_graph(env):
    fb, J = env
    proto, coef, boxes = W.make_yolact_inputs(2)
    want_masks, want_logits = torch.jit.script(W.YolactMasks())(proto, coef, boxes)
    fn = J.build(W.YolactMasks())
    assert J.functor_regions(fn.graph) == ["yolact_masks_logits"]
    (masks, logits), launches = run_counted(fb, J, fn, proto.cuda(), coef.cuda(), boxes.cuda())
    assert launches == 1
    assert logits.shape == want_logits.shape
    mag = torch.einsum("bhwk,bnk->bhwn", proto.abs(), coef.abs())
    close(logits.cpu(), want_logits, rtol=1e-5, scale=mag, what="mask logits")
    diff = masks.cpu() != want_masks
    if bool(diff.any()):
        l64 = torch.einsum("bhwk,bnk->bnhw", proto.double(), coef.double())
        assert bool((l64[diff].abs() < 1e-5).all())
    from functs_b200 import patterns
    fast = J.build(patterns.YolactMasksOnly())
    masks2, launches = run_counted(fb, J, fast, proto.cuda(), coef.cuda(), boxes.cuda())
    assert launches == 1 and torch.equal(masks2, masks)


def test_get_started_program_through_the_graph(env):
    fb, J = env
    a, b, n = W.make_get_started_inputs()
    fn = J.build(W.get_started)
    out, launches = run_counted(fb, J, fn, a.cuda(), b.cuda(), n)
    assert launches == 1
    assert torch.equal(out.cpu(), W.get_started(a, b, n))


def test_region_rejects_cpu_tensors(env):
    fb, J = env
    fn = J.build(W.YolactMasks())
    proto, coef, boxes = W.make_yolact_inputs(1, size=20, num_det=3)
    with pytest.raises(RuntimeError, match="CUDA"):
        fn(proto, coef, boxes)
