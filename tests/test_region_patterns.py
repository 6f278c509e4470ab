"""Precompiled regions on CPU: the functionalized graphs of the oracle programs must reach the kernel adapters.

Builds every oracle module with functs_b200.jit.build and checks which adapter each tssa::ParallelFunctor node is bound
to (no GPU needed: nothing is executed).  Also checks what a signature does and does not depend on."""
import pytest
import torch

from oracle import workloads as W


@pytest.fixture(scope="module")
def J():
    from functs_b200 import jit
    return jit


def lstm_module(hidden=256):
    _, w_ih, w_hh, b_ih, b_hh = W.make_lstm_inputs(2, 2, hidden)
    return W.LSTMSeq(w_ih, w_hh, b_ih, b_hh)


@pytest.mark.parametrize("make,adapter", [
    (lambda: W.YOLOV3Post(), "yolov3_post_dense"),
    (lambda: W.YOLOV3Post(sizes=(2, 4, 8), score_thr=0.3, topk=100, iou_thr=0.6), "yolov3_post_dense"),
    (lambda: W.SSDPost(), "ssd_post"),
    (lambda: W.SSDPost(score_thr=0.05, topk=50, iou_thr=0.5), "ssd_post"),
    (lambda: lstm_module(256), "lstm_seq"),
    (lambda: lstm_module(512), "lstm_seq"),
    (lambda: W.YolactMasks(), "yolact_masks_logits"),
    (lambda: W.YolactMasks(thr=0.7), "yolact_masks_logits"),
])
def test_oracle_programs_reach_their_kernels(J, make, adapter):
    f = J.build(make())
    assert J.functor_regions(f.graph) == [adapter]
    kinds = {n.kind() for n in f.graph.nodes()}
    assert "prim::Loop" not in kinds, "the whole loop nest must have gone into the functor"


def functor_node(graph):
    return next(n for n in graph.nodes() if n.kind() == "tssa::ParallelFunctor")


def test_free_constants_travel_as_attributes(J):
    f = J.build(W.SSDPost(score_thr=0.05, topk=50, iou_thr=0.5))
    n = functor_node(f.graph)
    assert n.s("region") == "ssd_post"
    assert n.f("score_thr") == 0.05 and n.f("iou_thr") == 0.5 and n.f("clamp_max") == 300.0 and n.i("topk") == 50
    f = J.build(lstm_module(512))
    assert functor_node(f.graph).i("hidden") == 512
    f = J.build(W.YOLOV3Post(score_thr=0.3, topk=100, iou_thr=0.6))
    n = functor_node(f.graph)
    assert n.f("score_thr") == 0.3 and n.f("iou_thr") == 0.6 and n.i("topk") == 100


def test_results_only_variants(J):
    from functs_b200 import patterns
    f = J.build(patterns.YOLOV3Det())
    assert J.functor_regions(f.graph) == ["yolov3_post"]
    f = J.build(patterns.YolactMasksOnly())
    assert J.functor_regions(f.graph) == ["yolact_masks"]


class SSDOtherVariance(W.SSDPost):
    """Same structure, but the wh variance is a structural constant of the decode: 0.25 instead of 0.2."""

    def forward(self, loc, conf):
        num_imgs = loc.size(0)
        scores = conf.softmax(-1)[..., :-1]
        bboxes = torch.zeros_like(loc)
        for b in range(num_imgs):
            pxy = self.priors[:, 0:2]
            pwh = self.priors[:, 2:4]
            gxy = pxy + pwh * (loc[b][:, 0:2] * 0.1)
            gwh = pwh * (loc[b][:, 2:4] * 0.25).exp()
            bboxes[b] = torch.cat([gxy - gwh * 0.5, gxy + gwh * 0.5], dim=-1)
        return bboxes, scores


def test_structural_change_does_not_match(J):
    f = J.build(SSDOtherVariance())
    assert "ssd_post" not in J.functor_regions(f.graph)


class Embedded(torch.nn.Module):
    """The mask assembly inside a larger program: ops before and after the region."""

    def __init__(self):
        super().__init__()
        self.inner = W.YolactMasks()

    def forward(self, proto, coef, boxes):
        proto = proto * 2.0
        masks, logits = self.inner(proto, torch.tanh(coef), boxes)
        return masks.sum(), logits


def test_region_inside_a_larger_program(J):
    f = J.build(Embedded())
    regions = J.functor_regions(f.graph)
    assert "yolact_masks_logits" in regions
    kinds = [n.kind() for n in f.graph.nodes()]
    assert "aten::sum" in kinds and "prim::Loop" not in kinds
    # the ops in front of the region form a group of their own (mul, tanh); the region's inputs are its results
    assert regions.index("yolact_masks_logits") == len(regions) - 1


def test_signature_ignores_shapes_and_names(J):
    from functs_b200 import patterns
    d = patterns.register_all()
    assert set(d) == {"yolov3_post_dense", "yolov3_post", "ssd_post", "lstm_seq", "yolact_masks_logits", "yolact_masks"}
    for name, desc in d.items():
        assert desc["num_nodes"] > 0 and "f?" in desc["signature"] or name == "lstm_seq"
        assert "Float(" not in desc["signature"]  # no static shapes in a signature


def test_dump_graph_writes_stage_files(J, tmp_path, monkeypatch):
    """DUMP_GRAPH=<dir>: the IR after every pipeline stage is written to after_<stage>.rb."""
    monkeypatch.setenv("DUMP_GRAPH", str(tmp_path))
    J.build(W.YolactMasks())
    names = sorted(p.name for p in tmp_path.iterdir())
    assert names == ["after_fuse_ops.rb", "after_match_regions.rb", "after_parallel_functors.rb",
                     "after_parallelize_loops.rb", "after_split_parallel_maps.rb", "after_tensorssa.rb",
                     "after_unroll_loops.rb"]
    assert "prim::Loop" in (tmp_path / "after_tensorssa.rb").read_text()
    assert "tssa::ParallelFunctor" in (tmp_path / "after_match_regions.rb").read_text()
