"""Generates the golden fixtures in this folder by running the REFERENCE's own Python functions on CPU.

Run once, in a container that has the reference checked out, with the path of that checkout:
    python tests/golden/make_golden.py <reference_root>
The fixtures (small ``.pt`` files: seeded inputs + the reference's outputs) are committed; the tests only read them.

The reference's benchmark modules cannot be instantiated on CPU (their constructors call ``.cuda()`` and load
feature files that are not shipped), so the functions are taken from the source files directly: plain functions
are imported by file path; methods are called unbound on a stand-in ``self``; ``examples/get_started.py`` executes
``functs._C`` code at import time, so only the ``func`` definition is extracted from its syntax tree (likewise ``LSTMCell`` from lstm.py, which imports
``functs.utils``).
"""
import ast
import importlib.util
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_module(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def extract_function(path: str, func_name: str):
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, (ast.FunctionDef, ast.ClassDef)) and node.name == func_name:
            ns = {"torch": torch, "nn": torch.nn}
            exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), ns)
            return ns[func_name]
    raise KeyError(func_name)


def gen(seed: int) -> torch.Generator:
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def main(ref_root: str) -> None:
    bench = os.path.join(ref_root, "functs", "benchmark", "ai_model")
    out = {}

    # ---- get_started: examples/get_started.py:10-15 ----
    func = extract_function(os.path.join(ref_root, "examples", "get_started.py"), "func")
    g = gen(11)
    a, b = torch.randn(8, 16, generator=g), torch.randn(8, 16, generator=g)
    out["get_started"] = {"a": a, "b": b, "n": 5, "out": func(a, b, 5)}

    # ---- class-offset NMS: yolov3_bbox.py:139-179 (batched_nms + nms_wrapper) ----
    yolo = load_module(os.path.join(bench, "yolov3", "yolov3_bbox.py"), "ref_yolov3_bbox")
    g = gen(12)
    n = 300
    ctr = torch.rand(n, 2, generator=g) * 100
    wh = torch.rand(n, 2, generator=g) * 40 + 2
    boxes = torch.cat([ctr - wh / 2, ctr + wh / 2], dim=1)
    scores = torch.rand(n, generator=g)
    scores, _ = scores.sort(descending=True)
    labels = torch.randint(0, 4, (n,), generator=g)
    dets, keep = yolo.batched_nms(boxes, scores, labels)
    out["batched_nms"] = {"boxes": boxes, "scores": scores, "labels": labels, "iou_thr": 0.45, "dets": dets, "keep": keep}

    # ---- YOLOv3 box decode: yolov3_bbox.py:12-23 (decode_bboxes) on the anchors of YOLOAnchorGenerator (:26-100), fed as
    # YOLOV3BBox.forward feeds them (:209-222): permute/reshape, sigmoid on the xy slice, strides expanded per box.
    # gen_single_level_base_anchors ends in .cuda(); on this CPU-only run that one method is made the identity.
    g = gen(17)
    sizes, strides = (2, 3, 5), (32, 16, 8)
    maps = [torch.randn(1, 255, s, s, generator=g) for s in sizes]
    cuda_saved = torch.Tensor.cuda
    torch.Tensor.cuda = lambda self, *a, **k: self
    try:
        agen = yolo.YOLOAnchorGenerator(strides=[32, 16, 8], base_sizes=[[(116, 90), (156, 198), (373, 326)],
                                                                       [(30, 61), (62, 45), (59, 119)],
                                                                       [(10, 13), (16, 30), (33, 23)]])
    finally:
        torch.Tensor.cuda = cuda_saved
    anchors = torch.cat(agen([(s, s) for s in sizes], dtype=torch.float32, device=torch.device("cpu")))
    preds, strs = [], []
    for pred, stride in zip(maps, strides):
        pred = pred.permute(0, 2, 3, 1).reshape(1, -1, 85).clone()
        pred[..., :2].sigmoid_()
        preds.append(pred.clone())
        strs.append(torch.tensor(stride).expand(pred.size(1)))
    flat = torch.cat(preds, dim=1)
    out["yolo_decode"] = {"maps": maps, "sizes": sizes,
                          "bboxes": yolo.decode_bboxes(anchors, flat[..., :4], torch.cat(strs).unsqueeze(-1)),
                          "objectness": flat[..., 4].sigmoid(), "cls_scores": flat[..., 5:].sigmoid()}

    # ---- mask -> nonzero -> sort -> top-k: ssd_bbox.py:163-172 (filter_scores_and_topk) ----
    ssd = load_module(os.path.join(bench, "ssd", "ssd_bbox.py"), "ref_ssd_bbox")
    g = gen(13)
    sc = torch.rand(500, 7, generator=g)
    s, lab, keep_idxs = ssd.filter_scores_and_topk(sc, 0.3, 200)
    out["filter_topk"] = {"scores": sc, "thr": 0.3, "topk": 200, "out_scores": s, "out_labels": lab, "out_rows": keep_idxs}

    # ---- box decode with the strided clamp: ssd_bbox.py:121-154 (delta2bbox) ----
    # priors with exactly representable corners, so that corner form -> centre/size is exact
    g = gen(14)
    m = 400
    cxy = torch.randint(8, 300, (m, 2), generator=g).float()
    pwh = (torch.randint(2, 60, (m, 2), generator=g) * 2).float()
    rois = torch.cat([cxy - pwh / 2, cxy + pwh / 2], dim=1)
    deltas = torch.randn(m, 4, generator=g)
    out["delta2bbox"] = {"priors": torch.cat([cxy, pwh], dim=1), "rois": rois, "deltas": deltas, "clamp_max": 320.0,
                         "out": ssd.delta2bbox(rois, deltas)}

    # ---- one LSTM cell step: lstm.py:79-98 (LSTMCell.forward, called on a stand-in self) ----
    # (lstm.py imports functs.utils at module level, so only the LSTMCell class definition is extracted)
    lstm_cell_cls = extract_function(os.path.join(bench, "lstm", "lstm.py"), "LSTMCell")
    g = gen(15)
    hid, bat = 32, 6
    self_ = types.SimpleNamespace(
        weight_ih_l0_t=(torch.rand(4, hid, hid, generator=g) - 0.5) * 0.4,
        weight_hh_l0_t=(torch.rand(4, hid, hid, generator=g) - 0.5) * 0.4,
        bias_ih_l0_t=(torch.rand(4, 1, hid, generator=g) - 0.5) * 0.4,
        bias_hh_l0_t=(torch.rand(4, 1, hid, generator=g) - 0.5) * 0.4)
    x = torch.randn(bat, hid, generator=g)
    h0 = torch.randn(bat, hid, generator=g) * 0.5
    c0 = torch.randn(bat, hid, generator=g) * 0.5
    _, h1, c1 = lstm_cell_cls.forward(self_, x, h0, c0)
    out["lstm_cell"] = {"w_ih": self_.weight_ih_l0_t, "w_hh": self_.weight_hh_l0_t, "b_ih": self_.bias_ih_l0_t,
                        "b_hh": self_.bias_hh_l0_t, "x": x, "h0": h0, "c0": c0, "h1": h1, "c1": c1}

    # ---- crop to the sanitised box: yolact_mask.py:306-333 (crop + sanitize_coordinates, unbound) ----
    yolact = load_module(os.path.join(bench, "yolact", "yolact_mask.py"), "ref_yolact_mask")
    cls = yolact.YolactBBoxMask
    self_ = types.SimpleNamespace(sanitize_coordinates=lambda x1, x2, size: cls.sanitize_coordinates(None, x1, x2, size))
    g = gen(16)
    hgt, wid, nd = 20, 24, 9
    masks = torch.rand(hgt, wid, nd, generator=g) + 0.1
    u = torch.rand(nd, 4, generator=g)
    bx = torch.stack([u[:, 0] * wid, u[:, 1] * hgt, u[:, 2] * wid, u[:, 3] * hgt], dim=1)  # unsorted on purpose
    out["yolact_crop"] = {"masks": masks, "boxes": bx, "out": cls.crop(self_, masks, bx)}

    for name, blob in out.items():
        torch.save(blob, os.path.join(HERE, f"{name}.pt"))
        print("wrote", name, {k: (tuple(v.shape) if isinstance(v, torch.Tensor) else v) for k, v in blob.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <reference_root>")
    main(sys.argv[1])
