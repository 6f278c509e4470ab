"""Two single-group programs for the generic program kernel: small imperative functions whose whole body, once
functionalized, is one fusion group of Access / Assign and elementwise operators.  The reference times the same two access
patterns beside its models (examples/kernel_fusion.py:7-17: channel swap through `select` / `select_rev` on the innermost
dimension of an [800, 1333, 3] image; functs/benchmark/simpleops/offset2bbox/offset2bbox.py:8-44: step-4 slices read and
written on [3000, 4] boxes)."""
import torch


def normalize(src: torch.Tensor, mean: float, scale: float):
    out = src.clone()
    out[..., 0] = src[..., 2]
    out[..., 2] = src[..., 0]
    return (out - mean) * scale


def offset2bbox(boxes: torch.Tensor, offset: torch.Tensor):
    w = boxes[:, 2] - boxes[:, 0] + 1
    h = boxes[:, 3] - boxes[:, 1] + 1
    cx = boxes[:, 0] + 0.5 * w
    cy = boxes[:, 1] + 0.5 * h
    dx = offset[:, 0::4] / 1.0
    dy = offset[:, 1::4] / 1.0
    dw = torch.clamp(offset[:, 2::4] / 1.0, max=4.135)
    dh = torch.clamp(offset[:, 3::4] / 1.0, max=4.135)
    pcx = dx * w[:, None] + cx[:, None]
    pcy = dy * h[:, None] + cy[:, None]
    pw = torch.exp(dw) * w[:, None]
    ph = torch.exp(dh) * h[:, None]
    out = offset.clone()
    out[:, 0::4] = pcx - 0.5 * pw
    out[:, 1::4] = pcy - 0.5 * ph
    out[:, 2::4] = pcx + 0.5 * pw - 1
    out[:, 3::4] = pcy + 0.5 * ph - 1
    return out
