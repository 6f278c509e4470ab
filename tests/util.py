"""Helpers shared by the parity tests."""
import torch

IDX_MASK = 0xFFFFFFFF


def key_scores(keys: torch.Tensor) -> torch.Tensor:
    """int64 keys -> fp32 scores (high word reinterpreted)."""
    return (keys >> 32).to(torch.int32).view(torch.float32)


def key_index(keys: torch.Tensor) -> torch.Tensor:
    return IDX_MASK - (keys & IDX_MASK)


def make_keys(scores: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    bits = scores.contiguous().view(torch.int32).to(torch.int64)
    return (bits << 32) | (IDX_MASK - idx.to(torch.int64))


def close(actual: torch.Tensor, expected: torch.Tensor, rtol: float = 1e-5, atol: float = 0.0, scale=None, what=""):
    """|actual - expected| <= atol + rtol * max(|expected|, scale).  `scale` is the magnitude of the operands a
    value was formed from (a difference of two large numbers is only accurate relative to them)."""
    a, e = actual.double().cpu(), expected.double().cpu()
    mag = e.abs()
    if scale is not None:
        mag = torch.maximum(mag, torch.as_tensor(scale, dtype=torch.float64).expand_as(mag))
    err = (a - e).abs()
    bad = err > atol + rtol * mag
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())} of {bad.numel()} elements outside rtol={rtol} atol={atol}; "
        f"max abs err {float(err.max()):.3e}, worst rel {float((err / mag.clamp_min(1e-30)).max()):.3e}")
    return float((err / mag.clamp_min(1e-30)).max())
