"""Host-side index descriptions of the Access family against torch view ops (CPU).  The case list restates the
shapes of the reference's lowering tests (fait/testing/lowering_tests.json) and of test/test_immut_tensorexpr.py."""
import numpy as np
import pytest
import torch

from functs_b200 import access_desc as ad
from oracle import immut_ref as R


def run(src: torch.Tensor, a: ad.Access) -> torch.Tensor:
    out = R.eval_access(src.numpy(), a.out_shape, a.src_stride, a.src_mod, a.src_offset)
    return torch.from_numpy(np.ascontiguousarray(out))


def rnd(*shape):
    g = torch.Generator().manual_seed(sum(shape) + len(shape))
    return torch.rand(*shape, generator=g)


CASES = [
    ("select", lambda x: x.select(0, 0), lambda s: ad.select(s, 0, 0), (10, 20)),
    ("select_neg", lambda x: x.select(1, -1), lambda s: ad.select(s, 1, -1), (2, 3, 4)),
    ("select_mid", lambda x: x.select(-2, 1), lambda s: ad.select(s, -2, 1), (2, 3, 4)),
    ("slice_0_3_4", lambda x: x[:, 0:3:4], lambda s: ad.slice_(s, 1, 0, 3, 4), (3000, 4)),
    ("slice_neg_start", lambda x: x[:, -3:], lambda s: ad.slice_(s, 1, -3, None, 1), (2, 5)),
    ("slice_step2", lambda x: x[:, 1::2], lambda s: ad.slice_(s, 1, 1, None, 2), (2, 7)),
    ("slice_big_end", lambda x: x[1:100], lambda s: ad.slice_(s, 0, 1, 100, 1), (4, 3)),
    ("slice_empty", lambda x: x[3:1], lambda s: ad.slice_(s, 0, 3, 1, 1), (4, 3)),
    ("squeeze", lambda x: x.squeeze(1), lambda s: ad.squeeze(s, 1), (3, 1, 4)),
    ("squeeze_noop", lambda x: x.squeeze(0), lambda s: ad.squeeze(s, 0), (3, 1, 4)),
    ("unsqueeze0", lambda x: x.unsqueeze(0), lambda s: ad.unsqueeze(s, 0), (3000, 4)),
    ("unsqueeze_neg", lambda x: x.unsqueeze(-1), lambda s: ad.unsqueeze(s, -1), (2, 3)),
    ("reshape_m1", lambda x: x.reshape(-1, 6), lambda s: ad.view(s, (-1, 6)), (2, 3, 4)),
    ("view", lambda x: x.view(4, 6), lambda s: ad.view(s, (4, 6)), (2, 3, 4)),
    ("permute", lambda x: x.permute(2, 0, 1), lambda s: ad.permute(s, (2, 0, 1)), (2, 3, 4)),
    ("permute_neg", lambda x: x.permute(0, -1, 1), lambda s: ad.permute(s, (0, -1, 1)), (2, 3, 4)),
    ("expand_m1", lambda x: x.expand(5, -1, 4), lambda s: ad.expand(s, (5, -1, 4)), (1, 3, 1)),
    ("expand_lead", lambda x: x.expand(2, 3, 4), lambda s: ad.expand(s, (2, 3, 4)), (3, 4)),
    ("repeat", lambda x: x.repeat(2, 3), lambda s: ad.repeat(s, (2, 3)), (2, 3)),
    ("repeat_lead", lambda x: x.repeat(2, 1, 2), lambda s: ad.repeat(s, (2, 1, 2)), (3, 2)),
]


@pytest.mark.parametrize("name,torch_fn,desc_fn,shape", CASES, ids=[c[0] for c in CASES])
def test_access_matches_torch(name, torch_fn, desc_fn, shape):
    x = rnd(*shape)
    want = torch_fn(x)
    a = desc_fn(tuple(shape))
    assert list(a.out_shape) == list(want.shape)
    got = run(x, a)
    assert torch.equal(got.reshape(want.shape), want.contiguous())


def test_errors_follow_aten():
    with pytest.raises(IndexError):
        ad.select((3, 4), 0, 3)
    with pytest.raises(IndexError):
        ad.select((3, 4), 2, 0)
    with pytest.raises(ValueError):
        ad.view((3, 4), (5, -1))
    with pytest.raises(ValueError):
        ad.expand((3, 4), (2, 4))
    with pytest.raises(ValueError):
        ad.permute((3, 4), (0, 0))
    assert ad.normalize_slice(10, None, None, 1) == (0, 10, 10)
    assert ad.normalize_slice(10, -3, None, 2) == (7, 10, 2)
    assert ad.normalize_slice(10, 8, 2, 1) == (8, 8, 0)


def test_rev_reference_semantics():
    x = rnd(5, 4)
    s = rnd(5)
    want = x.clone()
    want[:, 2] = s
    assert np.array_equal(R.select_rev(x.numpy(), s.numpy(), 1, 2), want.numpy())
    src = rnd(5, 2)
    want = x.clone()
    want[:, 0::2] = src
    assert np.array_equal(R.slice_rev(x.numpy(), src.numpy(), 1, 0, 4, 2), want.numpy())
