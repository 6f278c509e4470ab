"""GPU parity for the stand-alone immut:: Access / Assign launches against the ATen view ops they stand for
(bit-exact: pure data movement).  Cases restate the reference's test/test_immut_tensorexpr.py:12-95 and the
immut-related suites of fait/testing/lowering_tests.json."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def im(cuda_device):
    from functs_b200 import immut
    return immut


def rnd(*shape, dtype=torch.float32):
    g = torch.Generator().manual_seed(sum(shape) * 3 + len(shape))
    if dtype in (torch.int64, torch.uint8, torch.int16):
        return torch.randint(0, 100, shape, generator=g).to(dtype)
    return torch.rand(*shape, generator=g).to(dtype)


ACCESS = [
    ("select_10x20", (10, 20), lambda im, x: im.select(x, 0, 0), lambda x: x.select(0, 0)),
    ("select_neg", (2, 3, 4), lambda im, x: im.select(x, 1, -1), lambda x: x.select(1, -1)),
    ("slice_3000x4", (3000, 4), lambda im, x: im.slice(x, 1, 0, 3, 4), lambda x: x[:, 0:3:4]),
    ("slice_neg_none", (2, 9), lambda im, x: im.slice(x, 1, -5, None, 2), lambda x: x[:, -5::2]),
    ("squeeze", (3, 1, 4), lambda im, x: im.squeeze(x, 1), lambda x: x.squeeze(1)),
    ("unsqueeze", (3000, 4), lambda im, x: im.unsqueeze(x, 0), lambda x: x.unsqueeze(0)),
    ("reshape", (2, 3, 4), lambda im, x: im.reshape(x, (-1, 6)), lambda x: x.reshape(-1, 6)),
    ("view", (2, 3, 4), lambda im, x: im.view(x, (4, 6)), lambda x: x.view(4, 6)),
    ("permute", (2, 3, 4), lambda im, x: im.permute(x, (2, 0, 1)), lambda x: x.permute(2, 0, 1)),
    ("expand", (1, 3, 1), lambda im, x: im.expand(x, (5, -1, 4)), lambda x: x.expand(5, -1, 4)),
    ("repeat", (2, 3), lambda im, x: im.repeat(x, (2, 3)), lambda x: x.repeat(2, 3)),
    ("repeat_lead", (3, 2), lambda im, x: im.repeat(x, (2, 1, 2)), lambda x: x.repeat(2, 1, 2)),
    ("normalize_800x1333x3", (800, 1333, 3), lambda im, x: im.select(x, 2, 1), lambda x: x.select(2, 1)),
]


@pytest.mark.parametrize("name,shape,ours,theirs", ACCESS, ids=[c[0] for c in ACCESS])
@pytest.mark.parametrize("dtype", [torch.float32, torch.int64, torch.uint8, torch.float16])
def test_access_ops(im, name, shape, ours, theirs, dtype):
    x = rnd(*shape, dtype=dtype)
    want = theirs(x).contiguous()
    got = ours(im, x.cuda())
    assert got.shape == want.shape and got.dtype == want.dtype
    assert torch.equal(got.cpu(), want)


def test_expand_as_and_index(im):
    x = rnd(1, 4)
    other = rnd(3, 4)
    assert torch.equal(im.expand_as(x.cuda(), other.cuda()).cpu(), x.expand_as(other).contiguous())
    src = rnd(5, 3, 2)
    idx = torch.tensor([[[0, 4], [2, 2]], [[1, -1], [3, 0]]])  # 3-D Long indices, one negative
    assert torch.equal(im.index(src.cuda(), [idx.cuda()]).cpu(), src[idx])
    with pytest.raises(IndexError):
        im.index(src.cuda(), [torch.tensor([5]).cuda()])
    with pytest.raises(TypeError):
        im.index(src.cuda(), [torch.tensor([True, False, True, False, True]).cuda()])


def test_select_rev_and_slice_rev(im):
    x, s = rnd(3000, 4), rnd(3000)
    want = x.clone()
    want[:, 0] = s
    assert torch.equal(im.select_rev(x.cuda(), s.cuda(), 1, 0).cpu(), want)
    src = rnd(3000, 1)
    want = x.clone()
    want[:, 0:3:4] = src
    assert torch.equal(im.slice_rev(x.cuda(), src.cuda(), 1, 0, 3, 4).cpu(), want)
    # strided assignment (offset2bbox / clamp on [..., 0::2])
    y, src2 = rnd(7, 5, 8), rnd(7, 5, 4)
    want = y.clone()
    want[..., 1::2] = src2
    assert torch.equal(im.slice_rev(y.cuda(), src2.cuda(), -1, 1, None, 2).cpu(), want)
    # negative bounds, middle dimension, None end
    src3 = rnd(7, 2, 8)
    want = y.clone()
    want[:, -3:-1] = src3
    assert torch.equal(im.slice_rev(y.cuda(), src3.cuda(), 1, -3, -1, 1).cpu(), want)
    # empty region: self comes back unchanged
    assert torch.equal(im.slice_rev(y.cuda(), rnd(7, 0, 8).cuda(), 1, 4, 2, 1).cpu(), y)
    with pytest.raises(IndexError):
        im.select_rev(x.cuda(), s.cuda(), 1, 4)


def test_other_rev_forms(im):
    x = rnd(2, 3, 4)
    src = rnd(4, 2, 3)
    # permute_rev: the tensor whose permute(dims) equals src
    got = im.permute_rev(x.cuda(), src.cuda(), (2, 0, 1)).cpu()
    assert torch.equal(got.permute(2, 0, 1), src)
    v = rnd(6, 4)
    assert torch.equal(im.view_rev(x.cuda(), v.cuda(), (6, 4)).cpu(), v.reshape(2, 3, 4))
    assert im.unsqueeze_rev(x.cuda(), rnd(2, 1, 3, 4).cuda(), 1).shape == x.shape
    with pytest.raises(RuntimeError):
        im.expand_rev(rnd(1, 4).cuda(), rnd(3, 4).cuda(), (3, 4))
    assert torch.equal(im.repeat_rev(x.cuda(), rnd(4, 3, 4).cuda(), (2, 1, 1)).cpu(), x)
    base, rows = rnd(6, 5), rnd(3, 5)
    idx = torch.tensor([4, 0, 2])
    want = base.clone()
    want[idx] = rows
    assert torch.equal(im.index_rev(base.cuda(), rows.cuda(), [idx.cuda()]).cpu(), want)


def test_normalize_program(im):
    """examples/kernel_fusion.py style: channel swap through two select_rev's on an 800x1333x3 image."""
    img = rnd(800, 1333, 3)
    want = img.clone()
    want[:, :, 0] = img[:, :, 2]
    want[:, :, 2] = img[:, :, 0]
    d = img.cuda()
    c0, c2 = im.select(d, 2, 0), im.select(d, 2, 2)
    out = im.select_rev(im.select_rev(d, c2, 2, 0), c0, 2, 2)
    assert torch.equal(out.cpu(), want)
