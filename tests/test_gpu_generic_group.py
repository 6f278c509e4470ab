"""Fusion groups without a precompiled kernel: the generic program kernel runs a whole group (all map iterations included)
in ONE launch; the result must equal the eager program on the same device bit for bit (the kernel evaluates sigmoid /
exp / tanh with the same expressions and every elementwise step rounds on its own, as ATen's kernels do)."""
from typing import List

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(cuda_device):
    import functs_b200
    from functs_b200 import jit
    return functs_b200, jit


def scales(feats: List[torch.Tensor], offs: List[torch.Tensor]):
    outs: List[torch.Tensor] = []
    for i in range(3):
        x = feats[i].clone()
        x[:, 0:2] = torch.sigmoid(x[:, 0:2]) + offs[i]
        x[:, 2:4] = torch.exp(x[:, 2:4]) * 2.0
        outs.append(x * 8.0)
    return outs


def normalize(img: torch.Tensor):
    # channel swap + per-channel affine through select / select_rev on the last dimension (examples/kernel_fusion.py style)
    out = img.clone()
    out[..., 0] = (img[..., 2] - 0.406) / 0.225
    out[..., 1] = (img[..., 1] - 0.456) / 0.224
    out[..., 2] = (img[..., 0] - 0.485) / 0.229
    return out


def mixed(x: torch.Tensor, y: torch.Tensor):
    t = x.clone()
    t[:, 1::2] = torch.clamp(t[:, 1::2] * 2.0, min=0.1, max=0.9)
    u = torch.cat([t[:, 0:3], torch.tanh(t[:, 3:8])], dim=1) + y
    v = torch.stack([u, u * 0.5], dim=0).permute(1, 0, 2)
    w = torch.maximum(u, y.unsqueeze(0).expand(6, 8)) - torch.minimum(u, y)
    return v, u > 0.5, w


def with_softmax(x: torch.Tensor):
    t = x.clone()
    t[:, 0:2] = torch.sigmoid(t[:, 0:2])
    return torch.softmax(t * 2.0, dim=1) + t


def check(env, fn, args, expect_generic=True):
    fb, J = env
    built = J.build(fn, args)
    n_groups = J.count_groups(built.graph)
    assert n_groups >= 1
    assert all(r == "" for r in J.functor_regions(built.graph)), "these programs match no precompiled region"
    want = fn(*[[t.clone() for t in a] if isinstance(a, list) else (a.clone() if isinstance(a, torch.Tensor) else a) for a in args])
    built(*args)  # first run builds the executor
    torch.cuda.synchronize()
    l0, g0, i0 = fb.launch_count(), J.generic_group_runs(), J.interpreted_functor_runs()
    got = built(*args)
    torch.cuda.synchronize()
    launches, generic, interp = fb.launch_count() - l0, J.generic_group_runs() - g0, J.interpreted_functor_runs() - i0
    flat_w = want if isinstance(want, (list, tuple)) else [want]
    flat_g = got if isinstance(got, (list, tuple)) else [got]
    assert len(flat_w) == len(flat_g)
    for a, b in zip(flat_g, flat_w):
        assert a.dtype == b.dtype and a.shape == b.shape
        assert torch.equal(a, b), (fn.__name__, float((a.float() - b.float()).abs().max()))
    if expect_generic:
        assert interp == 0, f"{fn.__name__}: a group was interpreted: {J.last_generic_refusal()}"
        assert generic == n_groups and launches == n_groups, (generic, launches, n_groups)
    return n_groups, launches, generic, interp


def test_map_over_scales_is_one_launch(env):
    g = torch.Generator().manual_seed(3)
    feats = [torch.randn(50 + i, 6, generator=g).cuda() for i in range(3)]
    offs = [torch.randn(50 + i, 2, generator=g).cuda() for i in range(3)]
    n_groups, launches, generic, _ = check(env, scales, (feats, offs))
    assert n_groups == 1 and launches == 1  # three iterations of different shapes, one launch


def test_normalize_group(env):
    g = torch.Generator().manual_seed(4)
    img = torch.rand(80, 133, 3, generator=g).cuda()
    check(env, normalize, (img,))


def test_mixed_access_assign_elementwise(env):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(6, 8, generator=g).cuda()
    y = torch.randn(8, generator=g).cuda()
    check(env, mixed, (x, y))


def test_group_the_program_format_cannot_express_is_interpreted(env):
    fb, J = env
    g = torch.Generator().manual_seed(6)
    x = torch.randn(5, 7, generator=g).cuda()
    n_groups, launches, generic, interp = check(env, with_softmax, (x,), expect_generic=False)
    assert interp >= 1 and "softmax" in J.last_generic_refusal()


def split_body(feats: List[torch.Tensor]):
    outs: List[torch.Tensor] = []
    for i in range(len(feats)):
        x = feats[i].clone()
        x[:, 0:2] = torch.sigmoid(x[:, 0:2]) * 2.0
        s = x.sum()
        y = x * 3.0 + s
        outs.append(torch.tanh(y))
    return outs


def test_split_map_runs_two_launches_plus_the_loop_between(env):
    """[group, sum, group] inside a map: each group is ONE launch over all iterations; the sums stay a loop of ATen calls."""
    fb, J = env
    g = torch.Generator().manual_seed(8)
    feats = [torch.randn(20 + 3 * i, 6, generator=g).cuda() for i in range(4)]
    built = J.build(split_body, (feats,))
    want = split_body(feats)
    built(feats)
    torch.cuda.synchronize()
    l0, g0, i0 = fb.launch_count(), J.generic_group_runs(), J.interpreted_functor_runs()
    got = built(feats)
    torch.cuda.synchronize()
    assert fb.launch_count() - l0 == 2 and J.generic_group_runs() - g0 == 2 and J.interpreted_functor_runs() == i0, J.last_generic_refusal()
    for a, b in zip(got, want):
        assert torch.allclose(a, b, rtol=1e-6, atol=1e-6)


def test_reference_simple_programs_are_one_launch_each(env):
    """The channel-swap normalisation on [800, 1333, 3] and the step-4 box decoding on [3000, 4]: one generic launch each,
    equal to eager bit for bit."""
    from functs_b200 import simpleops
    g = torch.Generator().manual_seed(5)
    img = torch.rand(800, 1333, 3, generator=g).cuda()
    assert check(env, simpleops.normalize, (img, 0.45, 4.4)) == (1, 1, 1, 0)
    boxes = (torch.rand(3000, 4, generator=g) * 100).cuda()
    offs = torch.randn(3000, 4, generator=g).cuda()
    assert check(env, simpleops.offset2bbox, (boxes, offs)) == (1, 1, 1, 0)


def rank5(x: torch.Tensor, y: torch.Tensor):
    t = x.clone()
    t[:, :, 1, :, 0:3] = torch.relu(t[:, :, 1, :, 0:3]) - y
    u = t.permute(0, 2, 1, 3, 4) * 0.5
    return u, t[:, 0, :, 1:3, :] > 0.25


def test_rank_five_program_and_bool_output(env):
    """Index arithmetic over five dimensions (the rank-8 instantiation), a permuted output and a bool output."""
    g = torch.Generator().manual_seed(11)
    x = torch.randn(3, 4, 5, 6, 7, generator=g).cuda()
    y = torch.randn(6, 3, generator=g).cuda()
    check(env, rank5, (x, y))


def scaled(x: torch.Tensor, s: float):
    t = x.clone()
    t[1:, :] = t[1:, :] * s
    return t + 1.0


def test_cached_programs_follow_shapes_and_scalars(env):
    """The flattened program of a functor is kept between calls: another shape or another scalar value rebuilds it, the
    same ones only re-point it; the results are those of the eager program every time."""
    fb, J = env
    g = torch.Generator().manual_seed(12)
    a = torch.randn(9, 17, generator=g).cuda()
    b = torch.randn(33, 5, generator=g).cuda()
    built = J.build(scaled, (a, 2.0))
    for x, s in ((a, 2.0), (a, 2.0), (a, -0.75), (b, -0.75), (a, 2.0), (b.t().contiguous().t(), 3.5)):
        i0 = J.interpreted_functor_runs()
        got = built(x, s)
        assert J.interpreted_functor_runs() == i0, J.last_generic_refusal()
        assert torch.equal(got, scaled(x, s))


def strided_big(x: torch.Tensor, y: torch.Tensor):
    t = x.clone()
    t[:, 1::2] = torch.clamp(t[:, 1::2] * 2.0, min=-0.5, max=0.5)
    return torch.tanh(t) + y, t[:, 3:50] > 0.0


def test_four_elements_per_thread_with_divided_coordinates(env):
    """Large enough for four elements per thread along the untested dimension (4099 rows: a ragged last block), with a read
    below a strided assignment (a divided coordinate in the load) and a broadcast operand."""
    g = torch.Generator().manual_seed(13)
    x = torch.randn(4099, 96, generator=g).cuda()
    y = torch.randn(96, generator=g).cuda()
    check(env, strided_big, (x, y))
