"""Functionalized TorchScript graphs executed on the GPU: the immut:: operators run as CUDA launches of the C-ABI
library.  Programs restate the reference's test/test_basic.py:6-38 and examples/get_started.py:10-15; the result must
equal the eager program run on the same device bit for bit (and the CPU eager program within 1e-5)."""
from typing import List

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fjit(cuda_device):
    from functs_b200 import jit
    return jit


def get_started(a: torch.Tensor, b: torch.Tensor, n: int):
    a = a.clone()
    b = b.clone()
    for i in range(n):
        b[i] = b[i] + 1
    return b


def dataflow(a: torch.Tensor, b: torch.Tensor):
    a = a.clone()
    a[0].copy_(b[0])
    a[1].copy_(b[1])
    a[0:1] = b[0:1]
    return a + a[0:1]


def branch_loop(a: torch.Tensor, c: torch.Tensor, d: torch.Tensor):
    tmp_0 = d.clone()
    tmp_1 = tmp_0[1]
    if a.nonzero().sum():
        tmp_0 = tmp_0 + 1
        for i in range(10):
            tmp_1.copy_(tmp_0[i + 1])
    else:
        tmp_0 = tmp_0 + tmp_1
        tmp_1.copy_(tmp_0[2])
    return tmp_1 + tmp_0


def strided_views(x: torch.Tensor, y: torch.Tensor):
    t = x.clone()
    t[..., 0:2].sigmoid_()
    t[:, 1::2].clamp_(min=0.1, max=0.6)
    t[2].add_(y[2])
    u = t.permute(1, 0)
    u[0] = u[0] * 3
    v = t.unsqueeze(0)
    v[0, 3] = t[4] * 2
    return t + u.permute(1, 0)


def rnd(*shape, seed=0):
    return torch.rand(*shape, generator=torch.Generator().manual_seed(seed + sum(shape)))


def run(fjit, fn, *args):
    g = torch.jit.script(fn).graph.copy()
    fjit.functionalize_graph(g)
    kinds = [n.kind() for n in g.nodes()]
    f = torch._C._create_function_from_graph(fn.__name__, g)
    dev_args = [a.cuda() if isinstance(a, torch.Tensor) else a for a in args]
    want = fn(*[a.clone() if isinstance(a, torch.Tensor) else a for a in dev_args])  # eager program on the same device
    got = f(*dev_args)
    assert got.is_cuda and torch.equal(got, want), fn.__name__
    assert torch.allclose(got.cpu(), fn(*args), rtol=1e-5, atol=1e-6), fn.__name__
    return kinds


def test_get_started_on_gpu(fjit):
    kinds = run(fjit, get_started, rnd(64, 1024), rnd(64, 1024, seed=1), 64)
    assert "prim::Loop" in kinds and "aten::copy_" not in kinds


def test_reference_programs_on_gpu(fjit):
    run(fjit, dataflow, rnd(64, 32), rnd(64, 32, seed=1))
    run(fjit, branch_loop, torch.ones(3), rnd(2, 2), rnd(12, 40, seed=2))
    run(fjit, branch_loop, torch.zeros(3), rnd(2, 2), rnd(12, 40, seed=2))
    run(fjit, strided_views, rnd(6, 8), rnd(6, 8, seed=3))


def test_script_front_door(fjit):
    f = fjit.script(get_started)
    a, b = rnd(8, 16), rnd(8, 16, seed=1)
    assert torch.equal(f(a.cuda(), b.cuda(), 5).cpu(), get_started(a, b, 5))


def scales(feats: List[torch.Tensor], offs: List[torch.Tensor]):
    outs: List[torch.Tensor] = []
    for i in range(3):
        x = feats[i].clone()
        x[:, 0:2] = torch.sigmoid(x[:, 0:2]) + offs[i]
        x[:, 2:4] = torch.exp(x[:, 2:4]) * 2.0
        outs.append(x * 8.0)
    return outs


def test_build_launches_the_precompiled_group(fjit):
    """jit.build: the get_started loop becomes ONE tssa::ParallelFunctor that launches the library's kernel (one launch
    for the whole loop), with the bit-exact result of the eager program."""
    from functs_b200._lib import launch_count
    fn = fjit.build(get_started, (rnd(64, 1024), rnd(64, 1024, seed=1), 64))
    nodes = [n for n in fn.graph.nodes() if n.kind() == "tssa::ParallelFunctor"]
    assert len(nodes) == 1 and fjit.count_groups(fn.graph) == 1
    assert "prim::Loop" not in [n.kind() for n in fn.graph.nodes()]
    a, b = rnd(64, 1024), rnd(64, 1024, seed=1)
    ca, cb = a.cuda(), b.cuda()
    fn(ca, cb, 64)  # warm-up (first run of the graph executor)
    torch.cuda.synchronize()
    before = launch_count()
    got = fn(ca, cb, 64)
    torch.cuda.synchronize()
    assert launch_count() - before == 1
    assert torch.equal(got.cpu(), get_started(a, b, 64))
    assert torch.equal(fn(ca, cb, 17).cpu(), get_started(a, b, 17))


def test_build_parallel_map_on_gpu(fjit):
    """A loop over three scales becomes one tssa::ParallelFunctor(is_parallel_map); without a precompiled kernel for its
    signature the operator runs the subgraph per index on the immut:: CUDA kernels: same bits as eager on the device."""
    g = torch.Generator().manual_seed(3)
    feats = [torch.randn(50 + i, 6, generator=g).cuda() for i in range(3)]
    offs = [torch.randn(50 + i, 2, generator=g).cuda() for i in range(3)]
    fn = fjit.build(scales, (feats, offs))
    nodes = [n for n in fn.graph.nodes() if n.kind() == "tssa::ParallelFunctor"]
    assert len(nodes) == 1 and nodes[0].i("is_parallel_map") == 1 and nodes[0].i("parallel_degree") == 3
    want = scales(feats, offs)
    got = fn(feats, offs)
    torch.cuda.synchronize()
    assert len(got) == 3
    for a, b in zip(got, want):
        assert torch.equal(a, b)
