"""Host logic of the multi-GPU path on CPU: contiguous sharding + the detection gather, two gloo ranks."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from functs_b200 import dist as fdist  # noqa: E402  (imports only torch; no CUDA needed)


def test_shard_range_covers_everything():
    for total in (1, 7, 64, 65):
        for world in (1, 2, 4, 8):
            spans = [fdist.shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1


def test_pack_unpack_roundtrip():
    g = torch.Generator().manual_seed(3)
    b, k = 3, 10
    dets = torch.randn(b, k, 5, generator=g)
    labels = torch.randint(0, 80, (b, k), generator=g)
    ids = torch.randint(0, 851760, (b, k), generator=g)
    counts = torch.tensor([0, 4, 10], dtype=torch.int32)
    d2, l2, i2, c2 = fdist.unpack_detections(fdist.pack_detections(dets, labels, ids, counts))
    assert torch.equal(d2, dets) and torch.equal(l2, labels) and torch.equal(i2, ids) and torch.equal(c2, counts)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, total, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(100)
        k = 6
        dets = torch.randn(total, k, 5, generator=g)
        labels = torch.randint(0, 80, (total, k), generator=g)
        ids = torch.randint(0, 1000, (total, k), generator=g)
        counts = torch.randint(0, k + 1, (total,), generator=g).to(torch.int32)
        s, e = fdist.shard_range(total, rank, world)
        rec = fdist.pack_detections(dets[s:e], labels[s:e], ids[s:e], counts[s:e])
        full = fdist.gather_ragged(rec, total)
        d2, l2, i2, c2 = fdist.unpack_detections(full)
        ok = torch.equal(d2, dets) and torch.equal(l2, labels) and torch.equal(i2, ids) and torch.equal(c2, counts)
        if total % world == 0:
            full2 = fdist.gather_records(rec)
            ok = ok and torch.equal(full2, full)
            # gather to one rank: rank 0 gets everything, the others get nothing back
            full3 = fdist.gather_records_to(rec, 0)
            ok = ok and ((rank == 0 and torch.equal(full3, full)) or (rank != 0 and full3 is None))
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


def test_gather_two_ranks_gloo(tmp_path):
    for total in (8, 7):
        port = _free_port()
        mp.spawn(_worker, args=(2, port, total, str(tmp_path)), nprocs=2, join=True)
        for r in range(2):
            assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def _one_sided_worker(rank, world, port, q):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        g = fdist.OneSidedGather((3, 5, fdist.RECORD_WORDS), 2, "cpu", dst=0)
        out = []
        for step in range(4):
            rec = torch.full((3, 5, fdist.RECORD_WORDS), 100 * step + rank, dtype=torch.int32)
            g.push(rec, step % 2)
            g.landed()
            if rank == 0:
                out.append(g.gathered(step % 2).clone())
            else:
                assert g.gathered(step % 2) is None
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


def test_one_sided_gather_host_logic():
    """On gloo / CPU tensors the pushes are plain gathers: every rank's shard ends up in its slot of the destination's
    buffer, buffer after buffer."""
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_one_sided_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for step, full in enumerate(res[0]):
        assert full.shape == (6, 5, 8)
        assert int(full[:3].min()) == int(full[:3].max()) == 100 * step
        assert int(full[3:].min()) == int(full[3:].max()) == 100 * step + 1
    assert res[1] == []
