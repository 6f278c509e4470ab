"""Batch sharding across the GPUs of one box and the one exchange step of the path: gathering final detections.

Images (and LSTM sequences) are independent, so a batch is split into contiguous shards, one per rank, with no
data-path collective; only the fixed-capacity detection records of the last kernel are gathered: to one rank
(gather_records_to) or to all of them (gather_records), NCCL over NVLink on GPUs; the same code runs on gloo / CPU
tensors, which is how the host logic is tested.
"""
from typing import List, Tuple

import torch
import torch.distributed as dist

RECORD_WORDS = 8  # x1, y1, x2, y2, score (fp32 bits), label, flat id, valid flag  -- 32 bytes per detection


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous split of `total` items; the first total % world ranks get one extra item."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def pack_detections(dets: torch.Tensor, labels: torch.Tensor, flat_ids: torch.Tensor, counts: torch.Tensor,
                    out: torch.Tensor = None) -> torch.Tensor:
    """[B,K,5] fp32 + [B,K] int64 + [B,K] int64 + [B] int32 -> [B,K,8] int32 records (bit-preserving)."""
    b, k, _ = dets.shape
    rec = out if out is not None else torch.empty(b, k, RECORD_WORDS, dtype=torch.int32, device=dets.device)
    if dets.is_cuda:  # one launch of the library's pack kernel on the current stream
        from ._lib import check, lib
        if not (dets.is_contiguous() and labels.is_contiguous() and flat_ids.is_contiguous() and rec.is_contiguous()
                and counts.is_contiguous() and counts.dtype == torch.int32):
            raise ValueError("pack_detections: contiguous tensors (counts int32) expected")
        check(lib.functs_b200_pack_detections(dets.data_ptr(), labels.data_ptr(), flat_ids.data_ptr(), counts.data_ptr(), b, k,
                                              rec.data_ptr(), torch.cuda.current_stream(dets.device).cuda_stream),
              "pack_detections")
        return rec
    rec[:, :, 0:5] = dets.view(torch.int32)
    rec[:, :, 5] = labels.to(torch.int32)
    rec[:, :, 6] = flat_ids.to(torch.int32)
    rec[:, :, 7] = (torch.arange(k, device=dets.device)[None, :] < counts[:, None]).to(torch.int32)
    return rec


def unpack_detections(rec: torch.Tensor):
    """Inverse of pack_detections -> (dets [B,K,5], labels [B,K] int64, flat_ids [B,K] int64, counts [B] int32)."""
    dets = rec[:, :, 0:5].contiguous().view(torch.float32)
    labels = rec[:, :, 5].to(torch.int64)
    flat_ids = rec[:, :, 6].to(torch.int64)
    counts = rec[:, :, 7].sum(dim=1).to(torch.int32)
    return dets, labels, flat_ids, counts


def gather_records(rec: torch.Tensor, group=None, out: torch.Tensor = None) -> torch.Tensor:
    """All-gather of equally sized record shards along the batch dimension -> [world * B, K, 8] on every rank."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return rec
    world = dist.get_world_size(group)
    full = out if out is not None else torch.empty((world * rec.size(0),) + tuple(rec.shape[1:]), dtype=rec.dtype,
                                                   device=rec.device)
    if dist.get_backend(group) == "gloo":
        parts = list(full.chunk(world, dim=0))
        dist.all_gather(parts, rec.contiguous(), group=group)
    else:
        dist.all_gather_into_tensor(full, rec.contiguous(), group=group)
    return full


def gather_records_to(rec: torch.Tensor, dst: int = 0, group=None, out: torch.Tensor = None):
    """Gather of equally sized record shards to ONE rank: -> [world * B, K, 8] on rank `dst`, None on the others.
    "Only the final detections are gathered": the other ranks just send their 32-byte records (NCCL send / recv pairs
    over NVLink; the same code runs on gloo / CPU tensors).  `out` is only used on `dst`."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return rec
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    rec = rec.contiguous()
    if rank != dst:
        dist.gather(rec, None, dst=dst, group=group)
        return None
    full = out if out is not None else torch.empty((world * rec.size(0),) + tuple(rec.shape[1:]), dtype=rec.dtype,
                                                   device=rec.device)
    dist.gather(rec, list(full.chunk(world, dim=0)), dst=dst, group=group)
    return full


def gather_ragged(rec: torch.Tensor, total: int, group=None) -> torch.Tensor:
    """All-gather of shards made by shard_range (sizes may differ by one): pads to the largest shard, trims after."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return rec
    world = dist.get_world_size(group)
    sizes = [shard_range(total, r, world) for r in range(world)]
    cap = max(e - s for s, e in sizes)
    padded = torch.zeros((cap,) + tuple(rec.shape[1:]), dtype=rec.dtype, device=rec.device)
    padded[:rec.size(0)] = rec
    full = gather_records(padded, group)
    parts: List[torch.Tensor] = [full[r * cap:r * cap + (e - s)] for r, (s, e) in enumerate(sizes)]
    return torch.cat(parts, dim=0)



class OneSidedGather:
    """Gather of equally sized record shards to ONE rank without a kernel on either side: the destination rank owns
    `n_buffers` buffers [world * B, K, 8], the other ranks of the box open them through CUDA IPC handles and push their shard
    into their slot with an asynchronous copy (copy engine over NVLink, functs_b200_push_records).  NCCL's send / receive
    kernels need streaming multiprocessors that a bandwidth-bound kernel in flight has filled; a copy engine does not.
    `landed()` is one small all-reduce: when it has completed on a rank, every push that any rank issued before its own
    call (on the same stream) has arrived.  CUDA tensors on the GPUs of one box only; on gloo / CPU tensors (the host-side
    tests) the pushes are plain gathers.

    Setting it up is collective (every rank of the group must construct it with the same arguments)."""

    def __init__(self, shard_shape, n_buffers: int, device, dst: int = 0, group=None):
        self.group, self.dst = group, dst
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.shard_shape = tuple(shard_shape)
        self.device = torch.device(device)
        self.on_gpu = self.device.type == "cuda"
        full_shape = (self.world * self.shard_shape[0],) + self.shard_shape[1:]
        self.shard_bytes = 4
        for d in self.shard_shape:
            self.shard_bytes *= int(d)
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.buffers = None   # on dst: the owned buffers; elsewhere: the same memory, opened through IPC
        if self.rank == dst:
            self.buffers = [torch.empty(full_shape, dtype=torch.int32, device=self.device) for _ in range(n_buffers)]
        if not self.on_gpu:
            return
        if self.shard_bytes % 16 != 0:
            raise ValueError("OneSidedGather: a shard must be a multiple of 16 bytes")
        from torch.multiprocessing.reductions import reduce_tensor
        payload = [[reduce_tensor(b) for b in self.buffers] if self.rank == dst else None]
        dist.broadcast_object_list(payload, src=dst, group=group)
        problem = ""
        if self.rank != dst:
            try:
                self.buffers = [fn(*args) for fn, args in payload[0]]
                for b in self.buffers:
                    if tuple(b.shape) != full_shape or b.dtype != torch.int32 or not b.is_contiguous():
                        problem = "the opened buffer does not look like the destination's"
            except Exception as exc:  # noqa: BLE001 - every rank must learn of it, or the others would wait for ever
                problem = f"{type(exc).__name__}: {exc}"
        # every rank has opened the handles (or none goes on): the failure of one is the failure of all
        ok = torch.tensor([0 if problem else 1], dtype=torch.int32, device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            raise RuntimeError("OneSidedGather: a rank could not open the destination's buffers" + (f" ({problem})" if problem else ""))

    def push(self, rec: torch.Tensor, buffer: int) -> None:
        """Enqueues, on the current stream, the copy of this rank's shard into its slot of buffer `buffer` on the destination."""
        if tuple(rec.shape) != self.shard_shape or rec.dtype != torch.int32 or not rec.is_contiguous():
            raise ValueError("OneSidedGather.push: a contiguous int32 tensor of the shard shape is expected")
        if not self.on_gpu:
            parts = list(self.buffers[buffer].chunk(self.world, dim=0)) if self.rank == self.dst else None
            dist.gather(rec, parts, dst=self.dst, group=self.group)
            return
        from ._lib import check, lib
        target = self.buffers[buffer].data_ptr() + self.rank * self.shard_bytes
        check(lib.functs_b200_push_records(target, rec.data_ptr(), self.shard_bytes,
                                           torch.cuda.current_stream(rec.device).cuda_stream), "push_records")

    def landed(self) -> None:
        """One small collective on the current stream: behind it, every push issued before it by any rank has arrived."""
        dist.all_reduce(self._token, group=self.group)

    def gathered(self, buffer: int):
        """The destination's buffer (None on the other ranks)."""
        return self.buffers[buffer] if self.rank == self.dst else None
