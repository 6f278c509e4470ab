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

