"""Sequence sharding across the GPUs of one box and the hand-shake of the NCCL KV hop.

The per-token path shards by sequence only (each GPU is a full replica with its own KV pool,
relay's worker model: scripts/cluster.sh:26-48 of the reference); there is no data-path
collective. What ranks exchange is host-side and small: which sequences each one owns, the
tokens they produced, and the NCCL unique id of a prefill/decode pair. This module does that
over any torch.distributed backend (gloo on CPU in the tests, nccl on the box).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_range(n_items: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) of `n_items` owned by `rank`: sizes differ by at most one and
    the ranges of all ranks tile [0, n_items) in rank order."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    base, extra = divmod(n_items, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def owner_of(item: int, n_items: int, world: int) -> int:
    """The rank whose shard_range contains `item`."""
    if not 0 <= item < n_items:
        raise ValueError("item out of range")
    base, extra = divmod(n_items, world)
    cut = extra * (base + 1)
    return item // (base + 1) if item < cut else extra + (item - cut) // base


def gather_in_order(local: Sequence[int], n_items: int, group=None) -> List[int]:
    """All ranks' per-sequence results concatenated in sequence order (every rank gets them)."""
    world = dist.get_world_size(group)
    parts: List[list] = [None] * world  # type: ignore[list-item]
    dist.all_gather_object(parts, list(local), group=group)
    out = [x for p in parts for x in p]
    if len(out) != n_items:
        raise RuntimeError(f"gathered {len(out)} results for {n_items} sequences")
    return out


def max_over_ranks(value: float, device=None, group=None) -> float:
    """The slowest rank's time: the number a multi-GPU measurement reports."""
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def broadcast_bytes(payload: bytes, n: int, src: int, device=None, group=None) -> bytes:
    """`n` bytes from rank `src` to every rank (the NCCL unique id of a KV-hop pair; in relay
    it would ride in the Hello frame of the transfer connection)."""
    buf = torch.zeros(n, dtype=torch.uint8, device=device)
    if dist.get_rank(group) == src:
        if len(payload) != n:
            raise ValueError("payload size")
        buf.copy_(torch.frombuffer(bytearray(payload), dtype=torch.uint8))
    dist.broadcast(buf, src=src, group=group)
    return bytes(buf.cpu().numpy().tobytes())
