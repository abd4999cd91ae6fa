"""The multi-GPU host logic on CPU: two gloo ranks shard sequences, gather results in order,
reduce a time to the slowest rank and pass the KV hop's id bytes."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from relay_b200.parallel import broadcast_bytes, gather_in_order, max_over_ranks, owner_of, shard_range


def test_shards_tile_the_sequences():
    for n in (0, 1, 7, 8, 255, 256, 257):
        for world in (1, 2, 3, 4, 8):
            covered = []
            for r in range(world):
                b, e = shard_range(n, world, r)
                assert 0 <= b <= e <= n and e - b in (n // world, n // world + 1)
                covered += list(range(b, e))
                for i in range(b, e):
                    assert owner_of(i, n, world) == r
            assert covered == list(range(n))
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n = 11
        b, e = shard_range(n, world, rank)
        tokens = [100 + i for i in range(b, e)]  # what this rank's replica would have generated
        q.put((rank, "gather", gather_in_order(tokens, n)))
        q.put((rank, "max", max_over_ranks(1.5 + rank)))
        uid = bytes(range(128)) if rank == 1 else b""
        q.put((rank, "uid", broadcast_bytes(uid, 128, src=1)))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_gather_and_reduce():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=120) for _ in range(6)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, kind, val in got:
        if kind == "gather":
            assert val == [100 + i for i in range(11)]
        elif kind == "max":
            assert val == 2.5
        else:
            assert val == bytes(range(128))
