"""Two GPUs of one box: the prefill -> decode KV hop over NCCL, and sequence-sharded replicas.

Rank 0 prefills a prompt and streams every layer's blocks to rank 1 from inside the forward
pass (the layer callback enqueues gather -> ncclSend on the copy stream, ordered behind the
layer's event), rank 1 receives them into different block ids and decodes; the result must
equal, bit for bit, rank 0 decoding on its own cache (the reference's
"disaggregated == colocated", tests/test_transfer.cpp:236-330, with NVLink in place of the
socket). Skipped on boxes with one GPU.
"""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _hop_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from relay_b200.backend import Backend, make_cuda_backend
    from relay_b200.parallel import broadcast_bytes
    from relay_b200.types import ForwardBatch, SeqChunk
    from tests.test_gpu_model import WIDE_CONFIGS, synthetic
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.cuda.set_device(rank)
        cfg = WIDE_CONFIGS["d128_g4"]
        w = synthetic(cfg, 12)
        be = make_cuda_backend(w, 64, 16, device=rank, max_batch_tokens=512)
        uid = Backend.nccl_unique_id() if rank == 0 else b""
        uid = broadcast_bytes(uid, 128, src=0)
        be.nccl_init(uid, world, rank)
        rng = np.random.Generator(np.random.PCG64(21))
        prompt = rng.integers(0, cfg.vocab, 300).tolist()
        src_blocks = list(range(3, 3 + 19))          # the prefill side's block ids
        dst_blocks = list(range(40, 40 + 19))[::-1]  # the decode side's own, different ids
        if rank == 0:
            first = be.forward(ForwardBatch([SeqChunk(prompt, 0, src_blocks + [30])]),
                               observer=lambda layer: be.send_kv_layer(1, layer, src_blocks))
            be.kv_hop_sync(20000)
            tok = int(np.argmax(first[0]))
            dist.broadcast_object_list([tok], src=0)
            table = src_blocks + [30]
        else:
            for layer in range(cfg.layers):
                be.recv_kv_layer(0, layer, dst_blocks)
            be.kv_hop_sync(20000)
            box = [None]
            dist.broadcast_object_list(box, src=0)
            tok = box[0]
            table = dst_blocks + [33]
        toks, rows = [], []
        for s in range(6):
            row = be.forward(ForwardBatch([SeqChunk([tok], 300 + s, table)]))[0]
            rows.append(row)
            tok = int(np.argmax(row))
            toks.append(tok)
        pages = [be.read_kv_layer(l, table[:19]) for l in range(cfg.layers)]
        be.nccl_finalize()
        q.put((rank, toks, np.stack(rows), [p.tobytes() for p in pages]))
    finally:
        dist.destroy_process_group()


def test_kv_hop_over_nccl_equals_colocated_decode():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_hop_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        rank, toks, rows, pages = q.get(timeout=300)
        got[rank] = (toks, rows, pages)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert got[0][0] == got[1][0]                    # same greedy tokens
    assert np.array_equal(got[0][1], got[1][1])      # same logits, bit for bit
    assert got[0][2] == got[1][2]                    # the pages that crossed NVLink are byte-identical


def _replica_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from relay_b200.backend import make_cuda_backend
    from relay_b200.parallel import gather_in_order, shard_range
    from relay_b200.types import ForwardBatch, SeqChunk
    from tests.workloads import c1_inputs
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.cuda.set_device(rank)
        w, _, _ = c1_inputs()
        be = make_cuda_backend(w, 64, 16, device=rank)
        rng = np.random.Generator(np.random.PCG64(5))
        prompts = [rng.integers(0, 256, int(n)).tolist() for n in rng.integers(5, 40, 7)]
        b, e = shard_range(len(prompts), world, rank)
        mine = []
        for i in range(b, e):  # each rank serves its own sequences in its own pool, no collective
            lg = be.forward(ForwardBatch([SeqChunk(prompts[i], 0, [2 * (i - b), 2 * (i - b) + 1, 20 + i])]))
            mine.append(int(np.argmax(lg[0])))
        q.put((rank, gather_in_order(mine, len(prompts))))
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_replicas_equal_one_gpu():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from relay_b200.backend import make_cuda_backend
    from relay_b200.types import ForwardBatch, SeqChunk
    from tests.workloads import c1_inputs
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_replica_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    w, _, _ = c1_inputs()
    be = make_cuda_backend(w, 64, 16)
    rng = np.random.Generator(np.random.PCG64(5))
    prompts = [rng.integers(0, 256, int(n)).tolist() for n in rng.integers(5, 40, 7)]
    want = [int(np.argmax(be.forward(ForwardBatch([SeqChunk(p, 0, [0, 1, 2])]))[0])) for p in prompts]
    assert got[0][1] == want and got[1][1] == want


def test_one_process_drives_backends_on_two_devices():
    # Kernel attributes (the dynamic shared-memory limit) belong to the device that was current
    # when they were set: a process with a backend on each of two GPUs must raise them on both.
    # Every kernel family runs on each device: tcgen05 prefill and GEMMs (D 128, 300-token
    # prompt), the split decode, the int8 few-token GEMM.
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from relay_b200.backend import make_cuda_backend
    from relay_b200.types import CudaOptions, ForwardBatch, SeqChunk
    from tests.test_gpu_model import WIDE_CONFIGS, synthetic
    cfg = WIDE_CONFIGS["d128_g4"]
    w = synthetic(cfg, 12)
    rng = np.random.Generator(np.random.PCG64(2))
    prompt = rng.integers(0, cfg.vocab, 300).tolist()
    table = list(range(20))
    for int8 in (False, True):
        rows = []
        for dev in (1, 0):  # the second device first: nothing has configured it yet
            be = make_cuda_backend(w, 64, 16, device=dev, max_batch_tokens=512, options=CudaOptions(int8_weights=int8))
            first = be.forward(ForwardBatch([SeqChunk(prompt, 0, table)]))
            step = be.forward(ForwardBatch([SeqChunk([int(np.argmax(first[0]))], 300, table)]))
            rows.append((first, step))
            be.close()
        assert np.array_equal(rows[0][0], rows[1][0]) and np.array_equal(rows[0][1], rows[1][1])


def _link_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from relay_b200 import _lib
    from relay_b200.backend import make_cuda_backend
    from relay_b200.types import ForwardBatch, SeqChunk
    from tests.test_gpu_model import WIDE_CONFIGS, synthetic
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.cuda.set_device(rank)
        cfg = WIDE_CONFIGS["d128_g4"]
        w = synthetic(cfg, 12)
        be = make_cuda_backend(w, 128, 16, device=rank, max_batch_tokens=512)
        # a ring of 3 slots of 4 blocks each: the 19-block layers travel as 5 messages, and the
        # 2 layers x 5 messages wrap the ring, so slot reuse behind the receiver's acknowledgements runs
        slot = 4 * 2 * be.kv_block_bytes()
        link, handle = be.kv_link_create(3, slot)
        handles = [None, None]
        dist.all_gather_object(handles, handle)
        be.kv_link_connect(link, handles[1 - rank])
        rng = np.random.Generator(np.random.PCG64(21))
        prompt = rng.integers(0, cfg.vocab, 300).tolist()
        src_blocks = list(range(3, 3 + 19))
        dst_blocks = list(range(40, 40 + 19))[::-1]
        if rank == 0:
            first = be.forward(ForwardBatch([SeqChunk(prompt, 0, src_blocks + [30])]),
                               observer=lambda layer: be.kv_link_send_layer(link, layer, src_blocks))
            be.kv_hop_sync(20000)
            tok = int(np.argmax(first[0]))
            dist.broadcast_object_list([tok], src=0)
            table = src_blocks + [30]
        else:
            for layer in range(cfg.layers):
                be.kv_link_recv_layer(link, layer, dst_blocks)
            be.kv_hop_sync(20000)
            box = [None]
            dist.broadcast_object_list(box, src=0)
            tok = box[0]
            table = dst_blocks + [33]
        toks, rows = [], []
        for s in range(6):
            row = be.forward(ForwardBatch([SeqChunk([tok], 300 + s, table)]))[0]
            rows.append(row)
            tok = int(np.argmax(row))
            toks.append(tok)
        pages = [be.read_kv_layer(l, table[:19]) for l in range(cfg.layers)]
        # the same request once more as a finished one: both layers in one message over a second
        # link whose slots hold two layers, into blocks nothing has written
        link2, handle2 = be.kv_link_create(2, 2 * 19 * 2 * be.kv_block_bytes())
        handles2 = [None, None]
        dist.all_gather_object(handles2, handle2)
        be.kv_link_connect(link2, handles2[1 - rank])
        if rank == 0:
            be.kv_link_send_layers(link2, 0, cfg.layers, src_blocks)
            be.kv_hop_sync(20000)
            pages2 = pages
        else:
            far = list(range(100, 119))
            be.kv_link_recv_layers(link2, 0, cfg.layers, far)
            be.kv_hop_sync(20000)
            pages2 = [be.read_kv_layer(l, far) for l in range(cfg.layers)]
        dist.barrier()
        be.kv_link_close(link2)
        # A receive nothing sends: the wait must run out on the host, the link is then refused,
        # and the backend goes on working (no GPU wait is left spinning).
        timed_out = refused = False
        if rank == 1:
            be.kv_link_recv_layer(link, 0, [60, 61])  # blocks no sequence uses
            try:
                be.kv_hop_sync(1500)
            except _lib.B200Error as e:
                timed_out = "timed out" in str(e)
            try:
                be.kv_link_recv_layer(link, 0, [60, 61])
            except _lib.B200Error as e:
                refused = "broken" in str(e)
        after = be.forward(ForwardBatch([SeqChunk([toks[-1]], 306, table)]))[0]
        dist.barrier()
        q.put((rank, toks, np.stack(rows), [p.tobytes() for p in pages], timed_out, refused, bool(np.isfinite(after).all()),
               [p.tobytes() for p in pages2]))
    finally:
        dist.destroy_process_group()


def test_kv_link_hop_equals_colocated_decode_and_its_waits_are_bounded():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_link_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        item = q.get(timeout=300)
        got[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert got[0][0] == got[1][0]                    # same greedy tokens
    assert np.array_equal(got[0][1], got[1][1])      # same logits, bit for bit
    assert got[0][2] == got[1][2]                    # the pages that crossed NVLink are byte-identical
    assert got[1][3] and got[1][4]                   # the unmatched receive timed out; the link is then refused
    assert got[0][5] and got[1][5]                   # both backends still compute
    assert got[0][6] == got[1][6]                    # the layer-range message landed the same bytes
