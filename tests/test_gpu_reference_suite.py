"""relay's own test programs, unmodified, on the B200 backend.

oracle/Makefile (`make reftests`) links the reference's tests/test_*.cpp against its engine
sources minus cuda_backend.cu, plus relay_b200/csrc/adapter.cpp and librelay_b200.so, into
oracle/_ref/bin/. With RELAY_TEST_BACKEND=cuda (tests/check.h:57-73 of the reference) every
model test in them runs through relay::make_cuda_backend, i.e. through this repository's
kernels. The binaries exist only where the reference checkout was present at build time.
"""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "bin")

# what each program pins on the path (the reference's files):
PROGRAMS = {
    "test_reference": "logits at every prompt position and 8 greedy steps against transformers, five fixtures",
    "test_batching": "batched == alone, chunked == whole, preemption, block sizes 1 and 32, prefix caching",
    "test_kv_cache": "KV blocks copied to another backend under other block ids decode identically",
    "test_attention": "fast kernels against the simple kernel over prompts 1..1300, chunked, mixed batches; int8 vs fp16",
    "test_transfer": "layer callbacks in order; disaggregated == colocated over TCP and shm; memory pressure; lost sender",
    "test_c_api": "C API tokens/logprobs, weight reload, resume, update_tensor",
}


@pytest.mark.parametrize("prog", list(PROGRAMS))
def test_reference_program_passes_on_the_b200_backend(prog):
    exe = os.path.join(BIN, prog)
    if not os.path.exists(exe):
        pytest.skip("relay's test programs were not built here (needs the reference checkout: make -C oracle reftests)")
    env = dict(os.environ, RELAY_TEST_BACKEND="cuda")
    r = subprocess.run([exe], cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "0 failed" in tail, tail


@pytest.mark.parametrize("devices", ["0,0", "0,1"])
def test_relays_transfer_engine_over_a_kv_link(devices):
    """tests/cpp/test_kv_link_transfer.cpp: relay's KVSender / KVReceiver / PrefillWorker / Engine,
    unmodified, with the Layer payloads on a K/V link (include/relay_b200_transfer.h): tokens equal
    one engine's, dropped frames, host-injected connection cuts. "0,0": both backends on one GPU;
    "0,1": prefill on GPU 0, decode on GPU 1 (skipped on a one-GPU box)."""
    exe = os.path.join(BIN, "test_kv_link_transfer")
    if not os.path.exists(exe):
        pytest.skip("not built here (needs the reference checkout: make -C oracle reftests)")
    if devices == "0,1":
        import torch
        if torch.cuda.device_count() < 2:
            pytest.skip("needs two GPUs")
    # A link orders its streams by counters the CUDA scheduler cannot see. With both ends on one
    # device, two of their streams may share a hardware queue, and a wait enqueued ahead of the work
    # that satisfies it would then hold that work back until the link's host deadline: give every
    # stream a queue of its own (two devices, the real use, have separate queues anyway).
    env = dict(os.environ, RB200_LINK_DEVICES=devices, CUDA_DEVICE_MAX_CONNECTIONS="32")
    r = subprocess.run([exe], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "\n0 failed" in tail, tail
