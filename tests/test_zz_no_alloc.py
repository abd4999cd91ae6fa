"""The decode-attention entry point that brings its own scratch (rb200_decode_attention_static).

Some callers cannot allocate device memory at the point where they need attention: the GPU's
free memory already belongs to their KV pool, or their loop cannot afford the device-wide
stall of an allocation. For them the library keeps the split-context partials in a fixed
array of its own. This file checks, through the C boundary, that the entry point gives the
same output as rb200_decode_attention (which takes the scratch from the caller) on two calls
in a row with different batches (so the second call runs over whatever the first one left
in the shared array), that both agree with the CPU checker (the two entry points share their
kernels, so agreeing with each other proves little on its own), that a batch whose partials
really exceed the array is refused with a clear error, and that a batch which only looks too
large by the 512-key upper bound is served. It is named to be collected last.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle  # noqa: E402  (the checker: tests only)
from tests.workloads import WideDecodeCase, paged_attention_case  # noqa: E402

ATTN_TOL = 3e-3  # the decode-attention tolerance of tests/test_gpu_ops.py


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def _row_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float((np.abs(a - b).max(1) / np.maximum(np.abs(b).max(1), 1e-6)).max())


def _run_both(ops, seed, ctxs, heads, kv_heads, D, bs):
    nb = sum((c + bs - 1) // bs for c in ctxs) + 3
    c = paged_attention_case(seed, ctxs, [1] * len(ctxs), heads, kv_heads, D, bs, nb)
    T = len(ctxs)
    shape = ops.attn_shape(heads, kv_heads, D, bs)
    meta = ops.TokenMeta.from_host(c["pos"], c["seq"], c["table_off"], c["tables"])
    q, kp, vp = _dev(c["q"]), _dev(c["k_pool"], torch.float16), _dev(c["v_pool"], torch.float16)
    toks = _dev(np.arange(T, dtype=np.int32))
    want = torch.zeros((T, heads * D), dtype=torch.float16, device="cuda")
    got = torch.zeros_like(want)
    ops.decode_attention(shape, q, meta, toks, max(ctxs), kp, vp, want)           # caller-owned scratch
    ops.decode_attention_static(shape, q, meta, toks, max(ctxs), kp, vp, got)     # the library's own array
    torch.cuda.synchronize()
    assert ops.decode_plan(shape, T, max(ctxs))[2] > 0  # the scratch is really used
    cpu = oracle.attention(c["q"], c["q"].shape[1], c["pos"], c["seq"], c["table_off"], c["tables"], c["k_pool"], c["v_pool"],
                           heads, kv_heads, D, bs)
    return got.cpu().numpy().astype(np.float32), want.cpu().numpy().astype(np.float32), cpu


def test_static_scratch_entry_point_matches_the_caller_scratch_one_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from relay_b200 import ops
    # both batches park partial results: 3 sequences in eight 512-key slices each (192 CTAs: more
    # than the SMs, so no cluster merges them on chip, and too few for the longer slices of the
    # one-wave rule), and 3 sequences of another model in ten
    got1, want1, cpu1 = _run_both(ops, 41, [4096, 700, 2048], 32, 8, 128, 16)
    got2, want2, cpu2 = _run_both(ops, 42, [600, 4700, 33], 8, 2, 64, 16)  # smaller: runs over the first call's leftovers
    for got, want, cpu in ((got1, want1, cpu1), (got2, want2, cpu2)):
        assert np.isfinite(got).all()
        assert _row_err(got, want) < ATTN_TOL
        assert np.array_equal(got, want)  # same kernels, same order of operations
        assert _row_err(got, cpu) < ATTN_TOL  # and both are right, not just alike


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from relay_b200 import _lib, ops
    shape = ops.attn_shape(32, 8, 128, 16)
    # 140 tokens leave room for two slices per context, and 131072 keys are sixteen of the largest
    # slice (512 table entries = 8192 keys): 16 slices x 140 x 32 heads x 130 floats = 37 MB
    n, ctx = 140, 131072
    _, parts, need = ops.decode_plan(shape, n, ctx)
    assert parts > 1 and need > _lib.STATIC_DECODE_SCRATCH_BYTES
    z = torch.zeros(16, device="cuda")
    meta = ops.TokenMeta(*(torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(4)))
    with pytest.raises(ValueError, match="built-in buffer holds 8388608"):
        ops.decode_attention_static(shape, z, meta, torch.zeros(n, dtype=torch.int32, device="cuda"), ctx, z, z, z)


def test_static_scratch_entry_point_serves_a_large_batch_that_needs_no_partials():
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from relay_b200 import _lib, ops
    # 160 tokens x 8 KV heads fill the GPU with one 2048-key slice per pair: nothing is parked,
    # although the 512-key upper bound (160 x 32 x 4 x 130 floats = 10.6 MB) is above the array.
    heads, kv_heads, D, bs, n, ctx = 32, 8, 128, 16, 160, 2048
    shape = ops.attn_shape(heads, kv_heads, D, bs)
    assert ops.decode_scratch_bytes(shape, n, ctx) > _lib.STATIC_DECODE_SCRATCH_BYTES
    assert ops.decode_plan(shape, n, ctx)[1:] == (1, 0)
    case = WideDecodeCase(9, n, ctx, heads, kv_heads, D, bs)
    k16, v16 = case.pools16()
    meta = ops.TokenMeta.from_host(case.pos, case.seq, case.table_off, case.tables)
    out = torch.zeros((n, heads * D), dtype=torch.float16, device="cuda")
    ops.decode_attention_static(shape, _dev(case.q), meta, _dev(np.arange(n, dtype=np.int32)), ctx, _dev(k16), _dev(v16), out)
    torch.cuda.synchronize()
    got = out.cpu().numpy().astype(np.float32)
    for g in range(n // case.group):
        c = case.group_case(g)
        cpu = oracle.attention(c["q"], c["q"].shape[1], c["pos"], c["seq"], c["table_off"], c["tables"], c["k_pool"],
                               c["v_pool"], heads, kv_heads, D, bs)
        assert _row_err(got[g * case.group:(g + 1) * case.group], cpu) < ATTN_TOL
