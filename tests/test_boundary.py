"""The C boundary on a machine without a GPU: the library loads, exports every symbol the
header declares, its host-only entry points agree with the oracle, and everything that needs
a device fails loudly instead of falling back."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oracle import oracle
from relay_b200 import _lib
from relay_b200.types import CudaOptions, ForwardBatch, ModelConfig, SeqChunk, flatten
from tests.helpers import load_fixture
from tests.workloads import c1_inputs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    hdr = open(os.path.join(ROOT, "include", "relay_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b(rb200_[a-z0-9_]+)\s*\(", hdr)))


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 45
    L = C.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/relay_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "the ctypes table and the header list different symbols"


def test_rope_inv_freq_matches_the_oracle():
    # bit for bit without Llama-3 scaling; with it, the interpolated band may differ by one ulp
    # (whether the compiler fuses the multiply-add of that expression is not part of the contract)
    L = _lib.lib()
    for name in ("llama3-rope", "llama-mha", "llama-gqa-tied-bf16"):
        cfg = load_fixture(name)[0].config
        out = np.zeros(cfg.head_dim // 2, np.float32)
        c = cfg.to_c()
        assert L.rb200_rope_inv_freq(C.byref(c), out.ctypes.data_as(C.c_void_p)) == cfg.head_dim // 2
        want = oracle.rope_inv_freq(cfg)
        assert np.array_equal(out, want) if not cfg.rope_scaling_type else np.allclose(out, want, rtol=1.3e-7, atol=0)
    big = ModelConfig(4096, 14336, 32, 32, 8, 128, 128256, rope_theta=500000.0, rope_scaling_type="llama3",
                      rope_factor=8.0, rope_original_max_position=8192.0)
    out = np.zeros(64, np.float32)
    c = big.to_c()
    L.rb200_rope_inv_freq(C.byref(c), out.ctypes.data_as(C.c_void_p))
    assert np.allclose(out, oracle.rope_inv_freq(big), rtol=1.3e-7, atol=0)


def test_host_int8_quantisation_matches_the_oracle_bit_for_bit():
    rng = np.random.Generator(np.random.PCG64(4))
    w = (rng.standard_normal((37, 172)) * 0.02).astype(np.float32)
    w[5] = 0
    w[6, :] = 0.5  # every value is the row maximum
    q, s = np.empty((37, 172), np.int8), np.empty(37, np.float32)
    assert _lib.lib().rb200_quantize_rows_int8(w.ctypes.data_as(C.c_void_p), 37, 172, q.ctypes.data_as(C.c_void_p),
                                               s.ctypes.data_as(C.c_void_p)) == 0
    wq, ws = oracle.quantize_rows_int8(w)
    assert np.array_equal(q, wq) and np.array_equal(s, ws)
    assert s[5] == 1.0 and np.all(q[5] == 0) and np.all(q[6] == 127)


def test_flags_follow_the_reference_environment_switches(monkeypatch):
    L = _lib.lib()
    monkeypatch.delenv("RELAY_CUDA_ATTENTION", raising=False)
    monkeypatch.delenv("RELAY_CUDA_INT8", raising=False)
    assert L.rb200_flags_from_env() == 0 and CudaOptions.from_env().flags() == 0
    monkeypatch.setenv("RELAY_CUDA_ATTENTION", "m0")
    monkeypatch.setenv("RELAY_CUDA_INT8", "1")
    assert L.rb200_flags_from_env() == 3 and CudaOptions.from_env().flags() == 3
    monkeypatch.setenv("RELAY_CUDA_ATTENTION", "m1")
    monkeypatch.setenv("RELAY_CUDA_INT8", "0")
    assert L.rb200_flags_from_env() == 0


def test_scratch_sizes_are_host_computable():
    L = _lib.lib()
    shape = _lib.CAttnShape(32, 8, 128, 16, 6144, 4096)
    # 32 tokens, contexts up to 4096: 8 slices of 512 keys, (D + 2) floats per (token, head, slice)
    assert L.rb200_decode_scratch_bytes(C.byref(shape), 32, 4096) == 32 * 32 * 8 * 130 * 4
    assert L.rb200_gemv_scratch_bytes(4096, 4096) >= 256
    assert L.rb200_kernel_launches() == 0


def test_decode_slice_plan_is_host_computable():
    # (keys per slice, slices per context, bytes of partials) for the benchmark model's head layout
    # on a 148-SM device (the count the planner assumes when no device is present)
    L = _lib.lib()
    if L.rb200_device_count() > 0:
        pytest.skip("the plan follows the SM count of the device that is present")
    shape = _lib.CAttnShape(32, 8, 128, 16, 6144, 4096)

    def plan(n, ctx):
        sl, parts = C.c_int32(0), C.c_int32(0)
        nbytes = L.rb200_decode_plan(C.byref(shape), n, ctx, C.byref(sl), C.byref(parts))
        return sl.value, parts.value, nbytes

    # one or two sequences: 512-key slices, merged on chip as clusters of up to eight
    assert plan(1, 4096) == (512, 8, 0) and plan(2, 4096) == (512, 8, 0) and plan(1, 3000) == (512, 6, 0)
    # three: 192 CTAs of 512 keys, more than the SMs and too few for longer slices: partials and the merge kernel
    assert plan(3, 4096) == (512, 8, 3 * 32 * 8 * 130 * 4)
    # 4 - 16: at most four longer slices per pair, one wave, merged on chip
    assert plan(4, 4096) == (1024, 4, 0) and plan(8, 4096) == (1024, 4, 0)
    assert plan(12, 4096) == (2048, 2, 0) and plan(16, 4096) == (2048, 2, 0)
    # from 17 sequences (136 pairs): one slice per pair
    for n in (17, 32, 64, 256):
        assert plan(n, 4096) == (4096, 1, 0)
    # a slice's table holds 512 block ids: longer contexts are cut evenly and merged from partials
    assert plan(32, 9024) == (4608, 2, 32 * 32 * 2 * 130 * 4)
    assert plan(140, 131072)[:2] == (8192, 16)
    assert L.rb200_kernel_launches() == 0


def test_kv_link_message_plan_is_host_computable():
    from relay_b200.backend import Backend
    bb = 8 * 16 * 128 * 2                       # a Llama-3-8B block: 8 KV heads x 16 keys x 128 x fp16
    layer = 2 * 128 * bb                        # a 2048-token prompt: 128 blocks, K and V
    assert Backend.kv_link_plan(layer, bb, 1, 128) == (1, 1)          # a streamed layer: one message
    assert Backend.kv_link_plan(layer, bb, 32, 128) == (32, 1)        # a finished prompt over such a ring
    assert Backend.kv_link_plan(8 * layer, bb, 32, 128) == (4, 8)     # slots of 8 layers: four messages
    assert Backend.kv_link_plan(5 * layer, bb, 32, 128) == (7, 5)     # 6 x 5 layers + 2
    assert Backend.kv_link_plan(8 * layer, bb, 3, 128) == (1, 3)      # a short range does not fill the slot
    # a layer larger than a slot travels as messages of blocks, layer by layer
    assert Backend.kv_link_plan(4 * 2 * bb, bb, 2, 19) == (10, 0)
    # more blocks than ride in one kernel's parameters (480): also cut by blocks, whatever the slot
    assert Backend.kv_link_plan(4096 * 2 * bb, bb, 1, 1000) == (3, 0)
    assert Backend.kv_link_plan(layer, bb, 32, 0) == (0, 0)
    for bad in ((bb, bb, 1, 1), (layer + 1, bb, 1, 1), (layer, 0, 1, 1), (layer, bb, 0, 1), (layer, bb, 1, -1)):
        with pytest.raises(ValueError):
            Backend.kv_link_plan(*bad)
    assert _lib.lib().rb200_kernel_launches() == 0


@pytest.mark.skipif(_lib.lib().rb200_device_count() > 0, reason="a CUDA device is present")
def test_no_cpu_fallback_without_a_device():
    from relay_b200.backend import make_cuda_backend
    with pytest.raises(_lib.B200Error, match="no CUDA device"):
        make_cuda_backend(c1_inputs()[0], 16, 16)
    L = _lib.lib()
    assert L.rb200_f32_to_f16(None, None, 16, None) == -1
    assert b"CUDA" in L.rb200_last_error()
    assert L.rb200_last_error_kind() == _lib.ERR_RUNTIME


def test_create_rejects_bad_configs_before_touching_a_device():
    from relay_b200.backend import Backend
    bad = ModelConfig(hidden=64, intermediate=64, layers=1, heads=3, kv_heads=2, head_dim=16, vocab=8)
    with pytest.raises(ValueError, match="multiple of num_key_value_heads"):
        Backend(bad, None, 4, 16)
    odd = ModelConfig(hidden=64, intermediate=64, layers=1, heads=2, kv_heads=2, head_dim=15, vocab=8)
    with pytest.raises(ValueError, match="head_dim must be even"):
        Backend(odd, None, 4, 16)
    small = ModelConfig(hidden=64, intermediate=64, layers=1, heads=1, kv_heads=1, head_dim=2, vocab=8)
    with pytest.raises(ValueError, match="multiple of 16 bytes"):
        Backend(small, None, 4, 1)


def test_flatten_is_the_reference_batch_walk():
    b = ForwardBatch([SeqChunk([1, 2, 3], 4, [9, 8]), SeqChunk([7], 20, [1, 2, 3], want_logits=False), SeqChunk([], 0, [])])
    fb = flatten(b)
    assert fb.tokens.tolist() == [1, 2, 3, 7] and fb.chunk_len.tolist() == [3, 1, 0]
    assert fb.start_pos.tolist() == [4, 20, 0] and fb.table_len.tolist() == [2, 3, 0]
    assert fb.tables.tolist() == [9, 8, 1, 2, 3] and fb.n_rows == 1
    b.all_logits = True
    assert flatten(b).n_rows == 4
