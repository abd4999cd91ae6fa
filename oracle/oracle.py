"""TEST INFRASTRUCTURE: ctypes faces of the two checkers.

`lib()` is this repo's plain-C restatement (oracle/relay_oracle.c); `ref_lib()` is relay's
own CPU backend compiled from its sources (oracle/_ref/librelay_ref.so, present only
where oracle/Makefile's `ref` target was built). Only tests/, __graft_entry__.smoke() and
bench.py's CPU-baseline legs import this module; the product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional

import numpy as np

from relay_b200.types import (CLayerWeights, CModelConfig, CWeights, FlatBatch, ForwardBatch, HostWeights,
                              ModelConfig, flatten, ptr)

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "librelay_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "librelay_ref.so")

_lib = None
_ref = None


def reference_root() -> Optional[str]:
    """The relay checkout to compile the reference checker from: $RELAY_REFERENCE, else a
    directory named `reference` beside this repository; None where neither holds relay's sources."""
    for cand in (os.environ.get("RELAY_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "engine", "src")):
            return cand
    return None


def build(reference: bool = True) -> None:
    """Compiles the restatement, and relay's CPU backend too where its sources are present."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    ref_root = reference_root()
    if reference and ref_root:
        subprocess.run(["make", "-s", "-j8", "-C", HERE, "ref", f"REF={ref_root}"], check=True)
        if os.path.exists(os.path.join(os.path.dirname(HERE), "relay_b200", "librelay_b200.so")):
            # relay's own test programs linked against the B200 backend (tests/test_gpu_reference_suite.py)
            subprocess.run(["make", "-s", "-j8", "-C", HERE, "reftests", f"REF={ref_root}"], check=True)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build(reference=False)
        L = C.CDLL(ORACLE_SO)
        L.ro_f32_to_f16.restype = C.c_uint16
        L.ro_f32_to_f16.argtypes = [C.c_float]
        L.ro_f16_to_f32.restype = C.c_float
        L.ro_f16_to_f32.argtypes = [C.c_uint16]
        L.ro_dot.restype = C.c_float
        L.ro_model_new.restype = C.c_void_p
        L.ro_model_new.argtypes = [C.POINTER(CModelConfig), C.POINTER(CWeights), C.c_int, C.c_int]
        L.ro_model_free.argtypes = [C.c_void_p]
        L.ro_kv_block_bytes.restype = C.c_size_t
        L.ro_kv_block_bytes.argtypes = [C.c_void_p]
        L.ro_forward.restype = C.c_int
        L.ro_forward.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 6 + [C.c_int, C.c_void_p, C.c_size_t]
        L.ro_read_kv_block.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.ro_write_kv_block.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.ro_uniform01.restype = C.c_double
        L.ro_uniform01.argtypes = [C.c_uint64, C.c_uint64]
        L.ro_sample.restype = C.c_int
        L.ro_sample.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_int, C.c_uint64, C.c_uint64, C.c_void_p]
        L.ro_set_threads.restype = C.c_int
        L.ro_set_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def have_ref() -> bool:
    return os.path.exists(REF_SO)


def ref_lib() -> C.CDLL:
    global _ref
    if _ref is None:
        R = C.CDLL(REF_SO)
        R.ref_last_error.restype = C.c_char_p
        R.ref_create.restype = C.c_void_p
        R.ref_create.argtypes = [C.POINTER(CModelConfig), C.POINTER(CWeights), C.c_int, C.c_int]
        R.ref_load.restype = C.c_void_p
        R.ref_load.argtypes = [C.c_char_p, C.c_int, C.c_int]
        R.ref_destroy.argtypes = [C.c_void_p]
        R.ref_get_config.argtypes = [C.c_void_p, C.POINTER(CModelConfig)]
        R.ref_tensor.restype = C.POINTER(C.c_float)
        R.ref_tensor.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_longlong)]
        R.ref_forward.restype = C.c_int
        R.ref_forward.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 6 + [C.c_int, C.c_void_p, C.c_size_t]
        R.ref_forward_observed.restype = C.c_int
        R.ref_forward_observed.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 6 + [C.c_int]
        R.ref_kv_block_bytes.restype = C.c_size_t
        R.ref_kv_block_bytes.argtypes = [C.c_void_p]
        R.ref_read_kv_block.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        R.ref_write_kv_block.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        R.ref_rope_inv_freq.argtypes = [C.POINTER(CModelConfig), C.c_void_p]
        R.ref_f32_to_f16.restype = C.c_uint16
        R.ref_f32_to_f16.argtypes = [C.c_float]
        R.ref_f16_to_f32.restype = C.c_float
        R.ref_f16_to_f32.argtypes = [C.c_uint16]
        R.ref_argmax.argtypes = [C.c_void_p, C.c_int]
        R.ref_sample.restype = C.c_int
        R.ref_sample.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_int, C.c_ulonglong, C.c_ulonglong, C.c_void_p]
        R.ref_uniform01.restype = C.c_double
        R.ref_uniform01.argtypes = [C.c_ulonglong, C.c_ulonglong]
        R.ref_set_threads.restype = C.c_int
        R.ref_set_threads.argtypes = [C.c_int]
        R.ref_generate_greedy.restype = C.c_int
        R.ref_generate_greedy.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        _ref = R
    return _ref


def set_threads(n: Optional[int] = None) -> int:
    """Runs both checkers' OpenMP loops on n threads (default: every core this process may run
    on), whatever OMP_NUM_THREADS says: a multi-process launcher exports OMP_NUM_THREADS=1 to
    its ranks. Returns the count in force."""
    n = len(os.sched_getaffinity(0)) if n is None else n
    got = lib().ro_set_threads(int(n))
    if have_ref():
        got = ref_lib().ref_set_threads(int(n))
    return int(got)


def f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


# ---- element-wise and op-level restatements ---------------------------------------------

def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    L = lib()
    flat = f32(x).ravel()
    return np.fromiter((L.ro_f32_to_f16(float(v)) for v in flat), dtype=np.uint16, count=flat.size).reshape(np.shape(x))


def round_to_f16(x: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest fp16 (what the GPU path stores), as float32."""
    x = f32(x)
    out = np.empty_like(x)
    lib().ro_round_to_f16(ptr(x), ptr(out), C.c_size_t(x.size))
    return out


def rope_inv_freq(cfg: ModelConfig) -> np.ndarray:
    out = np.zeros(cfg.head_dim // 2, np.float32)
    c = cfg.to_c()
    lib().ro_rope_inv_freq(C.byref(c), ptr(out))
    return out


def matmul(x: np.ndarray, W: np.ndarray, y: Optional[np.ndarray] = None) -> np.ndarray:
    """y[T,N] = x[T,K] W[N,K]^T (+ y), relay's fixed-order fp32 dot."""
    x, W = f32(x), f32(W)
    T, K = x.shape
    N = W.shape[0]
    acc = y is not None
    out = f32(y).copy() if acc else np.empty((T, N), np.float32)
    lib().ro_matmul(ptr(x), ptr(W), ptr(out), T, K, N, int(acc))
    return out


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x, w = f32(x), f32(w)
    out = np.empty_like(x)
    for r in range(x.shape[0]):
        lib().ro_rmsnorm(ptr(x[r]), ptr(w), C.c_void_p(out[r].ctypes.data), x.shape[1], C.c_float(eps))
    return out


def swiglu(gu: np.ndarray) -> np.ndarray:
    gu = f32(gu)
    T, I2 = gu.shape
    out = np.empty((T, I2 // 2), np.float32)
    lib().ro_swiglu(ptr(gu), ptr(out), T, I2 // 2)
    return out


def attention(q, q_stride, pos, seq, table_off, tables, k_pool, v_pool, heads, kv_heads, D, block_size) -> np.ndarray:
    q, k_pool, v_pool = f32(q), f32(k_pool), f32(v_pool)
    T = len(pos)
    out = np.zeros((T, heads * D), np.float32)
    lib().ro_attention(ptr(q), q_stride, ptr(pos), ptr(seq), ptr(table_off), ptr(tables), T, ptr(k_pool),
                       ptr(v_pool), heads, kv_heads, D, block_size, ptr(out))
    return out


def qkv_post(qkv, bias, inv_freq, pos, seq, table_off, tables, k_pool, v_pool, heads, kv_heads, D, block_size):
    """In place on qkv, k_pool, v_pool (float32 arrays)."""
    T = len(pos)
    lib().ro_qkv_post(ptr(qkv), ptr(bias), ptr(inv_freq), ptr(pos), ptr(seq), ptr(table_off), ptr(tables), T,
                      ptr(k_pool), ptr(v_pool), heads, kv_heads, D, block_size)


def quantize_rows_int8(w: np.ndarray):
    w = f32(w)
    N, K = w.shape
    q = np.empty((N, K), np.int8)
    s = np.empty(N, np.float32)
    lib().ro_quantize_rows_int8(ptr(w), N, K, ptr(q), ptr(s))
    return q, s


def gemv_int8(q: np.ndarray, scale: np.ndarray, x: np.ndarray, y: Optional[np.ndarray] = None, beta: float = 0.0):
    q = np.ascontiguousarray(q, dtype=np.int8)
    x = f32(x)
    T, K = x.shape
    N = q.shape[0]
    out = f32(y).copy() if y is not None else np.zeros((T, N), np.float32)
    lib().ro_gemv_int8(ptr(q), ptr(f32(scale)), ptr(x), ptr(out), T, K, N, C.c_float(beta))
    return out


def lse_merge(part_o: np.ndarray, part_ml: np.ndarray) -> np.ndarray:
    part_o, part_ml = f32(part_o), f32(part_ml)
    parts, D = part_o.shape
    out = np.empty(D, np.float32)
    lib().ro_lse_merge(ptr(part_o), ptr(part_ml), parts, D, ptr(out))
    return out


def argmax(logits: np.ndarray) -> int:
    logits = f32(logits)
    return int(lib().ro_argmax(ptr(logits), logits.size))


def sample(logits: np.ndarray, temperature: float, top_p: float, top_k: int, seed: int, index: int,
           prefer_reference: bool = True):
    """(token, log-probability) relay's sampler gives for one row of logits: relay's own code
    where it was compiled, else the restatement."""
    logits = f32(logits)
    lp = C.c_double(0.0)
    if prefer_reference and have_ref():
        tok = ref_lib().ref_sample(ptr(logits), logits.size, temperature, top_p, top_k, seed, index, C.byref(lp))
    else:
        tok = lib().ro_sample(ptr(logits), logits.size, temperature, top_p, top_k, seed, index, C.byref(lp))
    return int(tok), float(lp.value)


def uniform01(seed: int, index: int) -> float:
    return float(lib().ro_uniform01(seed, index))


def kv_gather(k_pool: np.ndarray, v_pool: np.ndarray, blocks, block_bytes: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.int32)
    out = np.empty(2 * len(blocks) * block_bytes, np.uint8)
    lib().ro_kv_gather(ptr(k_pool), ptr(v_pool), ptr(blocks), len(blocks), C.c_size_t(block_bytes), ptr(out))
    return out


def kv_scatter(k_pool: np.ndarray, v_pool: np.ndarray, blocks, block_bytes: int, staging: np.ndarray) -> None:
    blocks = np.ascontiguousarray(blocks, dtype=np.int32)
    lib().ro_kv_scatter(ptr(k_pool), ptr(v_pool), ptr(blocks), len(blocks), C.c_size_t(block_bytes), ptr(staging))


# ---- whole-model checkers ----------------------------------------------------------------

class _Model:
    """Shared shape of the two whole-model checkers (same methods as relay::Backend)."""

    config: ModelConfig

    def _forward(self, fb: FlatBatch, out: np.ndarray) -> int:
        raise NotImplementedError

    def forward(self, batch: ForwardBatch) -> np.ndarray:
        fb = flatten(batch)
        out = np.empty((max(fb.n_rows, 1), self.config.vocab), np.float32)
        rows = self._forward(fb, out)
        if rows < 0:
            raise ValueError({-1: "block table too short", -2: "token id out of range"}.get(rows, f"error {rows}"))
        return out[:rows]


class OracleModel(_Model):
    """The restatement's forward pass with its own fp32 paged cache."""

    def __init__(self, weights: HostWeights, num_blocks: int, block_size: int):
        self.config = weights.config
        self._w = weights
        cw, self._keep = weights.to_c()
        cc = weights.config.to_c()
        self._h = lib().ro_model_new(C.byref(cc), C.byref(cw), num_blocks, block_size)
        self.block_size = block_size

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ro_model_free(self._h)
            self._h = None

    def _forward(self, fb, out):
        return lib().ro_forward(self._h, fb.n_seqs, ptr(fb.tokens), ptr(fb.chunk_len), ptr(fb.start_pos),
                                ptr(fb.table_len), ptr(fb.tables), ptr(fb.want_logits.astype(np.uint8)),
                                int(fb.all_logits), ptr(out), C.c_size_t(out.size))

    def kv_block_bytes(self) -> int:
        return lib().ro_kv_block_bytes(self._h)

    def read_kv_block(self, layer: int, block: int):
        n = self.kv_block_bytes() // 4
        k, v = np.empty(n, np.float32), np.empty(n, np.float32)
        lib().ro_read_kv_block(self._h, layer, block, ptr(k), ptr(v))
        return k, v

    def write_kv_block(self, layer: int, block: int, k: np.ndarray, v: np.ndarray) -> None:
        lib().ro_write_kv_block(self._h, layer, block, ptr(f32(k)), ptr(f32(v)))


class RefModel(_Model):
    """relay's own CpuBackend (engine/src/cpu_backend.cpp), through oracle/ref_shim.cpp."""

    def __init__(self, weights: Optional[HostWeights] = None, num_blocks: int = 64, block_size: int = 16,
                 model_dir: Optional[str] = None):
        R = ref_lib()
        if model_dir is not None:
            self._h = R.ref_load(model_dir.encode(), num_blocks, block_size)
        else:
            cw, self._keep = weights.to_c()
            cc = weights.config.to_c()
            self._h = R.ref_create(C.byref(cc), C.byref(cw), num_blocks, block_size)
        if not self._h:
            raise RuntimeError(R.ref_last_error().decode())
        cc = CModelConfig()
        R.ref_get_config(self._h, C.byref(cc))
        self.config = ModelConfig.from_c(cc)
        self.block_size = block_size

    def __del__(self):
        if getattr(self, "_h", None):
            ref_lib().ref_destroy(self._h)
            self._h = None

    def tensor(self, name: str) -> Optional[np.ndarray]:
        n = C.c_longlong(0)
        p = ref_lib().ref_tensor(self._h, name.encode(), C.byref(n))
        if not p:
            return None
        return np.ctypeslib.as_array(p, shape=(n.value,)).copy()

    def _forward(self, fb, out):
        r = ref_lib().ref_forward(self._h, fb.n_seqs, ptr(fb.tokens), ptr(fb.chunk_len), ptr(fb.start_pos),
                                  ptr(fb.table_len), ptr(fb.tables), ptr(fb.want_logits.astype(np.uint8)),
                                  int(fb.all_logits), ptr(out), C.c_size_t(out.size))
        if r < 0:
            raise ValueError(ref_lib().ref_last_error().decode())
        return r

    def forward_observed(self, batch: ForwardBatch):
        fb = flatten(batch)
        seen = np.zeros(self.config.layers + 8, np.int32)
        n = ref_lib().ref_forward_observed(self._h, fb.n_seqs, ptr(fb.tokens), ptr(fb.chunk_len), ptr(fb.start_pos),
                                           ptr(fb.table_len), ptr(fb.tables), ptr(seen), seen.size)
        return seen[:n].tolist()

    def kv_block_bytes(self) -> int:
        return ref_lib().ref_kv_block_bytes(self._h)

    def read_kv_block(self, layer: int, block: int):
        n = self.kv_block_bytes() // 4
        k, v = np.empty(n, np.float32), np.empty(n, np.float32)
        ref_lib().ref_read_kv_block(self._h, layer, block, ptr(k), ptr(v))
        return k, v

    def write_kv_block(self, layer: int, block: int, k, v) -> None:
        ref_lib().ref_write_kv_block(self._h, layer, block, ptr(f32(k)), ptr(f32(v)))

    def generate_greedy(self, prompt, steps: int):
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        toks = np.zeros(steps, np.int32)
        lg = np.zeros((steps, self.config.vocab), np.float32)
        n = ref_lib().ref_generate_greedy(self._h, ptr(prompt), prompt.size, steps, ptr(toks), ptr(lg))
        if n < 0:
            raise RuntimeError(ref_lib().ref_last_error().decode())
        return toks[:n], lg[:n]


def cpu_model(weights: HostWeights, num_blocks: int, block_size: int, prefer_reference: bool = True) -> _Model:
    """relay's CPU backend where it was compiled, else the restatement."""
    if prefer_reference and have_ref():
        return RefModel(weights, num_blocks, block_size)
    return OracleModel(weights, num_blocks, block_size)
