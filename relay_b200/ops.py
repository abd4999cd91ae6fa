"""The path's kernels on caller-owned device tensors (torch is only the allocator here).

Each function forwards to one operator entry point of include/relay_b200.h on the current
CUDA stream of torch. Used by the parity tests and by bench.py at shapes the model-level
path does not reach; the backend (backend.py) calls the same kernels internally.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import CAttnShape, CTokenMeta


def _p(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dev_i32(a, device) -> torch.Tensor:
    return torch.as_tensor(a, dtype=torch.int32).to(device).contiguous()


@dataclass
class TokenMeta:
    """Device copies of the batch's position metadata (engine/src/cuda_kernels.cuh:16-26)."""

    pos: torch.Tensor
    seq: torch.Tensor
    table_off: torch.Tensor
    tables: torch.Tensor

    @staticmethod
    def from_host(pos, seq, table_off, tables, device="cuda") -> "TokenMeta":
        return TokenMeta(*(_dev_i32(a, device) for a in (pos, seq, table_off, tables)))

    def c(self) -> CTokenMeta:
        return CTokenMeta(self.pos.data_ptr(), self.seq.data_ptr(), self.table_off.data_ptr(), self.tables.data_ptr())


def attn_shape(heads, kv_heads, head_dim, block_size, q_stride=None, o_stride=None) -> CAttnShape:
    q_stride = (heads + 2 * kv_heads) * head_dim if q_stride is None else q_stride
    o_stride = heads * head_dim if o_stride is None else o_stride
    return CAttnShape(heads, kv_heads, head_dim, block_size, q_stride, o_stride)


def decode_scratch_bytes(shape: CAttnShape, n_decode: int, max_ctx: int) -> int:
    return _lib.lib().rb200_decode_scratch_bytes(C.byref(shape), n_decode, max_ctx)


def decode_plan(shape: CAttnShape, n_decode: int, max_ctx: int):
    """(keys per slice, slices per context, bytes of partial results) of such a decode launch."""
    sl, parts = C.c_int32(0), C.c_int32(0)
    nbytes = _lib.lib().rb200_decode_plan(C.byref(shape), n_decode, max_ctx, C.byref(sl), C.byref(parts))
    return sl.value, parts.value, nbytes


def decode_attention(shape: CAttnShape, q: torch.Tensor, meta: TokenMeta, decode_tokens: torch.Tensor, max_ctx: int,
                     k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                     scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    n = decode_tokens.numel()
    if scratch is None:
        scratch = torch.empty(max(decode_scratch_bytes(shape, n, max_ctx), 16), dtype=torch.uint8, device=q.device)
    m = meta.c()
    _lib.check(_lib.lib().rb200_decode_attention(C.byref(shape), _p(q), C.byref(m), _p(decode_tokens), n, max_ctx,
                                                 _p(k_pool), _p(v_pool), _p(scratch), scratch.numel(), _p(out), _stream()))
    return out


def decode_attention_static(shape: CAttnShape, q, meta: TokenMeta, decode_tokens, max_ctx: int, k_pool, v_pool,
                            out) -> torch.Tensor:
    """decode_attention without caller scratch: the partial results go to the fixed buffer
    inside the library (at most _lib.STATIC_DECODE_SCRATCH_BYTES; larger batches raise
    ValueError). Allocates nothing; calls sharing a GPU must not overlap."""
    m = meta.c()
    _lib.check(_lib.lib().rb200_decode_attention_static(C.byref(shape), _p(q), C.byref(m), _p(decode_tokens),
                                                        decode_tokens.numel(), max_ctx, _p(k_pool), _p(v_pool), _p(out),
                                                        _stream()))
    return out


def prefill_attention(shape: CAttnShape, q, meta: TokenMeta, tiles: torch.Tensor, k_pool, v_pool, out) -> torch.Tensor:
    m = meta.c()
    _lib.check(_lib.lib().rb200_prefill_attention(C.byref(shape), _p(q), C.byref(m), _p(tiles), tiles.numel() // 2,
                                                  _p(k_pool), _p(v_pool), _p(out), _stream()))
    return out


def reference_attention(shape: CAttnShape, q, meta: TokenMeta, n_tokens: int, k_pool, v_pool, out) -> torch.Tensor:
    m = meta.c()
    _lib.check(_lib.lib().rb200_reference_attention(C.byref(shape), _p(q), C.byref(m), n_tokens, _p(k_pool), _p(v_pool),
                                                    _p(out), _stream()))
    return out


def gemv_scratch(N: int, K: int, device="cuda") -> torch.Tensor:
    return torch.zeros(_lib.lib().rb200_gemv_scratch_bytes(N, K), dtype=torch.uint8, device=device)


def gemv_int8(wq, scale, x, y, beta=0.0, scratch=None) -> torch.Tensor:
    """y[T,N] (+)= scale * (wq[N,K] . x[T,K]); T <= 8."""
    N, K = wq.shape
    T = x.shape[0]
    scratch = gemv_scratch(N, K, wq.device) if scratch is None else scratch
    _lib.check(_lib.lib().rb200_gemv_int8(_p(wq), _p(scale), _p(x), _p(y), T, K, N, wq.stride(0), x.stride(0), beta,
                                          _p(scratch), scratch.numel(), _stream()))
    return y


def gemv_f16(w, x, y, beta=0.0, scratch=None) -> torch.Tensor:
    N, K = w.shape
    T = x.shape[0]
    scratch = gemv_scratch(N, K, w.device) if scratch is None else scratch
    _lib.check(_lib.lib().rb200_gemv_f16(_p(w), _p(x), _p(y), T, K, N, w.stride(0), x.stride(0), beta, _p(scratch),
                                         scratch.numel(), _stream()))
    return y


def gemm(w, x, y, beta=0.0, scale=None) -> torch.Tensor:
    """y[T,N] (+)= x[T,K] w[N,K]^T; w fp16, or int8 with per-row `scale`."""
    N, K = w.shape
    T = x.shape[0]
    i8 = w.dtype == torch.int8
    _lib.check(_lib.lib().rb200_gemm(None if i8 else _p(w), _p(w) if i8 else None, _p(scale), _p(x), _p(y), T, K, N,
                                     w.stride(0), x.stride(0), beta, _stream()))
    return y


def gemm_status() -> int:
    return _lib.lib().rb200_gemm_status()


def rmsnorm(x, w, out, eps, rows=None) -> torch.Tensor:
    R = out.shape[0]
    _lib.check(_lib.lib().rb200_rmsnorm(_p(x), _p(rows), _p(w), _p(out), R, x.shape[1], out.stride(0), eps, _stream()))
    return out


def embed(tokens, table, x) -> torch.Tensor:
    _lib.check(_lib.lib().rb200_embed(_p(tokens), _p(table), _p(x), tokens.numel(), x.shape[1], table.stride(0), _stream()))
    return x


def qkv_post(qkv, bias, inv_freq, meta: TokenMeta, k_pool, v_pool, heads, kv_heads, head_dim, block_size) -> None:
    m = meta.c()
    _lib.check(_lib.lib().rb200_qkv_post(_p(qkv), _p(bias), _p(inv_freq), C.byref(m), qkv.shape[0], _p(k_pool), _p(v_pool),
                                         heads, kv_heads, head_dim, block_size, _stream()))


def silu_mul(gu, act) -> torch.Tensor:
    T, I2 = gu.shape
    _lib.check(_lib.lib().rb200_silu_mul(_p(gu), _p(act), T, I2 // 2, act.stride(0), _stream()))
    return act


def f32_to_f16(x, out) -> torch.Tensor:
    _lib.check(_lib.lib().rb200_f32_to_f16(_p(x), _p(out), x.numel(), _stream()))
    return out


def kv_gather(k_pool, v_pool, blocks, block_bytes, staging) -> torch.Tensor:
    _lib.check(_lib.lib().rb200_kv_gather(_p(k_pool), _p(v_pool), _p(blocks), blocks.numel(), block_bytes, _p(staging),
                                          _stream()))
    return staging


def kv_scatter(k_pool, v_pool, blocks, block_bytes, staging) -> None:
    _lib.check(_lib.lib().rb200_kv_scatter(_p(k_pool), _p(v_pool), _p(blocks), blocks.numel(), block_bytes, _p(staging),
                                           _stream()))


def argmax_rows(logits, token_out, logit_out=None):
    R, V = logits.shape
    _lib.check(_lib.lib().rb200_argmax_rows(_p(logits), R, V, _p(token_out), _p(logit_out), _stream()))
    return token_out


def sample_rows(logits, params: torch.Tensor, token_out, logprob_out=None):
    """The device sampler on logits [R][V]; `params`: a device uint8 tensor holding R
    rb200_sampling_params (32 bytes each); logprob_out: float64 [R] or None."""
    R, V = logits.shape
    _lib.check(_lib.lib().rb200_sample_rows(_p(logits), R, V, _p(params), _p(token_out), _p(logprob_out), _stream()))
    return token_out
