"""Seeded synthetic workloads shared by the tests, the golden-vector generator and bench.py.

No public dataset or suite is involved in this path: the reference's own benchmarks draw
random token ids (tools/relay_attention_bench.cpp:40-42), and so do these.
"""
from __future__ import annotations

import numpy as np

from relay_b200.types import HostWeights, ModelConfig


def c1_config() -> ModelConfig:
    """The tiny random Llama fixture: hidden 64, 4 layers, 4 q / 2 kv heads, head_dim 16,
    SwiGLU 172, vocab 256, theta 1e4, eps 1e-5."""
    return ModelConfig(hidden=64, intermediate=172, layers=4, heads=4, kv_heads=2, head_dim=16, vocab=256,
                       max_position=1024, rms_eps=1e-5, rope_theta=10000.0)


def c1_inputs(seed: int = 1234):
    """(weights N(0,0.02) with norm weights 1+N(0,0.02), 37 uniform token ids, 4 blocks drawn
    in random order from a 64-block pool)."""
    w = HostWeights.random(c1_config(), seed)
    rng = np.random.Generator(np.random.PCG64(seed + 1))
    prompt = rng.integers(0, 256, 37).astype(np.int32)
    table = rng.permutation(64)[:4].astype(np.int32)
    return w, prompt, table


def round_f16(a: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest fp16 (IEEE round-to-nearest-even), as float32."""
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


def paged_attention_case(seed: int, ctxs, chunk_lens, heads: int, kv_heads: int, D: int, bs: int, num_blocks: int,
                         pad_tables_to: int = 4):
    """A batch of sequence chunks over a paged fp16 KV pool, as the kernels see it.

    Sequence i has ctxs[i] keys in the cache and its chunk is the LAST chunk_lens[i] of them
    (1 = a decode token). Q, K, V ~ N(0,1) rounded to fp16; the block tables are consecutive
    runs of a seeded permutation of the pool. Returns a dict of numpy arrays:
    q [T, (heads+2kv)*D] fp32 (only the q part is filled), k_pool/v_pool
    [num_blocks, kv_heads, bs, D] fp32 (fp16-representable), pos, seq, table_off, tables.
    """
    rng = np.random.Generator(np.random.PCG64(seed))
    perm = rng.permutation(num_blocks).astype(np.int32)
    k_pool = np.zeros((num_blocks, kv_heads, bs, D), np.float32)
    v_pool = np.zeros_like(k_pool)
    pos, seq, table_off, tables = [], [], [], []
    used = 0
    for i, (ctx, n) in enumerate(zip(ctxs, chunk_lens)):
        nb = (ctx + bs - 1) // bs
        if used + nb > num_blocks:
            raise ValueError("pool too small for the case")
        blocks = perm[used:used + nb]
        used += nb
        while len(tables) % pad_tables_to:
            tables.append(0)
        table_off.append(len(tables))
        tables.extend(blocks.tolist())
        kk = round_f16(rng.standard_normal((ctx, kv_heads, D)))
        vv = round_f16(rng.standard_normal((ctx, kv_heads, D)))
        for j in range(ctx):
            k_pool[blocks[j // bs], :, j % bs, :] = kk[j]
            v_pool[blocks[j // bs], :, j % bs, :] = vv[j]
        for r in range(n):
            pos.append(ctx - n + r)
            seq.append(i)
    T = len(pos)
    qkv = np.zeros((T, (heads + 2 * kv_heads) * D), np.float32)
    qkv[:, :heads * D] = round_f16(rng.standard_normal((T, heads * D)))
    i32 = lambda a: np.asarray(a, np.int32)
    return dict(q=qkv, k_pool=k_pool, v_pool=v_pool, pos=i32(pos), seq=i32(seq), table_off=i32(table_off),
                tables=i32(tables), heads=heads, kv_heads=kv_heads, D=D, bs=bs, ctxs=list(ctxs),
                chunk_lens=list(chunk_lens))


def c2_contexts(seed: int = 2, n: int = 32, lo: int = 1024, hi: int = 4096):
    """Context lengths of the paged split-decode workload: n sequences, uniform in [lo, hi]."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(lo, hi + 1, n).tolist()
