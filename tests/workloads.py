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


def sampler_cases(seed: int = 31, n: int = 160):
    """Rows of logits with sampling parameters for the sampler checks: vocabularies of 5 to 3000
    ids, logits N(0, s) for s in {0.5, 2, 8}, some rows with their maximum repeated (ties), and
    every mix of temperature {0, 0.7, 1, 1.5}, top_p {1, 0.9, 0.5}, top_k {0, 1, 5, 50, > vocab}.
    Returns a list of (logits float32, temperature, top_p, top_k, seed, index)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    out = []
    for trial in range(n):
        V = int(rng.integers(5, 3000))
        lg = (rng.standard_normal(V) * rng.choice([0.5, 2.0, 8.0])).astype(np.float32)
        if trial % 7 == 0:
            lg[rng.integers(0, V, 3)] = lg.max()
        out.append((lg, float(rng.choice([0.0, 0.7, 1.0, 1.5])), float(rng.choice([1.0, 0.9, 0.5])),
                    int(rng.choice([0, 1, 5, 50, V + 3])), int(rng.integers(0, 2 ** 62)), int(rng.integers(0, 1000))))
    return out


def c2_contexts(seed: int = 2, n: int = 32, lo: int = 1024, hi: int = 4096):
    """Context lengths of the paged split-decode workload: n sequences, uniform in [lo, hi]."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(lo, hi + 1, n).tolist()


class WideDecodeCase:
    """A decode batch too large to hold as one float32 case: `n_seqs` single-token chunks, every
    sequence with `ctx` keys in the cache (ctx a multiple of the block size), pages placed by a
    seeded permutation of a pool that holds exactly the batch.

    The K/V values of one group of `group` sequences are drawn once (N(0,1) rounded to fp16) and
    every group reuses them with its own sign pattern per KV head, its own block ids and its own
    queries, so that the whole pool costs one group's worth of random numbers. `pools16()` is the
    device's view ([num_blocks, kv_heads, bs, D] fp16, K and V); `group_case(g)` is group g as a
    self-contained float32 case over a compacted pool (block ids renumbered), in the format of
    paged_attention_case, for the CPU checker."""

    def __init__(self, seed: int, n_seqs: int, ctx: int, heads: int, kv_heads: int, D: int, bs: int, group: int = 32):
        if ctx % bs or n_seqs % group:
            raise ValueError("ctx must be a multiple of bs and n_seqs of group")
        self.n_seqs, self.ctx, self.heads, self.kv_heads, self.D, self.bs, self.group = n_seqs, ctx, heads, kv_heads, D, bs, group
        rng = np.random.Generator(np.random.PCG64(seed))
        self.per = ctx // bs
        self.num_blocks = n_seqs * self.per
        self.perm = rng.permutation(self.num_blocks).astype(np.int32)
        # one group's pages, already in pool order: [group * per, kv_heads, bs, D]
        shape = (group * self.per, kv_heads, bs, D)
        self.k16 = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
        self.v16 = rng.standard_normal(shape, dtype=np.float32).astype(np.float16)
        self.signs = rng.choice(np.asarray([-1.0, 1.0], np.float16), size=(n_seqs // group, 2, kv_heads))
        self.q = np.zeros((n_seqs, (heads + 2 * kv_heads) * D), np.float32)
        self.q[:, :heads * D] = round_f16(rng.standard_normal((n_seqs, heads * D), dtype=np.float32))
        self.pos = np.full(n_seqs, ctx - 1, np.int32)
        self.seq = np.arange(n_seqs, dtype=np.int32)
        self.table_off = (np.arange(n_seqs, dtype=np.int32) * self.per).astype(np.int32)  # per % 4 == 0 for ctx >= 4 bs
        self.tables = self.perm.copy()  # sequence i owns perm[i * per : (i + 1) * per]

    def _group_pages(self, g: int):
        s = self.signs[g]
        return self.k16 * s[0][None, :, None, None], self.v16 * s[1][None, :, None, None]

    def pools16(self):
        k = np.empty((self.num_blocks, self.kv_heads, self.bs, self.D), np.float16)
        v = np.empty_like(k)
        n = self.group * self.per
        for g in range(self.n_seqs // self.group):
            kg, vg = self._group_pages(g)
            ids = self.perm[g * n:(g + 1) * n]
            k[ids], v[ids] = kg, vg
        return k, v

    def group_case(self, g: int) -> dict:
        kg, vg = self._group_pages(g)
        lo, hi = g * self.group, (g + 1) * self.group
        i32 = lambda a: np.asarray(a, np.int32)
        return dict(q=self.q[lo:hi], k_pool=kg.astype(np.float32), v_pool=vg.astype(np.float32), pos=self.pos[lo:hi],
                    seq=i32(np.arange(self.group)), table_off=i32(np.arange(self.group) * self.per),
                    tables=i32(np.arange(self.group * self.per)), heads=self.heads, kv_heads=self.kv_heads, D=self.D,
                    bs=self.bs, ctxs=[self.ctx] * self.group, chunk_lens=[1] * self.group)
