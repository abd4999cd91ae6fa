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
