"""Helpers shared by the CPU and GPU parity tests."""
from __future__ import annotations

import dataclasses
import json
import os

import numpy as np

from relay_b200.types import HostWeights, ModelConfig

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FIXTURES = ("llama-mha", "llama-gqa-tied-bf16", "llama3-rope", "qwen2-bias", "chat-tiny")


def load_fixture(name: str):
    """(HostWeights, dict of golden arrays) of one converted reference fixture."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg = ModelConfig(**json.loads(bytes(z["config_json"]).decode()))
    tensors = {k[2:]: np.ascontiguousarray(z[k]) for k in z.files if k.startswith("w:")}
    gold = {k: z[k] for k in z.files if not k.startswith("w:") and k != "config_json"}
    return HostWeights(cfg, tensors), gold


def rel_err_rows(a: np.ndarray, b: np.ndarray) -> float:
    """The reference's logit metric (tests/test_reference.cpp:50-57): per row,
    max|a-b| / max(|b|, 1e-6); returns the worst row."""
    a = np.asarray(a, np.float64).reshape(-1, a.shape[-1])
    b = np.asarray(b, np.float64).reshape(-1, b.shape[-1])
    diff = np.abs(a - b).max(axis=1)
    scale = np.maximum(np.abs(b).max(axis=1), 1e-6)
    return float((diff / scale).max())


def argmax_lowest(row: np.ndarray) -> int:
    """Greedy token with the reference's tie rule (engine/src/sampler.cpp:17-22)."""
    return int(np.argmax(row))  # numpy returns the first maximum: the lowest id
