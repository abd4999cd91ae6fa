"""Host-side mirror of the reference's batch and model structs for the per-token path.

`ModelConfig` follows relay::ModelConfig (engine/include/relay/config.h:20-47),
`HostWeights` relay::HostWeights / LayerWeights (engine/include/relay/weights.h:13-34),
`SeqChunk` / `ForwardBatch` the structs of engine/include/relay/backend.h:22-32, and
`CudaOptions` backend.h:85-94. `flatten` is the batch walk both backends of the reference
do at the top of forward() (engine/src/cuda_backend.cu:508-526).
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np


class CModelConfig(C.Structure):
    """rb200_model_config (include/relay_b200.h)."""

    _fields_ = [
        ("hidden", C.c_int32), ("intermediate", C.c_int32), ("layers", C.c_int32), ("heads", C.c_int32),
        ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("vocab", C.c_int32), ("max_position", C.c_int32),
        ("rms_eps", C.c_double), ("rope_theta", C.c_double),
        ("rope_scaling_type", C.c_int32),
        ("rope_factor", C.c_double), ("rope_low_freq_factor", C.c_double),
        ("rope_high_freq_factor", C.c_double), ("rope_original_max_position", C.c_double),
        ("tie_embeddings", C.c_int32), ("qkv_bias", C.c_int32),
    ]


class CLayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("attn_norm", "wqkv", "bqkv", "wo", "mlp_norm", "w_gate_up", "w_down")]


class CWeights(C.Structure):
    _fields_ = [("embed", C.c_void_p), ("final_norm", C.c_void_p), ("lm_head", C.c_void_p),
                ("layers", C.POINTER(CLayerWeights))]


@dataclass
class ModelConfig:
    hidden: int
    intermediate: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    vocab: int
    max_position: int = 4096
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling_type: str = ""  # "" or "llama3"
    rope_factor: float = 1.0
    rope_low_freq_factor: float = 1.0
    rope_high_freq_factor: float = 4.0
    rope_original_max_position: float = 8192.0
    tie_embeddings: bool = False
    qkv_bias: bool = False

    @property
    def q_dim(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    def to_c(self) -> CModelConfig:
        return CModelConfig(
            self.hidden, self.intermediate, self.layers, self.heads, self.kv_heads, self.head_dim, self.vocab,
            self.max_position, self.rms_eps, self.rope_theta, 1 if self.rope_scaling_type == "llama3" else 0,
            self.rope_factor, self.rope_low_freq_factor, self.rope_high_freq_factor,
            self.rope_original_max_position, int(self.tie_embeddings), int(self.qkv_bias))

    @staticmethod
    def from_c(c: CModelConfig) -> "ModelConfig":
        return ModelConfig(
            c.hidden, c.intermediate, c.layers, c.heads, c.kv_heads, c.head_dim, c.vocab, c.max_position,
            c.rms_eps, c.rope_theta, "llama3" if c.rope_scaling_type == 1 else "", c.rope_factor,
            c.rope_low_freq_factor, c.rope_high_freq_factor, c.rope_original_max_position,
            bool(c.tie_embeddings), bool(c.qkv_bias))


LAYER_TENSORS = ("attn_norm", "wqkv", "bqkv", "wo", "mlp_norm", "w_gate_up", "w_down")


def tensor_shapes(c: ModelConfig) -> Dict[str, tuple]:
    """Relay's weight names (backend.h:72-75) and their shapes in the fused layout."""
    shapes = {"embed": (c.vocab, c.hidden), "final_norm": (c.hidden,)}
    if not c.tie_embeddings:
        shapes["lm_head"] = (c.vocab, c.hidden)
    for l in range(c.layers):
        p = f"layers.{l}."
        shapes[p + "attn_norm"] = (c.hidden,)
        shapes[p + "wqkv"] = (c.qkv_dim, c.hidden)
        if c.qkv_bias:
            shapes[p + "bqkv"] = (c.qkv_dim,)
        shapes[p + "wo"] = (c.hidden, c.q_dim)
        shapes[p + "mlp_norm"] = (c.hidden,)
        shapes[p + "w_gate_up"] = (2 * c.intermediate, c.hidden)
        shapes[p + "w_down"] = (c.hidden, c.intermediate)
    return shapes


@dataclass
class HostWeights:
    """float32 host weights by relay's tensor names ("embed", "layers.0.wqkv", ...)."""

    config: ModelConfig
    tensors: Dict[str, np.ndarray] = field(default_factory=dict)

    def validate(self) -> None:
        for name, shape in tensor_shapes(self.config).items():
            t = self.tensors.get(name)
            if t is None:
                raise ValueError(f"missing weight {name}")
            if t.dtype != np.float32 or tuple(t.shape) != shape or not t.flags.c_contiguous:
                raise ValueError(f"weight {name}: want contiguous float32 {shape}, got {t.dtype} {t.shape}")

    def to_c(self):
        """(CWeights, keepalive) pointing into the numpy arrays."""
        self.validate()
        c = self.config
        layers = (CLayerWeights * c.layers)()
        for l in range(c.layers):
            for n in LAYER_TENSORS:
                t = self.tensors.get(f"layers.{l}.{n}")
                setattr(layers[l], n, t.ctypes.data if t is not None else None)
        lm = self.tensors.get("lm_head")
        w = CWeights(self.tensors["embed"].ctypes.data, self.tensors["final_norm"].ctypes.data,
                     lm.ctypes.data if lm is not None else None, layers)
        return w, layers

    @staticmethod
    def random(config: ModelConfig, seed: int, std: float = 0.02, norm_std: Optional[float] = None) -> "HostWeights":
        """Seeded N(0, std) matrices; norm weights 1 + N(0, norm_std) (std if None).

        numpy's PCG64 stream by tensor name order, so any process regenerates the same values.
        """
        rng = np.random.Generator(np.random.PCG64(seed))
        out: Dict[str, np.ndarray] = {}
        for name, shape in tensor_shapes(config).items():
            if name.endswith("norm"):
                s = std if norm_std is None else norm_std
                out[name] = (1.0 + s * rng.standard_normal(shape)).astype(np.float32)
            else:
                out[name] = (std * rng.standard_normal(shape)).astype(np.float32)
        return HostWeights(config, out)


@dataclass
class SeqChunk:
    tokens: List[int]
    start_pos: int = 0
    block_table: List[int] = field(default_factory=list)
    want_logits: bool = True


@dataclass
class ForwardBatch:
    seqs: List[SeqChunk] = field(default_factory=list)
    all_logits: bool = False


@dataclass
class FlatBatch:
    n_seqs: int
    tokens: np.ndarray
    chunk_len: np.ndarray
    start_pos: np.ndarray
    table_len: np.ndarray
    tables: np.ndarray
    want_logits: np.ndarray
    all_logits: bool

    @property
    def n_tokens(self) -> int:
        return int(self.tokens.size)

    @property
    def n_rows(self) -> int:
        if self.all_logits:
            return self.n_tokens
        return int(np.count_nonzero(self.want_logits & (self.chunk_len > 0)))


def flatten(batch: ForwardBatch) -> FlatBatch:
    i32 = np.int32
    toks = [np.asarray(s.tokens, dtype=i32).ravel() for s in batch.seqs]
    tabs = [np.asarray(s.block_table, dtype=i32).ravel() for s in batch.seqs]
    cat = lambda xs: np.ascontiguousarray(np.concatenate(xs)) if xs else np.zeros(0, i32)
    return FlatBatch(
        n_seqs=len(batch.seqs), tokens=cat(toks).astype(i32, copy=False),
        chunk_len=np.asarray([t.size for t in toks], dtype=i32),
        start_pos=np.asarray([s.start_pos for s in batch.seqs], dtype=i32),
        table_len=np.asarray([t.size for t in tabs], dtype=i32), tables=cat(tabs).astype(i32, copy=False),
        want_logits=np.asarray([bool(s.want_logits) for s in batch.seqs], dtype=np.bool_),
        all_logits=bool(batch.all_logits))


@dataclass
class CudaOptions:
    """relay::CudaOptions (backend.h:85-94)."""

    reference_attention: bool = False
    int8_weights: bool = False
    gpu_argmax: bool = False  # not in the reference: enables Backend.forward_greedy

    @staticmethod
    def from_env() -> "CudaOptions":
        """RELAY_CUDA_ATTENTION=m0, RELAY_CUDA_INT8=1 (engine/src/cuda_backend.cu:37-42)."""
        return CudaOptions(os.environ.get("RELAY_CUDA_ATTENTION") == "m0", os.environ.get("RELAY_CUDA_INT8") == "1")

    def flags(self) -> int:
        return (1 if self.int8_weights else 0) | (2 if self.reference_attention else 0) | (4 if self.gpu_argmax else 0)


def ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def i32(a: Sequence[int]) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32))
