"""relay_b200: the per-token compute path of the relay inference engine for B200 (sm_100a).

Hand-written CUDA kernels behind a C boundary (include/relay_b200.h, librelay_b200.so) and
a host-side mirror of relay's backend interface. Nothing here falls back to the CPU.
"""
from .types import CudaOptions, ForwardBatch, HostWeights, ModelConfig, SeqChunk, flatten  # noqa: F401


def __getattr__(name):
    if name in ("Backend", "make_cuda_backend", "KVLayout"):
        from . import backend
        return getattr(backend, name)
    raise AttributeError(name)
