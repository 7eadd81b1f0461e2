"""cacheir_b200: the CacheIR batched decode step as hand-written sm_100a CUDA.

Public surface (mirrors the reference names for this path):
  B200DecodeRuntime / create_runtime   -- drop-in for CudaRuntime on decode
  B200KVPageAllocator, B200PagedKVCache -- paged KV pool + page tables
  quantization, ops                     -- pack format and C-ABI wrappers
Importing the package does not need a GPU; calling a kernel without the built
library or without CUDA raises (there is no fallback path).
"""
from .artifact import CompileArtifact, Graph, ModelConfig, Node, build_decoder_artifact, build_decoder_graph
from .kv_cache import B200KVPageAllocator, B200PagedKVCache, KVPage
from .registry import B200_BACKEND, Backend, BackendRegistry, default_registry

__all__ = [
    "B200DecodeRuntime", "create_runtime", "b200_runtime_available",
    "B200KVPageAllocator", "B200PagedKVCache", "KVPage",
    "CompileArtifact", "Graph", "ModelConfig", "Node", "build_decoder_artifact", "build_decoder_graph",
    "B200_BACKEND", "Backend", "BackendRegistry", "default_registry",
]


def __getattr__(name):  # torch is imported only when the runtime is actually used
    if name in {"B200DecodeRuntime", "create_runtime", "b200_runtime_available"}:
        from . import runtime
        return getattr(runtime, name)
    raise AttributeError(name)
