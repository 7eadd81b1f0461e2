"""Backend registry entry for the B200 decode backend.

Same declarative shape as the reference registry (cacheir/backends/registry.py:6-67):
a `Backend` names its devices and the kernel-level names it provides. The op
names a compiled graph carries (`paged_attention_decode`, `quantized_matmul`,
`quantized_fused_rmsnorm_qkv_rope`, `quantized_fused_swiglu`, ...) and the
`attrs["kernel"]` strings written by the reference's `KernelSelection` pass
(cacheir/passes/transformer.py:356-388) are accepted unchanged; `KERNEL_FOR_OP`
records which C entry point serves each of them.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Backend:
    name: str
    devices: tuple[str, ...]
    kernels: tuple[str, ...]
    notes: str = ""


class BackendRegistry:
    def __init__(self) -> None:
        self._backends: dict[str, Backend] = {}

    def register(self, backend: Backend) -> None:
        self._backends[backend.name] = backend

    def get(self, name: str) -> Backend:
        return self._backends[name]

    def names(self) -> list[str]:
        return sorted(self._backends)


# graph op  ->  (kernel name in attrs["kernel"] for cuda targets, C entry points that execute it)
KERNEL_FOR_OP: dict[str, tuple[str, tuple[str, ...]]] = {
    "token_embedding": ("triton.embedding_gather", ("cacheir_b200_embedding_gather",)),
    "rms_norm": ("triton.rms_norm", ("cacheir_b200_rms_norm",)),
    "matmul": ("triton.matmul_tensorcore", ("cacheir_b200_qgemv",)),
    "quantized_matmul": ("triton.awq_int4_tensorcore", ("cacheir_b200_qgemv",)),
    "fused_rmsnorm_qkv_rope": ("triton.fused_rmsnorm_qkv_rope",
                               ("cacheir_b200_rms_norm", "cacheir_b200_qgemv", "cacheir_b200_rope_inplace")),
    "quantized_fused_rmsnorm_qkv_rope": ("triton.awq_fused_rmsnorm_qkv_rope",
                                         ("cacheir_b200_rms_norm", "cacheir_b200_qgemv", "cacheir_b200_rope_inplace")),
    "paged_attention_decode": ("triton.paged_attention_decode",
                               ("cacheir_b200_kv_append", "cacheir_b200_paged_attention_decode_batch")),
    "fused_swiglu": ("triton.fused_swiglu", ("cacheir_b200_qgemv",)),
    "quantized_fused_swiglu": ("triton.awq_fused_swiglu", ("cacheir_b200_qgemv",)),
    "add": ("triton.vector_add", ("cacheir_b200_add", "cacheir_b200_qgemv")),
}

B200_BACKEND = Backend(
    name="cuda-b200",
    devices=("sm100a",),
    kernels=(
        "embedding_gather",
        "rms_norm",
        "fused_rmsnorm_qkv_rope",
        "awq_fused_rmsnorm_qkv_rope",
        "paged_attention_decode",
        "paged_attention_decode_batch_splitk",
        "fused_swiglu",
        "awq_fused_swiglu",
        "awq_int4_tensorcore",
        "qgemv_int8",
        "qgemv_int4",
        "qgemv_int4_group128",
        "matmul_tensorcore",
        "kv_page_append",
        "quant_pack_rows",
        "cuda_graph_decode_replay",
    ),
    notes="Hand-written sm_100a kernels behind a C ABI (libcacheir_b200.so): split-K paged decode attention over a "
          "shared page pool, packed int4/int8 dequant-GEMV, fused glue ops; decode step replayed as a CUDA graph.",
)


def default_registry() -> BackendRegistry:
    registry = BackendRegistry()
    registry.register(B200_BACKEND)
    return registry
