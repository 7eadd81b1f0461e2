"""ctypes binding of libcacheir_b200.so (the C ABI declared in include/cacheir_b200.h).

There is no fallback: if the shared library is missing the import of any
compute entry point raises, telling the user to build it.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libcacheir_b200.so"

# name -> (restype, argtypes); mirrors include/cacheir_b200.h one to one
SIGNATURES: dict[str, tuple[object, list[object]]] = {
    "cacheir_b200_version": (c_int, []),
    "cacheir_b200_build_info": (c_char_p, []),
    "cacheir_b200_error_string": (c_char_p, [c_int]),
    "cacheir_b200_paged_attention_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "cacheir_b200_paged_attention_auto_splits": (c_int, [c_int] * 6),
    "cacheir_b200_paged_attention_decode_batch": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,  # q k v page_table seq_lens out
         c_int, c_int, c_int, c_int, c_int, c_int, c_int,              # batch heads kv_heads max_pages page D dtype
         c_longlong, c_longlong, c_float, c_int,                       # q_stride out_stride scale num_splits
         c_void_p, c_size_t, c_void_p]),                               # workspace bytes stream
    "cacheir_b200_paged_attention_decode_batch_ex": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int,
         c_longlong, c_longlong, c_float, c_int,
         c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p]),      # workspace bytes num_slots kv_dtype kv_scales stream
    "cacheir_b200_paged_attention_decode_batch_quantize": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int,
         c_longlong, c_float, c_int, c_void_p, c_size_t, c_void_p]),  # q_stride scale num_slots gemm_workspace bytes stream
    "cacheir_b200_paged_attention_quantize_supported": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "cacheir_b200_paged_attention_noalloc_max_workspace_bytes": (c_size_t, []),
    "cacheir_b200_paged_attention_decode_batch_noalloc": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int,
         c_longlong, c_longlong, c_float, c_int, c_void_p]),
    "cacheir_b200_qgemv": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,  # x packed scales zero_points residual y
         c_int, c_int, c_int, c_int, c_int, c_int, c_int,              # M N K bits group x_dtype scale_dtype
         c_longlong, c_int, c_void_p]),                                # x_stride epilogue stream
    "cacheir_b200_qgemv_workspace_bytes": (c_size_t, [c_int, c_int]),
    "cacheir_b200_qgemv_ex": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int,
         c_longlong, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "cacheir_b200_rmsnorm_qgemv": (
        c_int,
        [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,   # x norm_w eps packed scales zero residual y
         c_int, c_int, c_int, c_int, c_int, c_longlong, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "cacheir_b200_qgemv_plan": (c_int, [c_int] * 8),
    "cacheir_b200_rmsnorm_qkv_rope_append": (
        c_int,
        [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_int,
         c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
         c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "cacheir_b200_qkv_rope_append": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_int,  # x..qkv M N K scale_dtype stride layout
         c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,             # q_dim k_dim hd theta table n pos table maxp page
         c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),                                             # k v ws bytes stream
    "cacheir_b200_rope_table": (c_int, [c_void_p, c_int, c_int, c_float, c_void_p]),
    "cacheir_b200_quantize_activations": (c_int, [c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_size_t, c_void_p]),
    "cacheir_b200_rms_norm_quantize": (
        c_int, [c_void_p] * 5 + [c_int, c_int, c_float, c_int, c_void_p, c_size_t, c_void_p]),
    "cacheir_b200_pack_tiled_bytes": (c_size_t, [c_int, c_int, c_int]),
    "cacheir_b200_pack_relayout": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "cacheir_b200_pack_unrelayout": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "cacheir_b200_peer_alloc": (c_int, [c_size_t, c_void_p, c_void_p]),
    "cacheir_b200_peer_open": (c_int, [c_void_p, c_void_p]),
    "cacheir_b200_peer_close": (c_int, [c_void_p]),
    "cacheir_b200_peer_free": (c_int, [c_void_p]),
    "cacheir_b200_peer_all_reduce": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_void_p, c_void_p]),
    "cacheir_b200_peer_all_reduce_two_step": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_void_p,
                                                      c_void_p]),
    "cacheir_b200_peer_all_reduce_ll": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_int, c_int, c_void_p,
                                                c_void_p]),
    "cacheir_b200_peer_all_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_int, c_int, c_int, c_void_p, c_void_p]),
    "cacheir_b200_device_status": (c_int, [c_int]),
    "cacheir_b200_pack_rows": (c_int, [c_void_p] * 5 + [c_int, c_int, c_int, c_void_p]),
    "cacheir_b200_dequantize_rows": (c_int, [c_void_p] * 4 + [c_int, c_int, c_int, c_int, c_void_p]),
    "cacheir_b200_rms_norm": (c_int, [c_void_p] * 5 + [c_int, c_int, c_float, c_int, c_void_p]),
    "cacheir_b200_rope_inplace": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_longlong, c_void_p]),
    "cacheir_b200_rope_append": (c_int, [c_void_p] * 5 + [c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_longlong, c_void_p]),
    "cacheir_b200_kv_append": (
        c_int, [c_void_p] * 6 + [c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p]),
    "cacheir_b200_kv_append_q8": (
        c_int, [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p]),
    "cacheir_b200_silu_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "cacheir_b200_add": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "cacheir_b200_embedding_gather": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "cacheir_b200_argmax_rows": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "cacheir_b200_advance_positions": (c_int, [c_void_p, c_void_p, c_int, c_void_p]),
}

_LIB: ctypes.CDLL | None = None


class CacheIRB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def load() -> ctypes.CDLL:
    """Load the library once and attach the prototypes. Raises if it is not built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not LIB_PATH.exists():
        raise CacheIRB200Error(
            f"{LIB_PATH} is missing: build the CUDA library first (python -m cacheir_b200.build). "
            "cacheir_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _LIB = lib
    return lib


def check(code: int, what: str) -> None:
    if code != 0:
        text = load().cacheir_b200_error_string(int(code)).decode("utf-8", "replace")
        raise CacheIRB200Error(f"{what} failed with status {code}: {text}")
