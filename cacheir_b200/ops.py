"""Torch-tensor wrappers over the C ABI (include/cacheir_b200.h).

PyTorch supplies device memory and the current stream, nothing else: every
function below validates its arguments, passes raw device pointers to
libcacheir_b200.so on `torch.cuda.current_stream()`, and raises
`CacheIRB200Error` on a non-zero status. Output tensors can be passed in (no
allocation, CUDA-graph friendly) or are allocated here.
"""
from __future__ import annotations

import math

import torch

from . import _lib
from ._lib import CacheIRB200Error, check

F32, F16, BF16 = 0, 1, 2
EPI_NONE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2

_DTYPE_CODES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODES[dtype]
    except KeyError:
        raise TypeError(f"cacheir_b200 supports float32/float16/bfloat16 activations, got {dtype}") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _require_cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise CacheIRB200Error("cacheir_b200 kernels run on CUDA tensors only; there is no CPU fallback")


def _rows_dense(t: torch.Tensor, what: str) -> None:
    if t.stride(-1) != 1:
        raise ValueError(f"{what}: innermost dimension must be contiguous")


# ------------------------------------------------------------------------------
def attention_auto_splits(batch: int, heads: int, kv_heads: int, max_pages: int, page_size: int, head_dim: int) -> int:
    return int(_lib.load().cacheir_b200_paged_attention_auto_splits(batch, heads, kv_heads, max_pages, page_size, head_dim))


def attention_workspace_bytes(batch: int, heads: int, head_dim: int, num_splits: int) -> int:
    return int(_lib.load().cacheir_b200_paged_attention_workspace_bytes(batch, heads, head_dim, num_splits))


def attention_quantize_supported(batch: int, heads: int, kv_heads: int, max_pages: int, page_size: int, head_dim: int,
                                 dtype: torch.dtype) -> bool:
    """Can `paged_attention_decode_batch_quantize` take these extents (single split, fp16, head_dim 128, ...)?"""
    if dtype != torch.float16:
        return False
    return bool(_lib.load().cacheir_b200_paged_attention_quantize_supported(int(batch), int(heads), int(kv_heads), int(max_pages),
                                                                            int(page_size), int(head_dim), dtype_code(dtype)))


def paged_attention_decode_batch_quantize(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                          page_table: torch.Tensor, seq_lens: torch.Tensor, *, out: torch.Tensor,
                                          gemm_workspace: torch.Tensor, softmax_scale: float | None = None) -> torch.Tensor:
    """`paged_attention_decode_batch` in one split that also leaves `out` ([B, H, D], dense rows) in
    `gemm_workspace` as the activation planes of the integer GEMM, exactly as `quantize_activations(out.view(B, H*D),
    gemm_workspace)` would: the projection behind it runs with `prequantized=True` and no pre-pass launch."""
    _require_cuda(q, k_cache, v_cache, page_table, seq_lens, out, gemm_workspace)
    if q.dim() != 3 or k_cache.dim() != 4 or v_cache.shape != k_cache.shape:
        raise ValueError("expected q [B,H,D] and k_cache/v_cache [slots,KVH,page,D]")
    batch, heads, head_dim = (int(s) for s in q.shape)
    _, kv_heads, page_size, pool_dim = (int(s) for s in k_cache.shape)
    if pool_dim != head_dim or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise ValueError("q and the KV pool must share head_dim and dtype")
    if page_table.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise TypeError("page_table and seq_lens must be int32")
    if page_table.dim() != 2 or page_table.shape[0] != batch or seq_lens.numel() != batch:
        raise ValueError("page_table must be [B, max_pages] and seq_lens [B]")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous() and page_table.is_contiguous() and seq_lens.is_contiguous()):
        raise ValueError("KV pool, page_table and seq_lens must be contiguous")
    if q.stride(2) != 1 or q.stride(1) != head_dim:
        raise ValueError("q heads must be dense: only the batch stride may differ from H*D")
    if out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor of q's shape and dtype")
    if gemm_workspace.dtype != torch.uint8 or not gemm_workspace.is_contiguous():
        raise ValueError("gemm_workspace must be a contiguous uint8 tensor")
    check(_lib.load().cacheir_b200_paged_attention_decode_batch_quantize(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), page_table.data_ptr(), seq_lens.data_ptr(), out.data_ptr(),
        batch, heads, kv_heads, int(page_table.shape[1]), page_size, head_dim, dtype_code(q.dtype), q.stride(0),
        float(softmax_scale or 0.0), int(k_cache.shape[0]), gemm_workspace.data_ptr(), gemm_workspace.numel(), _stream()),
        "paged_attention_decode_batch_quantize")
    return out


def paged_attention_decode_batch(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                 page_table: torch.Tensor, seq_lens: torch.Tensor, *,
                                 out: torch.Tensor | None = None, softmax_scale: float | None = None,
                                 num_splits: int = 0, workspace: torch.Tensor | None = None,
                                 kv_scales: torch.Tensor | None = None) -> torch.Tensor:
    """out[b,h,:] = softmax(scale * q[b,h].K_b^T) V_b over the pages of sequence b.

    q: [B, H, D] (rows may be strided views of a wider buffer); k_cache/v_cache:
    [slots, KVH, page, D] contiguous, same dtype as q; page_table: int32
    [B, max_pages]; seq_lens: int32 [B]. Same contract as the reference's
    Triton launch (cacheir/runtime/cuda.py:1238-1251). With `kv_scales` (fp16
    [slots, KVH, 2, page]) the pools are uint8: value = (byte - 128) * scale of its row."""
    _require_cuda(q, k_cache, v_cache, page_table, seq_lens, out, workspace, kv_scales)
    if q.dim() != 3 or k_cache.dim() != 4 or v_cache.shape != k_cache.shape:
        raise ValueError("expected q [B,H,D] and k_cache/v_cache [slots,KVH,page,D]")
    batch, heads, head_dim = (int(s) for s in q.shape)
    _, kv_heads, page_size, pool_dim = (int(s) for s in k_cache.shape)
    kv8 = kv_scales is not None
    if kv8:
        if k_cache.dtype != torch.uint8 or v_cache.dtype != torch.uint8 or pool_dim != head_dim:
            raise ValueError("8-bit KV pools must be uint8 with q's head_dim")
        if kv_scales.dtype != torch.float16 or tuple(kv_scales.shape) != (int(k_cache.shape[0]), kv_heads, 2, page_size) or not kv_scales.is_contiguous():
            raise ValueError("kv_scales must be a contiguous fp16 [slots, KVH, 2, page] tensor")
    elif pool_dim != head_dim or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise ValueError("q and the KV pool must share head_dim and dtype")
    if page_table.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise TypeError("page_table and seq_lens must be int32")
    if page_table.dim() != 2 or page_table.shape[0] != batch or seq_lens.numel() != batch:
        raise ValueError("page_table must be [B, max_pages] and seq_lens [B]")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous() and page_table.is_contiguous() and seq_lens.is_contiguous()):
        raise ValueError("KV pool, page_table and seq_lens must be contiguous")
    if q.stride(2) != 1 or q.stride(1) != head_dim:
        raise ValueError("q heads must be dense: only the batch stride may differ from H*D")
    if out is None:
        out = torch.empty((batch, heads, head_dim), device=q.device, dtype=q.dtype)
    elif out.shape != q.shape or out.dtype != q.dtype or out.stride(2) != 1 or out.stride(1) != head_dim:
        raise ValueError("out must match q's shape/dtype with dense heads")
    max_pages = int(page_table.shape[1])
    lib = _lib.load()
    splits = num_splits if num_splits > 0 else attention_auto_splits(batch, heads, kv_heads, max_pages, page_size, head_dim)
    need = attention_workspace_bytes(batch, heads, head_dim, splits)
    if need > 0 and workspace is None:
        workspace = torch.empty((need + 3) // 4, device=q.device, dtype=torch.float32)
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    check(lib.cacheir_b200_paged_attention_decode_batch_ex(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), page_table.data_ptr(), seq_lens.data_ptr(),
        out.data_ptr(), batch, heads, kv_heads, max_pages, page_size, head_dim, dtype_code(q.dtype),
        q.stride(0), out.stride(0), float(softmax_scale or 0.0), int(splits), _ptr(workspace), ws_bytes,
        int(k_cache.shape[0]), 1 if kv8 else 0, _ptr(kv_scales), _stream()),
        "paged_attention_decode_batch")
    return out


def qgemv_workspace_bytes(m: int, k: int) -> int:
    return int(_lib.load().cacheir_b200_qgemv_workspace_bytes(int(m), int(k)))


def qgemv(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor | None, zero_points: torch.Tensor | None, *,
          bits: int, n: int, k: int, group_size: int = 0, epilogue: int = EPI_NONE,
          residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
          workspace: torch.Tensor | None = None, tiled: bool = False, prequantized: bool = False,
          paired: bool = False, norm_weight: torch.Tensor | None = None, norm_eps: float = 1e-6) -> torch.Tensor:
    """y[M, N_out] = x[M, K] . deq(W)[N, K]^T with the reference's pack format
    (bits 8/4; bits 0 = dense weights of x's dtype). x: [..., K] with dense rows.
    `norm_weight` puts an RMSNorm of x in front (integer tensor-core path only)."""
    _require_cuda(x, packed, scales, zero_points, residual, out, norm_weight)
    if x.shape[-1] != k:
        raise ValueError(f"x has {x.shape[-1]} input features, weight expects {k}")
    _rows_dense(x, "x")
    x2 = x.reshape(-1, k) if x.is_contiguous() else x
    if x2.dim() != 2:
        raise ValueError("non-contiguous x must be 2-D [M, K] with a row stride")
    m = int(x2.shape[0])
    n_out = n // 2 if epilogue == EPI_SWIGLU else n
    if bits == 0:
        if packed.dtype != x.dtype or tuple(packed.shape) != (n, k) or not packed.is_contiguous():
            raise ValueError("dense weights must be a contiguous [N, K] tensor of x's dtype")
    else:
        row_bytes = k if bits == 8 else (k + 1) // 2
        if tiled:
            if packed.dtype != torch.uint8 or packed.numel() != pack_tiled_bytes(n, k, bits) or not packed.is_contiguous():
                raise ValueError("tiled weights must be the uint8 buffer produced by pack_relayout")
        elif packed.dtype != torch.uint8 or tuple(packed.shape) != (n, row_bytes) or not packed.is_contiguous():
            raise ValueError(f"packed int{bits} weights must be contiguous uint8 [{n}, {row_bytes}]")
        if scales is None or scales.dtype not in (torch.float32, torch.float16) or not scales.is_contiguous():
            raise ValueError("scales must be a contiguous float32 or float16 tensor")
        want = n * (k // group_size) if group_size else n
        if scales.numel() != want:
            raise ValueError(f"scales has {scales.numel()} entries, expected {want}")
        if zero_points is not None and (zero_points.dtype != torch.float32 or zero_points.numel() != n):
            raise ValueError("zero_points must be float32 [N] (the reference's device format)")
    if out is None:
        out = torch.empty((m, n_out), device=x.device, dtype=x.dtype)
    elif out.numel() != m * n_out or out.dtype != x.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous [M, N_out] tensor of x's dtype")
    if residual is not None and (residual.numel() != m * n_out or residual.dtype != x.dtype or not residual.is_contiguous()):
        raise ValueError("residual must be a contiguous [M, N_out] tensor of x's dtype")
    _require_cuda(workspace)
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    layout = (1 if tiled else 0) | (2 if prequantized else 0) | (4 if paired else 0)
    scale_code = F16 if (scales is not None and scales.dtype == torch.float16) else F32
    if norm_weight is not None:
        if x.dtype != torch.float16 or norm_weight.dtype != torch.float16 or norm_weight.numel() != k or group_size:
            raise ValueError("the fused RMSNorm needs fp16 activations, an fp16 norm weight [K] and per-row weights")
        check(_lib.load().cacheir_b200_rmsnorm_qgemv(
            x2.data_ptr(), norm_weight.data_ptr(), float(norm_eps), packed.data_ptr(), _ptr(scales), _ptr(zero_points),
            _ptr(residual), out.data_ptr(), m, n, k, bits, scale_code, x2.stride(0), epilogue, layout, _ptr(workspace),
            ws_bytes, _stream()), "rmsnorm_qgemv")
        return out
    check(_lib.load().cacheir_b200_qgemv_ex(
        x2.data_ptr(), packed.data_ptr(), _ptr(scales), _ptr(zero_points), _ptr(residual), out.data_ptr(),
        m, n, k, bits, group_size, dtype_code(x.dtype), scale_code,
        x2.stride(0), epilogue, layout, _ptr(workspace), ws_bytes, _stream()), "qgemv")
    return out


def qgemv_plan(m: int, n: int, k: int, *, bits: int, group_size: int = 0, epilogue: int = EPI_NONE, tiled: bool = False,
               prequantized: bool = False, paired: bool = False, workspace: bool = True) -> dict:
    """Which kernel `qgemv` launches for these extents: {"family": "i8"|"f16"|"cuda_core"|"stream_int4", "split_k"}.
    epilogue 3 asks about `qkv_rope_append`."""
    layout = (1 if tiled else 0) | (2 if prequantized else 0) | (4 if paired else 0)
    code = int(_lib.load().cacheir_b200_qgemv_plan(int(m), int(n), int(k), int(bits), int(group_size), int(epilogue), layout,
                                                   1 if workspace else 0))
    check(code if code < 0 else 0, "qgemv_plan")
    family = {1: "i8", 2: "f16", 3: "cuda_core", 4: "stream_int4"}[code >> 8]
    return {"family": family, "split_k": (code & 255) if family == "i8" else 1}


def pack_tiled_bytes(n: int, k: int, bits: int) -> int:
    return int(_lib.load().cacheir_b200_pack_tiled_bytes(int(n), int(k), int(bits)))


def pack_relayout(packed: torch.Tensor, *, n: int, k: int, bits: int, paired: bool = False) -> torch.Tensor:
    """Reference row-major codes -> the 128x128 tile order the tensor-core kernels stream (exactly invertible).
    `paired` builds the [gate; up] form: each tile holds 64 gate rows and the 64 up rows of the same columns."""
    _require_cuda(packed)
    size = pack_tiled_bytes(n, k, bits)
    if size == 0 or packed.dtype != torch.uint8 or not packed.is_contiguous():
        raise ValueError("pack_relayout needs contiguous uint8 codes and K % 128 == 0")
    tiled = torch.empty((size,), device=packed.device, dtype=torch.uint8)
    check(_lib.load().cacheir_b200_pack_relayout(packed.data_ptr(), tiled.data_ptr(), n, k, bits, int(paired), _stream()), "pack_relayout")
    return tiled


def pack_unrelayout(tiled: torch.Tensor, *, n: int, k: int, bits: int, paired: bool = False) -> torch.Tensor:
    _require_cuda(tiled)
    row_bytes = k if bits == 8 else k // 2
    packed = torch.empty((n, row_bytes), device=tiled.device, dtype=torch.uint8)
    check(_lib.load().cacheir_b200_pack_unrelayout(tiled.data_ptr(), packed.data_ptr(), n, k, bits, int(paired), _stream()), "pack_unrelayout")
    return packed


def pack_rows(weight: torch.Tensor, bits: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Device quantization loader: fp32 [N,K] -> (packed uint8, scales f32, zero_points i32, zero_points f32),
    bit-exact with the reference's NumPy packer (cacheir/quantization.py:96-130)."""
    _require_cuda(weight)
    if weight.dim() != 2 or weight.dtype != torch.float32 or not weight.is_contiguous():
        raise ValueError("pack_rows expects a contiguous float32 [N, K] CUDA tensor")
    n, k = (int(s) for s in weight.shape)
    row_bytes = k if bits == 8 else (k + 1) // 2
    packed = torch.empty((n, row_bytes), device=weight.device, dtype=torch.uint8)
    scales = torch.empty((n,), device=weight.device, dtype=torch.float32)
    zp_i = torch.empty((n,), device=weight.device, dtype=torch.int32)
    zp_f = torch.empty((n,), device=weight.device, dtype=torch.float32)
    check(_lib.load().cacheir_b200_pack_rows(weight.data_ptr(), packed.data_ptr(), scales.data_ptr(), zp_i.data_ptr(),
                                             zp_f.data_ptr(), n, k, bits, _stream()), "pack_rows")
    return packed, scales, zp_i, zp_f


def dequantize_rows(packed: torch.Tensor, scales: torch.Tensor, zero_points: torch.Tensor | None, *, bits: int,
                    k: int, dtype: torch.dtype) -> torch.Tensor:
    _require_cuda(packed, scales, zero_points)
    n = int(packed.shape[0])
    out = torch.empty((n, k), device=packed.device, dtype=dtype)
    check(_lib.load().cacheir_b200_dequantize_rows(packed.data_ptr(), scales.data_ptr(), _ptr(zero_points),
                                                   out.data_ptr(), n, k, bits, dtype_code(dtype), _stream()),
          "dequantize_rows")
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, *, residual: torch.Tensor | None = None,
             sum_out: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """out = rmsnorm(x [+ residual]) * weight; with a residual the rounded sum is stored to sum_out."""
    _require_cuda(x, weight, residual, sum_out, out)
    hidden = int(x.shape[-1])
    if not x.is_contiguous() or weight.numel() != hidden or weight.dtype != x.dtype:
        raise ValueError("rms_norm expects contiguous x and a weight of x's dtype and width")
    rows = x.numel() // hidden
    if out is None:
        out = torch.empty_like(x)
    if residual is not None:
        if residual.shape != x.shape or not residual.is_contiguous():
            raise ValueError("residual must match x")
        if sum_out is None:
            sum_out = torch.empty_like(x)
    check(_lib.load().cacheir_b200_rms_norm(x.data_ptr(), _ptr(residual), weight.data_ptr(), _ptr(sum_out),
                                            out.data_ptr(), rows, hidden, float(eps), dtype_code(x.dtype), _stream()),
          "rms_norm")
    return out


def quantize_activations(x: torch.Tensor, workspace: torch.Tensor) -> None:
    """x [M, K] fp16 -> 16-bit fixed point per row in `workspace` (the integer GEMM's pre-pass)."""
    _require_cuda(x, workspace)
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("quantize_activations expects x [M, K] with dense rows")
    check(_lib.load().cacheir_b200_quantize_activations(x.data_ptr(), int(x.shape[0]), int(x.shape[1]), x.stride(0),
                                                        dtype_code(x.dtype), workspace.data_ptr(),
                                                        workspace.numel() * workspace.element_size(), _stream()),
          "quantize_activations")


def rms_norm_quantize(x: torch.Tensor, weight: torch.Tensor, eps: float, workspace: torch.Tensor, *,
                      residual: torch.Tensor | None = None, sum_out: torch.Tensor | None = None,
                      out: torch.Tensor | None = None) -> None:
    """RMSNorm fused with the integer GEMM's activation pre-pass; the fp16 result is stored only if `out` is given."""
    _require_cuda(x, weight, residual, sum_out, out, workspace)
    hidden = int(x.shape[-1])
    if not x.is_contiguous() or weight.numel() != hidden or weight.dtype != x.dtype:
        raise ValueError("rms_norm_quantize expects contiguous x and a weight of x's dtype and width")
    if residual is not None and sum_out is None:
        raise ValueError("a residual needs sum_out")
    check(_lib.load().cacheir_b200_rms_norm_quantize(x.data_ptr(), _ptr(residual), weight.data_ptr(), _ptr(sum_out), _ptr(out),
                                                     x.numel() // hidden, hidden, float(eps), dtype_code(x.dtype),
                                                     workspace.data_ptr(), workspace.numel() * workspace.element_size(),
                                                     _stream()), "rms_norm_quantize")


def rope_inplace(x: torch.Tensor, positions: torch.Tensor, *, num_heads: int, head_dim: int, theta: float) -> torch.Tensor:
    """Interleaved-pair RoPE applied in place to x [B, num_heads*head_dim] (row-strided views allowed)."""
    _require_cuda(x, positions)
    if positions.dtype != torch.int32 or x.dim() != 2 or x.stride(1) != 1 or x.shape[1] != num_heads * head_dim:
        raise ValueError("rope_inplace expects x [B, H*D] with dense rows and int32 positions")
    check(_lib.load().cacheir_b200_rope_inplace(x.data_ptr(), positions.data_ptr(), int(x.shape[0]), num_heads,
                                                head_dim, float(theta), dtype_code(x.dtype), x.stride(0), _stream()),
          "rope_inplace")
    return x


def kv_append(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              page_table: torch.Tensor, positions: torch.Tensor) -> None:
    """Write one new K/V row per request (k, v: [B, KVH*D], row-strided views allowed) into the page pool."""
    _require_cuda(k, v, k_cache, v_cache, page_table, positions)
    _, kv_heads, page_size, head_dim = (int(s) for s in k_cache.shape)
    batch = int(k.shape[0])
    if k.shape != v.shape or k.shape[1] != kv_heads * head_dim or k.stride(1) != 1 or v.stride(1) != 1:
        raise ValueError("k and v must be [B, KVH*D] with dense rows")
    if k.dtype != k_cache.dtype or page_table.dtype != torch.int32 or positions.dtype != torch.int32:
        raise TypeError("dtype mismatch in kv_append")
    check(_lib.load().cacheir_b200_kv_append(k.data_ptr(), v.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                             page_table.data_ptr(), positions.data_ptr(), batch, kv_heads,
                                             int(page_table.shape[1]), page_size, head_dim, dtype_code(k.dtype),
                                             k.stride(0), v.stride(0), _stream()), "kv_append")


def rope_append(qkv: torch.Tensor, positions: torch.Tensor, page_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *,
                q_dim: int, k_dim: int, head_dim: int, theta: float) -> None:
    """`rope_inplace` on the q and k heads of the fused rows qkv [B, q_dim + 2*k_dim] followed by `kv_append` of the
    rotated k and the v columns, in one launch (the same bits)."""
    _require_cuda(qkv, positions, page_table, k_cache, v_cache)
    _, kv_heads, page_size, pool_dim = (int(s) for s in k_cache.shape)
    if qkv.dim() != 2 or int(qkv.shape[1]) != q_dim + 2 * k_dim or qkv.stride(1) != 1:
        raise ValueError("qkv must be [B, q_dim + 2*k_dim] with dense rows")
    if pool_dim != head_dim or kv_heads * head_dim != k_dim or v_cache.shape != k_cache.shape:
        raise ValueError("the pools must hold k_dim / head_dim heads of head_dim values")
    if qkv.dtype != k_cache.dtype or v_cache.dtype != k_cache.dtype or page_table.dtype != torch.int32 or positions.dtype != torch.int32:
        raise TypeError("dtype mismatch in rope_append")
    check(_lib.load().cacheir_b200_rope_append(qkv.data_ptr(), positions.data_ptr(), page_table.data_ptr(), k_cache.data_ptr(),
                                               v_cache.data_ptr(), int(qkv.shape[0]), int(q_dim), int(k_dim), int(head_dim),
                                               float(theta), int(page_table.shape[1]), page_size, dtype_code(qkv.dtype),
                                               qkv.stride(0), _stream()), "rope_append")


def kv_append_q8(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_scales: torch.Tensor,
                 page_table: torch.Tensor, positions: torch.Tensor) -> None:
    """`kv_append` into uint8 pools: each new row is quantised with its own fp16 scale (kv_scales [slots, KVH, 2, page])."""
    _require_cuda(k, v, k_cache, v_cache, kv_scales, page_table, positions)
    _, kv_heads, page_size, head_dim = (int(s) for s in k_cache.shape)
    batch = int(k.shape[0])
    if k.shape != v.shape or k.shape[1] != kv_heads * head_dim or k.stride(1) != 1 or v.stride(1) != 1:
        raise ValueError("k and v must be [B, KVH*D] with dense rows")
    if k_cache.dtype != torch.uint8 or v_cache.dtype != torch.uint8 or kv_scales.dtype != torch.float16:
        raise TypeError("8-bit KV pools are uint8 with fp16 scales")
    if page_table.dtype != torch.int32 or positions.dtype != torch.int32:
        raise TypeError("page_table and positions must be int32")
    check(_lib.load().cacheir_b200_kv_append_q8(k.data_ptr(), v.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                                kv_scales.data_ptr(), page_table.data_ptr(), positions.data_ptr(), batch,
                                                kv_heads, int(page_table.shape[1]), page_size, head_dim, dtype_code(k.dtype),
                                                k.stride(0), v.stride(0), _stream()), "kv_append_q8")


def silu_mul(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _require_cuda(gate, up, out)
    if gate.shape != up.shape or not gate.is_contiguous() or not up.is_contiguous():
        raise ValueError("silu_mul expects contiguous tensors of equal shape")
    out = torch.empty_like(gate) if out is None else out
    check(_lib.load().cacheir_b200_silu_mul(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(),
                                            dtype_code(gate.dtype), _stream()), "silu_mul")
    return out


def add(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _require_cuda(a, b, out)
    if a.shape != b.shape or not a.is_contiguous() or not b.is_contiguous():
        raise ValueError("add expects contiguous tensors of equal shape")
    out = torch.empty_like(a) if out is None else out
    check(_lib.load().cacheir_b200_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), dtype_code(a.dtype),
                                       _stream()), "add")
    return out


def embedding_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _require_cuda(table, ids, out)
    if ids.dtype != torch.int64 or not ids.is_contiguous() or not table.is_contiguous():
        raise ValueError("embedding_gather expects contiguous int64 ids and a contiguous table")
    rows, hidden = ids.numel(), int(table.shape[1])
    out = torch.empty((rows, hidden), device=table.device, dtype=table.dtype) if out is None else out
    check(_lib.load().cacheir_b200_embedding_gather(table.data_ptr(), ids.data_ptr(), out.data_ptr(), rows, hidden,
                                                    int(table.shape[0]), dtype_code(table.dtype), _stream()),
          "embedding_gather")
    return out


def argmax_rows(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _require_cuda(logits, out)
    vocab = int(logits.shape[-1])
    rows = logits.numel() // vocab
    if not logits.is_contiguous():
        raise ValueError("argmax_rows expects contiguous logits")
    out = torch.empty((rows,), device=logits.device, dtype=torch.int64) if out is None else out
    check(_lib.load().cacheir_b200_argmax_rows(logits.data_ptr(), out.data_ptr(), rows, vocab, dtype_code(logits.dtype),
                                               _stream()), "argmax_rows")
    return out


def advance_positions(positions: torch.Tensor, seq_lens: torch.Tensor) -> None:
    _require_cuda(positions, seq_lens)
    check(_lib.load().cacheir_b200_advance_positions(positions.data_ptr(), seq_lens.data_ptr(), seq_lens.numel(),
                                                     _stream()), "advance_positions")


def default_softmax_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(float(head_dim))


def rope_table(positions: int, head_dim: int, theta: float, device: torch.device) -> torch.Tensor:
    """(cos, sin) of every (position, pair): float32 [positions, head_dim/2, 2], the values rope_inplace evaluates."""
    table = torch.empty((int(positions), head_dim // 2, 2), device=device, dtype=torch.float32)
    check(_lib.load().cacheir_b200_rope_table(table.data_ptr(), int(positions), int(head_dim), float(theta), _stream()), "rope_table")
    return table


def qkv_rope_append(x: torch.Tensor | None, packed: torch.Tensor, scales: torch.Tensor, zero_points: torch.Tensor | None,
                    out: torch.Tensor, *, n: int, k: int, q_dim: int, k_dim: int, head_dim: int, theta: float,
                    table: torch.Tensor, positions: torch.Tensor, page_table: torch.Tensor, k_cache: torch.Tensor,
                    v_cache: torch.Tensor, workspace: torch.Tensor, tiled: bool = False, prequantized: bool = False,
                    norm_weight: torch.Tensor | None = None, norm_eps: float = 1e-6) -> torch.Tensor:
    """Fused QKV projection (int8 weights) + RoPE on q and k + append of the new k/v rows to the page pool.
    `out` [M, N] fp16 receives q (roped), k (roped), v. `norm_weight` puts the RMSNorm of the reference's
    fused_rmsnorm_qkv_rope op in front. Raises CacheIRB200Error (unsupported) outside the
    integer tensor-core shapes; the caller then uses qgemv + rope_inplace + kv_append."""
    _require_cuda(x, packed, scales, zero_points, out, table, positions, page_table, k_cache, v_cache, workspace, norm_weight)
    m = int(out.shape[0])
    if out.dtype != torch.float16 or tuple(out.shape) != (m, n) or not out.is_contiguous():
        raise ValueError("out must be a contiguous fp16 [M, N] tensor")
    if k_cache.dtype != torch.float16 or v_cache.dtype != torch.float16 or k_cache.shape != v_cache.shape:
        raise ValueError("the page pool must be fp16")
    if positions.dtype != torch.int32 or page_table.dtype != torch.int32 or positions.numel() != m or page_table.shape[0] != m:
        raise ValueError("positions [M] and page_table [M, max_pages] must be int32")
    if x is not None and (x.dtype != torch.float16 or x.dim() != 2 or x.stride(1) != 1 or tuple(x.shape) != (m, k)):
        raise ValueError("x must be fp16 [M, K] with dense rows")
    _, kv_heads, page_size, hd = (int(v) for v in k_cache.shape)
    if hd != head_dim or kv_heads * head_dim != k_dim:
        raise ValueError("pool geometry does not match k_dim / head_dim")
    if table.dtype != torch.float32 or not table.is_contiguous() or table.shape[1:] != (head_dim // 2, 2):
        raise ValueError("rope table must be float32 [positions, head_dim/2, 2]")
    layout = (1 if tiled else 0) | (2 if prequantized else 0)
    if norm_weight is not None:
        if x is None or norm_weight.dtype != torch.float16 or norm_weight.numel() != k:
            raise ValueError("the fused RMSNorm needs x and an fp16 norm weight [K]")
        check(_lib.load().cacheir_b200_rmsnorm_qkv_rope_append(
            x.data_ptr(), norm_weight.data_ptr(), float(norm_eps), packed.data_ptr(), scales.data_ptr(), _ptr(zero_points),
            out.data_ptr(), m, n, k, F16 if scales.dtype == torch.float16 else F32, x.stride(0), layout, q_dim, k_dim,
            head_dim, float(theta), table.data_ptr(), int(table.shape[0]), positions.data_ptr(), page_table.data_ptr(),
            int(page_table.shape[1]), page_size, k_cache.data_ptr(), v_cache.data_ptr(), workspace.data_ptr(),
            workspace.numel() * workspace.element_size(), _stream()), "rmsnorm_qkv_rope_append")
        return out
    check(_lib.load().cacheir_b200_qkv_rope_append(
        _ptr(x), packed.data_ptr(), scales.data_ptr(), _ptr(zero_points), out.data_ptr(), m, n, k,
        F16 if scales.dtype == torch.float16 else F32, 0 if x is None else x.stride(0),
        layout, q_dim, k_dim, head_dim, float(theta),
        table.data_ptr(), int(table.shape[0]), positions.data_ptr(), page_table.data_ptr(),
        int(page_table.shape[1]), page_size, k_cache.data_ptr(), v_cache.data_ptr(), workspace.data_ptr(),
        workspace.numel() * workspace.element_size(), _stream()), "qkv_rope_append")
    return out
