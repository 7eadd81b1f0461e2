"""Device-side quantized weights in the reference's pack format.

`B200PackedWeight` is the GPU counterpart of the reference's
`CudaPackedQuantizedTensor` (cacheir/runtime/cuda.py:96-105): uint8 codes
(`packed_values`: [N, K] for int8, [N, ceil(K/2)] for int4 with the even
column in the low nibble), fp32 `scales` [N] and fp32 `zero_points` [N]
(the reference uploads its int32 zero points as fp32, cuda.py:83). The codes
are exactly what `cacheir/quantization.py:_asymmetric_pack` produces; packing
runs on the GPU (`ops.pack_rows`). Group-wise symmetric weights (scales
[N, K/group], zero point 2^(bits-1)) use the same code layout.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from . import ops


def quant_bits(quant: str | None) -> int | None:
    """Bit width by quant name, the rule of cacheir/quantization.py:63-71."""
    if not quant:
        return None
    name = quant.lower()
    if "int4" in name or "awq" in name or "gptq" in name:
        return 4
    if "int8" in name or "8bit" in name:
        return 8
    return None


@dataclass
class B200PackedWeight:
    packed_values: torch.Tensor          # uint8 [N, K] or [N, ceil(K/2)]
    scales: torch.Tensor                 # f32 [N]  |  f16/f32 [N, K/group]
    zero_points: torch.Tensor | None     # f32 [N]  |  None (midpoint)
    bits: int
    shape: tuple[int, int]
    axis: int = 1
    group_size: int | None = None
    zero_points_i32: torch.Tensor | None = None   # the reference's int32 form, kept for parity checks
    tiled: bool = False                           # packed_values is in the 128x128 tile order (ops.pack_relayout)
    paired: bool = False                          # tiled as [gate; up] pairs: 64 + 64 rows per tile (SwiGLU, int8)

    @property
    def nbytes(self) -> int:
        total = self.packed_values.numel() + self.scales.numel() * self.scales.element_size()
        if self.zero_points is not None:
            total += self.zero_points.numel() * 4
        return int(total)


def quant_group_size(quant: str | None) -> int:
    """Group size named by a quant string such as "int4_g128" (0: the reference's per-row affine format)."""
    if not quant:
        return 0
    for part in quant.lower().replace("-", "_").split("_"):
        if part.startswith("g") and part[1:].isdigit():
            return int(part[1:])
    return 0


def pack_group_int4(weight: torch.Tensor, group_size: int = 128) -> B200PackedWeight:
    """Group-wise symmetric int4: w[n, k] ~ (code - 8) * scale[n, k // group], fp16 scales, the nibble order
    of the reference's int4 pack (even column in the low nibble, cacheir/quantization.py:123-130). The
    reference has the `group_size` field (cacheir/quantization.py:25) but no packer for it; its nearest
    relative is the GGUF Q4_0 block format, `(nibble - 8) * d` (cacheir/importers/gguf.py:297-310).
    scale = max|w| / 7 per group (rounded to fp16), code = clip(rint(w / scale) + 8, 0, 15)."""
    w = weight.to(dtype=torch.float32).contiguous()
    n, k = int(w.shape[0]), int(w.shape[1])
    if w.dim() != 2 or k % group_size != 0 or group_size % 2 != 0:
        raise ValueError("group-wise int4 needs a 2D weight whose width is a multiple of the (even) group size")
    groups = w.view(n, k // group_size, group_size)
    scales = (groups.abs().amax(dim=2) / 7.0).clamp_min(1e-8).to(torch.float16)
    q = torch.clamp(torch.round(groups / scales.float().unsqueeze(2)) + 8.0, 0.0, 15.0).to(torch.uint8).view(n, k)
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()
    return B200PackedWeight(packed, scales.contiguous(), None, 4, (n, k), group_size=group_size)


def pack_weight_device(weight: torch.Tensor, quant: str | None) -> B200PackedWeight | None:
    """`pack_quantized_weight` (cacheir/quantization.py:63-71) on the GPU; None when `quant` names no packed format.
    A group size in the name ("int4_g128") selects the group-wise symmetric int4 extension."""
    bits = quant_bits(quant)
    if bits is None:
        return None
    w = weight.to(dtype=torch.float32).contiguous()
    if w.dim() != 2:
        raise ValueError("packed quantization expects a 2D out_features x in_features weight")
    group = quant_group_size(quant)
    if group:
        if bits != 4:
            raise ValueError("group-wise quantization is defined for int4 only")
        return pack_group_int4(w, group)
    packed, scales, zp_i, zp_f = ops.pack_rows(w, bits)
    return B200PackedWeight(packed, scales, zp_f, bits, (int(w.shape[0]), int(w.shape[1])), zero_points_i32=zp_i)


def upload_reference_pack(packed: Any, device: torch.device | str) -> B200PackedWeight:
    """Upload a host `PackedQuantizedTensor`-like object (numpy fields packed_values, scales, zero_points, bits,
    shape, group_size) the way `CudaWeightStore.get_quantized` does (cacheir/runtime/cuda.py:77-94)."""
    values = torch.from_numpy(packed.packed_values).to(device).contiguous()
    group = int(packed.group_size) if getattr(packed, "group_size", None) else None
    if group:
        scales = torch.from_numpy(packed.scales).to(device).contiguous()   # keeps fp16 scales as fp16
        zero_points = None
    else:
        scales = torch.from_numpy(packed.scales).to(device=device, dtype=torch.float32).contiguous()
        zero_points = torch.from_numpy(packed.zero_points).to(device=device, dtype=torch.float32).contiguous()
    return B200PackedWeight(values, scales, zero_points, int(packed.bits), (int(packed.shape[0]), int(packed.shape[1])),
                            group_size=group)


def concat_rows(weights: list[B200PackedWeight]) -> B200PackedWeight:
    """Stack packed weights along the output dimension (Q|K|V, gate|up): same K, bits and grouping."""
    first = weights[0]
    for w in weights[1:]:
        if w.bits != first.bits or w.shape[1] != first.shape[1] or w.group_size != first.group_size:
            raise ValueError("cannot concatenate packed weights of different formats")
    zero_points = None
    if first.zero_points is not None:
        zero_points = torch.cat([w.zero_points for w in weights]).contiguous()
    return B200PackedWeight(
        packed_values=torch.cat([w.packed_values for w in weights], dim=0).contiguous(),
        scales=torch.cat([w.scales for w in weights], dim=0).contiguous(),
        zero_points=zero_points,
        bits=first.bits,
        shape=(sum(w.shape[0] for w in weights), first.shape[1]),
        group_size=first.group_size,
    )


def to_tiled(w: B200PackedWeight, *, paired: bool = False) -> B200PackedWeight:
    """The same weight with its codes in the tile order of the tensor-core kernels (K % 128 == 0).
    `paired` is the [gate; up] form consumed by the SwiGLU epilogue of the integer kernel."""
    if w.tiled:
        if w.paired != paired:
            return to_tiled(to_rows(w), paired=paired)
        return w
    n, k = w.shape
    return B200PackedWeight(ops.pack_relayout(w.packed_values, n=n, k=k, bits=w.bits, paired=paired), w.scales, w.zero_points,
                            w.bits, w.shape, group_size=w.group_size, zero_points_i32=w.zero_points_i32, tiled=True,
                            paired=paired)


def to_rows(w: B200PackedWeight) -> B200PackedWeight:
    """Back to the reference's row-major `packed_values` (bit-exact)."""
    if not w.tiled:
        return w
    n, k = w.shape
    return B200PackedWeight(ops.pack_unrelayout(w.packed_values, n=n, k=k, bits=w.bits, paired=w.paired), w.scales,
                            w.zero_points, w.bits, w.shape, group_size=w.group_size, zero_points_i32=w.zero_points_i32,
                            tiled=False)


def dequantize_device(w: B200PackedWeight, dtype: torch.dtype) -> torch.Tensor:
    """`dequantize_packed_weight` (cacheir/quantization.py:74-84) on the GPU (load time)."""
    if w.group_size:      # group-wise symmetric int4: (code - 8) * scale[n, k // group]
        n, k = w.shape
        codes = to_rows(w).packed_values if w.tiled else w.packed_values
        q = torch.empty((n, k), device=codes.device, dtype=torch.float32)
        q[:, 0::2] = (codes & 0xF).float()
        q[:, 1::2] = (codes >> 4).float()
        scale = w.scales.float().reshape(n, -1).repeat_interleave(w.group_size, dim=1)
        return ((q - 8.0) * scale).to(dtype)
    return ops.dequantize_rows(w.packed_values, w.scales, w.zero_points, bits=w.bits, k=w.shape[1], dtype=dtype)


def quantized_matmul(x: torch.Tensor, w: B200PackedWeight, *, epilogue: int = ops.EPI_NONE,
                     residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
                     workspace: torch.Tensor | None = None) -> torch.Tensor:
    """`_quantized_matmul` (cacheir/runtime/cuda.py:932-940) without materialising the dense weight.
    `workspace` (ops.qgemv_workspace_bytes) enables the integer tensor-core path for int8 weights."""
    return ops.qgemv(x, w.packed_values, w.scales, w.zero_points, bits=w.bits, n=w.shape[0], k=w.shape[1],
                     group_size=w.group_size or 0, epilogue=epilogue, residual=residual, out=out, workspace=workspace,
                     tiled=w.tiled, paired=w.paired)
