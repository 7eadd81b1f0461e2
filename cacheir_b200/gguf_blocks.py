"""llama.cpp block formats Q4_0 and Q8_0 as native pack layouts.

The reference reads these blocks and dequantises them to fp32 at import
(`_decode_q4_0`, `_decode_q8_0`, cacheir/importers/gguf.py:273-310): a block is 32
consecutive elements of a row with one fp16 scale `d`;
Q4_0: 16 bytes of nibbles, low nibbles = elements 0..15, high nibbles = elements 16..31,
      value = (nibble - 8) * d;
Q8_0: 32 signed bytes, value = int8 * d.
Here the blocks are re-arranged -- an exact permutation of the integer codes, no
arithmetic on them -- into the group-wise symmetric layout the GEMV kernels stream:
codes [N, K] (int4: even column in the low nibble, like the reference's own int4 pack,
cacheir/quantization.py:123-130), fp16 scales [N, K/32], implicit zero point
2**(bits-1). Q8_0's signed bytes become codes = value + 128. The weights then stay
4/8-bit in HBM and are dequantised inside the kernel.
"""
from __future__ import annotations

import numpy as np
import torch

from .quantization import B200PackedWeight

BLOCK = 32
Q4_0_BLOCK_BYTES = 2 + 16
Q8_0_BLOCK_BYTES = 2 + 32


def _blocks(raw: bytes | np.ndarray, n: int, k: int, block_bytes: int) -> np.ndarray:
    if k % BLOCK != 0:
        raise ValueError("block formats need a row width that is a multiple of 32")
    data = np.frombuffer(raw, dtype=np.uint8) if isinstance(raw, (bytes, bytearray, memoryview)) else np.asarray(raw, dtype=np.uint8).reshape(-1)
    want = n * (k // BLOCK) * block_bytes
    if data.size != want:
        raise ValueError(f"expected {want} bytes of blocks for a {n}x{k} tensor, got {data.size}")
    return data.reshape(n, k // BLOCK, block_bytes)


def q4_0_to_packed(raw: bytes | np.ndarray, n: int, k: int, device: torch.device | str = "cpu") -> B200PackedWeight:
    """Row-major Q4_0 blocks of an [n, k] weight -> group-32 symmetric int4 pack."""
    blocks = _blocks(raw, n, k, Q4_0_BLOCK_BYTES)
    scales = blocks[:, :, :2].copy().view(np.float16).reshape(n, k // BLOCK)
    nibbles = blocks[:, :, 2:]                                    # [n, blocks, 16]
    codes = np.empty((n, k // BLOCK, BLOCK), dtype=np.uint8)
    codes[:, :, :16] = nibbles & 0x0F                             # elements 0..15
    codes[:, :, 16:] = nibbles >> 4                               # elements 16..31
    codes = codes.reshape(n, k)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return B200PackedWeight(torch.from_numpy(np.ascontiguousarray(packed)).to(device),
                            torch.from_numpy(np.ascontiguousarray(scales)).to(device), None, 4, (n, k), group_size=BLOCK)


def q8_0_to_packed(raw: bytes | np.ndarray, n: int, k: int, device: torch.device | str = "cpu") -> B200PackedWeight:
    """Row-major Q8_0 blocks of an [n, k] weight -> group-32 symmetric int8 pack (code = value + 128)."""
    blocks = _blocks(raw, n, k, Q8_0_BLOCK_BYTES)
    scales = blocks[:, :, :2].copy().view(np.float16).reshape(n, k // BLOCK)
    codes = (blocks[:, :, 2:].view(np.int8).astype(np.int16) + 128).astype(np.uint8).reshape(n, k)
    return B200PackedWeight(torch.from_numpy(np.ascontiguousarray(codes)).to(device),
                            torch.from_numpy(np.ascontiguousarray(scales)).to(device), None, 8, (n, k), group_size=BLOCK)
