// 16-bit fixed-point activations of the integer GEMM: one row of x becomes two planes of signed bytes, a scale and
// the sum of its integers. Shared by the pre-pass kernels and by kernels that produce the planes in their epilogue.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace cb200 {

constexpr float kQMax = 32639.f;      // 127*256 + 127: every value splits into two signed bytes

// Fixed-point conversion of one activation: q = rint(v * inv) in [-32639, 32639], split as q = 256*hi + lo with
// signed bytes. Adding 1.5*2^23 + 128 inside one fused multiply-add leaves q + 128 in the low 16 bits of the
// float (one rounding, to nearest even, no conversion instruction): byte 1 is hi, byte 0 ^ 0x80 is lo.
constexpr float kRoundMagic = 12582912.f + 128.f;
__device__ __forceinline__ uint32_t fixed_point_bits(float v, float inv) { return __float_as_uint(fmaf(v, inv, kRoundMagic)); }
// Four converted values -> the word of their high bytes, the word of their low bytes, and their sum.
__device__ __forceinline__ void split_four(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t* hi, uint32_t* lo, int* sum) {
  const uint32_t ab = __byte_perm(a, b, 0x5410), cd = __byte_perm(c, d, 0x5410);
  *hi = __byte_perm(ab, cd, 0x7531);
  *lo = __byte_perm(ab, cd, 0x6420) ^ 0x80808080u;
  *sum = __dp4a(static_cast<int>(*lo), 0x01010101, *sum + 256 * __dp4a(static_cast<int>(*hi), 0x01010101, 0));
}

// The planes are stored the way the GEMM consumes them: per 128-column k block one contiguous tile
// [2*mp rows][128 bytes] (rows [0,mp): high bytes, [mp,2mp): low bytes; rows >= M are zero), with the 16-byte chunks
// of row R in the XOR order of a 128-byte swizzle (chunk c at c ^ (R & 7)), so that one contiguous bulk copy per
// stage lands it ready for the tensor core. After the planes of a [mp][K] matrix come 64 scales (fp32) and 64 sums.
__device__ __forceinline__ size_t plane_offset(int mp, int R, int k) {
  const int kb = k >> 7, j = k & 127;
  return (static_cast<size_t>(kb) * 2 * mp + R) * 128 + ((((j >> 4) ^ (R & 7)) << 4) | (j & 15));
}

}  // namespace cb200
