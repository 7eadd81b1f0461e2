// Quantization loader on the device: per-row asymmetric int8/int4 packing that
// reproduces the NumPy packer of the reference bit for bit, and its inverse.
//
// NumPy semantics reproduced here (cacheir/quantization.py:96-130):
//   scale = max((max - min) / qmax, 1e-8)            all in float32
//   zero  = rint(0 - min / scale)  -> int32          float32 divide, half-to-even
//   code  = clip(rint(double(w / scale) + double(zero)), 0, qmax) -> uint8
// (the float32 quotient plus an int32 array promotes to float64 in NumPy).
// int4 packs two codes per byte, even column in the low nibble, odd K padded
// with a zero nibble.
#include "common.cuh"

namespace cb200 {
namespace {

template <int BITS>
__global__ void __launch_bounds__(256)
pack_rows_kernel(const float* __restrict__ weight, uint8_t* __restrict__ packed, float* __restrict__ scales,
                 int32_t* __restrict__ zp_i32, float* __restrict__ zp_f32, int K) {
  __shared__ float s_min[8], s_max[8];
  __shared__ float s_scale;
  __shared__ int s_zero;
  const size_t n = blockIdx.x;
  const float* w = weight + n * K;
  float lo = INFINITY, hi = -INFINITY;
  for (int k = threadIdx.x; k < K; k += 256) {
    const float v = w[k];
    lo = fminf(lo, v);
    hi = fmaxf(hi, v);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
  }
  if ((threadIdx.x & 31) == 0) { s_min[threadIdx.x >> 5] = lo; s_max[threadIdx.x >> 5] = hi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) { lo = fminf(lo, s_min[i]); hi = fmaxf(hi, s_max[i]); }
    constexpr float qmax = static_cast<float>((1 << BITS) - 1);
    const float scale = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), qmax), 1.0e-8f);
    const float zf = rintf(__fsub_rn(0.0f, __fdiv_rn(lo, scale)));
    const int zero = static_cast<int>(zf);
    s_scale = scale;
    s_zero = zero;
    scales[n] = scale;
    if (zp_i32) zp_i32[n] = zero;
    if (zp_f32) zp_f32[n] = static_cast<float>(zero);
  }
  __syncthreads();
  const float scale = s_scale;
  const double zero = static_cast<double>(s_zero);
  constexpr double qmax_d = static_cast<double>((1 << BITS) - 1);
  if (BITS == 8) {
    uint8_t* dst = packed + n * K;
    for (int k = threadIdx.x; k < K; k += 256) {
      double q = rint(static_cast<double>(__fdiv_rn(w[k], scale)) + zero);
      q = fmin(fmax(q, 0.0), qmax_d);
      dst[k] = static_cast<uint8_t>(q);
    }
  } else {
    const int row_bytes = (K + 1) / 2;
    uint8_t* dst = packed + n * row_bytes;
    for (int j = threadIdx.x; j < row_bytes; j += 256) {
      uint32_t byte = 0;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int k = 2 * j + e;
        if (k < K) {
          double q = rint(static_cast<double>(__fdiv_rn(w[k], scale)) + zero);
          q = fmin(fmax(q, 0.0), qmax_d);
          byte |= (static_cast<uint32_t>(q) & 0xFu) << (4 * e);
        }
      }
      dst[j] = static_cast<uint8_t>(byte);
    }
  }
}

template <typename T, int BITS>
__global__ void dequantize_rows_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                                       const float* __restrict__ zero_points, T* __restrict__ out, int K) {
  const size_t n = blockIdx.x;
  const float scale = scales[n];
  const float zero = zero_points ? zero_points[n] : static_cast<float>(1 << (BITS - 1));
  const int row_bytes = BITS == 8 ? K : (K + 1) / 2;
  const uint8_t* src = packed + n * row_bytes;
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const uint32_t code = BITS == 8 ? src[k] : ((src[k >> 1] >> ((k & 1) * 4)) & 0xFu);
    // (float(code) - zero) * scale, each step rounded to fp32 like the NumPy expression
    Elem<T>::st(out + n * K + k, __fmul_rn(__fsub_rn(static_cast<float>(code), zero), scale));
  }
}

// Tile-major device layout of the packed codes: the matrix is cut into tiles of 128 rows x 128
// k elements (128 bytes per row for int8, 64 for int4) and each tile is stored contiguously,
// tiles of one 128-row band following each other along K:
//   tiled[((band * KB + kb) * 128 + r) * TB + swz(r, j)] = packed[(band*128 + r) * row_bytes + kb*TB + j]
// Inside a tile the 16-byte chunks of row r are stored in the XOR order that a 128-byte (int8) or
// 64-byte (int4) swizzled TMA copy would produce in shared memory -- chunk c of row r sits at
// c ^ (r & 7), respectively c ^ ((r >> 1) & 3) -- so a plain contiguous bulk copy of the tile lands
// in the bank-conflict-free layout the kernels read. A pure permutation of bytes (rows past N are
// zero), so it is exactly invertible.
template <bool INVERSE>
__global__ void __launch_bounds__(256)
relayout_tiles_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int N, int row_bytes, int tile_bytes_per_row,
                      int paired) {
  const int kb = blockIdx.x;
  const int band = blockIdx.y;
  const int kblocks = row_bytes / tile_bytes_per_row;
  const int chunks_per_row = tile_bytes_per_row / 16;
  for (int idx = threadIdx.x; idx < 128 * chunks_per_row; idx += 256) {
    const int r = idx / chunks_per_row;
    const int c = idx % chunks_per_row;
    // paired: tile rows 0..63 are rows 64*band.. of the first half of W, rows 64..127 the same rows of the second half
    const int n = paired ? (r < 64 ? band * 64 + r : N / 2 + band * 64 + (r - 64)) : band * 128 + r;
    const int cs = chunks_per_row == 8 ? (c ^ (r & 7)) : (c ^ ((r >> 1) & 3));
    const size_t tiled_off = ((static_cast<size_t>(band) * kblocks + kb) * 128 + r) * tile_bytes_per_row + cs * 16;
    const size_t rows_off = static_cast<size_t>(n) * row_bytes + static_cast<size_t>(kb) * tile_bytes_per_row + c * 16;
    if (INVERSE) {
      if (n < N) *reinterpret_cast<uint4*>(dst + rows_off) = *reinterpret_cast<const uint4*>(src + tiled_off);
    } else {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (n < N) v = *reinterpret_cast<const uint4*>(src + rows_off);
      *reinterpret_cast<uint4*>(dst + tiled_off) = v;
    }
  }
}

}  // namespace
}  // namespace cb200

using namespace cb200;

extern "C" size_t cacheir_b200_pack_tiled_bytes(int N, int K, int bits) {
  if (N <= 0 || K <= 0 || (bits != 4 && bits != 8) || K % 128 != 0) return 0;
  const size_t row_bytes = bits == 8 ? static_cast<size_t>(K) : static_cast<size_t>(K / 2);
  return static_cast<size_t>((N + 127) / 128) * 128 * row_bytes;
}

static int relayout_impl(const uint8_t* src, uint8_t* dst, int N, int K, int bits, int paired, bool inverse, void* stream) {
  if (N <= 0 || K <= 0) return 0;
  if (!src || !dst || (bits != 4 && bits != 8) || K % 128 != 0) return CACHEIR_B200_EINVAL;
  if (paired && N % 128 != 0) return CACHEIR_B200_EINVAL;   // both halves must be whole 64-row groups
  if (!aligned_to(src, 16) || !aligned_to(dst, 16)) return CACHEIR_B200_EALIGN;
  const int row_bytes = bits == 8 ? K : K / 2;
  const int tile_bytes_per_row = bits == 8 ? 128 : 64;
  const dim3 grid(row_bytes / tile_bytes_per_row, (N + 127) / 128);
  if (grid.y > 65535) return CACHEIR_B200_ELIMIT;
  if (inverse) relayout_tiles_kernel<true><<<grid, 256, 0, as_stream(stream)>>>(src, dst, N, row_bytes, tile_bytes_per_row, paired);
  else relayout_tiles_kernel<false><<<grid, 256, 0, as_stream(stream)>>>(src, dst, N, row_bytes, tile_bytes_per_row, paired);
  return launch_status();
}

extern "C" int cacheir_b200_pack_relayout(const uint8_t* packed, uint8_t* tiled, int N, int K, int bits, int paired, void* stream) {
  return relayout_impl(packed, tiled, N, K, bits, paired != 0, false, stream);
}

extern "C" int cacheir_b200_pack_unrelayout(const uint8_t* tiled, uint8_t* packed, int N, int K, int bits, int paired, void* stream) {
  return relayout_impl(tiled, packed, N, K, bits, paired != 0, true, stream);
}

extern "C" int cacheir_b200_pack_rows(const float* weight, uint8_t* packed, float* scales,
                                      int32_t* zero_points_i32, float* zero_points_f32, int N,
                                      int K, int bits, void* stream) {
  if (N <= 0 || K <= 0) return 0;
  if (!weight || !packed || !scales) return CACHEIR_B200_EINVAL;
  if (bits == 8) {
    pack_rows_kernel<8><<<N, 256, 0, as_stream(stream)>>>(weight, packed, scales, zero_points_i32, zero_points_f32, K);
  } else if (bits == 4) {
    pack_rows_kernel<4><<<N, 256, 0, as_stream(stream)>>>(weight, packed, scales, zero_points_i32, zero_points_f32, K);
  } else {
    return CACHEIR_B200_EINVAL;
  }
  return launch_status();
}

extern "C" int cacheir_b200_dequantize_rows(const uint8_t* packed, const float* scales,
                                            const float* zero_points, void* out, int N, int K,
                                            int bits, int out_dtype, void* stream) {
  if (N <= 0 || K <= 0) return 0;
  if (!packed || !scales || !out) return CACHEIR_B200_EINVAL;
  if (bits != 4 && bits != 8) return CACHEIR_B200_EINVAL;
  cudaStream_t st = as_stream(stream);
#define CB200_DEQ(T)                                                                            \
  do {                                                                                          \
    if (bits == 8)                                                                              \
      dequantize_rows_kernel<T, 8><<<N, 256, 0, st>>>(packed, scales, zero_points, static_cast<T*>(out), K); \
    else                                                                                        \
      dequantize_rows_kernel<T, 4><<<N, 256, 0, st>>>(packed, scales, zero_points, static_cast<T*>(out), K); \
  } while (0)
  switch (out_dtype) {
    case CACHEIR_B200_F32: CB200_DEQ(float); break;
    case CACHEIR_B200_F16: CB200_DEQ(__half); break;
    case CACHEIR_B200_BF16: CB200_DEQ(__nv_bfloat16); break;
    default: return CACHEIR_B200_EINVAL;
  }
#undef CB200_DEQ
  return launch_status();
}
