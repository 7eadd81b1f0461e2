// Shared device/host helpers for the cacheir_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "cacheir_b200.h"

namespace cb200 {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

// ---- element access in fp32 -------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float ld(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ void st(__half* p, float v) { *p = __float2half_rn(v); }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// Load VEC consecutive elements (VEC*sizeof(T) is 16 bytes, or VEC == 1) as fp32.
template <typename T, int VEC>
struct VecIO;

template <typename T>
struct VecIO<T, 1> {
  static __device__ __forceinline__ void ld(const T* p, float (&out)[1]) { out[0] = Elem<T>::ld(p); }
  static __device__ __forceinline__ void st(T* p, const float (&in)[1]) { Elem<T>::st(p, in[0]); }
};
template <>
struct VecIO<float, 4> {
  static __device__ __forceinline__ void ld(const float* p, float (&out)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
  static __device__ __forceinline__ void st(float* p, const float (&in)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
  }
};
template <>
struct VecIO<__half, 8> {
  static __device__ __forceinline__ void ld(const __half* p, float (&out)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void st(__half* p, const float (&in)[8]) {
    uint4 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};
template <>
struct VecIO<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // bf16 -> fp32 is a 16-bit shift
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, const float (&in)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// silu(g) = g / (1 + e^-g) for the fused epilogues. The quotient uses the reciprocal unit directly:
// when e^-g overflows (g below about -88) the denominator is infinite and a full IEEE division would
// detour through its slow path on every such element; here the reciprocal is 0 and the result -0.
__device__ __forceinline__ float silu_fast(float g) { return __fdividef(g, 1.f + __expf(-g)); }

// ---- RoPE arithmetic shared by the stand-alone kernel, the table builder and the fused epilogue
// (one definition, so the three produce the same bits). Interleaved pairs (2i, 2i+1);
// angle = pos * theta^(-2i/D), evaluated in fp32 like the reference (cacheir/runtime/cuda.py:1072-1102).
__device__ __forceinline__ void rope_cos_sin(int pos, int i, int head_dim, float theta, float* c, float* s) {
  const float freq = 1.0f / powf(theta, static_cast<float>(i) * 2.0f / static_cast<float>(head_dim));
  const float angle = static_cast<float>(pos) * freq;
  sincosf(angle, s, c);
}
__device__ __forceinline__ void rope_rotate(float e, float o, float c, float s, float* re, float* ro) {
  *re = __fmaf_rn(e, c, -__fmul_rn(o, s));
  *ro = __fmaf_rn(e, s, __fmul_rn(o, c));
}

// ---- host side ----------------------------------------------------------------
inline int dtype_size(int dtype) {
  switch (dtype) {
    case CACHEIR_B200_F32: return 4;
    case CACHEIR_B200_F16: return 2;
    case CACHEIR_B200_BF16: return 2;
    default: return 0;
  }
}
inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline int launch_status() { return static_cast<int>(cudaGetLastError()); }
inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

}  // namespace cb200
