// Packed int4/int8 dequant-GEMV on the CUDA cores: y[M,N] = x[M,K] . deq(W)[N,K]^T.
//
// One warp owns one output row (or a gate/up row pair for the SwiGLU
// epilogue) and streams it with 128-bit loads: a lane's 16-byte unit holds 16
// int8 or 32 int4 codes, unpacked in registers (codes become fp32 through the
// 2^23 mantissa trick, no integer->float conversion instructions), multiplied
// against up to MT rows of x and reduced with warp shuffles. This kernel is
// the path for fp32 activations, for dense (unquantized) weights and for shapes
// the tensor-core kernel does not take.
#include "common.cuh"
#include "paged_attention_common.cuh"
#include "qgemv_common.cuh"

namespace cb200 {
namespace {

constexpr int kWarpsPerBlock = 8;

// 8 consecutive x elements as fp32 (k0 is a multiple of 8 and x rows are 16-byte aligned).
template <typename XT>
__device__ __forceinline__ void load_x8(const XT* p, float (&out)[8]) {
  VecIO<XT, 8>::ld(p, out);
}
template <>
__device__ __forceinline__ void load_x8<float>(const float* p, float (&out)[8]) {
  float a[4], b[4];
  VecIO<float, 4>::ld(p, a);
  VecIO<float, 4>::ld(p + 4, b);
#pragma unroll
  for (int i = 0; i < 4; ++i) { out[i] = a[i]; out[4 + i] = b[i]; }
}

__device__ __forceinline__ float code_from_byte(uint32_t word, int i) {
  // byte i of `word` placed in the mantissa of 2^23: exact integer -> fp32.
  return __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540u + i)) - 8388608.f;
}
__device__ __forceinline__ float code_from_nibble(uint32_t word, int i) {
  return __uint_as_float(((word >> (4 * i)) & 0xFu) | 0x4B000000u) - 8388608.f;
}

template <typename XT>
__device__ __forceinline__ float scale_at(const void* scales, int scale_dtype, size_t idx) {
  return scale_dtype == CACHEIR_B200_F16 ? __half2float(static_cast<const __half*>(scales)[idx])
                                         : static_cast<const float*>(scales)[idx];
}

// BITS: 8, 4 or 0 (dense weights of type XT).
template <typename XT, int BITS, int MT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
qgemv_cuda_core_kernel(const QGemvParams p) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_out = blockIdx.x * kWarpsPerBlock + warp;
  const int n_out_total = p.epilogue == CACHEIR_B200_EPI_SWIGLU ? p.N / 2 : p.N;
  if (n_out >= n_out_total) return;
  const int m0 = blockIdx.y * MT;
  const int K = p.K;
  const XT* x = static_cast<const XT*>(p.x);
  const int halves = p.epilogue == CACHEIR_B200_EPI_SWIGLU ? 2 : 1;
  // elements per lane and iteration: a 16-byte unit of codes, or 8 dense weights
  constexpr int EPU = BITS == 8 ? 16 : (BITS == 4 ? 32 : 8);
  const int k_main = p.vector_ok ? (K / EPU) * EPU : 0;
  const size_t row_bytes = BITS == 8 ? static_cast<size_t>(K)
                         : BITS == 4 ? static_cast<size_t>((K + 1) / 2)
                                     : static_cast<size_t>(K) * sizeof(XT);
  float result[2][MT];

  for (int half = 0; half < halves; ++half) {
    const int n = n_out + half * (p.N / 2);
    const uint8_t* wrow = static_cast<const uint8_t*>(p.packed) + static_cast<size_t>(n) * row_bytes;
    float zp = 0.f;
    if (BITS != 0) {
      zp = (p.group_size == 0 && p.zero_points) ? p.zero_points[n] : static_cast<float>(BITS > 0 ? (1 << (BITS > 0 ? BITS - 1 : 0)) : 0);
    }
    const int groups_per_row = p.group_size > 0 ? K / p.group_size : 1;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;

    for (int k0 = lane * EPU; k0 < k_main; k0 += 32 * EPU) {
      uint32_t words[4] = {0u, 0u, 0u, 0u};
      if (BITS != 0) {
        const uint4 raw = *reinterpret_cast<const uint4*>(wrow + (BITS == 8 ? k0 : k0 / 2));
        words[0] = raw.x; words[1] = raw.y; words[2] = raw.z; words[3] = raw.w;
      }
      float part[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) part[m] = 0.f;
#pragma unroll
      for (int c = 0; c < EPU / 8; ++c) {  // 8 weights at a time
        float w8[8];
        if (BITS == 8) {
#pragma unroll
          for (int i = 0; i < 8; ++i) w8[i] = code_from_byte(words[c * 2 + i / 4], i % 4) - zp;
        } else if (BITS == 4) {
#pragma unroll
          for (int i = 0; i < 8; ++i) w8[i] = code_from_nibble(words[c], i) - zp;
        } else {
          load_x8<XT>(reinterpret_cast<const XT*>(wrow) + k0 + c * 8, w8);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (m0 + m < p.M) {
            float x8[8];
            load_x8<XT>(x + static_cast<size_t>(m0 + m) * p.x_stride + k0 + c * 8, x8);
#pragma unroll
            for (int i = 0; i < 8; ++i) part[m] = fmaf(x8[i], w8[i], part[m]);
          }
        }
      }
      const float gs = p.group_size > 0
                           ? scale_at<XT>(p.scales, p.scale_dtype, static_cast<size_t>(n) * groups_per_row + k0 / p.group_size)
                           : 1.f;
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[m] = fmaf(part[m], gs, acc[m]);
    }
    // scalar remainder (and the whole row when 128-bit access is not possible)
    for (int k = k_main + lane; k < K; k += 32) {
      float w;
      if (BITS == 8) {
        w = static_cast<float>(wrow[k]) - zp;
      } else if (BITS == 4) {
        w = static_cast<float>((wrow[k >> 1] >> ((k & 1) * 4)) & 0xF) - zp;
      } else {
        w = Elem<XT>::ld(reinterpret_cast<const XT*>(wrow) + k);
      }
      if (p.group_size > 0)
        w *= scale_at<XT>(p.scales, p.scale_dtype, static_cast<size_t>(n) * groups_per_row + k / p.group_size);
#pragma unroll
      for (int m = 0; m < MT; ++m)
        if (m0 + m < p.M) acc[m] = fmaf(Elem<XT>::ld(x + static_cast<size_t>(m0 + m) * p.x_stride + k), w, acc[m]);
    }
    const float row_scale = (BITS != 0 && p.group_size == 0) ? scale_at<XT>(p.scales, p.scale_dtype, n) : 1.f;
#pragma unroll
    for (int m = 0; m < MT; ++m) result[half][m] = warp_sum(acc[m]) * row_scale;
  }

  if (lane == 0) {
    XT* y = static_cast<XT*>(p.y);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m0 + m >= p.M) continue;
      const size_t o = static_cast<size_t>(m0 + m) * n_out_total + n_out;
      float v = result[0][m];
      if (p.epilogue == CACHEIR_B200_EPI_SWIGLU) {
        v = silu_fast(v) * result[1][m];
      } else if (p.epilogue == CACHEIR_B200_EPI_RESIDUAL) {
        v += Elem<XT>::ld(static_cast<const XT*>(p.residual) + o);
      }
      Elem<XT>::st(y + o, v);
    }
  }
}

template <typename XT, int BITS>
int launch_mt(const QGemvParams& p, cudaStream_t stream) {
  const int n_out_total = p.epilogue == CACHEIR_B200_EPI_SWIGLU ? p.N / 2 : p.N;
  const int mt = p.M >= 8 ? 8 : (p.M > 2 ? 4 : p.M);
  const dim3 grid((n_out_total + kWarpsPerBlock - 1) / kWarpsPerBlock, (p.M + mt - 1) / mt);
  if (grid.y > 65535) return CACHEIR_B200_ELIMIT;
  switch (mt) {
    case 8: qgemv_cuda_core_kernel<XT, BITS, 8><<<grid, kWarpsPerBlock * 32, 0, stream>>>(p); break;
    case 4: qgemv_cuda_core_kernel<XT, BITS, 4><<<grid, kWarpsPerBlock * 32, 0, stream>>>(p); break;
    case 2: qgemv_cuda_core_kernel<XT, BITS, 2><<<grid, kWarpsPerBlock * 32, 0, stream>>>(p); break;
    default: qgemv_cuda_core_kernel<XT, BITS, 1><<<grid, kWarpsPerBlock * 32, 0, stream>>>(p); break;
  }
  return launch_status();
}

template <typename XT>
int launch_bits(const QGemvParams& p, cudaStream_t stream) {
  switch (p.bits) {
    case 8: return launch_mt<XT, 8>(p, stream);
    case 4: return launch_mt<XT, 4>(p, stream);
    default: return launch_mt<XT, 0>(p, stream);
  }
}

}  // namespace

int launch_qgemv_cuda_core(const QGemvParams& p, cudaStream_t stream) {
  switch (p.x_dtype) {
    case CACHEIR_B200_F32: return launch_bits<float>(p, stream);
    case CACHEIR_B200_F16: return launch_bits<__half>(p, stream);
    default: return launch_bits<__nv_bfloat16>(p, stream);
  }
}

}  // namespace cb200

using namespace cb200;

extern "C" size_t cacheir_b200_qgemv_workspace_bytes(int M, int K) { return qgemm_i8_workspace_bytes(M, K); }

namespace {

// Shared body of cacheir_b200_qgemv_ex and cacheir_b200_rmsnorm_qgemv (norm_weight == nullptr: no norm).
int qgemv_dispatch(const void* x, const void* norm_weight, float norm_eps, const void* packed, const void* scales,
                   const float* zero_points, const void* residual, void* y, int M, int N, int K, int bits, int group_size,
                   int x_dtype, int scale_dtype, long long x_stride, int epilogue, int weight_layout, void* workspace,
                   size_t workspace_bytes, void* stream, bool plan_only) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (!plan_only && (!x || !packed || !y)) return CACHEIR_B200_EINVAL;
  const int esize = dtype_size(x_dtype);
  if (esize == 0) return CACHEIR_B200_EINVAL;
  if (bits != 0 && bits != 4 && bits != 8) return CACHEIR_B200_EINVAL;
  if (epilogue < CACHEIR_B200_EPI_NONE || epilogue > CACHEIR_B200_EPI_SWIGLU) return CACHEIR_B200_EINVAL;
  if (epilogue == CACHEIR_B200_EPI_SWIGLU && (N % 2) != 0) return CACHEIR_B200_EINVAL;
  if (!plan_only && epilogue == CACHEIR_B200_EPI_RESIDUAL && !residual) return CACHEIR_B200_EINVAL;
  if (bits != 0) {
    if (!plan_only && !scales) return CACHEIR_B200_EINVAL;
    if (scale_dtype != CACHEIR_B200_F32 && scale_dtype != CACHEIR_B200_F16) return CACHEIR_B200_EINVAL;
    if (group_size < 0) return CACHEIR_B200_EINVAL;
    if (group_size > 0 && (group_size % 32 != 0 || K % group_size != 0 || zero_points != nullptr))
      return CACHEIR_B200_EINVAL;
  } else if (group_size != 0) {
    return CACHEIR_B200_EINVAL;
  }
  QGemvParams p{};
  p.x = x; p.packed = packed; p.scales = scales; p.zero_points = zero_points;
  p.residual = residual; p.y = y;
  p.M = M; p.N = N; p.K = K; p.bits = bits; p.group_size = group_size;
  p.x_dtype = x_dtype; p.scale_dtype = scale_dtype;
  p.x_stride = x_stride > 0 ? x_stride : K;
  p.epilogue = epilogue;
  p.norm_weight = norm_weight; p.norm_eps = norm_eps;
  constexpr int kAllFlags = CACHEIR_B200_LAYOUT_TILED | CACHEIR_B200_X_PREQUANTIZED | CACHEIR_B200_LAYOUT_PAIRED;
  if (weight_layout < 0 || (weight_layout & ~kAllFlags) != 0) return CACHEIR_B200_EINVAL;
  p.tiled = (weight_layout & CACHEIR_B200_LAYOUT_TILED) != 0;
  p.paired = (weight_layout & CACHEIR_B200_LAYOUT_PAIRED) != 0;
  if (p.paired && !(p.tiled && epilogue == CACHEIR_B200_EPI_SWIGLU)) return CACHEIR_B200_EINVAL;
  p.x_prequantized = (weight_layout & CACHEIR_B200_X_PREQUANTIZED) != 0;
  if (p.x_prequantized && norm_weight) return CACHEIR_B200_EINVAL;
  const size_t row_bytes = bits == 8 ? static_cast<size_t>(K)
                         : bits == 4 ? static_cast<size_t>((K + 1) / 2)
                                     : static_cast<size_t>(K) * esize;
  p.vector_ok = aligned_to(packed, 16) && row_bytes % 16 == 0 && aligned_to(x, 16) &&
                (p.x_stride * esize) % 16 == 0;
  cudaStream_t st = as_stream(stream);
  if (M > 64 && !p.x_prequantized && !norm_weight) {
    // The integer tensor-core kernel takes up to 64 batch rows per launch, the fp16 one up to 128. A taller
    // batch runs as chunks of that height (the weights stream once per chunk, still far cheaper than the
    // CUDA-core kernel at these heights) when a chunk-sized problem of the same shape is tensor-core eligible.
    QGemvParams c = p;
    c.M = 64;
    const bool i8_ok = qgemm_i8_supported(c, workspace, workspace_bytes);
    if (i8_ok || (!c.paired && qgemm_tc_supported(c))) {
      if (plan_only) return i8_ok ? ((1 << 8) | qgemm_i8_plan(c)) : (2 << 8);
      const int rows = i8_ok ? 64 : 128;
      const size_t n_out = epilogue == CACHEIR_B200_EPI_SWIGLU ? static_cast<size_t>(N) / 2 : static_cast<size_t>(N);
      for (int m0 = 0; m0 < M; m0 += rows) {
        c.M = M - m0 < rows ? M - m0 : rows;
        c.x = static_cast<const char*>(x) + static_cast<size_t>(m0) * p.x_stride * esize;
        c.y = static_cast<char*>(y) + static_cast<size_t>(m0) * n_out * esize;
        c.residual = residual ? static_cast<const char*>(residual) + static_cast<size_t>(m0) * n_out * esize : nullptr;
        const int rc = i8_ok ? launch_qgemm_i8(c, workspace, st) : launch_qgemm_tc(c, st);
        if (rc != 0) return rc;
      }
      return 0;
    }
  }
  // up to 8 batch rows of int4 codes in row order: the streaming GEMV reads every code once and needs no pre-pass
  if (qgemv_mma_supported(p)) return plan_only ? (4 << 8) : launch_qgemv_mma(p, st);
  if (qgemm_i8_supported(p, workspace, workspace_bytes))
    return plan_only ? ((1 << 8) | qgemm_i8_plan(p)) : launch_qgemm_i8(p, workspace, st);
  if (norm_weight) return CACHEIR_B200_EUNSUPPORTED;  // the fused norm exists on the integer path only: run cacheir_b200_rms_norm first
  if (p.x_prequantized) return CACHEIR_B200_EINVAL;   // only the integer path can consume a quantized workspace
  if (p.paired) return CACHEIR_B200_EUNSUPPORTED;     // only the integer tensor-core kernel reads paired tiles
  if (qgemm_tc_supported(p)) return plan_only ? (2 << 8) : launch_qgemm_tc(p, st);
  if (p.tiled) return CACHEIR_B200_EUNSUPPORTED;   // the tile order only exists for the tensor-core kernels
  return plan_only ? (3 << 8) : launch_qgemv_cuda_core(p, st);
}

}  // namespace

extern "C" int cacheir_b200_qgemv_ex(const void* x, const void* packed, const void* scales,
                                     const float* zero_points, const void* residual, void* y, int M,
                                     int N, int K, int bits, int group_size, int x_dtype,
                                     int scale_dtype, long long x_stride, int epilogue, int weight_layout,
                                     void* workspace, size_t workspace_bytes, void* stream) {
  return qgemv_dispatch(x, nullptr, 0.f, packed, scales, zero_points, residual, y, M, N, K, bits, group_size, x_dtype,
                        scale_dtype, x_stride, epilogue, weight_layout, workspace, workspace_bytes, stream, false);
}

extern "C" int cacheir_b200_rmsnorm_qgemv(const void* x, const void* norm_weight, float eps, const void* packed,
                                          const void* scales, const float* zero_points, const void* residual, void* y,
                                          int M, int N, int K, int bits, int scale_dtype, long long x_stride, int epilogue,
                                          int weight_layout, void* workspace, size_t workspace_bytes, void* stream) {
  if (M > 0 && N > 0 && K > 0 && !norm_weight) return CACHEIR_B200_EINVAL;
  return qgemv_dispatch(x, norm_weight, eps, packed, scales, zero_points, residual, y, M, N, K, bits, 0, CACHEIR_B200_F16,
                        scale_dtype, x_stride, epilogue, weight_layout, workspace, workspace_bytes, stream, false);
}

extern "C" int cacheir_b200_qgemv_plan(int M, int N, int K, int bits, int group_size, int epilogue, int weight_layout,
                                       int with_workspace) {
  // Dummy, suitably aligned addresses: the choice depends on extents, flags and alignment only.
  void* aligned = reinterpret_cast<void*>(static_cast<uintptr_t>(1) << 20);
  const size_t ws_bytes = with_workspace ? qgemm_i8_workspace_bytes(M, K) : 0;
  if (epilogue == kEpiQkvRopeAppend) {
    QGemvParams p{};
    p.x = aligned; p.packed = aligned; p.scales = aligned; p.y = aligned;
    p.M = M; p.N = N; p.K = K; p.bits = 8; p.x_dtype = CACHEIR_B200_F16; p.x_stride = K; p.epilogue = kEpiQkvRopeAppend;
    p.tiled = (weight_layout & CACHEIR_B200_LAYOUT_TILED) != 0;
    p.x_prequantized = (weight_layout & CACHEIR_B200_X_PREQUANTIZED) != 0;
    if (!qgemm_i8_supported(p, with_workspace ? aligned : nullptr, ws_bytes)) return CACHEIR_B200_EUNSUPPORTED;
    return (1 << 8) | qgemm_i8_plan(p);
  }
  return qgemv_dispatch(aligned, nullptr, 0.f, aligned, aligned, nullptr, aligned, aligned, M, N, K, bits, group_size, CACHEIR_B200_F16,
                        CACHEIR_B200_F32, K, epilogue, weight_layout, with_workspace ? aligned : nullptr, ws_bytes, nullptr, true);
}

extern "C" int cacheir_b200_qgemv(const void* x, const void* packed, const void* scales,
                                  const float* zero_points, const void* residual, void* y, int M,
                                  int N, int K, int bits, int group_size, int x_dtype,
                                  int scale_dtype, long long x_stride, int epilogue, void* stream) {
  return cacheir_b200_qgemv_ex(x, packed, scales, zero_points, residual, y, M, N, K, bits, group_size, x_dtype,
                               scale_dtype, x_stride, epilogue, CACHEIR_B200_LAYOUT_ROWS, nullptr, 0, stream);
}

namespace cb200 {
int peer_collectives_device_status(bool reset);
}

extern "C" int cacheir_b200_device_status(int reset) {
  const int gemm = qgemm_tc_device_status(reset != 0);
  const int attn = paged_attention_device_status(reset != 0);
  const int i8 = qgemm_i8_device_status(reset != 0);
  const int peer = peer_collectives_device_status(reset != 0);
  const int gemv = qgemv_mma_device_status(reset != 0);
  return gemm != 0 ? gemm : (attn != 0 ? attn : (i8 != 0 ? i8 : (peer != 0 ? peer : gemv)));
}

extern "C" int cacheir_b200_quantize_activations(const void* x, int M, int K, long long x_stride, int x_dtype,
                                                 void* workspace, size_t workspace_bytes, void* stream) {
  if (M <= 0 || K <= 0) return 0;
  if (!x || x_dtype != CACHEIR_B200_F16 || M > 64 || K % 128 != 0) return CACHEIR_B200_EUNSUPPORTED;
  if (!workspace || workspace_bytes < qgemm_i8_workspace_bytes(M, K) || !aligned_to(workspace, 128)) return CACHEIR_B200_EWORKSPACE;
  const long long stride = x_stride > 0 ? x_stride : K;
  if (!aligned_to(x, 16) || (stride * 2) % 16 != 0) return CACHEIR_B200_EALIGN;
  return qgemm_i8_quantize_activations(x, stride, M, K, workspace, as_stream(stream));
}

extern "C" int cacheir_b200_rms_norm_quantize(const void* x, const void* residual, const void* weight, void* sum_out,
                                              void* out, int rows, int hidden, float eps, int dtype, void* workspace,
                                              size_t workspace_bytes, void* stream) {
  if (rows <= 0 || hidden <= 0) return 0;
  if (!x || !weight || (residual && !sum_out)) return CACHEIR_B200_EINVAL;
  if (dtype != CACHEIR_B200_F16 || rows > 64 || hidden % 128 != 0 || hidden > 8192) return CACHEIR_B200_EUNSUPPORTED;
  if (!workspace || workspace_bytes < qgemm_i8_workspace_bytes(rows, hidden) || !aligned_to(workspace, 128)) return CACHEIR_B200_EWORKSPACE;
  if (!aligned_to(x, 16) || !aligned_to(weight, 16) || (residual && (!aligned_to(residual, 16) || !aligned_to(sum_out, 16))) ||
      (out && !aligned_to(out, 16)))
    return CACHEIR_B200_EALIGN;
  return qgemm_i8_rms_norm_quantize(x, residual, weight, sum_out, out, rows, hidden, eps, workspace, as_stream(stream));
}

static int qkv_rope_append_dispatch(const void* x, const void* norm_weight, float norm_eps, const void* packed, const void* scales,
                                    const float* zero_points, void* qkv, int M, int N, int K, int scale_dtype, long long x_stride,
                                    int weight_layout, int q_dim, int k_dim, int head_dim, float theta,
                                    const float* rope_table, int rope_table_positions, const int32_t* positions,
                                    const int32_t* page_table, int max_pages_per_seq, int page_size, void* k_cache,
                                    void* v_cache, void* workspace, size_t workspace_bytes, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (!packed || !scales || !qkv || !positions || !page_table || !k_cache || !v_cache) return CACHEIR_B200_EINVAL;
  if (head_dim <= 0 || (head_dim % 2) != 0 || q_dim <= 0 || k_dim <= 0 || q_dim % head_dim != 0 || k_dim % head_dim != 0 ||
      N != q_dim + 2 * k_dim || max_pages_per_seq <= 0 || page_size <= 0)
    return CACHEIR_B200_EINVAL;
  if (scale_dtype != CACHEIR_B200_F32 && scale_dtype != CACHEIR_B200_F16) return CACHEIR_B200_EINVAL;
  if (weight_layout < 0 || (weight_layout & ~(CACHEIR_B200_LAYOUT_TILED | CACHEIR_B200_X_PREQUANTIZED)) != 0) return CACHEIR_B200_EINVAL;
  if (!rope_table || rope_table_positions <= 0 || !aligned_to(rope_table, 8)) return CACHEIR_B200_EINVAL;
  QGemvParams p{};
  p.x = x; p.packed = packed; p.scales = scales; p.zero_points = zero_points; p.residual = nullptr; p.y = qkv;
  p.M = M; p.N = N; p.K = K; p.bits = 8; p.group_size = 0;
  p.x_dtype = CACHEIR_B200_F16; p.scale_dtype = scale_dtype;
  p.x_stride = x_stride > 0 ? x_stride : K;
  p.epilogue = kEpiQkvRopeAppend;
  p.tiled = (weight_layout & CACHEIR_B200_LAYOUT_TILED) != 0;
  p.x_prequantized = (weight_layout & CACHEIR_B200_X_PREQUANTIZED) != 0;
  p.norm_weight = norm_weight; p.norm_eps = norm_eps;
  if (!p.x_prequantized && !x) return CACHEIR_B200_EINVAL;
  if (p.x_prequantized && norm_weight) return CACHEIR_B200_EINVAL;
  p.vector_ok = true;
  p.rope.table = rope_table; p.rope.table_positions = rope_table_positions;
  p.rope.positions = positions; p.rope.page_table = page_table; p.rope.k_cache = k_cache; p.rope.v_cache = v_cache;
  p.rope.q_dim = q_dim; p.rope.k_dim = k_dim; p.rope.head_dim = head_dim; p.rope.kv_heads = k_dim / head_dim;
  p.rope.max_pages = max_pages_per_seq; p.rope.page_size = page_size; p.rope.theta = theta;
  // only the integer tensor-core kernel carries this epilogue; other shapes use the separate kernels
  if (!qgemm_i8_supported(p, workspace, workspace_bytes)) return CACHEIR_B200_EUNSUPPORTED;
  return launch_qgemm_i8(p, workspace, as_stream(stream));
}

extern "C" int cacheir_b200_qkv_rope_append(const void* x, const void* packed, const void* scales, const float* zero_points,
                                            void* qkv, int M, int N, int K, int scale_dtype, long long x_stride,
                                            int weight_layout, int q_dim, int k_dim, int head_dim, float theta,
                                            const float* rope_table, int rope_table_positions, const int32_t* positions,
                                            const int32_t* page_table, int max_pages_per_seq, int page_size, void* k_cache,
                                            void* v_cache, void* workspace, size_t workspace_bytes, void* stream) {
  return qkv_rope_append_dispatch(x, nullptr, 0.f, packed, scales, zero_points, qkv, M, N, K, scale_dtype, x_stride, weight_layout,
                                  q_dim, k_dim, head_dim, theta, rope_table, rope_table_positions, positions, page_table,
                                  max_pages_per_seq, page_size, k_cache, v_cache, workspace, workspace_bytes, stream);
}

extern "C" int cacheir_b200_rmsnorm_qkv_rope_append(const void* x, const void* norm_weight, float eps, const void* packed,
                                                    const void* scales, const float* zero_points, void* qkv, int M, int N, int K,
                                                    int scale_dtype, long long x_stride, int weight_layout, int q_dim, int k_dim,
                                                    int head_dim, float theta, const float* rope_table, int rope_table_positions,
                                                    const int32_t* positions, const int32_t* page_table, int max_pages_per_seq,
                                                    int page_size, void* k_cache, void* v_cache, void* workspace,
                                                    size_t workspace_bytes, void* stream) {
  if (M > 0 && N > 0 && K > 0 && (!norm_weight || !x)) return CACHEIR_B200_EINVAL;
  return qkv_rope_append_dispatch(x, norm_weight, eps, packed, scales, zero_points, qkv, M, N, K, scale_dtype, x_stride, weight_layout,
                                  q_dim, k_dim, head_dim, theta, rope_table, rope_table_positions, positions, page_table,
                                  max_pages_per_seq, page_size, k_cache, v_cache, workspace, workspace_bytes, stream);
}
