// Paged decode attention over a shared KV page pool: general kernel (any head
// size, page size and element type), split-K partials and the deterministic
// combine, plus the C entry points.
//
// Mapping: one CTA per (context split, KV head x query-head chunk, sequence).
// All GC query heads of a GQA group that share a KV head are served from ONE
// read of each K/V row. Inside a warp a K/V row is spread over LPT lanes, each
// lane owning a 16-byte chunk (128-bit loads, a row is read as one contiguous
// 16*LPT-byte segment), so 32/LPT rows are in flight per warp instruction.
// Scores are reduced over the LPT lanes with shuffles; every lane group keeps
// its own online-softmax state, merged once per CTA in a fixed order.
#include <float.h>

#include "common.cuh"
#include "paged_attention_common.cuh"

namespace cb200 {
namespace {

constexpr int kWarps = 4;

// VEC consecutive cached values as fp32: elements of type T, or (KV8) unsigned bytes with the row's scale.
template <typename T, int VEC, bool KV8>
__device__ __forceinline__ void load_cached(const void* cache, size_t elem, float scale, float (&out)[VEC]) {
  if constexpr (!KV8) {
    VecIO<T, VEC>::ld(static_cast<const T*>(cache) + elem, out);
  } else {
    const uint8_t* src = static_cast<const uint8_t*>(cache) + elem;
    uint8_t bytes[VEC];
    if constexpr (VEC == 8) *reinterpret_cast<uint2*>(bytes) = *reinterpret_cast<const uint2*>(src);
    else if constexpr (VEC == 4) *reinterpret_cast<uint32_t*>(bytes) = *reinterpret_cast<const uint32_t*>(src);
    else bytes[0] = src[0];
#pragma unroll
    for (int v = 0; v < VEC; ++v) out[v] = (static_cast<float>(bytes[v]) - 128.f) * scale;
  }
}

template <typename T, int VEC, int LPT, int R, int GC, bool KV8>
__global__ void __launch_bounds__(kWarps * 32)
paged_decode_general_kernel(const AttnParams p) {
  constexpr int TPW = 32 / LPT;         // rows handled per warp instruction
  constexpr int SLOTS = kWarps * TPW;   // independent softmax streams per CTA
  extern __shared__ float smem[];
  float* s_m = smem;                    // [SLOTS][GC]
  float* s_l = smem + SLOTS * GC;       // [SLOTS][GC]
  float* s_acc = smem + 2 * SLOTS * GC; // [SLOTS][GC][DP]
  constexpr int DP = VEC * LPT * R;

  const int split = blockIdx.x;
  const int kvh = blockIdx.y / p.head_chunks;
  const int hc = blockIdx.y % p.head_chunks;
  const int b = blockIdx.z;
  const int D = p.head_dim;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int sub = lane % LPT;   // chunk owner inside a row
  const int slot_in_warp = lane / LPT;

  const int seq_len = p.seq_lens[b];
  const int t_begin = split * p.chunk_tokens;
  if (p.splits > 1 && t_begin >= seq_len) return;  // combine never reads this split
  const int t_end = min(seq_len, t_begin + p.chunk_tokens);

  const T* qb = static_cast<const T*>(p.q) + static_cast<size_t>(b) * p.q_stride;
  const int g0 = hc * GC;       // first head of this chunk inside the group
  const int h0 = kvh * p.group + g0;

  float qreg[GC][R][VEC];
  float acc[GC][R][VEC];
  float m[GC], l[GC];
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
    const bool head_ok = (g0 + g) < p.group;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d0 = (sub + r * LPT) * VEC;
      float tmp[VEC];
#pragma unroll
      for (int v = 0; v < VEC; ++v) tmp[v] = 0.f;
      if (head_ok && d0 < D) VecIO<T, VEC>::ld(qb + static_cast<size_t>(h0 + g) * D + d0, tmp);
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        qreg[g][r][v] = tmp[v] * p.scale_log2;
        acc[g][r][v] = 0.f;
      }
    }
  }

  const int32_t* pt = p.page_table + static_cast<size_t>(b) * p.max_pages;
  for (int tb = t_begin + warp * TPW; tb < t_end; tb += kWarps * TPW) {
    const int t = tb + slot_in_warp;
    const bool valid = t < t_end;
    float kf[R][VEC], vf[R][VEC];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int v = 0; v < VEC; ++v) { kf[r][v] = 0.f; vf[r][v] = 0.f; }
    if (valid) {
      const int page = pt[t / p.page_size];
      const size_t row = ((static_cast<size_t>(page) * p.kv_heads + kvh) * p.page_size +
                          (t % p.page_size)) * static_cast<size_t>(D);
      float ks = 1.f, vs = 1.f;
      if constexpr (KV8) {
        const __half* sc = static_cast<const __half*>(p.kv_scales) +
                           (static_cast<size_t>(page) * p.kv_heads + kvh) * 2 * p.page_size + (t % p.page_size);
        ks = __half2float(sc[0]);
        vs = __half2float(sc[p.page_size]);
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int d0 = (sub + r * LPT) * VEC;
        if (d0 < D) {
          load_cached<T, VEC, KV8>(p.k_cache, row + d0, ks, kf[r]);
          load_cached<T, VEC, KV8>(p.v_cache, row + d0, vs, vf[r]);
        }
      }
    }
    float s[GC];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      float part = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int v = 0; v < VEC; ++v) part = fmaf(qreg[g][r][v], kf[r][v], part);
#pragma unroll
      for (int off = LPT / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
      s[g] = part;
    }
    if (valid) {
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        const float m_new = fmaxf(m[g], s[g]);
        const float corr = exp2f(m[g] - m_new);  // first row: exp2(-inf) = 0
        const float pw = exp2f(s[g] - m_new);
        l[g] = fmaf(l[g], corr, pw);
        m[g] = m_new;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int v = 0; v < VEC; ++v) acc[g][r][v] = fmaf(acc[g][r][v], corr, pw * vf[r][v]);
      }
    }
  }

  // ---- merge the SLOTS streams of this CTA in slot order -----------------------
  const int slot = warp * TPW + slot_in_warp;
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    if (sub == 0) {
      s_m[slot * GC + g] = m[g];
      s_l[slot * GC + g] = l[g];
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int v = 0; v < VEC; ++v)
        s_acc[(slot * GC + g) * DP + (sub + r * LPT) * VEC + v] = acc[g][r][v];
  }
  __syncthreads();

  for (int idx = threadIdx.x; idx < GC * DP; idx += kWarps * 32) {
    const int g = idx / DP;
    const int d = idx % DP;
    if (d >= D || (g0 + g) >= p.group) continue;
    float m_tot = -INFINITY;
    for (int sl = 0; sl < SLOTS; ++sl) m_tot = fmaxf(m_tot, s_m[sl * GC + g]);
    float l_tot = 0.f, o = 0.f;
    for (int sl = 0; sl < SLOTS; ++sl) {
      const float mi = s_m[sl * GC + g];
      const float w = (mi == -INFINITY) ? 0.f : exp2f(mi - m_tot);
      l_tot = fmaf(s_l[sl * GC + g], w, l_tot);
      o = fmaf(s_acc[(sl * GC + g) * DP + d], w, o);
    }
    const int h = h0 + g;
    if (p.splits == 1) {
      T* ob = static_cast<T*>(p.out) + static_cast<size_t>(b) * p.out_stride;
      Elem<T>::st(ob + static_cast<size_t>(h) * D + d, l_tot > 0.f ? o / l_tot : 0.f);
    } else {
      const size_t unit = (static_cast<size_t>(b) * p.heads + h) * p.splits + split;
      p.ws_acc[unit * D + d] = o;
      if (d == 0) {
        p.ws_ml[unit * 2] = m_tot;
        p.ws_ml[unit * 2 + 1] = l_tot;
      }
    }
  }
}

template <typename T, int VEC, int LPT, int R, bool KV8 = false>
int launch_general_gc(const AttnParams& p0, cudaStream_t stream) {
  AttnParams p = p0;
  const int gc = p.group >= 8 ? 8 : (p.group > 2 ? 4 : (p.group > 1 ? 2 : 1));
  p.head_chunks = (p.group + gc - 1) / gc;
  const dim3 grid(p.splits, p.kv_heads * p.head_chunks, p.batch);
  const int tpw = 32 / LPT;
  const int dp = VEC * LPT * R;
  const size_t smem = static_cast<size_t>(kWarps * tpw) * gc * (2 + dp) * sizeof(float);
#define CB200_LAUNCH_GC(GCV)                                                              \
  do {                                                                                    \
    auto kern = paged_decode_general_kernel<T, VEC, LPT, R, GCV, KV8>;                    \
    if (smem > 48 * 1024) {                                                               \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           static_cast<int>(smem));                       \
      if (e != cudaSuccess) return static_cast<int>(e);                                   \
    }                                                                                     \
    kern<<<grid, kWarps * 32, smem, stream>>>(p);                                         \
  } while (0)
  switch (gc) {
    case 8: CB200_LAUNCH_GC(8); break;
    case 4: CB200_LAUNCH_GC(4); break;
    case 2: CB200_LAUNCH_GC(2); break;
    default: CB200_LAUNCH_GC(1); break;
  }
#undef CB200_LAUNCH_GC
  return launch_status();
}

template <typename T, int VEC, bool KV8 = false>
int launch_general(const AttnParams& p, bool vector_ok, cudaStream_t stream) {
  const int D = p.head_dim;
  if (VEC > 1 && vector_ok && D % VEC == 0) {
    const int lpt = D / VEC;
    if (lpt == 32) return launch_general_gc<T, VEC, 32, 1, KV8>(p, stream);
    if (lpt == 16) return launch_general_gc<T, VEC, 16, 1, KV8>(p, stream);
    if (lpt == 8) return launch_general_gc<T, VEC, 8, 1, KV8>(p, stream);
  }
  // scalar lanes: lane i owns dims i, i+32, ...
  if (D <= 32) return launch_general_gc<T, 1, 32, 1, KV8>(p, stream);
  if (D <= 256) return launch_general_gc<T, 1, 32, 8, KV8>(p, stream);
  return CACHEIR_B200_EUNSUPPORTED;
}

// ---- split combine: fixed split order => bit-reproducible ------------------------
template <typename T>
__global__ void combine_splits_kernel(const AttnParams p) {
  const int h = blockIdx.x;
  const int b = blockIdx.y;
  const int D = p.head_dim;
  const int seq_len = p.seq_lens[b];
  int n = seq_len <= 0 ? 0 : (seq_len + p.chunk_tokens - 1) / p.chunk_tokens;
  n = min(n, p.splits);
  const size_t unit0 = (static_cast<size_t>(b) * p.heads + h) * p.splits;
  float m_tot = -INFINITY;
  for (int s = 0; s < n; ++s) m_tot = fmaxf(m_tot, p.ws_ml[(unit0 + s) * 2]);
  T* ob = static_cast<T*>(p.out) + static_cast<size_t>(b) * p.out_stride + static_cast<size_t>(h) * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float l_tot = 0.f, o = 0.f;
    for (int s = 0; s < n; ++s) {
      const float mi = p.ws_ml[(unit0 + s) * 2];
      const float w = (mi == -INFINITY) ? 0.f : exp2f(mi - m_tot);
      l_tot = fmaf(p.ws_ml[(unit0 + s) * 2 + 1], w, l_tot);
      o = fmaf(p.ws_acc[(unit0 + s) * D + d], w, o);
    }
    Elem<T>::st(ob + d, l_tot > 0.f ? o / l_tot : 0.f);
  }
}

template <typename T>
int launch_combine(const AttnParams& p, cudaStream_t stream) {
  const dim3 grid(p.heads, p.batch);
  const int threads = p.head_dim <= 32 ? 32 : (p.head_dim <= 64 ? 64 : 128);
  combine_splits_kernel<T><<<grid, threads, 0, stream>>>(p);
  return launch_status();
}

}  // namespace

void resolve_attention_splits(int batch, int heads, int kv_heads, int max_pages, int page_size,
                              int requested, int* splits, int* chunk_tokens) {
  const long long max_ctx = static_cast<long long>(max_pages) * page_size;
  int s = requested;
  if (s <= 0) {
    // Every extra split costs a few microseconds (partials + the combine launch), so split only as
    // far as needed: chunks of at most 4096 tokens bound the tail of the longest sequence of a
    // ragged batch, and small batches get enough splits to put one CTA on each of the 148 SMs.
    s = static_cast<int>((max_ctx + 4095) / 4096);
    long long units = static_cast<long long>(batch) * kv_heads * ((heads / kv_heads + 15) / 16);
    if (units < 1) units = 1;   // fewer query heads than KV heads: rejected by the entry points, but this must not divide by zero
    // Long contexts with few (sequence, kv head) units: a ragged batch then leaves about one wave of CTAs of very
    // different lengths (log-uniform 1k..32k tokens, 128 units: 140 us with 4096-token chunks, 124 us with 2048).
    if (s >= 4 && units < 2 * kNumSMs) s *= 2;
    const long long want = (kNumSMs + units - 1) / units;
    if (s < want) s = static_cast<int>(want);
    const int cap = static_cast<int>((max_ctx + 255) / 256);
    if (s > cap) s = cap;
  }
  if (s > kMaxAttentionSplits) s = kMaxAttentionSplits;
  if (s < 1) s = 1;
  long long chunk = (max_ctx + s - 1) / s;
  chunk = ((chunk + page_size - 1) / page_size) * page_size;  // splits start on page boundaries
  if (chunk < page_size) chunk = page_size;
  s = static_cast<int>((max_ctx + chunk - 1) / chunk);
  if (s < 1) s = 1;
  *splits = s;
  *chunk_tokens = static_cast<int>(chunk);
}

}  // namespace cb200

using namespace cb200;

extern "C" size_t cacheir_b200_paged_attention_workspace_bytes(int batch_size, int num_heads,
                                                               int head_dim, int num_splits) {
  if (batch_size <= 0 || num_heads <= 0 || head_dim <= 0 || num_splits <= 1) return 0;
  return static_cast<size_t>(batch_size) * num_heads * num_splits * (head_dim + 2) * sizeof(float);
}

extern "C" int cacheir_b200_paged_attention_auto_splits(int batch_size, int num_heads,
                                                        int num_kv_heads, int max_pages_per_seq,
                                                        int page_size, int head_dim) {
  (void)head_dim;
  if (batch_size <= 0 || num_heads <= 0 || num_kv_heads <= 0 || max_pages_per_seq <= 0 ||
      page_size <= 0 || num_heads % num_kv_heads != 0)
    return 1;
  int s = 1, chunk = 0;
  resolve_attention_splits(batch_size, num_heads, num_kv_heads, max_pages_per_seq, page_size, 0, &s,
                           &chunk);
  return s;
}

namespace cb200 {
size_t qgemm_i8_workspace_bytes(int M, int K);
int i8_plane_rows(int M);
}

namespace {
// `gemm_workspace` non-null: the launch must also leave the output as the integer GEMM's activation planes
// (CACHEIR_B200_EUNSUPPORTED when the fast single-split kernel cannot take the case). `probe`: decide only, launch nothing.
int attention_dispatch(
    const void* q, const void* k_cache, const void* v_cache, const int32_t* page_table,
    const int32_t* seq_lens, void* out, int batch_size, int num_heads, int num_kv_heads,
    int max_pages_per_seq, int page_size, int head_dim, int dtype, long long q_batch_stride,
    long long out_batch_stride, float softmax_scale, int num_splits, void* workspace,
    size_t workspace_bytes, int num_slots, int kv_dtype, const void* kv_scales, void* gemm_workspace,
    size_t gemm_workspace_bytes, bool probe, void* stream) {
  if (batch_size <= 0 || num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0) return 0;
  if (max_pages_per_seq <= 0 || page_size <= 0 || num_slots < 0) return CACHEIR_B200_EINVAL;
  if (num_heads % num_kv_heads != 0) return CACHEIR_B200_EINVAL;
  if (!q || !k_cache || !v_cache || !page_table || !seq_lens || !out) return CACHEIR_B200_EINVAL;
  const int esize = dtype_size(dtype);
  if (esize == 0 || num_splits < 0) return CACHEIR_B200_EINVAL;
  if (kv_dtype != CACHEIR_B200_KV_SAME && kv_dtype != CACHEIR_B200_KV_INT8) return CACHEIR_B200_EINVAL;
  const bool kv8 = kv_dtype == CACHEIR_B200_KV_INT8;
  if (kv8 && !kv_scales) return CACHEIR_B200_EINVAL;
  if (head_dim > 256) return CACHEIR_B200_EUNSUPPORTED;
  if (batch_size > 65535 || static_cast<long long>(num_heads) > 65535) return CACHEIR_B200_ELIMIT;

  AttnParams p{};
  p.q = q; p.k_cache = k_cache; p.v_cache = v_cache;
  p.kv_scales = kv_scales; p.kv8 = kv8 ? 1 : 0; p.num_slots = num_slots;
  p.page_table = page_table; p.seq_lens = seq_lens; p.out = out;
  p.batch = batch_size; p.heads = num_heads; p.kv_heads = num_kv_heads;
  p.max_pages = max_pages_per_seq; p.page_size = page_size; p.head_dim = head_dim;
  p.group = num_heads / num_kv_heads;
  p.q_stride = q_batch_stride > 0 ? q_batch_stride : static_cast<long long>(num_heads) * head_dim;
  p.out_stride = out_batch_stride > 0 ? out_batch_stride : static_cast<long long>(num_heads) * head_dim;
  const float scale = softmax_scale > 0.f ? softmax_scale : 1.0f / sqrtf(static_cast<float>(head_dim));
  p.scale_log2 = scale * kLog2e;
  resolve_attention_splits(batch_size, num_heads, num_kv_heads, max_pages_per_seq, page_size,
                           num_splits, &p.splits, &p.chunk_tokens);
  if (p.splits > 1) {
    const size_t need = cacheir_b200_paged_attention_workspace_bytes(batch_size, num_heads, head_dim, p.splits);
    if (!workspace || workspace_bytes < need) return CACHEIR_B200_EWORKSPACE;
    if (!aligned_to(workspace, 16)) return CACHEIR_B200_EALIGN;
    p.ws_ml = static_cast<float*>(workspace);
    p.ws_acc = p.ws_ml + static_cast<size_t>(batch_size) * num_heads * p.splits * 2;
  }
  if (gemm_workspace) {
    const int k_total = num_heads * head_dim;
    if (!paged_attention_quantize_supported(p, dtype)) return CACHEIR_B200_EUNSUPPORTED;
    if (gemm_workspace_bytes < qgemm_i8_workspace_bytes(batch_size, k_total)) return CACHEIR_B200_EWORKSPACE;
    if (!aligned_to(gemm_workspace, 128) || !aligned_to(out, 8)) return CACHEIR_B200_EALIGN;
    p.quant_rows = i8_plane_rows(batch_size);
    p.quant_planes = static_cast<int8_t*>(gemm_workspace);
    p.quant_sx = reinterpret_cast<float*>(p.quant_planes + static_cast<size_t>(2 * p.quant_rows) * k_total);
    p.quant_qsum = reinterpret_cast<int*>(p.quant_sx + 64);
    if (probe) return 0;
  }
  cudaStream_t st = as_stream(stream);
  // 128-bit row chunks need 16-byte aligned rows everywhere they are used (8-bit pools: 8-byte chunks of the cached rows).
  const int kv_esize = kv8 ? 1 : esize;
  const bool vector_ok = aligned_to(q, 16) && aligned_to(k_cache, 16) && aligned_to(v_cache, 16) &&
                         (p.q_stride * esize) % 16 == 0 &&
                         (static_cast<long long>(head_dim) * esize) % 16 == 0 &&
                         (static_cast<long long>(head_dim) * kv_esize) % 8 == 0;
  int rc;
  if (paged_attention_fast_supported(p, dtype)) {
    rc = launch_paged_attention_fast(p, dtype, st);
  } else if (kv8) {
    switch (dtype) {
      case CACHEIR_B200_F32: rc = launch_general<float, 4, true>(p, vector_ok, st); break;
      case CACHEIR_B200_F16: rc = launch_general<__half, 8, true>(p, vector_ok, st); break;
      default: rc = launch_general<__nv_bfloat16, 8, true>(p, vector_ok, st); break;
    }
  } else
  switch (dtype) {
    case CACHEIR_B200_F32: rc = launch_general<float, 4>(p, vector_ok, st); break;
    case CACHEIR_B200_F16: rc = launch_general<__half, 8>(p, vector_ok, st); break;
    default: rc = launch_general<__nv_bfloat16, 8>(p, vector_ok, st); break;
  }
  if (rc != 0 || p.splits == 1) return rc;
  switch (dtype) {
    case CACHEIR_B200_F32: return launch_combine<float>(p, st);
    case CACHEIR_B200_F16: return launch_combine<__half>(p, st);
    default: return launch_combine<__nv_bfloat16>(p, st);
  }
}
}  // namespace

extern "C" int cacheir_b200_paged_attention_decode_batch_ex(
    const void* q, const void* k_cache, const void* v_cache, const int32_t* page_table,
    const int32_t* seq_lens, void* out, int batch_size, int num_heads, int num_kv_heads,
    int max_pages_per_seq, int page_size, int head_dim, int dtype, long long q_batch_stride,
    long long out_batch_stride, float softmax_scale, int num_splits, void* workspace,
    size_t workspace_bytes, int num_slots, int kv_dtype, const void* kv_scales, void* stream) {
  return attention_dispatch(q, k_cache, v_cache, page_table, seq_lens, out, batch_size, num_heads, num_kv_heads,
                            max_pages_per_seq, page_size, head_dim, dtype, q_batch_stride, out_batch_stride, softmax_scale,
                            num_splits, workspace, workspace_bytes, num_slots, kv_dtype, kv_scales, nullptr, 0, false, stream);
}

extern "C" int cacheir_b200_paged_attention_decode_batch_quantize(
    const void* q, const void* k_cache, const void* v_cache, const int32_t* page_table,
    const int32_t* seq_lens, void* out, int batch_size, int num_heads, int num_kv_heads,
    int max_pages_per_seq, int page_size, int head_dim, int dtype, long long q_batch_stride,
    float softmax_scale, int num_slots, void* gemm_workspace, size_t gemm_workspace_bytes, void* stream) {
  if (!gemm_workspace) return CACHEIR_B200_EINVAL;
  return attention_dispatch(q, k_cache, v_cache, page_table, seq_lens, out, batch_size, num_heads, num_kv_heads,
                            max_pages_per_seq, page_size, head_dim, dtype, q_batch_stride, 0, softmax_scale, 1, nullptr, 0,
                            num_slots, CACHEIR_B200_KV_SAME, nullptr, gemm_workspace, gemm_workspace_bytes, false, stream);
}

extern "C" int cacheir_b200_paged_attention_quantize_supported(int batch_size, int num_heads, int num_kv_heads,
                                                               int max_pages_per_seq, int page_size, int head_dim, int dtype) {
  if (batch_size <= 0 || num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0) return 0;
  // Dummy, suitably aligned addresses: the answer depends on extents and alignment only.
  void* aligned = reinterpret_cast<void*>(static_cast<uintptr_t>(1) << 20);
  const int rc = attention_dispatch(aligned, aligned, aligned, static_cast<const int32_t*>(aligned), static_cast<const int32_t*>(aligned),
                                    aligned, batch_size, num_heads, num_kv_heads, max_pages_per_seq, page_size, head_dim, dtype, 0, 0,
                                    0.f, 1, nullptr, 0, 0, CACHEIR_B200_KV_SAME, nullptr, aligned,
                                    qgemm_i8_workspace_bytes(batch_size, num_heads * head_dim), true, nullptr);
  return rc == 0 ? 1 : 0;
}

extern "C" int cacheir_b200_paged_attention_decode_batch(
    const void* q, const void* k_cache, const void* v_cache, const int32_t* page_table,
    const int32_t* seq_lens, void* out, int batch_size, int num_heads, int num_kv_heads,
    int max_pages_per_seq, int page_size, int head_dim, int dtype, long long q_batch_stride,
    long long out_batch_stride, float softmax_scale, int num_splits, void* workspace,
    size_t workspace_bytes, void* stream) {
  return cacheir_b200_paged_attention_decode_batch_ex(q, k_cache, v_cache, page_table, seq_lens, out, batch_size, num_heads,
                                                      num_kv_heads, max_pages_per_seq, page_size, head_dim, dtype, q_batch_stride,
                                                      out_batch_stride, softmax_scale, num_splits, workspace, workspace_bytes, 0,
                                                      CACHEIR_B200_KV_SAME, nullptr, stream);
}

// ---- allocation-free variant -------------------------------------------------------
// Split-K scratch that lives inside the library image: callers that cannot obtain
// device memory themselves use this instead of passing a workspace.
#define CB200_NOALLOC_WORKSPACE_BYTES (16u * 1024u * 1024u)
static __device__ __align__(256) float g_noalloc_attention_workspace[CB200_NOALLOC_WORKSPACE_BYTES / sizeof(float)];

namespace {
constexpr int kMaxDevices = 64;
// Device address of the array above, looked up once per device. In host code the
// array's name is only a handle for the runtime, never a pointer a kernel may use.
// (Host threads may fill a slot concurrently without a lock: every thread that looks the
// symbol up for a device gets the same address, so a racing store writes the same value.)
void* g_noalloc_ws_ptr[kMaxDevices] = {};
}  // namespace

extern "C" size_t cacheir_b200_paged_attention_noalloc_max_workspace_bytes(void) {
  return CB200_NOALLOC_WORKSPACE_BYTES;
}

extern "C" int cacheir_b200_paged_attention_decode_batch_noalloc(
    const void* q, const void* k_cache, const void* v_cache, const int32_t* page_table,
    const int32_t* seq_lens, void* out, int batch_size, int num_heads, int num_kv_heads,
    int max_pages_per_seq, int page_size, int head_dim, int dtype, long long q_batch_stride,
    long long out_batch_stride, float softmax_scale, int num_splits, void* stream) {
  if (batch_size <= 0 || num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0) return 0;
  if (max_pages_per_seq <= 0 || page_size <= 0 || num_splits < 0 || num_heads % num_kv_heads != 0) return CACHEIR_B200_EINVAL;
  int splits = 1, chunk = 0;
  resolve_attention_splits(batch_size, num_heads, num_kv_heads, max_pages_per_seq, page_size, num_splits,
                           &splits, &chunk);
  const size_t need = cacheir_b200_paged_attention_workspace_bytes(batch_size, num_heads, head_dim, splits);
  if (need > CB200_NOALLOC_WORKSPACE_BYTES) return CACHEIR_B200_ELIMIT;
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (device < 0 || device >= kMaxDevices) return CACHEIR_B200_ELIMIT;
  void* ws = g_noalloc_ws_ptr[device];
  if (ws == nullptr) {  // first call on this device: resolve the symbol with this device current
    err = cudaGetSymbolAddress(&ws, g_noalloc_attention_workspace);
    if (err != cudaSuccess) return static_cast<int>(err);
    g_noalloc_ws_ptr[device] = ws;
  }
  return cacheir_b200_paged_attention_decode_batch(
      q, k_cache, v_cache, page_table, seq_lens, out, batch_size, num_heads, num_kv_heads,
      max_pages_per_seq, page_size, head_dim, dtype, q_batch_stride, out_batch_stride, softmax_scale,
      num_splits, ws, CB200_NOALLOC_WORKSPACE_BYTES, stream);
}
