// Glue ops of the decode graph: RMSNorm (+fused residual add), RoPE, KV page
// append, SiLU*mul, add, embedding gather, row argmax and the per-step
// position bookkeeping. All of them touch a few hundred KB per step; they are
// written as single-pass, 128-bit-access kernels so that their cost is the
// launch, not the traffic.
#include "common.cuh"

namespace cb200 {
namespace {

// ---- RMSNorm ---------------------------------------------------------------------
// One CTA per row; the row is read once (optionally summed with a residual row,
// the sum being written back for the later residual connection) and kept in
// registers between the statistics pass and the scaling pass when it fits.
template <typename T, int VEC, int PER_THREAD>
__global__ void __launch_bounds__(256)
rms_norm_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ weight,
                T* __restrict__ sum_out, T* __restrict__ out, int hidden, float eps) {
  __shared__ float red[8];
  const size_t row = blockIdx.x;
  const T* xr = x + row * hidden;
  const T* rr = residual ? residual + row * hidden : nullptr;
  const int nvec = hidden / VEC;  // host guarantees hidden % VEC == 0 on this path
  float cache[PER_THREAD][VEC];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PER_THREAD; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      VecIO<T, VEC>::ld(xr + c * VEC, cache[i]);
      if (rr) {
        float r[VEC];
        VecIO<T, VEC>::ld(rr + c * VEC, r);
#pragma unroll
        for (int v = 0; v < VEC; ++v) cache[i][v] += r[v];
        // the residual stream carries the rounded sum, so normalise what is stored
        T tmp[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) { Elem<T>::st(&tmp[v], cache[i][v]); cache[i][v] = Elem<T>::ld(&tmp[v]); }
        VecIO<T, VEC>::st(sum_out + row * hidden + c * VEC, cache[i]);
      }
#pragma unroll
      for (int v = 0; v < VEC; ++v) ss = fmaf(cache[i][v], cache[i][v], ss);
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += red[w];
  const float inv = rsqrtf(tot / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int i = 0; i < PER_THREAD; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      float w[VEC], o[VEC];
      VecIO<T, VEC>::ld(weight + c * VEC, w);
#pragma unroll
      for (int v = 0; v < VEC; ++v) o[v] = cache[i][v] * inv * w[v];
      VecIO<T, VEC>::st(out + row * hidden + c * VEC, o);
    }
  }
}

// Any hidden size / alignment: two passes over global memory, scalar access.
template <typename T>
__global__ void __launch_bounds__(256)
rms_norm_generic_kernel(const T* __restrict__ x, const T* __restrict__ residual,
                        const T* __restrict__ weight, T* __restrict__ sum_out, T* __restrict__ out,
                        int hidden, float eps) {
  __shared__ float red[8];
  const size_t row = blockIdx.x;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += 256) {
    float v = Elem<T>::ld(x + row * hidden + c);
    if (residual) {
      v += Elem<T>::ld(residual + row * hidden + c);
      Elem<T>::st(sum_out + row * hidden + c, v);
      v = Elem<T>::ld(sum_out + row * hidden + c);
    }
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += red[w];
  const float inv = rsqrtf(tot / static_cast<float>(hidden) + eps);
  const T* src = residual ? sum_out : x;
  for (int c = threadIdx.x; c < hidden; c += 256)
    Elem<T>::st(out + row * hidden + c, Elem<T>::ld(src + row * hidden + c) * inv * Elem<T>::ld(weight + c));
}

template <typename T, int VEC>
int launch_rms_norm(const void* x, const void* residual, const void* weight, void* sum_out, void* out,
                    int rows, int hidden, float eps, cudaStream_t st) {
  const T* xp = static_cast<const T*>(x);
  const T* rp = static_cast<const T*>(residual);
  const T* wp = static_cast<const T*>(weight);
  T* sp = static_cast<T*>(sum_out);
  T* op = static_cast<T*>(out);
  const bool vec_ok = hidden % VEC == 0 && aligned_to(x, 16) && aligned_to(weight, 16) &&
                      aligned_to(out, 16) && (!residual || (aligned_to(residual, 16) && aligned_to(sum_out, 16)));
  const int nvec = hidden / VEC;
  if (vec_ok && nvec <= 256 * 2) {
    rms_norm_kernel<T, VEC, 2><<<rows, 256, 0, st>>>(xp, rp, wp, sp, op, hidden, eps);
  } else if (vec_ok && nvec <= 256 * 8) {
    rms_norm_kernel<T, VEC, 8><<<rows, 256, 0, st>>>(xp, rp, wp, sp, op, hidden, eps);
  } else {
    rms_norm_generic_kernel<T><<<rows, 256, 0, st>>>(xp, rp, wp, sp, op, hidden, eps);
  }
  return launch_status();
}

// ---- RoPE (interleaved pairs) ----------------------------------------------------
// angle = pos * theta^(-2i/D); the reference evaluates pow/cos/sin in fp32.
template <typename T>
__global__ void rope_inplace_kernel(T* __restrict__ x, const int32_t* __restrict__ positions,
                                    int num_heads, int head_dim, float theta, long long stride) {
  const int b = blockIdx.y;
  const int half = head_dim / 2;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;  // (head, pair)
  if (idx >= num_heads * half) return;
  const int h = idx / half;
  const int i = idx % half;
  float s, c;
  rope_cos_sin(positions[b], i, head_dim, theta, &c, &s);
  T* p = x + static_cast<size_t>(b) * stride + static_cast<size_t>(h) * head_dim + 2 * i;
  float re, ro;
  rope_rotate(Elem<T>::ld(p), Elem<T>::ld(p + 1), c, s, &re, &ro);
  Elem<T>::st(p, re);
  Elem<T>::st(p + 1, ro);
}

// (cos, sin) of every (position, pair) for the fused QKV epilogue: table[pos][i] = float2(cos, sin)
__global__ void rope_table_kernel(float2* __restrict__ table, int positions, int head_dim, float theta) {
  const int half = head_dim / 2;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(positions) * half) return;
  float s, c;
  rope_cos_sin(static_cast<int>(idx / half), static_cast<int>(idx % half), head_dim, theta, &c, &s);
  table[idx] = make_float2(c, s);
}

// ---- KV append: one new row per (request, kv head) into its page ------------------
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ k_cache,
                                 T* __restrict__ v_cache, const int32_t* __restrict__ page_table,
                                 const int32_t* __restrict__ positions, int num_kv_heads, int max_pages,
                                 int page_size, int head_dim, long long k_stride, long long v_stride) {
  const int b = blockIdx.y;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;  // (kv head, dim)
  if (idx >= num_kv_heads * head_dim) return;
  const int kvh = idx / head_dim;
  const int d = idx % head_dim;
  const int pos = positions[b];
  const int page_idx = pos / page_size;
  if (pos < 0 || page_idx >= max_pages) return;  // no page reserved: drop rather than write out of range
  const int page = page_table[static_cast<size_t>(b) * max_pages + page_idx];
  const size_t dst = ((static_cast<size_t>(page) * num_kv_heads + kvh) * page_size + pos % page_size) *
                         static_cast<size_t>(head_dim) + d;
  k_cache[dst] = k[static_cast<size_t>(b) * k_stride + idx];
  v_cache[dst] = v[static_cast<size_t>(b) * v_stride + idx];
}

// ---- RoPE on the q and k heads of a fused [q | k | v] row and the append of the new k / v rows, one launch ----
// The same arithmetic as rope_inplace_kernel followed by kv_append_kernel (the pool receives the rotated, rounded k).
template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, const int32_t* __restrict__ positions,
                                   const int32_t* __restrict__ page_table, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                   int q_dim, int k_dim, int head_dim, float theta, int max_pages, int page_size, long long stride) {
  const int b = blockIdx.y;
  const int pair = blockIdx.x * blockDim.x + threadIdx.x;            // pair of adjacent elements of the row
  if (pair >= (q_dim + 2 * k_dim) / 2) return;
  const int col = 2 * pair;
  const int pos = positions[b];
  T* p = qkv + static_cast<size_t>(b) * stride + col;
  T e0 = p[0], e1 = p[1];
  if (col < q_dim + k_dim) {                                          // q and k heads rotate
    float s, c, re, ro;
    rope_cos_sin(pos, (col % head_dim) / 2, head_dim, theta, &c, &s);
    rope_rotate(Elem<T>::ld(p), Elem<T>::ld(p + 1), c, s, &re, &ro);
    Elem<T>::st(p, re);
    Elem<T>::st(p + 1, ro);
    e0 = p[0]; e1 = p[1];
  }
  if (col < q_dim) return;
  const int page_idx = pos / page_size;
  if (pos < 0 || page_idx >= max_pages) return;                       // no page reserved: drop rather than write out of range
  const int kv_col = (col - q_dim) % k_dim;                           // v follows k and has the same width
  const int page = page_table[static_cast<size_t>(b) * max_pages + page_idx];
  const size_t dst = ((static_cast<size_t>(page) * (k_dim / head_dim) + kv_col / head_dim) * page_size + pos % page_size) *
                         static_cast<size_t>(head_dim) + kv_col % head_dim;
  T* pool = col < q_dim + k_dim ? k_cache : v_cache;
  pool[dst] = e0;
  pool[dst + 1] = e1;
}

// ---- KV append into 8-bit pools: each new row is quantised with its own scale --------------------
// scale = fp16(max|row| / 127) (1 for an all-zero row), byte = clamp(rint(value / scale), -127, 127) + 128.
// One CTA per (kv head, request); k and v rows of head_dim values each.
template <typename T>
__global__ void __launch_bounds__(128)
kv_append_q8_kernel(const T* __restrict__ k, const T* __restrict__ v, uint8_t* __restrict__ k_cache, uint8_t* __restrict__ v_cache,
                    __half* __restrict__ kv_scales, const int32_t* __restrict__ page_table, const int32_t* __restrict__ positions,
                    int num_kv_heads, int max_pages, int page_size, int head_dim, long long k_stride, long long v_stride) {
  __shared__ float s_max[2][4];
  const int kvh = blockIdx.x, b = blockIdx.y;
  const int pos = positions[b];
  const int page_idx = pos / page_size;
  if (pos < 0 || page_idx >= max_pages) return;  // no page reserved: drop rather than write out of range
  const int page = page_table[static_cast<size_t>(b) * max_pages + page_idx];
  const size_t chunk = static_cast<size_t>(page) * num_kv_heads + kvh;
  const size_t dst = (chunk * page_size + pos % page_size) * static_cast<size_t>(head_dim);
  const T* src[2] = {k + static_cast<size_t>(b) * k_stride + static_cast<size_t>(kvh) * head_dim,
                     v + static_cast<size_t>(b) * v_stride + static_cast<size_t>(kvh) * head_dim};
  uint8_t* out[2] = {k_cache + dst, v_cache + dst};
  float vals[2][2];        // up to 256 dims: two per thread
  float amax[2] = {0.f, 0.f};
#pragma unroll
  for (int w = 0; w < 2; ++w)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int d = threadIdx.x + i * 128;
      vals[w][i] = d < head_dim ? Elem<T>::ld(src[w] + d) : 0.f;
      amax[w] = fmaxf(amax[w], fabsf(vals[w][i]));
    }
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    amax[w] = warp_max(amax[w]);
    if ((threadIdx.x & 31) == 0) s_max[w][threadIdx.x >> 5] = amax[w];
  }
  __syncthreads();
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    const float m = fmaxf(fmaxf(s_max[w][0], s_max[w][1]), fmaxf(s_max[w][2], s_max[w][3]));
    __half sh = __float2half_rn(m / 127.f);
    if (__half2float(sh) == 0.f) sh = __float2half_rn(1.f);
    const float scale = __half2float(sh);
    if (threadIdx.x == 0) kv_scales[(chunk * 2 + w) * page_size + pos % page_size] = sh;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int d = threadIdx.x + i * 128;
      if (d < head_dim) {
        const float qv = fminf(127.f, fmaxf(-127.f, rintf(__fdiv_rn(vals[w][i], scale))));
        out[w][d] = static_cast<uint8_t>(static_cast<int>(qv) + 128);
      }
    }
  }
}

// ---- elementwise ------------------------------------------------------------------
template <typename T, bool SILU_MUL>
__global__ void binary_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, size_t total) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float x = Elem<T>::ld(a + i);
  const float y = Elem<T>::ld(b + i);
  Elem<T>::st(out + i, SILU_MUL ? (x / (1.f + expf(-x))) * y : x + y);
}

template <typename T>
__global__ void embedding_gather_kernel(const T* __restrict__ table, const int64_t* __restrict__ ids,
                                        T* __restrict__ out, int hidden, int vocab) {
  const int r = blockIdx.x;
  long long id = ids[r];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // clamp instead of faulting on a bad id
  const T* src = table + static_cast<size_t>(id) * hidden;
  T* dst = out + static_cast<size_t>(r) * hidden;
  constexpr int VEC = 16 / sizeof(T);
  if (hidden % VEC == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {   // 16-byte copies
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int c = threadIdx.x; c < hidden / VEC; c += blockDim.x) d4[c] = s4[c];
    return;
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = src[c];
}

// Row argmax; ties resolve to the lowest index like torch/numpy argmax.
template <typename T>
__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const T* __restrict__ logits, int64_t* __restrict__ out_ids, int vocab) {
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  const T* row = logits + static_cast<size_t>(blockIdx.x) * vocab;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  constexpr int VEC = sizeof(T) == 2 ? 8 : 4;     // 16-byte loads when the row allows it
  int done = 0;
  if (vocab % VEC == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    for (int c = threadIdx.x * VEC; c < vocab; c += blockDim.x * VEC) {
      float v[VEC];
      VecIO<T, VEC>::ld(row + c, v);
#pragma unroll
      for (int i = 0; i < VEC; ++i)      // ascending index inside the vector: the first maximum wins
        if (v[i] > best || (v[i] == best && c + i < best_i)) { best = v[i]; best_i = c + i; }
    }
    done = vocab;
  }
  for (int c = done + threadIdx.x; c < vocab; c += blockDim.x) {
    const float v = Elem<T>::ld(row + c);
    if (v > best || (v == best && c < best_i)) { best = v; best_i = c; }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = best_i; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? s_val[threadIdx.x] : -INFINITY;
    best_i = threadIdx.x < nw ? s_idx[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, off);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (threadIdx.x == 0) out_ids[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

__global__ void advance_positions_kernel(int32_t* positions, int32_t* seq_lens, int batch) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < batch) {
    const int32_t len = seq_lens[b];
    positions[b] = len;
    seq_lens[b] = len + 1;
  }
}

}  // namespace
}  // namespace cb200

using namespace cb200;

#define CB200_DISPATCH_DTYPE(dtype, CALL)                 \
  switch (dtype) {                                        \
    case CACHEIR_B200_F32: { using T = float; CALL; } break;          \
    case CACHEIR_B200_F16: { using T = __half; CALL; } break;         \
    case CACHEIR_B200_BF16: { using T = __nv_bfloat16; CALL; } break; \
    default: return CACHEIR_B200_EINVAL;                  \
  }

extern "C" int cacheir_b200_rms_norm(const void* x, const void* residual, const void* weight,
                                     void* sum_out, void* out, int rows, int hidden, float eps,
                                     int dtype, void* stream) {
  if (rows <= 0 || hidden <= 0) return 0;
  if (!x || !weight || !out) return CACHEIR_B200_EINVAL;
  if (residual && !sum_out) return CACHEIR_B200_EINVAL;
  cudaStream_t st = as_stream(stream);
  switch (dtype) {
    case CACHEIR_B200_F32: return launch_rms_norm<float, 4>(x, residual, weight, sum_out, out, rows, hidden, eps, st);
    case CACHEIR_B200_F16: return launch_rms_norm<__half, 8>(x, residual, weight, sum_out, out, rows, hidden, eps, st);
    case CACHEIR_B200_BF16: return launch_rms_norm<__nv_bfloat16, 8>(x, residual, weight, sum_out, out, rows, hidden, eps, st);
    default: return CACHEIR_B200_EINVAL;
  }
}

extern "C" int cacheir_b200_rope_inplace(void* x, const int32_t* positions, int batch_size,
                                         int num_heads, int head_dim, float theta, int dtype,
                                         long long x_batch_stride, void* stream) {
  if (batch_size <= 0 || num_heads <= 0 || head_dim <= 0) return 0;
  if (!x || !positions || (head_dim % 2) != 0 || batch_size > 65535) return CACHEIR_B200_EINVAL;
  const long long stride = x_batch_stride > 0 ? x_batch_stride : static_cast<long long>(num_heads) * head_dim;
  const int pairs = num_heads * (head_dim / 2);
  const dim3 grid((pairs + 127) / 128, batch_size);
  CB200_DISPATCH_DTYPE(dtype, (rope_inplace_kernel<T><<<grid, 128, 0, as_stream(stream)>>>(
                                  static_cast<T*>(x), positions, num_heads, head_dim, theta, stride)));
  return launch_status();
}

extern "C" int cacheir_b200_rope_table(float* table, int positions, int head_dim, float theta, void* stream) {
  if (positions <= 0 || head_dim <= 0) return 0;
  if (!table || (head_dim % 2) != 0) return CACHEIR_B200_EINVAL;
  if (!aligned_to(table, 8)) return CACHEIR_B200_EALIGN;
  const size_t total = static_cast<size_t>(positions) * (head_dim / 2);
  rope_table_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, as_stream(stream)>>>(
      reinterpret_cast<float2*>(table), positions, head_dim, theta);
  return launch_status();
}

extern "C" int cacheir_b200_rope_append(void* qkv, const int32_t* positions, const int32_t* page_table, void* k_cache,
                                        void* v_cache, int batch_size, int q_dim, int k_dim, int head_dim, float theta,
                                        int max_pages_per_seq, int page_size, int dtype, long long qkv_batch_stride,
                                        void* stream) {
  if (batch_size <= 0 || q_dim < 0 || k_dim <= 0 || head_dim <= 0) return 0;
  if (!qkv || !positions || !page_table || !k_cache || !v_cache || max_pages_per_seq <= 0 || page_size <= 0 ||
      batch_size > 65535 || (head_dim % 2) != 0 || q_dim % head_dim != 0 || k_dim % head_dim != 0)
    return CACHEIR_B200_EINVAL;
  const long long stride = qkv_batch_stride > 0 ? qkv_batch_stride : static_cast<long long>(q_dim) + 2 * k_dim;
  const int pairs = (q_dim + 2 * k_dim) / 2;
  const dim3 grid((pairs + 127) / 128, batch_size);
  CB200_DISPATCH_DTYPE(dtype, (rope_append_kernel<T><<<grid, 128, 0, as_stream(stream)>>>(
                                  static_cast<T*>(qkv), positions, page_table, static_cast<T*>(k_cache), static_cast<T*>(v_cache),
                                  q_dim, k_dim, head_dim, theta, max_pages_per_seq, page_size, stride)));
  return launch_status();
}

extern "C" int cacheir_b200_kv_append(const void* k, const void* v, void* k_cache, void* v_cache,
                                      const int32_t* page_table, const int32_t* positions,
                                      int batch_size, int num_kv_heads, int max_pages_per_seq,
                                      int page_size, int head_dim, int dtype, long long k_batch_stride,
                                      long long v_batch_stride, void* stream) {
  if (batch_size <= 0 || num_kv_heads <= 0 || head_dim <= 0) return 0;
  if (!k || !v || !k_cache || !v_cache || !page_table || !positions || max_pages_per_seq <= 0 ||
      page_size <= 0 || batch_size > 65535)
    return CACHEIR_B200_EINVAL;
  const long long dense = static_cast<long long>(num_kv_heads) * head_dim;
  const long long ks = k_batch_stride > 0 ? k_batch_stride : dense;
  const long long vs = v_batch_stride > 0 ? v_batch_stride : dense;
  const dim3 grid((static_cast<int>(dense) + 127) / 128, batch_size);
  CB200_DISPATCH_DTYPE(dtype, (kv_append_kernel<T><<<grid, 128, 0, as_stream(stream)>>>(
                                  static_cast<const T*>(k), static_cast<const T*>(v), static_cast<T*>(k_cache),
                                  static_cast<T*>(v_cache), page_table, positions, num_kv_heads,
                                  max_pages_per_seq, page_size, head_dim, ks, vs)));
  return launch_status();
}

extern "C" int cacheir_b200_kv_append_q8(const void* k, const void* v, void* k_cache, void* v_cache, void* kv_scales,
                                         const int32_t* page_table, const int32_t* positions, int batch_size,
                                         int num_kv_heads, int max_pages_per_seq, int page_size, int head_dim, int dtype,
                                         long long k_batch_stride, long long v_batch_stride, void* stream) {
  if (batch_size <= 0 || num_kv_heads <= 0 || head_dim <= 0) return 0;
  if (!k || !v || !k_cache || !v_cache || !kv_scales || !page_table || !positions || max_pages_per_seq <= 0 ||
      page_size <= 0 || batch_size > 65535)
    return CACHEIR_B200_EINVAL;
  if (head_dim > 256) return CACHEIR_B200_EUNSUPPORTED;
  const long long dense = static_cast<long long>(num_kv_heads) * head_dim;
  const long long ks = k_batch_stride > 0 ? k_batch_stride : dense;
  const long long vs = v_batch_stride > 0 ? v_batch_stride : dense;
  const dim3 grid(num_kv_heads, batch_size);
  CB200_DISPATCH_DTYPE(dtype, (kv_append_q8_kernel<T><<<grid, 128, 0, as_stream(stream)>>>(
                                  static_cast<const T*>(k), static_cast<const T*>(v), static_cast<uint8_t*>(k_cache),
                                  static_cast<uint8_t*>(v_cache), static_cast<__half*>(kv_scales), page_table, positions,
                                  num_kv_heads, max_pages_per_seq, page_size, head_dim, ks, vs)));
  return launch_status();
}

extern "C" int cacheir_b200_silu_mul(const void* gate, const void* up, void* out, size_t total,
                                     int dtype, void* stream) {
  if (total == 0) return 0;
  if (!gate || !up || !out) return CACHEIR_B200_EINVAL;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  CB200_DISPATCH_DTYPE(dtype, (binary_kernel<T, true><<<blocks, 256, 0, as_stream(stream)>>>(
                                  static_cast<const T*>(gate), static_cast<const T*>(up), static_cast<T*>(out), total)));
  return launch_status();
}

extern "C" int cacheir_b200_add(const void* a, const void* b, void* out, size_t total, int dtype,
                                void* stream) {
  if (total == 0) return 0;
  if (!a || !b || !out) return CACHEIR_B200_EINVAL;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  CB200_DISPATCH_DTYPE(dtype, (binary_kernel<T, false><<<blocks, 256, 0, as_stream(stream)>>>(
                                  static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), total)));
  return launch_status();
}

extern "C" int cacheir_b200_embedding_gather(const void* table, const int64_t* ids, void* out,
                                             int rows, int hidden, int vocab, int dtype, void* stream) {
  if (rows <= 0 || hidden <= 0) return 0;
  if (!table || !ids || !out || vocab <= 0) return CACHEIR_B200_EINVAL;
  CB200_DISPATCH_DTYPE(dtype, (embedding_gather_kernel<T><<<rows, 256, 0, as_stream(stream)>>>(
                                  static_cast<const T*>(table), ids, static_cast<T*>(out), hidden, vocab)));
  return launch_status();
}

extern "C" int cacheir_b200_argmax_rows(const void* logits, int64_t* out_ids, int rows, int vocab,
                                        int dtype, void* stream) {
  if (rows <= 0 || vocab <= 0) return 0;
  if (!logits || !out_ids) return CACHEIR_B200_EINVAL;
  CB200_DISPATCH_DTYPE(dtype, (argmax_rows_kernel<T><<<rows, 1024, 0, as_stream(stream)>>>(
                                  static_cast<const T*>(logits), out_ids, vocab)));
  return launch_status();
}

extern "C" int cacheir_b200_advance_positions(int32_t* positions, int32_t* seq_lens, int batch_size,
                                              void* stream) {
  if (batch_size <= 0) return 0;
  if (!positions || !seq_lens) return CACHEIR_B200_EINVAL;
  advance_positions_kernel<<<(batch_size + 127) / 128, 128, 0, as_stream(stream)>>>(positions, seq_lens, batch_size);
  return launch_status();
}
