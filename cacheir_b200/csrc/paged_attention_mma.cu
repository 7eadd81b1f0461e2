// Paged decode attention, fast path: fp16/bf16 pools, head_dim 64 or 128, 16-token pages.
//
// One CTA per (context split, KV head, sequence). A producer warp walks the
// sequence's page table and brings each (page, kv head) chunk -- 16 rows of K and 16
// rows of V, 4 KB each at head_dim 128 -- into shared memory with TMA tensor copies
// (128-byte swizzle, so that the ldmatrix reads below are bank-conflict free),
// through a ring of stages guarded by mbarriers. Four consumer warps each take one
// page of a stage: S = Q K^T and O += P V run on the tensor cores (mma.sync
// m16n8k16, fp32 accumulation) with all query heads of the GQA group as the 16-row
// M dimension, so every K/V byte is read from HBM once for the whole group. The
// online softmax keeps its running max / sum per row in registers (quad shuffles);
// the four warps' states are merged once per CTA in warp order, and context splits
// are merged by the combine kernel in split order: bit-reproducible.
#include <cuda.h>

#include "common.cuh"
#include <type_traits>

#include "paged_attention_common.cuh"
#include "fixed_point.cuh"

namespace cb200 {
namespace {

constexpr int kPage = 16;
constexpr int kPagesPerStage = 4;
constexpr int kConsumerWarps = 4;
constexpr int kFastThreads = (kConsumerWarps + 1) * 32;
constexpr uint32_t kPollLimit = 8u * 1000u * 1000u;

__device__ int g_attn_status = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int id) {
  for (uint32_t i = 0; i < kPollLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(32);
  }
  atomicCAS(&g_attn_status, 0, (2 << 8) | id);
  return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// DSMEM helpers of the quantising epilogue: a 32-bit store into the same shared-memory offset of another CTA of the
// cluster, and the cluster barrier with release / acquire ordering (all threads of all CTAs, at uniform points).
__device__ __forceinline__ void store_to_rank(void* local_ptr, uint32_t rank, uint32_t value) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_ptr)), "r"(rank));
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(value) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// QUANT: single split, launched as clusters of the kv heads of one sequence (grid z = padded row count of the
// planes); the epilogue also writes the output row as the integer GEMM's fixed-point planes, bit for bit what the
// stand-alone pre-pass makes of the stored fp16 output.
template <typename T, int D, bool QUANT>
__global__ void __launch_bounds__(kFastThreads)
paged_decode_mma_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                        const AttnParams p, const int stages) {
  constexpr int kTileBytes = kPage * D * 2;       // one K or V page chunk: 4 KB at D=128
  constexpr int kPageBytes = 2 * kTileBytes;      // K + V
  constexpr int kStageBytes = kPagesPerStage * kPageBytes;
  constexpr int kKSteps = D / 16;                 // k steps of the QK^T product
  constexpr int kDimTiles = D / 8;                // n tiles of the PV product

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + stages * kStageBytes);
  uint64_t* empty = full + stages;

  const int split = blockIdx.x;
  const int kvh = blockIdx.y;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if constexpr (QUANT) {
    if (b >= p.batch) {        // padding rows of the planes (the whole cluster is here): zeros, no barrier
      const int k0 = kvh * p.group * D;
      for (int i = threadIdx.x; i < p.group * D / 4; i += kFastThreads) {
        *reinterpret_cast<uint32_t*>(p.quant_planes + plane_offset(p.quant_rows, b, k0 + 4 * i)) = 0u;
        *reinterpret_cast<uint32_t*>(p.quant_planes + plane_offset(p.quant_rows, p.quant_rows + b, k0 + 4 * i)) = 0u;
      }
      if (kvh == 0 && threadIdx.x == 0) { p.quant_sx[b] = 0.f; p.quant_qsum[b] = 0; }
      return;
    }
  }
  const int seq_len = p.seq_lens[b];
  const int t_begin = split * p.chunk_tokens;
  if (p.splits > 1 && t_begin >= seq_len) return;      // combine never reads this split
  const int t_end = min(seq_len, t_begin + p.chunk_tokens);
  const int page_begin = t_begin / kPage;              // chunk_tokens is a multiple of the page size
  const int n_pages = t_end > t_begin ? (t_end - t_begin + kPage - 1) / kPage : 0;
  const int n_iters = (n_pages + kPagesPerStage - 1) / kPagesPerStage;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), kConsumerWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // per-thread softmax / output state of the two rows (heads) this thread owns: g and g + 8
  const int g = lane >> 2;
  const int t4 = lane & 3;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float o[kDimTiles][4];
#pragma unroll
  for (int i = 0; i < kDimTiles; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  bool ok = true;

  if (warp == kConsumerWarps) {
    // ---------------- producer warp: lane j copies page j of each stage ----------------
    const int32_t* pt = p.page_table + static_cast<size_t>(b) * p.max_pages + page_begin;
    int next_id = lane < min(kPagesPerStage, n_pages) ? pt[lane] : 0;   // page ids are fetched one stage ahead
    for (int it = 0; it < n_iters && ok; ++it) {
      const int s = it % stages;
      const uint32_t ph = (it / stages) & 1;
      const int first = it * kPagesPerStage;
      const int cnt = min(kPagesPerStage, n_pages - first);
      const int page_id = next_id;
      if (first + kPagesPerStage + lane < n_pages && lane < kPagesPerStage) next_id = pt[first + kPagesPerStage + lane];
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&empty[s]), ph ^ 1, 1);
        if (ok) mbar_expect_tx(smem_u32(&full[s]), cnt * kPageBytes);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (ok && lane < cnt) {
        const uint32_t dst = smem_u32(smem + s * kStageBytes + lane * kPageBytes);
        const int row = (page_id * p.kv_heads + kvh) * kPage;
        tma_load_3d(dst, &tmap_k, smem_u32(&full[s]), 0, row, 0);
        tma_load_3d(dst + kTileBytes, &tmap_v, smem_u32(&full[s]), 0, row, 0);
      }
    }
  } else {
    // ---------------- consumer warps ----------------
    // Q as the A operand: rows = heads of the group (zero beyond the group), 16 dims per k step
    uint32_t qa[kKSteps][4];
    {
      const T* qb = static_cast<const T*>(p.q) + static_cast<size_t>(b) * p.q_stride + static_cast<size_t>(kvh) * p.group * D;
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int row = g + (r & 1) * 8;
          const int col = ks * 16 + 2 * t4 + (r >> 1) * 8;
          qa[ks][r] = row < p.group ? *reinterpret_cast<const uint32_t*>(qb + static_cast<size_t>(row) * D + col) : 0u;
        }
      }
    }
    const uint32_t lrow = lane & 7;        // row supplied by this lane to ldmatrix
    const uint32_t lmat = lane >> 3;       // which of the four 8x8 matrices
    for (int it = 0; it < n_iters && ok; ++it) {
      const int s = it % stages;
      ok = mbar_wait(smem_u32(&full[s]), (it / stages) & 1, 2);
      if (!ok) break;
      const int pg = it * kPagesPerStage + warp;       // this warp's page of the stage
      if (pg < n_pages) {
        const uint32_t kbase = smem_u32(smem + s * kStageBytes + warp * kPageBytes);
        const uint32_t vbase = kbase + kTileBytes;
        // ---- S = Q K^T for the 16 tokens of the page: two n tiles of 8 tokens ----
        float sc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
          const uint32_t token = nt * 8 + lrow;
#pragma unroll
          for (int kk = 0; kk < kKSteps / 2; ++kk) {
            const uint32_t c = 4 * kk + lmat;          // 16-byte chunk of the row
            uint32_t kb[4];
            ldmatrix_x4(kbase + (c >> 3) * (kPage * 128) + token * 128 + (((c & 7) ^ (token & 7)) << 4), kb);
            mma_16816<T>(sc[nt], qa[2 * kk], kb[0], kb[1]);
            mma_16816<T>(sc[nt], qa[2 * kk + 1], kb[2], kb[3]);
          }
        }
        // ---- online softmax over the page (rows g and g+8; columns 2*t4, 2*t4+1 of each tile) ----
        const int tok0 = t_begin + pg * kPage;
        float pmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int tok = tok0 + nt * 8 + 2 * t4 + (e & 1);
            const float v = tok < t_end ? sc[nt][e] * p.scale_log2 : -INFINITY;
            sc[nt][e] = v;
            pmax[e >> 1] = fmaxf(pmax[e >> 1], v);
          }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          pmax[r] = fmaxf(pmax[r], __shfl_xor_sync(0xffffffffu, pmax[r], 1));
          pmax[r] = fmaxf(pmax[r], __shfl_xor_sync(0xffffffffu, pmax[r], 2));
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float m_new = fmaxf(m_run[r], pmax[r]);    // finite: every loaded page has a valid token
          corr[r] = exp2f(m_run[r] - m_new);               // first page: exp2(-inf) = 0
          m_run[r] = m_new;
        }
        uint32_t pa[4];
        {
          float pr[2][4];
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) pr[nt][e] = exp2f(sc[nt][e] - m_run[e >> 1]);
#pragma unroll
          for (int r = 0; r < 2; ++r)
            l_run[r] = l_run[r] * corr[r] + (pr[0][2 * r] + pr[0][2 * r + 1] + pr[1][2 * r] + pr[1][2 * r + 1]);
          // P as the A operand of the PV product (16 heads x 16 tokens)
          pa[0] = pack2<T>(pr[0][0], pr[0][1]);
          pa[1] = pack2<T>(pr[0][2], pr[0][3]);
          pa[2] = pack2<T>(pr[1][0], pr[1][1]);
          pa[3] = pack2<T>(pr[1][2], pr[1][3]);
        }
        // ---- O = O * corr + P V ----
#pragma unroll
        for (int j = 0; j < kDimTiles / 2; ++j) {
          o[2 * j][0] *= corr[0]; o[2 * j][1] *= corr[0]; o[2 * j][2] *= corr[1]; o[2 * j][3] *= corr[1];
          o[2 * j + 1][0] *= corr[0]; o[2 * j + 1][1] *= corr[0]; o[2 * j + 1][2] *= corr[1]; o[2 * j + 1][3] *= corr[1];
          const uint32_t token = (lmat & 1) * 8 + lrow;
          const uint32_t c = 2 * j + (lmat >> 1);
          uint32_t vb[4];
          ldmatrix_x4_trans(vbase + (c >> 3) * (kPage * 128) + token * 128 + (((c & 7) ^ (token & 7)) << 4), vb);
          mma_16816<T>(o[2 * j], pa, vb[0], vb[1]);
          mma_16816<T>(o[2 * j + 1], pa, vb[2], vb[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty[s]));
    }
    // the row sums were kept per thread: finish them across the quad
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
  }

  // ---------------- merge the consumer warps in warp order ----------------
  __syncthreads();                        // every stage is consumed: the ring can be reused
  float* s_m = reinterpret_cast<float*>(smem);                  // [warps][16]
  float* s_l = s_m + kConsumerWarps * 16;                       // [warps][16]
  float* s_o = s_l + kConsumerWarps * 16;                       // [warps][16][D]
  if (warp < kConsumerWarps) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + r * 8;
      if (t4 == 0) { s_m[warp * 16 + row] = m_run[r]; s_l[warp * 16 + row] = l_run[r]; }
#pragma unroll
      for (int i = 0; i < kDimTiles; ++i) {
        s_o[(warp * 16 + row) * D + i * 8 + 2 * t4] = o[i][2 * r];
        s_o[(warp * 16 + row) * D + i * 8 + 2 * t4 + 1] = o[i][2 * r + 1];
      }
    }
  }
  __syncthreads();
  if constexpr (QUANT) {
    // One item (four consecutive dims of one head) per thread; exchange area behind the ring's barriers.
    float* x_amax = reinterpret_cast<float*>(empty + stages);      // [8] one slot per CTA of the cluster, written by it
    int* x_qsum = reinterpret_cast<int*>(x_amax + 8);              // [8] the same for the sums (read by rank 0)
    float* s_redf = reinterpret_cast<float*>(x_qsum + 8);          // [8] per warp
    int* s_redi = reinterpret_cast<int*>(s_redf + 8);              // [8] per warp
    const int item = threadIdx.x;
    const bool has = item < p.group * (D / 4);
    const int row = has ? item / (D / 4) : 0, d0 = (item % (D / 4)) * 4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (has) {
      float m_tot = -INFINITY;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) m_tot = fmaxf(m_tot, s_m[w * 16 + row]);
      float l_tot = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float mi = s_m[w * 16 + row];
        const float wgt = (mi == -INFINITY) ? 0.f : exp2f(mi - m_tot);
        l_tot = fmaf(s_l[w * 16 + row], wgt, l_tot);
        const float4 part = *reinterpret_cast<const float4*>(s_o + (w * 16 + row) * D + d0);
        acc[0] = fmaf(part.x, wgt, acc[0]); acc[1] = fmaf(part.y, wgt, acc[1]);
        acc[2] = fmaf(part.z, wgt, acc[2]); acc[3] = fmaf(part.w, wgt, acc[3]);
      }
      const int h = kvh * p.group + row;
      __half2 lo2 = __floats2half2_rn(l_tot > 0.f ? acc[0] / l_tot : 0.f, l_tot > 0.f ? acc[1] / l_tot : 0.f);
      __half2 hi2 = __floats2half2_rn(l_tot > 0.f ? acc[2] / l_tot : 0.f, l_tot > 0.f ? acc[3] / l_tot : 0.f);
      __half* ob = static_cast<__half*>(p.out) + static_cast<size_t>(b) * p.out_stride + static_cast<size_t>(h) * D + d0;
      *reinterpret_cast<uint2*>(ob) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo2), *reinterpret_cast<const uint32_t*>(&hi2));
      const float2 a = __half22float2(lo2), c = __half22float2(hi2);       // the stored (rounded) values are what gets quantised
      v[0] = a.x; v[1] = a.y; v[2] = c.x; v[3] = c.y;
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (lane == 0) s_redf[warp] = amax;
    __syncthreads();
    const uint32_t rank = static_cast<uint32_t>(kvh), ranks = static_cast<uint32_t>(p.kv_heads);     // cluster = (1, kv_heads, 1)
    if (threadIdx.x < ranks) {
      float cta_max = 0.f;
#pragma unroll
      for (int w = 0; w < kFastThreads / 32; ++w) cta_max = fmaxf(cta_max, s_redf[w]);
      store_to_rank(x_amax + rank, threadIdx.x, __float_as_uint(cta_max));
    }
    cluster_sync_all();
    amax = 0.f;
    for (uint32_t r = 0; r < ranks; ++r) amax = fmaxf(amax, x_amax[r]);
    const float inv = amax > 0.f ? kQMax / amax : 0.f;
    int sum = 0;
    if (has) {
      uint32_t hi_w, lo_w;
      split_four(fixed_point_bits(v[0], inv), fixed_point_bits(v[1], inv), fixed_point_bits(v[2], inv), fixed_point_bits(v[3], inv),
                 &hi_w, &lo_w, &sum);
      const int k = (kvh * p.group + row) * D + d0;
      *reinterpret_cast<uint32_t*>(p.quant_planes + plane_offset(p.quant_rows, b, k)) = hi_w;
      *reinterpret_cast<uint32_t*>(p.quant_planes + plane_offset(p.quant_rows, p.quant_rows + b, k)) = lo_w;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane == 0) s_redi[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
      int cta_sum = 0;
#pragma unroll
      for (int w = 0; w < kFastThreads / 32; ++w) cta_sum += s_redi[w];
      store_to_rank(x_qsum + rank, 0u, static_cast<uint32_t>(cta_sum));
    }
    cluster_sync_all();
    if (rank == 0 && threadIdx.x == 0) {
      int tot = 0;
      for (uint32_t r = 0; r < ranks; ++r) tot += x_qsum[r];
      p.quant_qsum[b] = tot;
      p.quant_sx[b] = amax > 0.f ? amax / kQMax : 0.f;
    }
  } else {
  for (int idx = threadIdx.x; idx < p.group * D; idx += kFastThreads) {
    const int row = idx / D;
    const int d = idx % D;
    float m_tot = -INFINITY;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) m_tot = fmaxf(m_tot, s_m[w * 16 + row]);
    float l_tot = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) {
      const float mi = s_m[w * 16 + row];
      const float wgt = (mi == -INFINITY) ? 0.f : exp2f(mi - m_tot);
      l_tot = fmaf(s_l[w * 16 + row], wgt, l_tot);
      acc = fmaf(s_o[(w * 16 + row) * D + d], wgt, acc);
    }
    const int h = kvh * p.group + row;
    if (p.splits == 1) {
      T* ob = static_cast<T*>(p.out) + static_cast<size_t>(b) * p.out_stride;
      Elem<T>::st(ob + static_cast<size_t>(h) * D + d, l_tot > 0.f ? acc / l_tot : 0.f);
    } else {
      const size_t unit = (static_cast<size_t>(b) * p.heads + h) * p.splits + split;
      p.ws_acc[unit * D + d] = acc;
      if (d == 0) {
        p.ws_ml[unit * 2] = m_tot;
        p.ws_ml[unit * 2 + 1] = l_tot;
      }
    }
  }
  }
}

// ---- 8-bit pools -----------------------------------------------------------------------------------------
// The same kernel shape for pools of unsigned bytes, value = (byte - 128) * scale[row] (fp16 queries, head_dim 128):
// a (page, kv head) chunk is 16 rows x 128 bytes of K, the same of V, and 64 bytes of scales (16 fp16 for K, 16 for V),
// half the bytes of the fp16 pool. ldmatrix reads the byte tiles as 16-bit units, so a thread receives four
// consecutive dims of a K row (or, transposed, two dims of two V rows); a byte permute with 0x64 high bytes turns two
// of them into the fp16 pair (1024 + b0, 1024 + b1) = (b - 128) + 1152, exact in fp16; the constant leaves through sums
// the MMAs' accumulators account for (scores start at -1152 * sum(q) of their row, outputs lose 1152 * sum(p) of their
// row at the end), so no subtraction is spent per value. The k order of the QK^T product
// inside a 16-dim step is therefore 4t, 4t+1 | 4t+2, 4t+3 for thread t of a quad, and Q is loaded in that order; the
// PV product yields the dims of a 16-dim block as two tiles, even dims and odd dims. The row scales multiply the scores
// (K) and the probabilities (V) instead of the 2 x 2048 cached values.
__device__ __forceinline__ void bulk_load_bytes(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y) : "memory");
}
// bytes i and j of w as the fp16 pair (b_i - 128, b_j - 128)
template <uint32_t SEL>
__device__ __forceinline__ uint32_t byte_pair(uint32_t w) {
  return __byte_perm(w, 0x64646464u, SEL);                                  // (1024 + b_i, 1024 + b_j), exact in fp16
}
constexpr float kByteBias = 1152.f;     // 1024 + 128: what every operand built by byte_pair carries on top of (b - 128)

// Six consumer warps (a page each per stage): the chain per page is longer than with fp16 pages (byte -> fp16
// conversions in front of every MMA) while the page has half the bytes, so more pages must be in work per SM (two CTAs of six warps).
constexpr int kQ8Warps = 6;
constexpr int kQ8Threads = (kQ8Warps + 1) * 32;

__global__ void __launch_bounds__(kQ8Threads, 2)
paged_decode_mma_q8_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                           const AttnParams p, const int stages) {
  constexpr int D = 128;
  constexpr int kTileBytes = kPage * D;            // one K or V page chunk of bytes: 2 KB
  constexpr int kScaleBytes = 2 * kPage * 2;       // 16 K scales + 16 V scales, fp16
  constexpr int kStageBytes = kQ8Warps * 2 * kTileBytes + 1024;   // tiles (1 KB aligned), then the pages' scales
  constexpr int kKSteps = D / 16;
  constexpr int kDimTiles = D / 8;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + stages * kStageBytes);
  uint64_t* empty = full + stages;

  const int split = blockIdx.x;
  const int kvh = blockIdx.y;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int seq_len = p.seq_lens[b];
  const int t_begin = split * p.chunk_tokens;
  if (p.splits > 1 && t_begin >= seq_len) return;      // combine never reads this split
  const int t_end = min(seq_len, t_begin + p.chunk_tokens);
  const int page_begin = t_begin / kPage;
  const int n_pages = t_end > t_begin ? (t_end - t_begin + kPage - 1) / kPage : 0;
  const int n_iters = (n_pages + kQ8Warps - 1) / kQ8Warps;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), kQ8Warps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int g = lane >> 2;
  const int t4 = lane & 3;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float o[kDimTiles][4];       // tile 2c: even dims of the 16-dim block c, tile 2c+1: its odd dims
#pragma unroll
  for (int i = 0; i < kDimTiles; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  bool ok = true;

  if (warp == kQ8Warps) {
    // ---------------- producer warp: lane j copies page j of each stage ----------------
    const int32_t* pt = p.page_table + static_cast<size_t>(b) * p.max_pages + page_begin;
    const __half* scales = static_cast<const __half*>(p.kv_scales);
    int next_id = lane < min(kQ8Warps, n_pages) ? pt[lane] : 0;
    for (int it = 0; it < n_iters && ok; ++it) {
      const int s = it % stages;
      const uint32_t ph = (it / stages) & 1;
      const int first = it * kQ8Warps;
      const int cnt = min(kQ8Warps, n_pages - first);
      const int page_id = next_id;
      if (first + kQ8Warps + lane < n_pages && lane < kQ8Warps) next_id = pt[first + kQ8Warps + lane];
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&empty[s]), ph ^ 1, 1);
        if (ok) mbar_expect_tx(smem_u32(&full[s]), cnt * (2 * kTileBytes + kScaleBytes));
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (ok && lane < cnt) {
        uint8_t* stage = smem + s * kStageBytes;
        const int chunk = page_id * p.kv_heads + kvh;
        tma_load_2d_tile(smem_u32(stage + lane * 2 * kTileBytes), &tmap_k, smem_u32(&full[s]), 0, chunk * kPage);
        tma_load_2d_tile(smem_u32(stage + lane * 2 * kTileBytes + kTileBytes), &tmap_v, smem_u32(&full[s]), 0, chunk * kPage);
        bulk_load_bytes(smem_u32(stage + kQ8Warps * 2 * kTileBytes + lane * kScaleBytes),
                        scales + static_cast<size_t>(chunk) * 2 * kPage, kScaleBytes, smem_u32(&full[s]));
      }
    }
  } else {
    // ---------------- consumer warps ----------------
    // Q as the A operand, k order of a 16-dim step: thread t of a quad holds dims 4t, 4t+1 (first half) and 4t+2, 4t+3
    uint32_t qa[kKSteps][4];
    {
      const __half* qb = static_cast<const __half*>(p.q) + static_cast<size_t>(b) * p.q_stride + static_cast<size_t>(kvh) * p.group * D;
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int row = g + (r & 1) * 8;
          const int col = ks * 16 + 4 * t4 + (r >> 1) * 2;
          qa[ks][r] = row < p.group ? *reinterpret_cast<const uint32_t*>(qb + static_cast<size_t>(row) * D + col) : 0u;
        }
      }
    }
    // -1152 * (sum of the row's query values, as the MMA sees them): where the score accumulators start
    float qbias[2] = {0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&qa[ks][r]));
        qbias[r & 1] += f.x + f.y;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      qbias[r] += __shfl_xor_sync(0xffffffffu, qbias[r], 1);
      qbias[r] += __shfl_xor_sync(0xffffffffu, qbias[r], 2);
      qbias[r] *= -kByteBias;
    }
    float p_run[2] = {0.f, 0.f};         // running sum of the probabilities (times V scales) fed to the PV product, per thread
    const uint32_t lrow = lane & 7;
    const uint32_t lmat = lane >> 3;
    for (int it = 0; it < n_iters && ok; ++it) {
      const int s = it % stages;
      ok = mbar_wait(smem_u32(&full[s]), (it / stages) & 1, 2);
      if (!ok) break;
      const int pg = it * kQ8Warps + warp;
      if (pg < n_pages) {
        const uint8_t* stage = smem + s * kStageBytes;
        const uint32_t kbase = smem_u32(stage + warp * 2 * kTileBytes);
        const uint32_t vbase = kbase + kTileBytes;
        const __half* sc_k = reinterpret_cast<const __half*>(stage + kQ8Warps * 2 * kTileBytes + warp * kScaleBytes);
        const __half* sc_v = sc_k + kPage;
        // ---- S = Q K^T for the 16 tokens of the page: two n tiles of 8 tokens; one ldmatrix covers four k steps ----
        float sc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          sc[nt][0] = sc[nt][1] = qbias[0]; sc[nt][2] = sc[nt][3] = qbias[1];
          const uint32_t token = nt * 8 + lrow;
#pragma unroll
          for (int kk = 0; kk < kKSteps / 4; ++kk) {
            const uint32_t c = 4 * kk + lmat;          // 16-byte chunk of the row = k step
            uint32_t kb[4];
            ldmatrix_x4(kbase + token * 128 + (((c & 7) ^ (token & 7)) << 4), kb);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              mma_16816<__half>(sc[nt], qa[4 * kk + i], byte_pair<0x4140>(kb[i]), byte_pair<0x4342>(kb[i]));
          }
        }
        // ---- online softmax over the page (rows g and g+8; columns 2*t4, 2*t4+1 of each tile) ----
        const int tok0 = t_begin + pg * kPage;
        float pmax[2] = {-INFINITY, -INFINITY};
        float vscale[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const float ks0 = __half2float(sc_k[nt * 8 + 2 * t4]), ks1 = __half2float(sc_k[nt * 8 + 2 * t4 + 1]);
          vscale[nt][0] = __half2float(sc_v[nt * 8 + 2 * t4]);
          vscale[nt][1] = __half2float(sc_v[nt * 8 + 2 * t4 + 1]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int tok = tok0 + nt * 8 + 2 * t4 + (e & 1);
            const float v = tok < t_end ? sc[nt][e] * ((e & 1) ? ks1 : ks0) * p.scale_log2 : -INFINITY;
            sc[nt][e] = v;
            pmax[e >> 1] = fmaxf(pmax[e >> 1], v);
          }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          pmax[r] = fmaxf(pmax[r], __shfl_xor_sync(0xffffffffu, pmax[r], 1));
          pmax[r] = fmaxf(pmax[r], __shfl_xor_sync(0xffffffffu, pmax[r], 2));
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float m_new = fmaxf(m_run[r], pmax[r]);
          corr[r] = exp2f(m_run[r] - m_new);
          m_run[r] = m_new;
        }
        uint32_t pa[4];
        {
          float pr[2][4];
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) pr[nt][e] = exp2f(sc[nt][e] - m_run[e >> 1]);
#pragma unroll
          for (int r = 0; r < 2; ++r)
            l_run[r] = l_run[r] * corr[r] + (pr[0][2 * r] + pr[0][2 * r + 1] + pr[1][2 * r] + pr[1][2 * r + 1]);
          // P times the V row scales as the A operand of the PV product (a masked token has p = 0; its stale scale must not turn that into NaN)
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) pr[nt][e] = pr[nt][e] > 0.f ? pr[nt][e] * vscale[nt][e & 1] : 0.f;
          pa[0] = pack2<__half>(pr[0][0], pr[0][1]);
          pa[1] = pack2<__half>(pr[0][2], pr[0][3]);
          pa[2] = pack2<__half>(pr[1][0], pr[1][1]);
          pa[3] = pack2<__half>(pr[1][2], pr[1][3]);
#pragma unroll
          for (int r = 0; r < 2; ++r) {     // the rounded values the MMA multiplies: their sum carries the byte offset out again
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&pa[r])), c = __half22float2(*reinterpret_cast<const __half2*>(&pa[2 + r]));
            p_run[r] = fmaf(p_run[r], corr[r], (a.x + a.y) + (c.x + c.y));
          }
        }
        // ---- O = O * corr + P V: one transposed ldmatrix covers two 16-dim blocks = four n tiles ----
#pragma unroll
        for (int j = 0; j < kDimTiles / 4; ++j) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            o[4 * j + i][0] *= corr[0]; o[4 * j + i][1] *= corr[0]; o[4 * j + i][2] *= corr[1]; o[4 * j + i][3] *= corr[1];
          }
          const uint32_t token = (lmat & 1) * 8 + lrow;
          const uint32_t c = 2 * j + (lmat >> 1);
          uint32_t vb[4];       // [block 2j: tokens 0-7, tokens 8-15], [block 2j+1: tokens 0-7, tokens 8-15]
          ldmatrix_x4_trans(vbase + token * 128 + (((c & 7) ^ (token & 7)) << 4), vb);
          mma_16816<__half>(o[4 * j], pa, byte_pair<0x4240>(vb[0]), byte_pair<0x4240>(vb[1]));          // even dims of block 2j
          mma_16816<__half>(o[4 * j + 1], pa, byte_pair<0x4341>(vb[0]), byte_pair<0x4341>(vb[1]));      // odd dims
          mma_16816<__half>(o[4 * j + 2], pa, byte_pair<0x4240>(vb[2]), byte_pair<0x4240>(vb[3]));      // block 2j+1
          mma_16816<__half>(o[4 * j + 3], pa, byte_pair<0x4341>(vb[2]), byte_pair<0x4341>(vb[3]));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty[s]));
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
      p_run[r] += __shfl_xor_sync(0xffffffffu, p_run[r], 1);
      p_run[r] += __shfl_xor_sync(0xffffffffu, p_run[r], 2);
      const float off = kByteBias * p_run[r];        // every output column of the row carries 1152 * sum(p)
#pragma unroll
      for (int i = 0; i < kDimTiles; ++i) { o[i][2 * r] -= off; o[i][2 * r + 1] -= off; }
    }
  }

  // ---------------- merge the consumer warps in warp order ----------------
  __syncthreads();
  float* s_m = reinterpret_cast<float*>(smem);
  float* s_l = s_m + kQ8Warps * 16;
  float* s_o = s_l + kQ8Warps * 16;
  if (warp < kQ8Warps) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + r * 8;
      if (t4 == 0) { s_m[warp * 16 + row] = m_run[r]; s_l[warp * 16 + row] = l_run[r]; }
#pragma unroll
      for (int i = 0; i < kDimTiles; ++i) {
        // tile i = block i/2, parity i&1; its columns 2*t4, 2*t4+1 are dims 16*(i/2) + 2*column + parity
        const int d0 = 16 * (i >> 1) + 4 * t4 + (i & 1);
        s_o[(warp * 16 + row) * D + d0] = o[i][2 * r];
        s_o[(warp * 16 + row) * D + d0 + 2] = o[i][2 * r + 1];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.group * D; idx += kQ8Threads) {
    const int row = idx / D;
    const int d = idx % D;
    float m_tot = -INFINITY;
#pragma unroll
    for (int w = 0; w < kQ8Warps; ++w) m_tot = fmaxf(m_tot, s_m[w * 16 + row]);
    float l_tot = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kQ8Warps; ++w) {
      const float mi = s_m[w * 16 + row];
      const float wgt = (mi == -INFINITY) ? 0.f : exp2f(mi - m_tot);
      l_tot = fmaf(s_l[w * 16 + row], wgt, l_tot);
      acc = fmaf(s_o[(w * 16 + row) * D + d], wgt, acc);
    }
    const int h = kvh * p.group + row;
    if (p.splits == 1) {
      __half* ob = static_cast<__half*>(p.out) + static_cast<size_t>(b) * p.out_stride;
      ob[static_cast<size_t>(h) * D + d] = __float2half_rn(l_tot > 0.f ? acc / l_tot : 0.f);
    } else {
      const size_t unit = (static_cast<size_t>(b) * p.heads + h) * p.splits + split;
      p.ws_acc[unit * D + d] = acc;
      if (d == 0) {
        p.ws_ml[unit * 2] = m_tot;
        p.ws_ml[unit * 2 + 1] = l_tot;
      }
    }
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// The pool [slots, kv_heads, 16, D] as a 3-D tensor [D/64 spans][rows][64 elements]: one box
// {64, 16, D/64} is one (page, kv head) chunk, landing as [span][16 rows][128 B] with the 128-byte swizzle.
bool encode_pool(CUtensorMap* map, const void* base, int dtype, uint64_t rows, int head_dim) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {64, rows, static_cast<cuuint64_t>(head_dim / 64)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2, 128};
  const cuuint32_t box[3] = {64, kPage, static_cast<cuuint32_t>(head_dim / 64)};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUtensorMapDataType type = dtype == CACHEIR_B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  return fn(map, type, 3, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int D>
int launch_fast(const AttnParams& p, int dtype, uint64_t pool_rows, cudaStream_t stream) {
  CUtensorMap tmap_k, tmap_v;
  if (!encode_pool(&tmap_k, p.k_cache, dtype, pool_rows, D) || !encode_pool(&tmap_v, p.v_cache, dtype, pool_rows, D))
    return CACHEIR_B200_EUNSUPPORTED;
  constexpr int kStageBytes = kPagesPerStage * 2 * kPage * D * 2;
  const int stages = D == 128 ? 3 : 4;
  size_t smem = 1024 + static_cast<size_t>(stages) * kStageBytes + 256;
  const size_t merge = static_cast<size_t>(kConsumerWarps) * 16 * (D + 2) * sizeof(float) + 1024;
  if (smem < merge) smem = merge;
  if constexpr (std::is_same<T, __half>::value && D == 128) {
    if (p.quant_planes) {      // the kv heads of a sequence form a cluster; grid z covers the padding rows of the planes too
      auto kern = paged_decode_mma_kernel<T, D, true>;
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(1, p.kv_heads, p.quant_rows);
      cfg.blockDim = dim3(kFastThreads, 1, 1);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = p.kv_heads;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      e = cudaLaunchKernelEx(&cfg, kern, tmap_k, tmap_v, p, stages);
      if (e != cudaSuccess) return static_cast<int>(e);
      return launch_status();
    }
  }
  auto kern = paged_decode_mma_kernel<T, D, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  const dim3 grid(p.splits, p.kv_heads, p.batch);
  kern<<<grid, kFastThreads, smem, stream>>>(tmap_k, tmap_v, p, stages);
  return launch_status();
}


// 8-bit pool [slots * kv_heads * 16 rows][128 bytes]: box {128, 16}, 128-byte swizzle.
bool encode_pool_q8(CUtensorMap* map, const void* base, uint64_t rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {128, rows};
  const cuuint64_t strides[1] = {128};
  const cuuint32_t box[2] = {128, kPage};
  const cuuint32_t elem_strides[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_fast_q8(const AttnParams& p, uint64_t pool_rows, cudaStream_t stream) {
  CUtensorMap tmap_k, tmap_v;
  if (!encode_pool_q8(&tmap_k, p.k_cache, pool_rows) || !encode_pool_q8(&tmap_v, p.v_cache, pool_rows)) return CACHEIR_B200_EUNSUPPORTED;
  constexpr int kStageBytes = kQ8Warps * 2 * kPage * 128 + 1024;
  const int stages = 4;
  size_t smem = 1024 + static_cast<size_t>(stages) * kStageBytes + 256;
  const size_t merge = static_cast<size_t>(kQ8Warps) * 16 * (128 + 2) * sizeof(float) + 1024;
  if (smem < merge) smem = merge;
  cudaError_t e = cudaFuncSetAttribute(paged_decode_mma_q8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  const dim3 grid(p.splits, p.kv_heads, p.batch);
  paged_decode_mma_q8_kernel<<<grid, kQ8Threads, smem, stream>>>(tmap_k, tmap_v, p, stages);
  return launch_status();
}

}  // namespace

bool paged_attention_fast_supported(const AttnParams& p, int dtype) {
  if (p.kv8) {
    return dtype == CACHEIR_B200_F16 && p.head_dim == 128 && p.page_size == kPage && p.group <= 16 && p.chunk_tokens % kPage == 0 &&
           aligned_to(p.k_cache, 128) && aligned_to(p.v_cache, 128) && aligned_to(p.kv_scales, 16) && aligned_to(p.q, 4) &&
           (p.q_stride % 2) == 0 && encode_fn() != nullptr;
  }
  if (dtype != CACHEIR_B200_F16 && dtype != CACHEIR_B200_BF16) return false;
  if (p.head_dim != 64 && p.head_dim != 128) return false;
  if (p.page_size != kPage || p.group > 16) return false;
  if (p.chunk_tokens % kPage != 0) return false;
  if (!aligned_to(p.k_cache, 16) || !aligned_to(p.v_cache, 16) || !aligned_to(p.q, 4) || (p.q_stride % 2) != 0) return false;
  return encode_fn() != nullptr;
}

bool paged_attention_quantize_supported(const AttnParams& p, int dtype) {
  if (p.kv8 || dtype != CACHEIR_B200_F16 || p.head_dim != 128 || p.splits != 1) return false;
  if (!paged_attention_fast_supported(p, dtype)) return false;
  if (p.kv_heads < 1 || p.kv_heads > 8 || p.heads != p.group * p.kv_heads) return false;      // one portable cluster per sequence
  if (p.group * (p.head_dim / 4) > kFastThreads) return false;                                // one four-dim item per thread
  if (p.batch > 64 || p.out_stride != static_cast<long long>(p.heads) * p.head_dim) return false;
  return true;
}

int launch_paged_attention_fast(const AttnParams& p, int dtype, cudaStream_t stream) {
  // With the pool's slot count the tensor maps carry the true row bound: the copy engine then zero-fills a chunk
  // whose page id lies outside the pool instead of reading past it. Without it (the reference's launcher signature
  // has no such argument) the bound is a formality and page ids are trusted.
  const uint64_t rows = p.num_slots > 0 ? static_cast<uint64_t>(p.num_slots) * p.kv_heads * kPage : (1ull << 30);
  if (p.kv8) return launch_fast_q8(p, rows, stream);
  if (dtype == CACHEIR_B200_F16)
    return p.head_dim == 128 ? launch_fast<__half, 128>(p, dtype, rows, stream) : launch_fast<__half, 64>(p, dtype, rows, stream);
  return p.head_dim == 128 ? launch_fast<__nv_bfloat16, 128>(p, dtype, rows, stream)
                           : launch_fast<__nv_bfloat16, 64>(p, dtype, rows, stream);
}

int paged_attention_device_status(bool reset) {
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_attn_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int));
  }
  return status;
}

}  // namespace cb200
