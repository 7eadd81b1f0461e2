// int8 dequant-GEMM on the integer tensor cores (tcgen05.mma kind::i8), sm_100a.
//
//   y[M, N] = x[M, K] . ((code[N, K] - zero[N]) * scale[N])^T      M <= 64, fp16 x/y
//
// The packed uint8 codes go from HBM through one bulk copy per 16 KB tile (tile-ordered,
// pre-swizzled weights) or a TMA tensor copy (reference row order) into shared memory and from
// there straight into the tensor core: nothing unpacks, converts or re-stores a weight.
// Activations are made integer instead. A pre-pass turns every row of x into 16-bit
// fixed point with its own scale, x[m,k] ~= sx[m] * q[m,k], |q| <= 32639 (2^-15 of the
// row maximum: far below fp16's own resolution), and splits q into two signed bytes,
// q = 256*hi + lo. With the weight tile as the 128-row operand and the [hi; lo] rows
// as the other one, a single accumulator row holds, for weight row n,
//   D[n, m] = sum_k code[n,k]*hi[m,k]      D[n, MP+m] = sum_k code[n,k]*lo[m,k]
// exactly (int32). The epilogue recombines in integers:
//   y[m,n] = scale[n] * sx[m] * (256*D[n,m] + D[n,MP+m] - zero[n] * sum_k q[m,k]).
//
// One CTA owns 128 weight rows (with the SwiGLU epilogue: 64 gate rows and the 64 up rows of the
// same columns) and a K range: thread 0 initialises the barriers and requests the first ring of
// tiles while the rest of the CTA sets up, then keeps the ring full; one thread of warp 1 issues
// the MMAs (K = 32 per instruction, 4 per 128-column stage) into an accumulator in tensor memory;
// warps 2-5 run the epilogue (plain, residual, SwiGLU, or the fused QKV form: RoPE + cache append).
// K ranges of one row tile form a thread-block cluster. Their partial sums are integers, so
// the order of addition cannot matter; each rank lays its partials out per destination in its
// drained ring and one bulk shared-to-shared copy per destination signals that rank's barrier;
// each CTA of the cluster finishes the outputs of its own slice of the batch. Two CTAs share an SM.
#include "common.cuh"
#include "qgemv_common.cuh"
#include "tc_ptx.cuh"
#include "fixed_point.cuh"

namespace cb200 {
namespace {

using namespace ptx;

constexpr int kBlockN = 128;          // weight rows per CTA (UMMA M)
constexpr int kBlockK = 128;          // bytes of a weight row per stage
constexpr int kThreads = 192;         // producer, MMA issuer, four epilogue warps
constexpr int kCtaBudget = 104 * 1024;   // ring + exchange buffer; two CTAs per SM: one issues MMAs while the other waits on a barrier
constexpr int kCtaBudgetWide = 200 * 1024;   // split-K with more than 32 batch rows: one CTA per SM
constexpr int kMaxSplitK = 8;

__device__ int g_i8_status = 0;

// (int4 weights add the raw 8 KB nibble tile in front of the 16 KB byte tile it is unpacked into)
__host__ __device__ constexpr int stage_bytes(int mp, int bits = 8) {
  return kBlockN * kBlockK + (bits == 4 ? kBlockN * kBlockK / 2 : 0) + 2 * mp * kBlockK;
}
// split-K: every rank receives, from each rank, 128 rows x 2*(mp/split) words
__host__ __device__ constexpr int exchange_bytes(int mp, int split) { return split > 1 ? kBlockN * 2 * mp * 4 : 0; }
__host__ __device__ constexpr int ring_bytes(int mp, int split) {
  return (split > 1 && mp > 32 ? kCtaBudgetWide : kCtaBudget) - exchange_bytes(mp, split);
}
__host__ __device__ constexpr int num_stages(int mp, int split, int bits = 8) {
  return ring_bytes(mp, split) / stage_bytes(mp, bits) > 8 ? 8 : ring_bytes(mp, split) / stage_bytes(mp, bits);
}

// ---- pre-pass: rows of x -> two planes of signed bytes + scale + sum ------------------
// The planes are stored the way the GEMM consumes them: per 128-column k block one contiguous
// tile [2*mp rows][128 bytes] (rows [0,mp): high bytes, [mp,2mp): low bytes; rows >= M are zero),
// with the 16-byte chunks of row R in the XOR order of a 128-byte swizzle (chunk c at c ^ (R & 7)),
// so that one contiguous bulk copy per stage lands it ready for the tensor core.
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const __half* __restrict__ x, long long x_stride, int M, int K, int mp,
                     int8_t* __restrict__ planes, float* __restrict__ sx, int* __restrict__ qsum) {
  __shared__ float s_red[8];
  __shared__ int s_sum[8];
  const int m = blockIdx.x;
  const int nvec = K / 8;
  if (m >= M) {
    for (int c = threadIdx.x; c < nvec; c += 256) {
      *reinterpret_cast<uint2*>(planes + plane_offset(mp, m, c * 8)) = make_uint2(0u, 0u);
      *reinterpret_cast<uint2*>(planes + plane_offset(mp, mp + m, c * 8)) = make_uint2(0u, 0u);
    }
    if (threadIdx.x == 0) { sx[m] = 0.f; qsum[m] = 0; }
    return;
  }
  const __half* xr = x + static_cast<size_t>(m) * x_stride;
  float amax = 0.f;
  for (int c = threadIdx.x; c < nvec; c += 256) {
    float v[8];
    VecIO<__half, 8>::ld(xr + c * 8, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) amax = fmaxf(amax, s_red[w]);
  const float inv = amax > 0.f ? kQMax / amax : 0.f;
  int sum = 0;
  for (int c = threadIdx.x; c < nvec; c += 256) {
    float v[8];
    VecIO<__half, 8>::ld(xr + c * 8, v);
    uint32_t hi_w[2], lo_w[2];
#pragma unroll
    for (int i = 0; i < 2; ++i)
      split_four(fixed_point_bits(v[4 * i], inv), fixed_point_bits(v[4 * i + 1], inv), fixed_point_bits(v[4 * i + 2], inv),
                 fixed_point_bits(v[4 * i + 3], inv), &hi_w[i], &lo_w[i], &sum);
    *reinterpret_cast<uint2*>(planes + plane_offset(mp, m, c * 8)) = make_uint2(hi_w[0], hi_w[1]);
    *reinterpret_cast<uint2*>(planes + plane_offset(mp, mp + m, c * 8)) = make_uint2(lo_w[0], lo_w[1]);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if ((threadIdx.x & 31) == 0) s_sum[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    int tot = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += s_sum[w];
    qsum[m] = tot;
    sx[m] = amax > 0.f ? amax / kQMax : 0.f;
  }
}

// Block-wide reductions for the single-pass kernels below (up to 32 warps).
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) t += scratch[w];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) t = fmaxf(t, scratch[w]);
  return t;
}

// One row of activations held in registers -> byte planes, scale and sum. Shared by the
// stand-alone pre-pass and the RMSNorm-fused form; `vals` are the fp16-rounded activations.
template <int PT>
__device__ __forceinline__ void quantize_row_from_registers(const float (&vals)[PT][8], int nvec, int8_t* planes, int mp, int m,
                                                            float* sx_out, int* qsum_out, float* scratch) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < PT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(vals[i][j]));
  amax = block_max(amax, scratch);
  const float inv = amax > 0.f ? kQMax / amax : 0.f;
  int sum = 0;
#pragma unroll
  for (int i = 0; i < PT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nvec) {
      uint32_t hi_w[2], lo_w[2];
#pragma unroll
      for (int j = 0; j < 2; ++j)
        split_four(fixed_point_bits(vals[i][4 * j], inv), fixed_point_bits(vals[i][4 * j + 1], inv),
                   fixed_point_bits(vals[i][4 * j + 2], inv), fixed_point_bits(vals[i][4 * j + 3], inv), &hi_w[j], &lo_w[j], &sum);
      *reinterpret_cast<uint2*>(planes + plane_offset(mp, m, c * 8)) = make_uint2(hi_w[0], hi_w[1]);
      *reinterpret_cast<uint2*>(planes + plane_offset(mp, mp + m, c * 8)) = make_uint2(lo_w[0], lo_w[1]);
    }
  }
  __shared__ int s_isum[32];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if ((threadIdx.x & 31) == 0) s_isum[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    int tot = 0;
    for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) tot += s_isum[w];
    *qsum_out = tot;
    *sx_out = amax > 0.f ? amax / kQMax : 0.f;
  }
}

__device__ __forceinline__ void zero_plane_rows(int8_t* planes, int mp, int m, int nvec) {
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    *reinterpret_cast<uint2*>(planes + plane_offset(mp, m, c * 8)) = make_uint2(0u, 0u);
    *reinterpret_cast<uint2*>(planes + plane_offset(mp, mp + m, c * 8)) = make_uint2(0u, 0u);
  }
}

// Stand-alone pre-pass, single pass: the row stays in registers between the max and the rounding.
template <int PT>
__global__ void __launch_bounds__(1024)
quantize_rows_fast_kernel(const __half* __restrict__ x, long long x_stride, int M, int K, int mp,
                          int8_t* __restrict__ planes, float* __restrict__ sx, int* __restrict__ qsum) {
  __shared__ float scratch[32];
  const int m = blockIdx.x;
  const int nvec = K / 8;
  if (m >= M) {
    zero_plane_rows(planes, mp, m, nvec);
    if (threadIdx.x == 0) { sx[m] = 0.f; qsum[m] = 0; }
    return;
  }
  float vals[PT][8];
#pragma unroll
  for (int i = 0; i < PT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) vals[i][j] = 0.f;
    if (c < nvec) VecIO<__half, 8>::ld(x + static_cast<size_t>(m) * x_stride + c * 8, vals[i]);
  }
  quantize_row_from_registers<PT>(vals, nvec, planes, mp, m, sx + m, qsum + m, scratch);
}

// RMSNorm (optionally of x + residual, the rounded sum going to sum_out) fused with the pre-pass:
// the normalised row is rounded to fp16 exactly as the stand-alone RMSNorm stores it, optionally
// written to `out`, and quantised from registers.
template <int PT>
__global__ void __launch_bounds__(512)
rms_norm_quantize_kernel(const __half* __restrict__ x, const __half* __restrict__ residual, const __half* __restrict__ weight,
                         __half* __restrict__ sum_out, __half* __restrict__ out, int M, int hidden, float eps, int mp,
                         int8_t* __restrict__ planes, float* __restrict__ sx, int* __restrict__ qsum) {
  __shared__ float scratch[32];
  const int m = blockIdx.x;
  const int nvec = hidden / 8;
  if (m >= M) {
    zero_plane_rows(planes, mp, m, nvec);
    if (threadIdx.x == 0) { sx[m] = 0.f; qsum[m] = 0; }
    return;
  }
  const size_t row = static_cast<size_t>(m) * hidden;
  float vals[PT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) vals[i][j] = 0.f;
    if (c < nvec) {
      VecIO<__half, 8>::ld(x + row + c * 8, vals[i]);
      if (residual) {
        float r[8];
        VecIO<__half, 8>::ld(residual + row + c * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[i][j] = __half2float(__float2half_rn(vals[i][j] + r[j]));
        VecIO<__half, 8>::st(sum_out + row + c * 8, vals[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(vals[i][j], vals[i][j], ss);
    }
  }
  float w[PT][8];      // the norm weights are requested before the reduction, not after it
#pragma unroll
  for (int i = 0; i < PT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nvec) VecIO<__half, 8>::ld(weight + c * 8, w[i]);
  }
  const float inv = rsqrtf(block_sum(ss, scratch) / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int i = 0; i < PT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) vals[i][j] = __half2float(__float2half_rn(vals[i][j] * inv * w[i][j]));
      if (out) VecIO<__half, 8>::st(out + row + c * 8, vals[i]);
    }
  }
  quantize_row_from_registers<PT>(vals, nvec, planes, mp, m, sx + m, qsum + m, scratch);
}

struct I8Params {
  const void* scales;
  const float* zero_points;
  const void* residual;
  void* y;
  const float* sx;
  const int* qsum;
  const uint8_t* w_tiled;     // tile-ordered codes (tiled != 0)
  const int8_t* x_planes;     // activation byte tiles written by the pre-pass
  int n_tiles;                // row tiles (128 output columns, or 64 gate|up pairs)
  int M, N, K;
  int n_out;
  int scale_dtype;
  int epilogue;
  int split_k;
  int tiled;        // weights in 128x128 tile order: tile (band, kb) starts at row (band*KB + kb)*128 of a 128-byte-wide tensor
  RopeAppendParams rope;   // epilogue == kEpiQkvRopeAppend
};
// With the SwiGLU epilogue a tile pairs 64 gate rows (tile rows 0..63, weight rows 64t..64t+63) with the
// 64 up rows of the same output columns (tile rows 64..127, weight rows N/2+64t..): one pass, one
// accumulator, and twice as many CTAs as whole-half tiles would give.
constexpr int kPairRows = 64;

// y value from the exact integer sums: (256*hi + lo - zero*qsum) as float. Integer zero points in
// [-255, 255] (what the reference packer produces) are handled in integers, anything else in double precision.
// (The double-precision form is rare and kept out of line so that the epilogues stay short.)
__device__ __noinline__ float recombine_fractional(int32_t hi, int32_t lo, float zero, int qsum) {
  return static_cast<float>(256.0 * hi + static_cast<double>(lo) - static_cast<double>(zero) * qsum);
}
// `zero_int` is the zero point as an integer and `zero_is_int` says whether that is exact; both are
// per-thread constants worked out once, outside the loops over the batch rows.
__device__ __forceinline__ float recombine(int32_t hi, int32_t lo, float zero, int zero_int, bool zero_is_int, int qsum) {
  if (zero_is_int) {
    // 32-bit arithmetic only (64-bit integer math and its conversion cost several times more issue
    // slots): with qsum = 256*qh + ql, v = 256*(hi - z*qh) + (lo - z*ql); both brackets fit in 32 bits
    // for |z| <= 255. The float of v is exact-rounded while the first bracket is below 2^24
    // (|v| < 2^32, far above what cancelled sums reach), and within 1.5 units in the last place beyond.
    const int a = hi - zero_int * (qsum >> 8);
    const int b = lo - zero_int * (qsum & 255);
    return fmaf(static_cast<float>(a), 256.f, static_cast<float>(b));
  }
  return recombine_fractional(hi, lo, zero, qsum);
}

constexpr int kTailBytes = 1024;   // scratch behind the ring and the exchange buffer: barriers, TMEM base, per-row constants

template <int MP, int SPLIT, bool ROPE, int BITS>
__global__ void __launch_bounds__(kThreads, 2)
qgemm_i8_kernel(const __grid_constant__ CUtensorMap tmap_w, const I8Params p) {
  constexpr int kStages = num_stages(MP, SPLIT, BITS);
  constexpr int kWBytes = kBlockN * kBlockK;          // 16 KB of byte codes per stage (what the tensor core reads)
  constexpr int kRawBytes = BITS == 4 ? kWBytes / 2 : 0;   // int4: the nibble tile as it comes from HBM
  constexpr int kLoadBytes = BITS == 4 ? kRawBytes : kWBytes;
  constexpr int kXBytes = 2 * MP * kBlockK;           // [hi; lo] rows per stage
  constexpr int kAccCols = 2 * MP;                    // one accumulator: MP high + MP low columns
  constexpr int kTmemCols = kAccCols;                 // 32, 64 or 128: a power of two, as the allocator wants
  // split-K exchange: rank j finishes batch rows [j*MS, (j+1)*MS); a partial row for one destination is
  // W words: [MS high | MS low]
  constexpr int MS = MP / SPLIT;
  constexpr int W = 2 * MS;
  constexpr int kSlotBytes = kBlockN * W * 4;         // what one rank sends to one other rank
  constexpr bool kReadyBar = BITS == 4;               // a stage passes through the epilogue warps before the tensor core reads it

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* s_w = smem;
  uint8_t* s_x = s_w + kStages * kWBytes;
  uint8_t* s_raw = s_x + kStages * kXBytes;              // int4 only
  int32_t* s_xch = reinterpret_cast<int32_t*>(s_raw + kStages * kRawBytes);   // [SPLIT senders][128 rows][W], written by the peers
  uint8_t* tail = reinterpret_cast<uint8_t*>(s_xch) + exchange_bytes(MP, SPLIT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
  uint64_t* full = bars;                  // [kStages] TMA landed
  uint64_t* empty = bars + kStages;       // [kStages] MMAs that read the stage have retired
  uint64_t* acc_full = empty + kStages;   // [1]
  uint64_t* xch_bar = acc_full + 1;       // [1] all partials of the other ranks have landed
  uint64_t* ready = xch_bar + 1;          // [kStages] the operand tiles of the stage are complete (epilogue warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ready + kStages);
  float* s_sx = reinterpret_cast<float*>(tmem_slot + 2);     // [MP] fixed-point step of each batch row
  int* s_qsum = reinterpret_cast<int*>(s_sx + MP);           // [MP] sum over k of the row's integers
  int32_t* s_stage = reinterpret_cast<int32_t*>(smem);       // outgoing partials [SPLIT dests][128 rows][W] reuse the drained ring

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool swiglu = p.epilogue == CACHEIR_B200_EPI_SWIGLU;
  constexpr int split = SPLIT;
  constexpr bool clustered = SPLIT > 1;
  const int krank = split > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int kblocks_all = p.K / kBlockK;
  const int kb_begin = (kblocks_all * krank) / split;
  const int kb_end = (kblocks_all * (krank + 1)) / split;
  const int total = kb_end - kb_begin;
  const int n0 = blockIdx.x * (swiglu ? kPairRows : kBlockN);   // first output column of this tile

  auto load_stage = [&](int i, int s) {
    const int kb = kb_begin + i;
    const uint32_t bar = smem_u32(&full[s]);
    mbar_expect_tx(bar, kLoadBytes + kXBytes);
    constexpr int kRowBytes = BITS == 4 ? kBlockK / 2 : kBlockK;      // bytes of one tile row as stored in HBM
    const uint32_t dst = BITS == 4 ? smem_u32(s_raw + s * kRawBytes) : smem_u32(s_w + s * kWBytes);
    if (p.tiled) {   // one contiguous, pre-swizzled tile (16 KB of bytes or 8 KB of nibbles)
      bulk_load(dst, p.w_tiled + (static_cast<size_t>(blockIdx.x) * kblocks_all + kb) * kLoadBytes, kLoadBytes, bar);
    } else if (swiglu) {   // the map's box is 64 rows: gate rows, then the up rows of the same columns
      tma_load_2d(dst, &tmap_w, bar, kb * kRowBytes, n0);
      tma_load_2d(dst + kPairRows * kRowBytes, &tmap_w, bar, kb * kRowBytes, p.N / 2 + n0);
    } else {
      tma_load_2d(dst, &tmap_w, bar, kb * kRowBytes, n0);
    }
    bulk_load(smem_u32(s_x + s * kXBytes), p.x_planes + static_cast<size_t>(kb) * kXBytes, kXBytes, bar);
  };
  const int pre = total < kStages ? total : kStages;

  // Set-up: thread 0 initialises the barriers and goes straight on to request the first ring of
  // tiles; warp 0 only arrives at the CTA-wide barrier below, the other warps wait on it.
  if (warp == 0) {
    if (lane == 0) {
      for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&full[s]), 1); mbar_init(smem_u32(&empty[s]), 1); }
      mbar_init(smem_u32(acc_full), 1);
      mbar_init(smem_u32(xch_bar), 1);
      if (kReadyBar)
        for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(&ready[s]), 128);
      mbar_fence_init();                       // visible to the copy engine and to the other CTAs of the cluster
      if (split > 1) mbar_expect_tx(smem_u32(xch_bar), (split - 1) * kSlotBytes);
    }
    __syncwarp();
    asm volatile("bar.arrive 2, %0;" ::"n"(kThreads) : "memory");
    if (clustered) cluster_arrive_relaxed();   // phase A: this CTA runs and its exchange barrier exists
    if (lane == 0) {
      for (int i = 0; i < pre; ++i) load_stage(i, i);
    }
  } else {
    if (warp == 1) tc_alloc(smem_u32(tmem_slot), kTmemCols);
    if (clustered) cluster_arrive_relaxed();
    tc_fence_before();
    asm volatile("bar.sync 2, %0;" ::"n"(kThreads) : "memory");
    tc_fence_after();
  }
  const uint32_t tmem_base = warp == 0 ? 0u : *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer (stages beyond the first ring) ----------------
      for (int i = pre; i < total; ++i) {
        const int s = i % kStages;
        if (!mbar_wait(smem_u32(&empty[s]), ((i / kStages) & 1) ^ 1, &g_i8_status, (3 << 8) | 1)) break;
        load_stage(i, s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      // D = s32, A (codes) unsigned 8 bit, B (activation bytes) signed 8 bit, both K-major, N = 2*MP, M = 128
      const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | (static_cast<uint32_t>(kAccCols >> 3) << 17) |
                             (static_cast<uint32_t>(kBlockN >> 4) << 24);
      for (int i = 0; i < total; ++i) {
        const int s = i % kStages;
        if (!mbar_wait(smem_u32(kReadyBar ? &ready[s] : &full[s]), (i / kStages) & 1, &g_i8_status, (3 << 8) | 2)) break;
        tc_fence_after();
        const uint32_t d = tmem_base;
        const uint32_t w_base = smem_u32(s_w + s * kWBytes);
        const uint32_t x_base = smem_u32(s_x + s * kXBytes);
#pragma unroll
        for (int j = 0; j < kBlockK / 32; ++j)   // 32 bytes of k per instruction inside the 128-byte swizzle span
          tc_mma_i8_ss(d, smem_desc_sw128(w_base + j * 32), smem_desc_sw128(x_base + j * 32), idesc, (i > 0 || j > 0) ? 1u : 0u);
        tc_commit(smem_u32(&empty[s]));
      }
      tc_commit(smem_u32(acc_full));
    }
  } else {
    // ---------------- epilogue warps: lane quarter = warp % 4 ----------------
    const int q = warp & 3;
    const int r = q * 32 + lane;                 // weight row of the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    // output column and weight row of this thread's accumulator row
    const bool is_up = swiglu && r >= kPairRows;
    const int n_out_idx = swiglu ? n0 + (r & (kPairRows - 1)) : n0 + r;
    const int w_row = is_up ? p.N / 2 + n_out_idx : n_out_idx;
    __half* y = static_cast<__half*>(p.y);
    const __half* res = static_cast<const __half*>(p.residual);
    // What the epilogue needs from global memory is requested here and first used after the main loop (a use
    // stalls the warp until the line has arrived, cold from HBM, and would hold back the loads behind it).
    if (threadIdx.x - 64 < MP) {
      s_sx[threadIdx.x - 64] = p.sx[threadIdx.x - 64];
      s_qsum[threadIdx.x - 64] = p.qsum[threadIdx.x - 64];
    }
    const bool col_ok = n_out_idx < p.n_out;
    uint32_t scale_raw = 0u;
    float zero = 128.f;
    if (col_ok) {
      scale_raw = p.scale_dtype == CACHEIR_B200_F16 ? static_cast<uint32_t>(static_cast<const uint16_t*>(p.scales)[w_row])
                                                    : static_cast<const uint32_t*>(p.scales)[w_row];
      if (p.zero_points) zero = p.zero_points[w_row];
    }
    uint16_t res_raw[MS];
#pragma unroll
    for (int j = 0; j < MS; ++j) {
      const int m = krank * MS + j;
      res_raw[j] = (split > 1 && p.epilogue == CACHEIR_B200_EPI_RESIDUAL && m < p.M && col_ok)
                       ? reinterpret_cast<const uint16_t*>(res)[static_cast<size_t>(m) * p.n_out + n_out_idx] : static_cast<uint16_t>(0);
    }
    // Fused QKV epilogue: per batch row, the (cos, sin) of this thread's pair and where its k/v element goes in the pool.
    [[maybe_unused]] constexpr bool rope_epi = ROPE;   // a template parameter: the other projections do not carry this code
    const RopeAppendParams& ra = p.rope;
    auto rope_row = [&](int m, float2* cs, long long* off) {
      *cs = make_float2(1.f, 0.f);
      *off = -1;
      if (m >= p.M || n_out_idx >= p.n_out) return;
      const int pos = ra.positions[m];
      if (n_out_idx < ra.q_dim + ra.k_dim) {
        const int i = (n_out_idx % ra.head_dim) >> 1;
        if (pos >= 0 && pos < ra.table_positions)
          *cs = reinterpret_cast<const float2*>(ra.table)[static_cast<size_t>(pos) * (ra.head_dim / 2) + i];
        else
          atomicCAS(&g_i8_status, 0, (3 << 8) | 5);   // position outside the cos/sin table: flagged, value left unrotated
      }
      if (n_out_idx >= ra.q_dim) {
        const int col = (n_out_idx - ra.q_dim) % ra.k_dim;      // v follows k and has the same width
        const int page_idx = pos / ra.page_size;
        if (pos >= 0 && page_idx < ra.max_pages) {               // no page reserved: drop rather than write out of range
          const int page = ra.page_table[static_cast<size_t>(m) * ra.max_pages + page_idx];
          *off = static_cast<long long>(((static_cast<size_t>(page) * ra.kv_heads + col / ra.head_dim) * ra.page_size +
                                         pos % ra.page_size) * ra.head_dim + col % ra.head_dim);
        }
      }
    };
    // all 32 lanes call this together (pairs are adjacent lanes); only `do_store` lanes write
    auto rope_finish = [&](float out, float2 cs, long long off, int m, bool do_store) {
      float v = __half2float(__float2half_rn(out));             // what the plain epilogue would have stored
      const float partner = __shfl_xor_sync(0xffffffffu, v, 1);
      const bool is_qk = n_out_idx < ra.q_dim + ra.k_dim;
      if (is_qk) {
        const bool odd = (n_out_idx & 1) != 0;
        float re, ro;
        rope_rotate(odd ? partner : v, odd ? v : partner, cs.x, cs.y, &re, &ro);
        v = odd ? ro : re;
      }
      const __half h = __float2half_rn(v);
      if (do_store) {
        y[static_cast<size_t>(m) * p.n_out + n_out_idx] = h;
        if (off >= 0) static_cast<__half*>(is_qk ? ra.k_cache : ra.v_cache)[off] = h;
      }
    };
    float2 cs_v[MS];
    long long off_v[MS];
    [[maybe_unused]] int pos_v[MS], page_v[MS];
    if constexpr (SPLIT > 1 && ROPE) {
      // Two levels of dependent loads (position, then table entry and page id): each level is issued for all of
      // this thread's rows at once, with clamped indices instead of branches, so the latencies overlap; the
      // values are put to use only after the main loop.
#pragma unroll
      for (int j = 0; j < MS; ++j) {
        const int m = krank * MS + j;
        pos_v[j] = (m < p.M && col_ok) ? ra.positions[m] : -1;
      }
    }
    if constexpr (SPLIT > 1 && ROPE) {
      const int pair = (n_out_idx % ra.head_dim) >> 1;
#pragma unroll
      for (int j = 0; j < MS; ++j) {
        const int m = min(krank * MS + j, p.M - 1);
        const int pos_t = min(max(pos_v[j], 0), ra.table_positions - 1);
        const int page_idx = min(max(pos_v[j], 0) / ra.page_size, ra.max_pages - 1);
        cs_v[j] = reinterpret_cast<const float2*>(ra.table)[static_cast<size_t>(pos_t) * (ra.head_dim / 2) + pair];
        page_v[j] = ra.page_table[static_cast<size_t>(m) * ra.max_pages + page_idx];
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps: s_sx / s_qsum are in place
    if constexpr (BITS == 4) {
      // int4 weights: while the main loop runs these warps turn each landed nibble tile into the byte tile the
      // tensor core reads. Thread r owns tile row r: 64 bytes of nibbles (four 16-byte chunks stored in the
      // 64-byte swizzle order, chunk c at c ^ ((r >> 1) & 3)) become 128 bytes of codes in the 128-byte
      // swizzle order (chunk c at c ^ (r & 7)); even columns sit in the low nibbles.
      for (int i = 0; i < total; ++i) {
        const int s = i % kStages;
        if (!mbar_wait(smem_u32(&full[s]), (i / kStages) & 1, &g_i8_status, (3 << 8) | 8)) break;
        const uint8_t* raw_row = s_raw + s * kRawBytes + r * (kBlockK / 2);
        uint8_t* out_row = s_w + s * kWBytes + r * kBlockK;
        uint4 raw[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) raw[c] = *reinterpret_cast<const uint4*>(raw_row + ((c ^ ((r >> 1) & 3)) * 16));
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
          uint32_t o[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t even = w[j] & 0x0F0F0F0Fu;
            const uint32_t odd = (w[j] >> 4) & 0x0F0F0F0Fu;
            o[2 * j] = __byte_perm(even, odd, 0x5140);         // columns 8j .. 8j+3
            o[2 * j + 1] = __byte_perm(even, odd, 0x7362);     // columns 8j+4 .. 8j+7
          }
          *reinterpret_cast<uint4*>(out_row + (((2 * c) ^ (r & 7)) * 16)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(out_row + (((2 * c + 1) ^ (r & 7)) * 16)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads these bytes through the async proxy
        mbar_arrive(smem_u32(&ready[s]));
      }
    }
    // Only now are the prefetched values put to use.
    const float scale = !col_ok ? 0.f : (p.scale_dtype == CACHEIR_B200_F16 ? __half2float(__ushort_as_half(static_cast<unsigned short>(scale_raw)))
                                                                             : __uint_as_float(scale_raw));
    const bool zero_is_int = zero == rintf(zero) && fabsf(zero) <= 255.f;
    const int zero_int = zero_is_int ? __float2int_rn(zero) : 0;
    float res_v[MS];
#pragma unroll
    for (int j = 0; j < MS; ++j) res_v[j] = __half2float(__ushort_as_half(res_raw[j]));
    if constexpr (SPLIT > 1 && ROPE) {
      const bool is_qk = n_out_idx < ra.q_dim + ra.k_dim;
      const int col = n_out_idx >= ra.q_dim ? (n_out_idx - ra.q_dim) % ra.k_dim : 0;
#pragma unroll
      for (int j = 0; j < MS; ++j) {
        const int pos = pos_v[j];
        const bool row_ok = pos >= 0;
        if (row_ok && is_qk && pos >= ra.table_positions) atomicCAS(&g_i8_status, 0, (3 << 8) | 5);   // outside the cos/sin table
        if (!(row_ok && is_qk && pos < ra.table_positions)) cs_v[j] = make_float2(1.f, 0.f);
        const bool write = row_ok && n_out_idx >= ra.q_dim && pos / ra.page_size < ra.max_pages;   // no page reserved: dropped
        off_v[j] = write ? static_cast<long long>(((static_cast<size_t>(page_v[j]) * ra.kv_heads + col / ra.head_dim) * ra.page_size +
                                                   pos % ra.page_size) * ra.head_dim + col % ra.head_dim)
                         : -1;
      }
    }
    bool ok = mbar_wait(smem_u32(acc_full), 0, &g_i8_status, (3 << 8) | 3);
    tc_fence_after();
    const bool store = ok && n_out_idx < p.n_out;
    if constexpr (SPLIT > 1) {
      // All-to-all over the cluster. Each rank lays its partial sums out per destination in its own
      // drained ring, one bulk copy per destination moves a slot into that rank's exchange buffer and
      // signals its barrier; the sums are integers, so the order of addition cannot matter.
      constexpr int G = MS >= 4 ? 4 : 2;
      {
        uint32_t acc[2 * MP];
        if (total > 0) {
#pragma unroll
          for (int c0 = 0; c0 < 2 * MP; c0 += 8) tc_ld_x8(tmem_base + lane_addr + c0, reinterpret_cast<uint32_t(&)[8]>(acc[c0]));
          tc_wait_ld();
        } else {
#pragma unroll
          for (int c = 0; c < 2 * MP; ++c) acc[c] = 0u;
        }
#pragma unroll
        for (int dest = 0; dest < SPLIT; ++dest) {
          int32_t* row = s_stage + (static_cast<size_t>(dest) * kBlockN + r) * W;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int u = 0; u < MS; u += G) {
              const int c = h * MP + dest * MS + u;
              if constexpr (G == 4) *reinterpret_cast<uint4*>(row + h * MS + u) = make_uint4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
              else *reinterpret_cast<uint2*>(row + h * MS + u) = make_uint2(acc[c], acc[c + 1]);
            }
          }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the bulk copies below read what was just stored
      asm volatile("bar.sync 1, 128;" ::: "memory");
      cluster_wait();                                // phase A: every rank of the cluster runs and has armed its barrier
      if (warp == 2 && lane < SPLIT - 1 && ok) {     // one lane per destination
        const int dest = (krank + 1 + lane) % SPLIT;
        bulk_copy_to_rank(smem_u32(reinterpret_cast<uint8_t*>(s_xch) + krank * kSlotBytes),
                          smem_u32(reinterpret_cast<uint8_t*>(s_stage) + dest * kSlotBytes), kSlotBytes,
                          smem_u32(xch_bar), dest);
      }
      __syncwarp();
      ok = mbar_wait(smem_u32(xch_bar), 0, &g_i8_status, (3 << 8) | 4) && ok;
      cluster_arrive_relaxed();                      // phase B: nothing more will be written into this CTA
#pragma unroll 1
      for (int u0 = 0; u0 < MS; u0 += G) {
        int32_t sum[2][4];                           // [half][word]
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int j = 0; j < 4; ++j) sum[h][j] = 0;
#pragma unroll
        for (int k = 0; k < SPLIT; ++k) {            // integer sums: exact, order-free
          const int32_t* src = (k == krank ? s_stage : s_xch) + (static_cast<size_t>(k) * kBlockN + r) * W + u0;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if constexpr (G == 4) {
              const int4 t = *reinterpret_cast<const int4*>(src + h * MS);
              sum[h][0] += t.x; sum[h][1] += t.y; sum[h][2] += t.z; sum[h][3] += t.w;
            } else {
              const int2 t = *reinterpret_cast<const int2*>(src + h * MS);
              sum[h][0] += t.x; sum[h][1] += t.y;
            }
          }
        }
#pragma unroll
        for (int j = 0; j < G; ++j) {
          const int m = krank * MS + u0 + j;
          if constexpr (ROPE) {
            float2 cs = make_float2(1.f, 0.f);
            long long off = -1;
#pragma unroll
            for (int jj = 0; jj < MS; ++jj)
              if (jj == u0 + j) { cs = cs_v[jj]; off = off_v[jj]; }
            rope_finish(recombine(sum[0][j], sum[1][j], zero, zero_int, zero_is_int, s_qsum[m]) * (scale * s_sx[m]), cs, off, m, m < p.M && store && ok);
          } else if (m < p.M && store && ok) {
            float out = recombine(sum[0][j], sum[1][j], zero, zero_int, zero_is_int, s_qsum[m]) * (scale * s_sx[m]);
            if (p.epilogue == CACHEIR_B200_EPI_RESIDUAL) {
              float rv = 0.f;
#pragma unroll
              for (int jj = 0; jj < MS; ++jj) rv = (jj == u0 + j) ? res_v[jj] : rv;   // register select, no local array
              out += rv;
            }
            y[static_cast<size_t>(m) * p.n_out + n_out_idx] = __float2half_rn(out);
          }
        }
      }
      cluster_wait();                                // phase B: every rank has received everything, this CTA's copies included
    } else if (swiglu) {
      // eight batch rows at a time: up rows hand their values over through the drained ring, gate rows finish
      float* s_up = reinterpret_cast<float*>(smem);          // [MP][64]
#pragma unroll 1
      for (int c0 = 0; c0 < MP; c0 += 8) {
        uint32_t hi[8], lo[8];
        if (total > 0) {
          tc_ld_x8(tmem_base + lane_addr + c0, hi);
          tc_ld_x8(tmem_base + lane_addr + MP + c0, lo);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) { hi[j] = 0u; lo[j] = 0u; }
        }
        float g[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int m = c0 + j;
          g[j] = recombine(static_cast<int32_t>(hi[j]), static_cast<int32_t>(lo[j]), zero, zero_int, zero_is_int, s_qsum[m]) * (scale * s_sx[m]);
          if (is_up) s_up[m * kPairRows + (r - kPairRows)] = g[j];
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!is_up && store) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int m = c0 + j;
            if (m < p.M) {
              const float u = s_up[m * kPairRows + r];
              y[static_cast<size_t>(m) * p.n_out + n_out_idx] = __float2half_rn(silu_fast(g[j]) * u);
            }
          }
        }
      }
    } else {
#pragma unroll 1
      for (int c0 = 0; c0 < MP; c0 += 8) {
        uint32_t hi[8], lo[8];
        if (total > 0) {
          tc_ld_x8(tmem_base + lane_addr + c0, hi);
          tc_ld_x8(tmem_base + lane_addr + MP + c0, lo);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) { hi[j] = 0u; lo[j] = 0u; }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int m = c0 + j;
          if constexpr (ROPE) {
            float2 cs;
            long long off;
            rope_row(m, &cs, &off);
            rope_finish(recombine(static_cast<int32_t>(hi[j]), static_cast<int32_t>(lo[j]), zero, zero_int, zero_is_int, s_qsum[m]) * (scale * s_sx[m]),
                        cs, off, m, m < p.M && store);
          } else if (m < p.M && store) {
            float out = recombine(static_cast<int32_t>(hi[j]), static_cast<int32_t>(lo[j]), zero, zero_int, zero_is_int, s_qsum[m]) * (scale * s_sx[m]);
            const size_t o = static_cast<size_t>(m) * p.n_out + n_out_idx;
            if (p.epilogue == CACHEIR_B200_EPI_RESIDUAL) out += __half2float(res[o]);
            y[o] = __float2half_rn(out);
          }
        }
      }
    }
  }
  if (warp < 2 && clustered) {   // warps without an epilogue still take part in every phase of the cluster barrier
    __syncwarp();
    cluster_wait();
    cluster_arrive_relaxed();
    cluster_wait();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tc_dealloc(tmem_base, kTmemCols);
  }
}

// CTAs per cluster along K. Every doubling adds cluster-barrier and exchange time to the epilogue, so the
// split only grows while the grid stays within two CTAs per SM; a power of two that leaves each rank at
// least two batch rows to finish and four k blocks to stream. With more than 32 batch rows a split CTA needs
// a whole SM (exchange buffer + ring), so the grid must then fit in one CTA per SM. The SwiGLU form (paired
// tiles, many of them) is not split.
int choose_split_k(int n_tiles, int kblocks, int epilogue, int mp) {
  if (epilogue == CACHEIR_B200_EPI_SWIGLU) return 1;
  const int slots = mp > 32 ? kNumSMs : 2 * kNumSMs;
  int s = 1;
  while (s * 2 <= kMaxSplitK && n_tiles * s * 2 <= slots && kblocks / (s * 2) >= 4 && mp / (s * 2) >= 2) s *= 2;
  return s;
}

int launch_quantize(const __half* x, long long x_stride, int M, int K, int mp, void* workspace, cudaStream_t stream) {
  int8_t* planes = static_cast<int8_t*>(workspace);
  float* sx = reinterpret_cast<float*>(planes + static_cast<size_t>(2 * mp) * K);
  int* qsum = reinterpret_cast<int*>(sx + 64);
  if (K <= 8192) quantize_rows_fast_kernel<1><<<mp, 1024, 0, stream>>>(x, x_stride, M, K, mp, planes, sx, qsum);
  else if (K <= 16384) quantize_rows_fast_kernel<2><<<mp, 1024, 0, stream>>>(x, x_stride, M, K, mp, planes, sx, qsum);
  else quantize_rows_kernel<<<mp, 256, 0, stream>>>(x, x_stride, M, K, mp, planes, sx, qsum);
  return launch_status();
}

template <int MP, int SPLIT, bool ROPE, int BITS>
cudaError_t launch_i8_split(const CUtensorMap& tmap_w, const I8Params& p, cudaStream_t stream) {
  constexpr size_t kSmem = 1024 + static_cast<size_t>(num_stages(MP, SPLIT, BITS)) * stage_bytes(MP, BITS) + exchange_bytes(MP, SPLIT) + kTailBytes;
  static_assert(num_stages(MP, SPLIT, BITS) >= 2, "the pipeline needs at least two stages");
  static_assert(num_stages(MP, SPLIT, BITS) * (kBlockN * kBlockK + 2 * MP * kBlockK) >= exchange_bytes(MP, SPLIT) || SPLIT == 1,
                "outgoing partials are staged in the drained byte and activation tiles at the head of the ring");
  static_assert(kTailBytes >= (3 * 8 + 2) * 8 + 8 + 2 * 64 * 4, "barriers, TMEM base and per-row constants fit behind the exchange buffer");
  auto kern = qgemm_i8_kernel<MP, SPLIT, ROPE, BITS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmem));
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.n_tiles, SPLIT, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = SPLIT;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, tmap_w, p);
}

template <int MP, bool ROPE, int BITS>
cudaError_t launch_i8_by_split(const CUtensorMap& tmap_w, const I8Params& p, cudaStream_t stream) {
  switch (p.split_k) {
    case 8: return launch_i8_split<MP, 8, ROPE, BITS>(tmap_w, p, stream);
    case 4: return launch_i8_split<MP, 4, ROPE, BITS>(tmap_w, p, stream);
    case 2: return launch_i8_split<MP, 2, ROPE, BITS>(tmap_w, p, stream);
    default: return launch_i8_split<MP, 1, ROPE, BITS>(tmap_w, p, stream);
  }
}

template <int MP>
int launch_i8(const QGemvParams& q, void* workspace, cudaStream_t stream) {
  int8_t* planes = static_cast<int8_t*>(workspace);
  float* sx = reinterpret_cast<float*>(planes + static_cast<size_t>(2 * MP) * q.K);
  int* qsum = reinterpret_cast<int*>(sx + 64);
  if (!q.x_prequantized) {   // the activation pre-pass, with the RMSNorm in front of it if one was asked for
    const int rc = q.norm_weight
        ? qgemm_i8_rms_norm_quantize(q.x, nullptr, q.norm_weight, nullptr, nullptr, q.M, q.K, q.norm_eps, workspace, stream)
        : launch_quantize(static_cast<const __half*>(q.x), q.x_stride, q.M, q.K, MP, workspace, stream);
    if (rc != 0) return rc;
  }

  CUtensorMap tmap_w;
  // (the tiled layout is fetched with plain bulk copies; its map is only a valid placeholder)
  const bool swiglu = q.epilogue == CACHEIR_B200_EPI_SWIGLU;
  const uint64_t bands = static_cast<uint64_t>((q.N + kBlockN - 1) / kBlockN);
  const uint64_t row_bytes = q.bits == 4 ? static_cast<uint64_t>(q.K / 2) : static_cast<uint64_t>(q.K);
  const bool w_ok = q.tiled
      ? encode_u8_rows_sw128(&tmap_w, q.packed, kBlockK, bands * (q.K / kBlockK) * (q.bits == 4 ? kBlockN / 2 : kBlockN), kBlockK, kBlockN)
      : (q.bits == 4 ? encode_u8_rows_sw64(&tmap_w, q.packed, row_bytes, static_cast<uint64_t>(q.N), row_bytes, swiglu ? kPairRows : kBlockN)
                     : encode_u8_rows_sw128(&tmap_w, q.packed, row_bytes, static_cast<uint64_t>(q.N), row_bytes, swiglu ? kPairRows : kBlockN));
  if (!w_ok) return CACHEIR_B200_EUNSUPPORTED;
  I8Params p{};
  p.scales = q.scales; p.zero_points = q.zero_points; p.residual = q.residual; p.y = q.y;
  p.sx = sx; p.qsum = qsum;
  p.w_tiled = static_cast<const uint8_t*>(q.packed); p.x_planes = planes;
  p.M = q.M; p.N = q.N; p.K = q.K;
  p.n_out = q.epilogue == CACHEIR_B200_EPI_SWIGLU ? q.N / 2 : q.N;
  p.scale_dtype = q.scale_dtype; p.epilogue = q.epilogue; p.tiled = q.tiled ? 1 : 0;
  p.rope = q.rope;
  p.n_tiles = swiglu ? (p.n_out + kPairRows - 1) / kPairRows : (p.n_out + kBlockN - 1) / kBlockN;
  p.split_k = choose_split_k(p.n_tiles, q.K / kBlockK, q.epilogue, MP);
  cudaError_t e;
  if (q.epilogue == kEpiQkvRopeAppend) e = launch_i8_by_split<MP, true, 8>(tmap_w, p, stream);
  else if (q.bits == 4) e = launch_i8_by_split<MP, false, 4>(tmap_w, p, stream);
  else e = launch_i8_by_split<MP, false, 8>(tmap_w, p, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  return launch_status();
}

}  // namespace

size_t qgemm_i8_workspace_bytes(int M, int K) {
  if (M <= 0 || K <= 0) return 0;
  return static_cast<size_t>(128) * K + 1024;   // two planes of up to 64 rows, then scales and sums
}

bool qgemm_i8_supported(const QGemvParams& q, const void* workspace, size_t workspace_bytes) {
  if (q.x_dtype != CACHEIR_B200_F16 || (q.bits != 8 && q.bits != 4) || q.group_size != 0) return false;
  if (q.bits == 4 && q.epilogue == kEpiQkvRopeAppend) return false;      // the fused QKV form is built for int8 only
  if (q.M < 1 || q.M > 64) return false;
  if (q.K % kBlockK != 0 || q.K < kBlockK || q.K > 32768) return false;   // 32-bit accumulators and epilogue arithmetic
  if (q.epilogue == CACHEIR_B200_EPI_SWIGLU && ((q.N / 2) % kPairRows != 0 || (q.tiled && !q.paired))) return false;
  if (q.paired && !(q.tiled && q.epilogue == CACHEIR_B200_EPI_SWIGLU)) return false;
  if (!workspace || workspace_bytes < qgemm_i8_workspace_bytes(q.M, q.K) || !aligned_to(workspace, 128)) return false;
  if (!aligned_to(q.packed, 16) || !aligned_to(q.x, 16) || (q.x_stride * 2) % 16 != 0) return false;
  // an RMSNorm in front runs inside the pre-pass kernel: dense rows, K <= 8192
  if (q.norm_weight && (!aligned_to(q.norm_weight, 16) || q.x_prequantized || q.K > 8192 || q.x_stride != q.K)) return false;
  return tensor_map_encoder() != nullptr;
}

// The split-K factor launch_qgemm_i8 would choose for these extents.
int qgemm_i8_plan(const QGemvParams& q) {
  const int mp = q.M <= 16 ? 16 : (q.M <= 32 ? 32 : 64);
  const bool swiglu = q.epilogue == CACHEIR_B200_EPI_SWIGLU;
  const int n_out = swiglu ? q.N / 2 : q.N;
  const int n_tiles = swiglu ? (n_out + kPairRows - 1) / kPairRows : (n_out + kBlockN - 1) / kBlockN;
  return choose_split_k(n_tiles, q.K / kBlockK, q.epilogue, mp);
}

int launch_qgemm_i8(const QGemvParams& q, void* workspace, cudaStream_t stream) {
  if (q.M <= 16) return launch_i8<16>(q, workspace, stream);
  if (q.M <= 32) return launch_i8<32>(q, workspace, stream);
  return launch_i8<64>(q, workspace, stream);
}

int i8_plane_rows(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }

int qgemm_i8_quantize_activations(const void* x, long long x_stride, int M, int K, void* workspace, cudaStream_t stream) {
  return launch_quantize(static_cast<const __half*>(x), x_stride, M, K, i8_plane_rows(M), workspace, stream);
}

int qgemm_i8_rms_norm_quantize(const void* x, const void* residual, const void* weight, void* sum_out, void* out, int M,
                               int hidden, float eps, void* workspace, cudaStream_t stream) {
  const int mp = i8_plane_rows(M);
  int8_t* planes = static_cast<int8_t*>(workspace);
  float* sx = reinterpret_cast<float*>(planes + static_cast<size_t>(2 * mp) * hidden);
  int* qsum = reinterpret_cast<int*>(sx + 64);
  const __half* xp = static_cast<const __half*>(x);
  const __half* rp = static_cast<const __half*>(residual);
  const __half* wp = static_cast<const __half*>(weight);
  __half* sp = static_cast<__half*>(sum_out);
  __half* op = static_cast<__half*>(out);
  if (hidden <= 4096) rms_norm_quantize_kernel<1><<<mp, 512, 0, stream>>>(xp, rp, wp, sp, op, M, hidden, eps, mp, planes, sx, qsum);
  else if (hidden <= 8192) rms_norm_quantize_kernel<2><<<mp, 512, 0, stream>>>(xp, rp, wp, sp, op, M, hidden, eps, mp, planes, sx, qsum);
  else return CACHEIR_B200_EUNSUPPORTED;
  return launch_status();
}

int qgemm_i8_device_status(bool reset) {
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_i8_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_i8_status, &zero, sizeof(int));
  }
  return status;
}

}  // namespace cb200
