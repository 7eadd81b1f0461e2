// Streaming int4 dequant-GEMV for up to 8 batch rows, fp16 activations, sm_100a.
//
//   y[M, N] = x[M, K] . deq(W)[N, K]^T,   M <= 8, K % 128 == 0
//   group-wise symmetric: deq = (code - 8) * scale[n, k / group]   (group a multiple of 128)
//   per-row affine:       deq = (code - zero[n]) * scale[n]        (the reference's int4 pack)
//
// HBM-bound byte streaming: the packed rows are read exactly once, in the reference's row-major layout, with
// 16-byte loads; nibbles become fp16 in registers (two per instruction: (w >> 4i) & 0x000F000F | 0x64006400 is
// the pair (1024 + n_i, 1024 + n_{i+4}), minus 1032 gives n - 8 exactly) and go straight into mma.sync m16n8k16
// as the 16-row operand, with the batch rows as the 8 columns and fp32 accumulation. A warp owns 16 weight rows
// and half of K; per 128-column block it issues 8 MMAs, then folds the block's sums into its running result
// with the group scales of its two rows. The k order inside an MMA is whatever the nibble pairing gives: x is
// staged in shared memory in the same order, so a lane's four (b0, b1) pairs of a packed word are one 16-byte
// load. The two K halves of a row tile meet in shared memory and are added in a fixed order.
#include "common.cuh"
#include "qgemv_common.cuh"

namespace cb200 {
namespace {

constexpr int kTileRows = 16;
constexpr int kChunkK = 4096;        // columns of x staged at a time
constexpr int kRowPadBytes = 64;     // staged rows are 64 bytes apart modulo 128: eight lanes of a load phase hit eight bank groups

struct MmaGemvParams {
  const __half* x;
  const uint8_t* packed;
  const void* scales;
  const float* zero_points;
  const __half* residual;
  __half* y;
  int M, N, K;
  int n_out;
  int group_size;     // 0: one scale (and zero point) per row
  int scale_dtype;
  int epilogue;
  long long x_stride;
};

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// nibbles i and i+4 of `w` as the fp16 pair (n_i - 8, n_{i+4} - 8)
__device__ __forceinline__ uint32_t nibble_pair(uint32_t w, int i) {
  const uint32_t biased = ((w >> (4 * i)) & 0x000F000Fu) | 0x64006400u;     // (1024 + n_i, 1024 + n_{i+4})
  const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&biased), __half2half2(__ushort_as_half(0x6408)));   // 0x6408 = 1032
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float scale_value(const void* scales, int scale_dtype, size_t idx) {
  return scale_dtype == CACHEIR_B200_F16 ? __half2float(static_cast<const __half*>(scales)[idx]) : static_cast<const float*>(scales)[idx];
}

// One CTA per SM: 8 tile slots x 2 K halves = 16 warps. x is staged once per CTA (per 4096-column chunk) and serves
// every row tile the CTA visits; tile t belongs to CTA t % grid, slot (t / grid) % 8, so the tiles spread evenly over
// the SMs. With the SwiGLU epilogue a slot handles the 16 gate rows and then the 16 up rows of its output columns.
// Shared memory: the staged chunk of x, [M batch rows][row_bytes], inside a row the 16-byte units of a 128-column
// block at unit (j*4 + q) for columns q*32 + j*8 .. +7, the eight values in the order 0,4,1,5,2,6,3,7; then the
// per-warp partial results and the row sums of x.
constexpr int kSlots = 8;
constexpr int kKSplit = 2;
constexpr int kThreadsMma = kSlots * kKSplit * 32;

struct CodeRegs {
  uint4 lo, hi;        // 32 codes of row g and of row g+8
  float s_lo, s_hi;    // their group scales
};

template <bool SWIGLU>
__global__ void __launch_bounds__(kThreadsMma, 1)
qgemv_mma_int4_kernel(const MmaGemvParams p) {
  constexpr int HALVES = SWIGLU ? 2 : 1;     // weight tiles per output tile
  extern __shared__ __align__(16) uint8_t smem[];
  const int chunk_cols = p.K < kChunkK ? p.K : kChunkK;
  const int row_bytes = chunk_cols * 2 + kRowPadBytes;
  uint8_t* xs = smem;
  float* s_red = reinterpret_cast<float*>(smem + p.M * row_bytes);    // [16 warps][HALVES][16 rows][8 columns]
  float* s_xsum = s_red + kSlots * kKSplit * HALVES * kTileRows * 8;  // [8]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int slot = warp >> 1, kh = warp & 1;
  const size_t row_stride = static_cast<size_t>(p.K) / 2;
  const int groups_per_row = p.group_size > 0 ? p.K / p.group_size : 1;
  const int n_units = (p.n_out + kTileRows - 1) / kTileRows;
  const uint8_t* x_lane = xs + min(g, p.M - 1) * row_bytes + q * 16;   // MMA column g is batch row g; columns past M repeat the last row and are never stored

  // Stage x[:, c0 : c0 + cols] in MMA order: 16-byte units (8 columns), four loads in flight per thread.
  auto stage_x = [&](int c0, int cols) {
    const int units = cols / 8;
    const int total_units = p.M * units;
    for (int u0 = threadIdx.x; u0 < total_units; u0 += 4 * kThreadsMma) {
      uint4 raw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int u = u0 + i * kThreadsMma;
        raw[i] = make_uint4(0u, 0u, 0u, 0u);
        if (u < total_units) {
          const int m = u / units, unit = u - m * units;
          raw[i] = *reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(m) * p.x_stride + c0 + unit * 8);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int u = u0 + i * kThreadsMma;
        if (u < total_units) {
          const int m = u / units, unit = u - m * units;
          const uint32_t w0 = raw[i].x, w1 = raw[i].y, w2 = raw[i].z, w3 = raw[i].w;   // (h0,h1) (h2,h3) (h4,h5) (h6,h7)
          const uint4 o = make_uint4(__byte_perm(w0, w2, 0x5410), __byte_perm(w0, w2, 0x7632),      // order 0,4,1,5,2,6,3,7
                                     __byte_perm(w1, w3, 0x5410), __byte_perm(w1, w3, 0x7632));
          const int kb = unit >> 4, in_block = unit & 15, qq = in_block >> 2, jj = in_block & 3;
          *reinterpret_cast<uint4*>(xs + m * row_bytes + (kb * 16 + jj * 4 + qq) * 16) = o;
        }
      }
    }
  };

  if (p.group_size == 0) {                   // per-row affine form: the sums of the batch rows, each by one warp in a fixed order
    for (int m = warp; m < p.M; m += kSlots * kKSplit) {
      const __half* xr = p.x + static_cast<size_t>(m) * p.x_stride;
      float s = 0.f;
      for (int k = lane * 8; k < p.K; k += 256) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr + k);
        const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h2[i]); s += f.x + f.y; }
      }
      s = warp_sum(s);
      if (lane == 0) s_xsum[m] = s;
    }
  }

  // Tiles of this slot: t = blockIdx.x + grid * (slot + 8 i). Every warp of the CTA runs the same number of rounds and
  // chunks (the barriers around the staging of x are CTA-wide); a warp without a tile in a round only takes part in them.
  const int rounds = (n_units + static_cast<int>(gridDim.x) * kSlots - 1) / (static_cast<int>(gridDim.x) * kSlots);
  for (int round = 0; round < rounds; ++round) {
    const int unit = static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) * (slot + kSlots * round);
    const bool have = unit < n_units;
    const int n0 = unit * kTileRows;                                       // first output column of the tile
    float acc[HALVES][4];
#pragma unroll
    for (int h = 0; h < HALVES; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[h][i] = 0.f;

    for (int c0 = 0; c0 < p.K; c0 += chunk_cols) {
      const int cols = min(chunk_cols, p.K - c0);
      if (round == 0 || chunk_cols < p.K) {   // (a single chunk stays staged for all rounds)
        __syncthreads();                      // the previous chunk has been consumed
        stage_x(c0, cols);
        __syncthreads();
      }
      if (!have) continue;
      const int blocks = cols / 128;
      const int b_begin = (blocks * kh) / kKSplit, b_end = (blocks * (kh + 1)) / kKSplit;
      const int kb0 = c0 / 128;
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        const int w_row0 = n0 + h * (p.N / 2);
        // rows this lane feeds (clamped: rows past N are computed on a valid row and never stored)
        const int r_lo = min(w_row0 + g, p.N - 1), r_hi = min(w_row0 + g + 8, p.N - 1);
        const uint8_t* w_lo = p.packed + static_cast<size_t>(r_lo) * row_stride + q * 16;
        const uint8_t* w_hi = p.packed + static_cast<size_t>(r_hi) * row_stride + q * 16;
        auto fetch = [&](int b) {
          CodeRegs r;
          r.lo = *reinterpret_cast<const uint4*>(w_lo + static_cast<size_t>(kb0 + b) * 64);
          r.hi = *reinterpret_cast<const uint4*>(w_hi + static_cast<size_t>(kb0 + b) * 64);
          r.s_lo = 1.f; r.s_hi = 1.f;
          if (p.group_size > 0) {
            const int grp = ((kb0 + b) * 128) / p.group_size;
            r.s_lo = scale_value(p.scales, p.scale_dtype, static_cast<size_t>(r_lo) * groups_per_row + grp);
            r.s_hi = scale_value(p.scales, p.scale_dtype, static_cast<size_t>(r_hi) * groups_per_row + grp);
          }
          return r;
        };
        // One 128-column block: 8 MMAs on the unpacked nibbles (two chains), then the block's sums join the result with the rows' group scales.
        auto do_block = [&](int b, const CodeRegs& r) {
          float c[4] = {0.f, 0.f, 0.f, 0.f}, d[4] = {0.f, 0.f, 0.f, 0.f};
          const uint32_t wa[4] = {r.lo.x, r.lo.y, r.lo.z, r.lo.w};
          const uint32_t wb[4] = {r.hi.x, r.hi.y, r.hi.z, r.hi.w};
          const uint8_t* xrow = x_lane + b * 256;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xrow + j * 64);     // (x0,x4) (x1,x5) (x2,x6) (x3,x7) of the word's 8 columns
            mma_16816(c, nibble_pair(wa[j], 0), nibble_pair(wb[j], 0), nibble_pair(wa[j], 1), nibble_pair(wb[j], 1), xv.x, xv.y);
            mma_16816(d, nibble_pair(wa[j], 2), nibble_pair(wb[j], 2), nibble_pair(wa[j], 3), nibble_pair(wb[j], 3), xv.z, xv.w);
          }
          acc[h][0] = fmaf(c[0] + d[0], r.s_lo, acc[h][0]); acc[h][1] = fmaf(c[1] + d[1], r.s_lo, acc[h][1]);
          acc[h][2] = fmaf(c[2] + d[2], r.s_hi, acc[h][2]); acc[h][3] = fmaf(c[3] + d[3], r.s_hi, acc[h][3]);
        };
        // four blocks of codes (and their scales) are on their way while one is multiplied
        CodeRegs ring[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (b_begin + i < b_end) ring[i] = fetch(b_begin + i);
        for (int b = b_begin; b < b_end; b += 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (b + i < b_end) {
              const CodeRegs cur = ring[i];
              if (b + 4 + i < b_end) ring[i] = fetch(b + 4 + i);
              do_block(b + i, cur);
            }
          }
        }
      }
    }

    // ---- the two K halves of a tile meet in shared memory and are added in order (named barrier of the slot's 64 threads) ----
    if (have) {
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        float* mine = s_red + ((warp * HALVES + h) * kTileRows) * 8;
        mine[g * 8 + 2 * q] = acc[h][0]; mine[g * 8 + 2 * q + 1] = acc[h][1];
        mine[(g + 8) * 8 + 2 * q] = acc[h][2]; mine[(g + 8) * 8 + 2 * q + 1] = acc[h][3];
      }
    }
    asm volatile("bar.sync %0, 64;" ::"r"(1 + slot) : "memory");
    if (have) {
      // 16 x 8 results, two per thread of the slot
      const int tt = (kh << 5) | lane;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int idx = tt * 2 + e, row = idx >> 3, m = idx & 7;
        const int n = n0 + row;
        if (m < p.M && n < p.n_out) {
          auto finish = [&](int h, int wrow) {     // halves in order; then the per-row scale / zero point of the affine form
            float v = 0.f;
#pragma unroll
            for (int k = 0; k < kKSplit; ++k) v += s_red[((((slot * kKSplit + k) * HALVES) + h) * kTileRows + row) * 8 + m];
            if (p.group_size == 0) {
              const float zp = p.zero_points ? p.zero_points[wrow] : 8.f;
              v = (v + (8.f - zp) * s_xsum[m]) * scale_value(p.scales, p.scale_dtype, wrow);
            }
            return v;
          };
          const size_t o = static_cast<size_t>(m) * p.n_out + n;
          if (SWIGLU) {
            p.y[o] = __float2half_rn(silu_fast(finish(0, n)) * finish(1, p.N / 2 + n));
          } else {
            float v = finish(0, n);
            if (p.epilogue == CACHEIR_B200_EPI_RESIDUAL) v += __half2float(p.residual[o]);
            p.y[o] = __float2half_rn(v);
          }
        }
      }
    }
    asm volatile("bar.sync %0, 64;" ::"r"(1 + slot) : "memory");     // the partial results are free for the slot's next tile
  }
}

size_t mma_gemv_smem_bytes(int M, int K, bool swiglu) {
  const int chunk_cols = K < kChunkK ? K : kChunkK;
  return static_cast<size_t>(M) * (chunk_cols * 2 + kRowPadBytes) + (kSlots * kKSplit * (swiglu ? 2 : 1) * kTileRows * 8 + 8) * sizeof(float);
}

}  // namespace

bool qgemv_mma_supported(const QGemvParams& q) {
  if (q.bits != 4 || q.x_dtype != CACHEIR_B200_F16 || q.tiled || q.paired || q.x_prequantized || q.norm_weight) return false;
  if (q.M < 1 || q.M > 8 || q.K % 128 != 0 || q.K < 128) return false;
  if (q.group_size != 0 && q.group_size % 128 != 0) return false;
  if (q.group_size != 0 && q.zero_points) return false;
  if (q.epilogue == CACHEIR_B200_EPI_SWIGLU && (q.N / 2) % kTileRows != 0) return false;
  if (q.epilogue == kEpiQkvRopeAppend) return false;
  return aligned_to(q.packed, 16) && aligned_to(q.x, 16) && (q.x_stride * 2) % 16 == 0;
}

int launch_qgemv_mma(const QGemvParams& q, cudaStream_t stream) {
  MmaGemvParams p{};
  p.x = static_cast<const __half*>(q.x);
  p.packed = static_cast<const uint8_t*>(q.packed);
  p.scales = q.scales; p.zero_points = q.zero_points;
  p.residual = static_cast<const __half*>(q.residual);
  p.y = static_cast<__half*>(q.y);
  p.M = q.M; p.N = q.N; p.K = q.K;
  const bool swiglu = q.epilogue == CACHEIR_B200_EPI_SWIGLU;
  p.n_out = swiglu ? q.N / 2 : q.N;
  p.group_size = q.group_size; p.scale_dtype = q.scale_dtype; p.epilogue = q.epilogue; p.x_stride = q.x_stride;
  const size_t smem = mma_gemv_smem_bytes(q.M, q.K, swiglu);
  // One CTA per SM (fewer when there are fewer tiles than slots); tiles are dealt out round robin over the CTAs first.
  const int n_units = (p.n_out + kTileRows - 1) / kTileRows;
  const int grid = n_units < kNumSMs ? n_units : kNumSMs;
  cudaError_t e;
  if (swiglu) {
    e = cudaFuncSetAttribute(qgemv_mma_int4_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    qgemv_mma_int4_kernel<true><<<grid, kThreadsMma, smem, stream>>>(p);
  } else {
    e = cudaFuncSetAttribute(qgemv_mma_int4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    qgemv_mma_int4_kernel<false><<<grid, kThreadsMma, smem, stream>>>(p);
  }
  return launch_status();
}

}  // namespace cb200
