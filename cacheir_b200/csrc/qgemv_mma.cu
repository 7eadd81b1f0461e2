// Streaming int4 dequant-GEMV for up to 8 batch rows, fp16 activations, sm_100a.
//
//   y[M, N] = x[M, K] . deq(W)[N, K]^T,   M <= 8, K % 128 == 0
//   group-wise symmetric: deq = (code - 8) * scale[n, k / group]   (group a multiple of 128)
//   per-row affine:       deq = (code - zero[n]) * scale[n]        (the reference's int4 pack)
//
// HBM-bound byte streaming: the packed rows are read exactly once, in the reference's row-major layout, with
// 16-byte loads; nibbles become fp16 in registers, two per shift-and-mask: (w >> 4i) & 0x000F000F | 0x64006400 is
// the pair (1024 + n_i, 1024 + n_{i+4}), exact in fp16. They go straight into mma.sync m16n8k16 as the 16-row
// operand, with the batch rows as the 8 columns and fp32 accumulation; the constant 1024 + zero leaves through the
// sum of x over the 128-column block, which the accumulators start from. The k order inside an MMA is whatever the
// nibble pairing gives: x is staged in shared memory in the same order, so a lane's four (b0, b1) pairs of a packed
// word are one 16-byte load.
#include <type_traits>

#include "common.cuh"
#include "qgemv_common.cuh"

namespace cb200 {
namespace {

constexpr int kTileRows = 16;
constexpr int kRowPadBytes = 64;     // staged rows are 64 bytes apart modulo 128: eight lanes of a load phase hit eight bank groups
constexpr int kWarps = 16;
constexpr int kThreadsMma = kWarps * 32;
constexpr int kRoundTiles = 16;      // weight tiles a CTA works on at a time: a warp's share of them spans at most two
constexpr int kRing = 4;             // 128-column blocks of codes in flight per warp
constexpr size_t kStageBudget = 160 * 1024;   // bytes of shared memory the staged activations may take

struct MmaGemvParams {
  const __half* x;
  const uint8_t* packed;
  const void* scales;
  const float* zero_points;
  const __half* residual;
  __half* y;
  int M, N, K;
  int n_out;
  int group_shift;    // group size = 128 << group_shift (group-wise form)
  int epilogue;
  int chunk_cols;     // columns of x staged at a time (a multiple of 128; K when everything fits)
  int max_tiles;      // weight tiles of the busiest CTA (sizes the cross-chunk sums)
  long long x_stride;
};

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// nibbles i and i+4 of `w` as the fp16 pair (1024 + n_i, 1024 + n_{i+4}): exact, one shift and one logic operation.
// The offset leaves through the block's sum of x: sum (n - z) x = sum (1024 + n) x - (1024 + z) sum x.
__device__ __forceinline__ uint32_t nibble_pair(uint32_t w, int i) {
  return ((w >> (4 * i)) & 0x000F000Fu) | 0x64006400u;
}
__device__ __forceinline__ uint4 load_codes(const uint8_t* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}

struct CodeRegs {
  uint4 lo, hi;        // 32 codes of row g and of row g+8
  float s_lo, s_hi;    // their group scales
};

// One CTA per SM, 16 warps. The CTA owns the output tiles blockIdx.x + grid * i (16 output columns each; with the
// SwiGLU epilogue a gate and an up weight tile per output tile). It takes its weight tiles 16 at a time and deals the
// (tile, 128-column block) units of such a round out evenly: warp w gets units [U w / 16, U (w+1) / 16), a run along K
// that crosses at most one tile boundary, so every warp streams the same number of bytes whatever the tile count.
// A warp keeps four blocks of codes in flight in registers; per block it issues 8 MMAs (two chains) whose
// accumulators start at -(1024 + zero) * sum(x over the block), then folds them into its running sums with the two
// rows' group scales. Partial sums meet in shared memory and are added in warp order.
// Shared memory: x of the current chunk, [M][row_bytes], inside a row the 16-byte units of a 128-column block at unit
// (j*4 + q) for columns q*32 + j*8 .. +7, the eight values in the order 0,4,1,5,2,6,3,7; the block sums of x
// [block][8]; the warps' partial sums [16][2][8][16]; their tile ranges; the cross-chunk sums [tile][8][16].
template <bool SWIGLU, bool GROUPED, bool F16SCALE>
__global__ void __launch_bounds__(kThreadsMma, 1)
qgemv_mma_int4_kernel(const MmaGemvParams p) {
  constexpr int HALVES = SWIGLU ? 2 : 1;     // weight tiles per output tile
  using scale_t = typename std::conditional<F16SCALE, __half, float>::type;
  extern __shared__ __align__(16) uint8_t smem[];
  const int row_bytes = p.chunk_cols * 2 + kRowPadBytes;
  uint8_t* xs = smem;
  float* s_xblk = reinterpret_cast<float*>(smem + p.M * row_bytes);
  float* s_part = s_xblk + (p.chunk_cols / 128) * 8;
  int* s_rng = reinterpret_cast<int*>(s_part + kWarps * 2 * 128);
  float* s_tile = reinterpret_cast<float*>(s_rng + kWarps * 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int grid = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
  const size_t row_stride = static_cast<size_t>(p.K) / 2;
  const int groups_per_row = GROUPED ? ((p.K / 128) >> p.group_shift) : 1;
  const scale_t* scales = static_cast<const scale_t*>(p.scales);
  const int n_units = (p.n_out + kTileRows - 1) / kTileRows;
  const int tiles = ((n_units - cta + grid - 1) / grid) * HALVES;            // weight tiles of this CTA (>= HALVES)
  const uint8_t* x_lane = xs + min(g, p.M - 1) * row_bytes + q * 16;         // MMA column g is batch row g; columns past M repeat the last row and are never stored
  const float* xblk_lane = s_xblk + 2 * q;
  const bool multi_chunk = p.chunk_cols < p.K;

  // first weight row of weight tile `wt` of this CTA
  auto tile_row0 = [&](int wt) {
    const int i = wt / HALVES, h = wt - i * HALVES;
    return (cta + grid * i) * kTileRows + h * (p.N / 2);
  };

  for (int i = threadIdx.x; i < (p.chunk_cols / 128) * 8; i += kThreadsMma)
    if ((i & 7) >= p.M) s_xblk[i] = 0.f;

  // Stage x[:, c0 : c0 + cols] in MMA order (16-byte units of 8 columns, four loads in flight per thread) and the
  // sum of every (128-column block, batch row): eight values in order, then a butterfly over the block's 16 lanes.
  auto stage_x = [&](int c0, int cols) {
    const int units = cols / 8;
    const int total_units = p.M * units;          // a multiple of 16: a half-warp is inside or outside as a whole
    for (int base = warp * 32; base < total_units; base += 4 * kThreadsMma) {
      uint4 raw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int u = base + lane + i * kThreadsMma;
        raw[i] = make_uint4(0u, 0u, 0u, 0u);
        if (u < total_units) {
          const int m = u / units, unit = u - m * units;
          raw[i] = *reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(m) * p.x_stride + c0 + unit * 8);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int u = base + lane + i * kThreadsMma;
        const bool valid = u < total_units;
        const int m = valid ? u / units : 0, unit = u - m * units;
        const uint32_t w0 = raw[i].x, w1 = raw[i].y, w2 = raw[i].z, w3 = raw[i].w;   // (h0,h1) (h2,h3) (h4,h5) (h6,h7)
        const int kb = unit >> 4, in_block = unit & 15, qq = in_block >> 2, jj = in_block & 3;
        if (valid) {
          const uint4 o = make_uint4(__byte_perm(w0, w2, 0x5410), __byte_perm(w0, w2, 0x7632),      // order 0,4,1,5,2,6,3,7
                                     __byte_perm(w1, w3, 0x5410), __byte_perm(w1, w3, 0x7632));
          *reinterpret_cast<uint4*>(xs + m * row_bytes + (kb * 16 + jj * 4 + qq) * 16) = o;
        }
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&w0)), f1 = __half22float2(*reinterpret_cast<const __half2*>(&w1));
        const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&w2)), f3 = __half22float2(*reinterpret_cast<const __half2*>(&w3));
        float sum = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (valid && (lane & 15) == 0) s_xblk[kb * 8 + m] = sum;
      }
    }
  };

  int chunk = 0;
  for (int c0 = 0; c0 < p.K; c0 += p.chunk_cols, ++chunk) {
    const int cols = min(p.chunk_cols, p.K - c0);
    const int kbc = cols / 128;                    // blocks of this chunk
    const int kb0 = c0 / 128;
    const bool last_chunk = c0 + cols >= p.K;
    for (int r0 = 0; r0 < tiles; r0 += kRoundTiles) {
      const int round_tiles = min(kRoundTiles, tiles - r0);
      const int units = round_tiles * kbc;
      const int ub = (units * warp) / kWarps, ue = (units * (warp + 1)) / kWarps;
      const int first_tile = ub / kbc;

      // ---- fetch cursor: the tile and block the next load reads ----
      int f_t = first_tile, f_b = ub - first_tile * kbc;
      const uint8_t *f_lo, *f_hi;
      const scale_t *f_slo, *f_shi;
      auto point_fetch_at = [&](int t) {
        const int row0 = tile_row0(r0 + min(t, round_tiles - 1));
        // rows this lane feeds (clamped: rows past N are computed on a valid row and never stored)
        const int r_lo = min(row0 + g, p.N - 1), r_hi = min(row0 + g + 8, p.N - 1);
        f_lo = p.packed + static_cast<size_t>(r_lo) * row_stride + (static_cast<size_t>(kb0) * 64 + q * 16);
        f_hi = p.packed + static_cast<size_t>(r_hi) * row_stride + (static_cast<size_t>(kb0) * 64 + q * 16);
        if (GROUPED) {
          f_slo = scales + static_cast<size_t>(r_lo) * groups_per_row;
          f_shi = scales + static_cast<size_t>(r_hi) * groups_per_row;
        }
      };
      point_fetch_at(f_t);
      auto fetch = [&](CodeRegs& r) {
        r.lo = load_codes(f_lo + f_b * 64);
        r.hi = load_codes(f_hi + f_b * 64);
        if (GROUPED) {
          const int grp = (kb0 + f_b) >> p.group_shift;
          r.s_lo = static_cast<float>(f_slo[grp]);
          r.s_hi = static_cast<float>(f_shi[grp]);
        }
        if (++f_b == kbc) { f_b = 0; point_fetch_at(++f_t); }
      };
      CodeRegs ring[kRing];
#pragma unroll
      for (int i = 0; i < kRing; ++i)
        if (ub + i < ue) fetch(ring[i]);

      if (r0 == 0) {                         // (the codes above are on their way while x is staged)
        stage_x(c0, cols);
        __syncthreads();
      }

      // ---- consume cursor ----
      int c_b = ub - first_tile * kbc, c_t = first_tile, pieces = 0;
      float kz_lo = -1032.f, kz_hi = -1032.f;                     // -(1024 + zero point) of the two rows
      auto point_consume_at = [&](int t) {
        if (!GROUPED && p.zero_points) {
          const int row0 = tile_row0(r0 + min(t, round_tiles - 1));
          kz_lo = -(1024.f + p.zero_points[min(row0 + g, p.N - 1)]);
          kz_hi = -(1024.f + p.zero_points[min(row0 + g + 8, p.N - 1)]);
        }
      };
      point_consume_at(c_t);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      auto flush = [&]() {
        if (pieces >= 2) return;                                   // (a warp's run never crosses two tile boundaries)
        float* mine = s_part + (warp * 2 + pieces) * 128;          // [m][row]
        mine[(2 * q) * 16 + g] = acc[0]; mine[(2 * q + 1) * 16 + g] = acc[1];
        mine[(2 * q) * 16 + g + 8] = acc[2]; mine[(2 * q + 1) * 16 + g + 8] = acc[3];
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        ++pieces;
      };
      auto consume = [&](const CodeRegs& r) {
        const float2 xb = *reinterpret_cast<const float2*>(xblk_lane + c_b * 8);
        float c[4], d[4] = {0.f, 0.f, 0.f, 0.f};
        if (GROUPED) { c[0] = c[2] = -1032.f * xb.x; c[1] = c[3] = -1032.f * xb.y; }
        else { c[0] = kz_lo * xb.x; c[1] = kz_lo * xb.y; c[2] = kz_hi * xb.x; c[3] = kz_hi * xb.y; }
        const uint32_t wa[4] = {r.lo.x, r.lo.y, r.lo.z, r.lo.w};
        const uint32_t wb[4] = {r.hi.x, r.hi.y, r.hi.z, r.hi.w};
        const uint8_t* xrow = x_lane + c_b * 256;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 xv = *reinterpret_cast<const uint4*>(xrow + j * 64);     // (x0,x4) (x1,x5) (x2,x6) (x3,x7) of the word's 8 columns
          mma_16816(c, nibble_pair(wa[j], 0), nibble_pair(wb[j], 0), nibble_pair(wa[j], 1), nibble_pair(wb[j], 1), xv.x, xv.y);
          mma_16816(d, nibble_pair(wa[j], 2), nibble_pair(wb[j], 2), nibble_pair(wa[j], 3), nibble_pair(wb[j], 3), xv.z, xv.w);
        }
        if (GROUPED) {
          acc[0] = fmaf(c[0] + d[0], r.s_lo, acc[0]); acc[1] = fmaf(c[1] + d[1], r.s_lo, acc[1]);
          acc[2] = fmaf(c[2] + d[2], r.s_hi, acc[2]); acc[3] = fmaf(c[3] + d[3], r.s_hi, acc[3]);
        } else {
          acc[0] += c[0] + d[0]; acc[1] += c[1] + d[1]; acc[2] += c[2] + d[2]; acc[3] += c[3] + d[3];
        }
        if (++c_b == kbc) { flush(); c_b = 0; point_consume_at(++c_t); }
      };
      for (int u = ub; u < ue; u += kRing) {
#pragma unroll
        for (int i = 0; i < kRing; ++i) {
          if (u + i < ue) {
            const CodeRegs cur = ring[i];
            if (u + i + kRing < ue) fetch(ring[i]);
            consume(cur);
          }
        }
      }
      if (c_b != 0 && ue > ub) flush();
      if (lane == 0) { s_rng[warp * 2] = first_tile; s_rng[warp * 2 + 1] = pieces; }
      __syncthreads();

      // ---- the warps' partial sums are added in warp order; the last chunk finishes the outputs ----
      const int out_tiles = round_tiles / HALVES;
      for (int idx = threadIdx.x; idx < out_tiles * 128; idx += kThreadsMma) {
        const int row = idx & 15, m = (idx >> 4) & 7, ot = idx >> 7;
        if (m >= p.M) continue;
        float v[HALVES];
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
          const int t = ot * HALVES + h;                // weight tile inside the round
          float sum = multi_chunk && chunk > 0 ? s_tile[((r0 + t) * 8 + m) * 16 + row] : 0.f;
          for (int w = 0; w < kWarps; ++w) {
            const int piece = t - s_rng[w * 2];
            if (piece >= 0 && piece < s_rng[w * 2 + 1]) sum += s_part[((w * 2 + piece) * 8 + m) * 16 + row];
          }
          v[h] = sum;
        }
        if (!last_chunk) {
#pragma unroll
          for (int h = 0; h < HALVES; ++h) s_tile[((r0 + ot * HALVES + h) * 8 + m) * 16 + row] = v[h];
          continue;
        }
        const int wrow0 = tile_row0(r0 + ot * HALVES) + row;      // weight row of v[0]; the output column too (h = 0)
        const int n = wrow0;
        if (n >= p.n_out) continue;
        if (!GROUPED) {
          v[0] *= static_cast<float>(scales[wrow0]);
          if (SWIGLU) v[HALVES - 1] *= static_cast<float>(scales[wrow0 + p.N / 2]);
        }
        const size_t o = static_cast<size_t>(m) * p.n_out + n;
        if (SWIGLU) {
          p.y[o] = __float2half_rn(silu_fast(v[0]) * v[HALVES - 1]);
        } else {
          float out = v[0];
          if (p.epilogue == CACHEIR_B200_EPI_RESIDUAL) out += __half2float(p.residual[o]);
          p.y[o] = __float2half_rn(out);
        }
      }
      __syncthreads();       // the partial sums (and, after a chunk's last round, the staged x) are free again
    }
  }
}

struct MmaGemvShape {
  int chunk_cols, grid, max_tiles;
  size_t smem;
};

MmaGemvShape mma_gemv_shape(int M, int N, int K, bool swiglu) {
  MmaGemvShape s{};
  const int kb = K / 128;
  const size_t per_block = static_cast<size_t>(M) * 256;
  int max_blocks = static_cast<int>((kStageBudget - static_cast<size_t>(M) * kRowPadBytes) / per_block);
  if (max_blocks < 1) max_blocks = 1;
  const int chunks = (kb + max_blocks - 1) / max_blocks;
  s.chunk_cols = ((kb + chunks - 1) / chunks) * 128;
  const int n_out = swiglu ? N / 2 : N;
  const int n_units = (n_out + kTileRows - 1) / kTileRows;
  s.grid = n_units < kNumSMs ? n_units : kNumSMs;
  s.max_tiles = ((n_units + s.grid - 1) / s.grid) * (swiglu ? 2 : 1);
  s.smem = static_cast<size_t>(M) * (s.chunk_cols * 2 + kRowPadBytes) + static_cast<size_t>(s.chunk_cols / 128) * 8 * sizeof(float) +
           kWarps * 2 * 128 * sizeof(float) + kWarps * 2 * sizeof(int) +
           (s.chunk_cols < K ? static_cast<size_t>(s.max_tiles) * 128 * sizeof(float) : 0);
  return s;
}

template <bool SWIGLU, bool GROUPED, bool F16SCALE>
int launch_mma_variant(const MmaGemvParams& p, int grid, size_t smem, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(qgemv_mma_int4_kernel<SWIGLU, GROUPED, F16SCALE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  qgemv_mma_int4_kernel<SWIGLU, GROUPED, F16SCALE><<<grid, kThreadsMma, smem, stream>>>(p);
  return launch_status();
}

}  // namespace

bool qgemv_mma_supported(const QGemvParams& q) {
  if (q.bits != 4 || q.x_dtype != CACHEIR_B200_F16 || q.tiled || q.paired || q.x_prequantized || q.norm_weight) return false;
  if (q.M < 1 || q.M > 8 || q.K % 128 != 0 || q.K < 128) return false;
  if (q.group_size != 0) {           // 128 << s columns per group, no zero points
    if (q.group_size % 128 != 0 || q.zero_points) return false;
    const int g = q.group_size / 128;
    if ((g & (g - 1)) != 0 || (q.K / 128) % g != 0) return false;
  }
  if (q.scale_dtype != CACHEIR_B200_F16 && q.scale_dtype != CACHEIR_B200_F32) return false;
  if (q.epilogue == CACHEIR_B200_EPI_SWIGLU && (q.N / 2) % kTileRows != 0) return false;
  if (q.epilogue == kEpiQkvRopeAppend) return false;
  if (mma_gemv_shape(q.M, q.N, q.K, q.epilogue == CACHEIR_B200_EPI_SWIGLU).smem > 220 * 1024) return false;
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
  const bool grouped = q.group_size != 0;
  p.group_shift = 0;
  for (int g = q.group_size / 128; g > 1; g >>= 1) ++p.group_shift;
  p.epilogue = q.epilogue; p.x_stride = q.x_stride;
  const MmaGemvShape shape = mma_gemv_shape(q.M, q.N, q.K, swiglu);
  p.chunk_cols = shape.chunk_cols; p.max_tiles = shape.max_tiles;
  const bool f16 = q.scale_dtype == CACHEIR_B200_F16;
  // One CTA per SM (fewer when there are fewer output tiles); output tiles are dealt out round robin over the CTAs.
#define CB200_MMA_GEMV(SW, GR, F16) launch_mma_variant<SW, GR, F16>(p, shape.grid, shape.smem, stream)
  if (swiglu) {
    if (grouped) return f16 ? CB200_MMA_GEMV(true, true, true) : CB200_MMA_GEMV(true, true, false);
    return f16 ? CB200_MMA_GEMV(true, false, true) : CB200_MMA_GEMV(true, false, false);
  }
  if (grouped) return f16 ? CB200_MMA_GEMV(false, true, true) : CB200_MMA_GEMV(false, true, false);
  return f16 ? CB200_MMA_GEMV(false, false, true) : CB200_MMA_GEMV(false, false, false);
#undef CB200_MMA_GEMV
}

}  // namespace cb200
