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
#include "tc_ptx.cuh"

namespace cb200 {
namespace {

constexpr int kTileRows = 16;
constexpr int kRowPadBytes = 64;     // staged rows are 64 bytes apart modulo 128: eight lanes of a load phase hit eight bank groups
#ifndef CB200_GEMV_TEAMS
#define CB200_GEMV_TEAMS 4
#endif
#ifndef CB200_GEMV_STAGE_BLOCKS
#define CB200_GEMV_STAGE_BLOCKS 16
#endif
constexpr int kTeams = CB200_GEMV_TEAMS;             // a team shares one ring of stages and one run of (tile, stage) units
constexpr int kTeamWarps = 4;         // each warp of a team multiplies a quarter of every stage
constexpr int kWarps = kTeams * kTeamWarps;
constexpr int kThreadsMma = kWarps * 32;
constexpr int kRoundTiles = 2 * kTeams;      // weight tiles a CTA works on at a time: a team's run then touches at most three
constexpr int kPieces = 3;
#ifndef CB200_GEMV_STAGES
#define CB200_GEMV_STAGES 2
#endif
constexpr int kStages = CB200_GEMV_STAGES;                   // stages per team ring
constexpr int kStageBlocks = CB200_GEMV_STAGE_BLOCKS;              // 128-column blocks per stage: 16 rows x 1024 bytes of codes, one TMA copy
constexpr int kStageRowBytes = kStageBlocks * 64;
constexpr int kStageBytes = kTileRows * kStageRowBytes;
constexpr int kWarpBlocks = kStageBlocks / kTeamWarps;
constexpr int kRingBytes = kTeams * kStages * kStageBytes;
constexpr size_t kSmemLimit = 227 * 1024;

__device__ int g_gemv_status = 0;    // 0 ok; otherwise (5 << 8 | id) of the first wait that gave up

struct MmaGemvParams {
  const __half* x;
  const void* scales;
  const float* zero_points;
  const __half* residual;
  __half* y;
  int M, N, K;
  int n_out;
  int group_shift;    // group size = 128 << group_shift (group-wise form)
  int epilogue;
  int chunk_cols;     // columns of x staged at a time (a multiple of 256; K when everything fits)
  int max_tiles;      // weight tiles of the busiest CTA (sizes the cross-chunk sums)
  long long x_stride;
};

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Nibbles to fp16 without a subtraction and with one shift per word: for a packed word w (nibble i = column i),
//   (w & 0x000F000F) | 0x64006400 = (1024 + n0, 1024 + n4)          (w >> 8 gives n2, n6)
//   (w & 0x00F000F0) | 0x64006400 = (1024 + 16 n1, 1024 + 16 n5)    (w >> 8 gives n3, n7)
// all exact in fp16. The second kind meets x / 16 in the MMA (staged that way), so its products are 64 x + n x. The
// constants leave through sums of the staged x that the accumulators start from: with P = -1024 (sum of all staged
// values of the block) and Q = sum of x, sum (n - z) x = [MMA result] + P - z Q.
constexpr uint32_t kNibLo = 0x000F000Fu, kNibHi = 0x00F000F0u, kFp16Magic = 0x64006400u;

// One CTA per SM. The CTA owns the output tiles blockIdx.x + grid * i (16 output columns each; with the SwiGLU
// epilogue a gate and an up weight tile per output tile). It takes its weight tiles 8 at a time and deals the
// (tile, stage) units of such a round out evenly over four teams of four warps: team t gets units [U t / 4, U (t+1) / 4),
// a run along K that touches at most three tiles, so every team streams the same number of bytes whatever the tile
// count. A stage is 16 rows x 2048 columns of codes: 1024 contiguous bytes of every row, fetched by one TMA copy, so
// that DRAM sees long runs per row. Each team keeps a ring of two stages: lane 0 of its first warp issues the copies,
// the four warps wait on the stage's `full` mbarrier, multiply four 128-column blocks each and arrive on its `empty`
// mbarrier. Per block a warp issues 8 MMAs (two chains) whose accumulators start at -(1024 + zero) * sum(x over the
// block), then folds them into its running sums with the two rows' group scales. Partial sums meet in shared memory
// and are added in warp order.
// Shared memory: the rings; x of the current chunk, [M][row_bytes], inside a row the 16-byte units of a 128-column
// block at unit (j*4 + q) for columns q*32 + j*8 .. +7, the eight values in the order 0,4,1,5,2,6,3,7; the block
// sums of x [block][8]; the warps' partial sums [W][3][8][16]; the teams' tile ranges; the mbarriers; the
// cross-chunk sums [tile][8][16].
template <bool SWIGLU, bool GROUPED, bool F16SCALE>
__global__ void __launch_bounds__(kThreadsMma, 1)
qgemv_mma_int4_kernel(const __grid_constant__ CUtensorMap tmap_w, const MmaGemvParams p) {
  using namespace ptx;
  constexpr int HALVES = SWIGLU ? 2 : 1;     // weight tiles per output tile
  using scale_t = typename std::conditional<F16SCALE, __half, float>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int row_bytes = p.chunk_cols * 2 + kRowPadBytes;
  uint8_t* ring = smem;
  uint8_t* xs = smem + kRingBytes;
  float* s_xblk = reinterpret_cast<float*>(xs + p.M * row_bytes);
  float* s_part = s_xblk + (p.chunk_cols / 128) * 16;
  int* s_rng = reinterpret_cast<int*>(s_part + kWarps * kPieces * 128);
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_rng + kTeams * 2);          // [team][full 0..3, empty 0..3]
  float* s_tile = reinterpret_cast<float*>(bars + kTeams * 2 * kStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int team = warp / kTeamWarps, tw = warp % kTeamWarps;
  const int g = lane >> 2, q = lane & 3;
  const int grid = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
  const int groups_per_row = GROUPED ? ((p.K / 128) >> p.group_shift) : 1;
  const scale_t* scales = static_cast<const scale_t*>(p.scales);
  const int n_units = (p.n_out + kTileRows - 1) / kTileRows;
  const int tiles = ((n_units - cta + grid - 1) / grid) * HALVES;            // weight tiles of this CTA (>= HALVES)
  const uint8_t* x_lane = xs + min(g, p.M - 1) * row_bytes + q * 16;         // MMA column g is batch row g; columns past M repeat the last row and are never stored
  const float* xblk_lane = s_xblk + 4 * q;
  const bool multi_chunk = p.chunk_cols < p.K;
  const bool producer = tw == 0 && lane == 0;
  uint8_t* team_ring = ring + team * (kStages * kStageBytes);
  // this lane's 16 bytes of (row g, first block of the warp's share) inside a stage; row g + 8 sits 8 rows further
  const uint32_t code_off = g * kStageRowBytes + (tw * kWarpBlocks) * 64 + q * 16;
  const uint32_t full0 = smem_u32(bars + team * 2 * kStages), empty0 = full0 + 8 * kStages;

  if (producer) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, kTeamWarps); }
    mbar_fence_init();
  }

  // first weight row of weight tile `wt` of this CTA
  auto tile_row0 = [&](int wt) {
    const int i = wt / HALVES, h = wt - i * HALVES;
    return (cta + grid * i) * kTileRows + h * (p.N / 2);
  };

  for (int i = threadIdx.x; i < (p.chunk_cols / 128) * 16; i += kThreadsMma)
    if (((i >> 1) & 7) >= p.M) s_xblk[i] = 0.f;
  __syncthreads();            // the mbarriers exist for every warp of their team

  // Stage x[:, c0 : c0 + cols] in MMA order (16-byte units of 8 columns; a thread's loads of all batch rows are in
  // flight together; the odd columns of every pair of nibbles divided by 16) and, per (128-column block, batch
  // row), P = -1024 * (sum of the staged values) and Q = sum of x: eight values in order, then a butterfly over the
  // block's 16 lanes.
  auto stage_x = [&](int c0, int cols) {
    const int units = cols / 8;                   // a multiple of 16: a half-warp is inside or outside as a whole
    for (int base = warp * 32; base < units; base += kThreadsMma) {
      const int unit = base + lane;
      const bool valid = unit < units;
      uint4 raw[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        raw[m] = make_uint4(0u, 0u, 0u, 0u);
        if (valid && m < p.M) raw[m] = *reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(m) * p.x_stride + c0 + unit * 8);
      }
      const int kb = unit >> 4, in_block = unit & 15, qq = in_block >> 2, jj = in_block & 3;
      uint8_t* dst = xs + (kb * 16 + jj * 4 + qq) * 16;
      const __half2 sixteenth = __float2half2_rn(0.0625f);
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        if (m < p.M) {                            // (uniform)
          const uint32_t w0 = raw[m].x, w1 = raw[m].y, w2 = raw[m].z, w3 = raw[m].w;   // (h0,h1) (h2,h3) (h4,h5) (h6,h7)
          uint4 o = make_uint4(__byte_perm(w0, w2, 0x5410), __byte_perm(w0, w2, 0x7632),            // order 0,4,1,5,2,6,3,7
                               __byte_perm(w1, w3, 0x5410), __byte_perm(w1, w3, 0x7632));
          __half2 odd0 = __hmul2(*reinterpret_cast<const __half2*>(&o.y), sixteenth);                // (x1, x5) / 16
          __half2 odd1 = __hmul2(*reinterpret_cast<const __half2*>(&o.w), sixteenth);                // (x3, x7) / 16
          o.y = *reinterpret_cast<const uint32_t*>(&odd0);
          o.w = *reinterpret_cast<const uint32_t*>(&odd1);
          if (valid) *reinterpret_cast<uint4*>(dst + m * row_bytes) = o;
          const float2 e0 = __half22float2(*reinterpret_cast<const __half2*>(&o.x)), e1 = __half22float2(*reinterpret_cast<const __half2*>(&o.z));
          const float2 d0 = __half22float2(odd0), d1 = __half22float2(odd1);
          float even = (e0.x + e0.y) + (e1.x + e1.y), odd = (d0.x + d0.y) + (d1.x + d1.y);
#pragma unroll
          for (int sh = 8; sh > 0; sh >>= 1) {
            even += __shfl_xor_sync(0xffffffffu, even, sh);
            odd += __shfl_xor_sync(0xffffffffu, odd, sh);
          }
          if (valid && (lane & 15) == 0)
            *reinterpret_cast<float2*>(s_xblk + (kb * 8 + m) * 2) = make_float2(-1024.f * (even + odd), even + 16.f * odd);
        }
      }
    }
  };

  uint32_t n_issued = 0, n_consumed = 0;       // stages the team has asked for / this warp has finished since the kernel began
  bool alive = true;                           // false once a wait has given up: the warp only keeps the barriers company
  int chunk = 0;
  for (int c0 = 0; c0 < p.K; c0 += p.chunk_cols, ++chunk) {
    const int cols = min(p.chunk_cols, p.K - c0);
    const int kbc = cols / 128;                                   // blocks of this chunk
    const int spt = (kbc + kStageBlocks - 1) / kStageBlocks;      // stages per tile (the last may reach past the row: zero codes)
    const int kb0 = c0 / 128;
    const bool last_chunk = c0 + cols >= p.K;
    for (int r0 = 0; r0 < tiles; r0 += kRoundTiles) {
      const int round_tiles = min(kRoundTiles, tiles - r0);
      const int units = round_tiles * spt;
      const int ub = (units * team) / kTeams, ue = (units * (team + 1)) / kTeams;
      const int first_tile = ub / spt;

      // ---- fetch cursor: the tile and stage the next copy reads (the producer issues; every lane keeps count) ----
      int f_t = first_tile, f_s = ub - first_tile * spt, fu = ub;
      auto issue = [&]() {
        if (producer) {
          const uint32_t s = n_issued % kStages, use = n_issued / kStages;
          bool ok = true;
          if (use > 0) ok = mbar_wait(empty0 + 8 * s, (use - 1) & 1, &g_gemv_status, (5 << 8) | 2);   // the four warps have read the stage's last contents
          if (ok) {
            mbar_expect_tx(full0 + 8 * s, kStageBytes);
            tma_load_2d(smem_u32(team_ring + s * kStageBytes), &tmap_w, full0 + 8 * s, (kb0 + f_s * kStageBlocks) * 16,
                        tile_row0(r0 + min(f_t, round_tiles - 1)));
          }
        }
        ++n_issued; ++fu;
        if (++f_s == spt) { f_s = 0; ++f_t; }
      };
#pragma unroll 1
      for (int i = 0; i < kStages - 1 && fu < ue && alive; ++i) issue();

      if (r0 == 0) {                         // (the codes above are on their way while x is staged)
        stage_x(c0, cols);
        __syncthreads();
      }

      // ---- consume cursor ----
      int c_s = ub - first_tile * spt, c_t = first_tile, pieces = 0;
      float nz_lo = -8.f, nz_hi = -8.f;                           // minus the zero point of the two rows
      const scale_t *sc_lo = scales, *sc_hi = scales;
      auto point_consume_at = [&](int t) {
        const int row0 = tile_row0(r0 + min(t, round_tiles - 1));
        const int r_lo = min(row0 + g, p.N - 1), r_hi = min(row0 + g + 8, p.N - 1);     // (rows past N: zero codes, never stored)
        if (GROUPED) {
          sc_lo = scales + static_cast<size_t>(r_lo) * groups_per_row;
          sc_hi = scales + static_cast<size_t>(r_hi) * groups_per_row;
        } else if (p.zero_points) {
          nz_lo = -p.zero_points[r_lo];
          nz_hi = -p.zero_points[r_hi];
        }
      };
      point_consume_at(c_t);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      auto flush = [&]() {
        if (pieces >= kPieces) return;                             // (a team's run never touches more tiles)
        float* mine = s_part + (warp * kPieces + pieces) * 128;    // [m][row]
        mine[(2 * q) * 16 + g] = acc[0]; mine[(2 * q + 1) * 16 + g] = acc[1];
        mine[(2 * q) * 16 + g + 8] = acc[2]; mine[(2 * q + 1) * 16 + g + 8] = acc[3];
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        ++pieces;
      };
      // One 128-column block: 8 MMAs on the unpacked nibbles (two chains), then the block's sums join the result.
      auto block = [&](const uint8_t* codes, int kb, float s_lo, float s_hi) {
        const uint4 lo = *reinterpret_cast<const uint4*>(codes);
        const uint4 hi = *reinterpret_cast<const uint4*>(codes + 8 * kStageRowBytes);
        const float4 pq = *reinterpret_cast<const float4*>(xblk_lane + kb * 16);     // (P, Q) of batch rows 2q and 2q+1
        float c[4], d[4] = {0.f, 0.f, 0.f, 0.f};
        c[0] = fmaf(nz_lo, pq.y, pq.x); c[1] = fmaf(nz_lo, pq.w, pq.z);
        c[2] = fmaf(nz_hi, pq.y, pq.x); c[3] = fmaf(nz_hi, pq.w, pq.z);
        const uint32_t wa[4] = {lo.x, lo.y, lo.z, lo.w};
        const uint32_t wb[4] = {hi.x, hi.y, hi.z, hi.w};
        const uint8_t* xrow = x_lane + kb * 256;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 xv = *reinterpret_cast<const uint4*>(xrow + j * 64);     // (x0,x4) (x1,x5)/16 (x2,x6) (x3,x7)/16 of the word's 8 columns
          const uint32_t ta = wa[j] >> 8, tb = wb[j] >> 8;
          mma_16816(c, (wa[j] & kNibLo) | kFp16Magic, (wb[j] & kNibLo) | kFp16Magic, (wa[j] & kNibHi) | kFp16Magic, (wb[j] & kNibHi) | kFp16Magic, xv.x, xv.y);
          mma_16816(d, (ta & kNibLo) | kFp16Magic, (tb & kNibLo) | kFp16Magic, (ta & kNibHi) | kFp16Magic, (tb & kNibHi) | kFp16Magic, xv.z, xv.w);
        }
        if (GROUPED) {
          acc[0] = fmaf(c[0] + d[0], s_lo, acc[0]); acc[1] = fmaf(c[1] + d[1], s_lo, acc[1]);
          acc[2] = fmaf(c[2] + d[2], s_hi, acc[2]); acc[3] = fmaf(c[3] + d[3], s_hi, acc[3]);
        } else {
          acc[0] += c[0] + d[0]; acc[1] += c[1] + d[1]; acc[2] += c[2] + d[2]; acc[3] += c[3] + d[3];
        }
      };
#pragma unroll 1
      for (int u = ub; u < ue && alive; ++u) {
        const int kb = c_s * kStageBlocks + tw * kWarpBlocks;      // first block of the warp's share inside the chunk
        float s_lo[kWarpBlocks], s_hi[kWarpBlocks];
#pragma unroll
        for (int b = 0; b < kWarpBlocks; ++b) {                    // asked for before the wait: they arrive with the codes
          s_lo[b] = 1.f; s_hi[b] = 1.f;
          if (GROUPED && kb + b < kbc) {
            const int grp = (kb0 + kb + b) >> p.group_shift;
            s_lo[b] = static_cast<float>(sc_lo[grp]); s_hi[b] = static_cast<float>(sc_hi[grp]);
          }
        }
        const uint32_t s = n_consumed % kStages;
        if (!mbar_wait(full0 + 8 * s, (n_consumed / kStages) & 1, &g_gemv_status, (5 << 8) | 1)) { alive = false; break; }
        const uint8_t* codes = team_ring + s * kStageBytes + code_off;
        if (kb + kWarpBlocks <= kbc) {                             // (one basic block: the blocks' instruction streams interleave)
#pragma unroll
          for (int b = 0; b < kWarpBlocks; ++b) block(codes + b * 64, kb + b, s_lo[b], s_hi[b]);
        } else {
#pragma unroll
          for (int b = 0; b < kWarpBlocks; ++b)
            if (kb + b < kbc) block(codes + b * 64, kb + b, s_lo[b], s_hi[b]);
        }
        ++n_consumed;
        __syncwarp();                                              // every lane has read the stage
        if (lane == 0) mbar_arrive(empty0 + 8 * s);
        if (fu < ue) issue();
        if (++c_s == spt) { flush(); c_s = 0; point_consume_at(++c_t); }
      }
      if (c_s != 0 && ue > ub) flush();
      if (tw == 0 && lane == 0) { s_rng[team * 2] = first_tile; s_rng[team * 2 + 1] = pieces; }
      __syncthreads();

      // ---- the warps' partial sums are added in warp order; the last chunk finishes the outputs ----
      const int out_tiles = round_tiles / HALVES;
      for (int idx = threadIdx.x; idx < out_tiles * p.M * 16; idx += kThreadsMma) {
        const int row = idx & 15, pair = idx >> 4, ot = pair / p.M, m = pair - ot * p.M;
        float v[HALVES];
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
          const int t = ot * HALVES + h;                // weight tile inside the round
          float sum = multi_chunk && chunk > 0 ? s_tile[((r0 + t) * 8 + m) * 16 + row] : 0.f;
#pragma unroll
          for (int tm = 0; tm < kTeams; ++tm) {
            const int piece = t - s_rng[tm * 2];
            if (piece >= 0 && piece < s_rng[tm * 2 + 1]) {
#pragma unroll
              for (int w = 0; w < kTeamWarps; ++w) sum += s_part[(((tm * kTeamWarps + w) * kPieces + piece) * 8 + m) * 16 + row];
            }
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
  const int n_out = swiglu ? N / 2 : N;
  const int n_units = (n_out + kTileRows - 1) / kTileRows;
  s.grid = n_units < kNumSMs ? n_units : kNumSMs;
  s.max_tiles = ((n_units + s.grid - 1) / s.grid) * (swiglu ? 2 : 1);
  const size_t fixed = 1024 + kRingBytes + kWarps * kPieces * 128 * sizeof(float) + kTeams * 2 * sizeof(int) + kTeams * 2 * kStages * sizeof(uint64_t);
  auto total = [&](int chunk_cols) {
    return fixed + static_cast<size_t>(M) * (chunk_cols * 2 + kRowPadBytes) + static_cast<size_t>(chunk_cols / 128) * 16 * sizeof(float) +
           (chunk_cols < K ? static_cast<size_t>(s.max_tiles) * 128 * sizeof(float) : 0);
  };
  // the fewest equal chunks of x (whole stages) that fit beside the rings
  const int stages = (K / 128 + kStageBlocks - 1) / kStageBlocks;
  for (int chunks = 1; chunks <= stages; ++chunks) {
    s.chunk_cols = ((stages + chunks - 1) / chunks) * kStageBlocks * 128;
    if (s.chunk_cols > K) s.chunk_cols = K;
    s.smem = total(s.chunk_cols);
    if (s.smem <= kSmemLimit) break;
  }
  return s;
}

template <bool SWIGLU, bool GROUPED, bool F16SCALE>
int launch_mma_variant(const CUtensorMap& tmap, const MmaGemvParams& p, int grid, size_t smem, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(qgemv_mma_int4_kernel<SWIGLU, GROUPED, F16SCALE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  qgemv_mma_int4_kernel<SWIGLU, GROUPED, F16SCALE><<<grid, kThreadsMma, smem, stream>>>(tmap, p);
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
  if (mma_gemv_shape(q.M, q.N, q.K, q.epilogue == CACHEIR_B200_EPI_SWIGLU).smem > kSmemLimit) return false;
  if (ptx::tensor_map_encoder() == nullptr) return false;
  return aligned_to(q.packed, 16) && aligned_to(q.x, 16) && (q.x_stride * 2) % 16 == 0;
}

int launch_qgemv_mma(const QGemvParams& q, cudaStream_t stream) {
  MmaGemvParams p{};
  p.x = static_cast<const __half*>(q.x);
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
  // the packed rows as a [N][K/8] matrix of 32-bit words, copied in tiles of 16 rows x 1024 bytes; what lies past N or K reads as zero
  CUtensorMap tmap;
  if (!ptx::encode_u32_rows_plain(&tmap, q.packed, static_cast<uint64_t>(q.K / 8), static_cast<uint64_t>(q.N), static_cast<uint64_t>(q.K / 2),
                                  kStageRowBytes / 4, kTileRows))
    return CACHEIR_B200_EUNSUPPORTED;
  // One CTA per SM (fewer when there are fewer output tiles); output tiles are dealt out round robin over the CTAs.
#define CB200_MMA_GEMV(SW, GR, F16) launch_mma_variant<SW, GR, F16>(tmap, p, shape.grid, shape.smem, stream)
  if (swiglu) {
    if (grouped) return f16 ? CB200_MMA_GEMV(true, true, true) : CB200_MMA_GEMV(true, true, false);
    return f16 ? CB200_MMA_GEMV(true, false, true) : CB200_MMA_GEMV(true, false, false);
  }
  if (grouped) return f16 ? CB200_MMA_GEMV(false, true, true) : CB200_MMA_GEMV(false, true, false);
  return f16 ? CB200_MMA_GEMV(false, false, true) : CB200_MMA_GEMV(false, false, false);
#undef CB200_MMA_GEMV
}

int qgemv_mma_device_status(bool reset) {
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_gemv_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gemv_status, &zero, sizeof(int));
  }
  return status;
}

}  // namespace cb200
