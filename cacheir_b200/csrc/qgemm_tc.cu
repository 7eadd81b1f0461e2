// Small-M dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
//   y[M, N] = x[M, K] . deq(W)[N, K]^T        M <= 128, fp16 activations
//
// The weight matrix is the 128-row MMA operand ("swap-AB"): one CTA owns 128
// weight rows and a K range, the M activation rows are the MMA's N dimension
// (padded to MP = 16/32/64), the fp32 accumulator D[128 x MP] lives in tensor
// memory. Weight codes exist in HBM only as the reference's packed bytes:
//
//   warp 0      TMA producer: raw code tile [128 rows x 128 k] (16 KB int8 / 8 KB
//               int4, hardware-swizzled so that row-per-thread reads are conflict
//               free) + the x tile [MP x 128 k] per pipeline stage
//   warps 4-11  converters: thread (r, half) owns half of weight row r of the tile;
//               unpacks its codes in registers (byte/nibble -> fp16 through the
//               0x6400 mantissa trick, zero point removed exactly) and stores the
//               fp16 operand tile into shared memory in the 128-byte swizzle order a
//               tensor copy would leave (two tiles rotate). Tensor memory was tried
//               as the hand-over (tcgen05.st): it sustains only ~23 B/clk per SM and
//               made the converters, not the MMAs, the bottleneck.
//   warp 1      one thread issues tcgen05.mma with both operands from shared memory
//               (M=128, N=MP, K=16; 8 per stage) and commits to the barriers that
//               recycle the stages
//   warps 4-11  epilogue: tcgen05.ld the accumulator, split-K reduction across the
//               CTAs of a cluster through distributed shared memory in rank order
//               (deterministic), row scale, residual add or SiLU*mul, store y
//
// Batches of 65..128 rows (MP = 128) run the same pipeline with the operand roles exchanged:
// the activation tile [128 rows x 128 k] is the 128-row MMA operand, the dequantised weight
// tile the N = 128 operand, so the weights stream once for the whole batch. The accumulator
// then holds batch rows on the tensor-memory lanes and weight rows along the columns; all
// sixteen converter warps share the epilogue (32 columns each).
//
// Every wait is bounded: a barrier that does not complete within the poll budget
// raises a device status flag and the CTA drains and exits instead of hanging.
#include <cuda.h>

#include "common.cuh"
#include "qgemv_common.cuh"

namespace cb200 {
namespace {

constexpr int kBlockN = 128;      // weight rows per CTA (UMMA M)
constexpr int kBlockK = 128;      // k elements per pipeline stage
// converted fp16 operand tiles in shared memory: three decouple the converters from the MMAs (two where the
// 128-row int8 stages leave no room for a third)
__host__ __device__ constexpr int a_stages(int bits, int mp) { return (bits == 8 && mp == 128) ? 2 : 3; }
constexpr int kABytes = kBlockN * kBlockK * 2;          // 32 KB: two 64-element halves of [128 rows x 128 B], 128-byte swizzled
constexpr int kAColBase = 256;                          // accumulators use tensor-memory columns [0, 256)
constexpr int kTmemCols = 256;
constexpr int kConvThreads = 512;                       // warps 4..19: the unpacking is latency-bound, more warps hide it
constexpr int kThreads = 128 + kConvThreads;
constexpr int kMaxSplitK = 4;
constexpr int kSmemBudget = 216 * 1024;                 // raw/x ring + fp16 operand tiles

__host__ __device__ constexpr int stage_bytes(int bits, int mp) {
  return (bits == 8 ? kBlockN * 128 : kBlockN * 64) + mp * kBlockK * 2;
}
__host__ __device__ constexpr int num_stages(int bits, int mp) {
  return (kSmemBudget - a_stages(bits, mp) * kABytes) / stage_bytes(bits, mp) > 8
             ? 8
             : (kSmemBudget - a_stages(bits, mp) * kABytes) / stage_bytes(bits, mp);
}
constexpr uint32_t kPollLimit = 8u * 1000u * 1000u;

__device__ int g_qgemm_status = 0;   // 0 ok; otherwise (code << 8 | barrier id) of the first wait that gave up

// ---- PTX wrappers ------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
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
// Bounded wait. Returns false (and records which barrier) when the poll budget runs out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int id) {
  for (uint32_t i = 0; i < kPollLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(32);
  }
  atomicCAS(&g_qgemm_status, 0, (1 << 8) | id);
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16_ss(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 fp16 (k0 .. k0+15 of tile row r) into a [2 halves][128 rows][128 B] operand tile whose 16-byte chunks sit in
// the 128-byte swizzle order (chunk c of row r at c ^ (r & 7)): what a TMA tensor copy of an fp16 tile would leave.
__device__ __forceinline__ void st_operand16(uint8_t* tile, int r, int k0, const uint32_t (&v)[8]) {
  uint8_t* row = tile + (k0 >> 6) * (kBlockN * 128) + r * 128;
  const int c = ((k0 & 63) >> 3);                      // first of the two 16-byte chunks (8 fp16 each)
  *reinterpret_cast<uint4*>(row + ((c ^ (r & 7)) * 16)) = make_uint4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<uint4*>(row + (((c + 1) ^ (r & 7)) * 16)) = make_uint4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void tc_ld_x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t local_addr, uint32_t rank, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Bulk copy from this CTA's shared memory into CTA `rank` of the cluster; completion is counted in
// bytes on that CTA's barrier at the same offset as `bar`.
__device__ __forceinline__ void bulk_copy_to_rank(uint32_t dst, uint32_t src, uint32_t bytes, uint32_t bar, uint32_t rank) {
  uint32_t rdst, rbar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rdst) : "r"(dst), "r"(rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(bar), "r"(rank));
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(rdst), "r"(src), "r"(bytes), "r"(rbar) : "memory");
}

// Shared-memory matrix descriptor (64 bit): start address, leading/stride byte offsets
// (all >> 4), descriptor version 1 at bit 46, swizzle mode at bits 61-63.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(layout_type & 0x7) << 61;
  return d;
}

struct TcParams {
  const void* scales;
  const float* zero_points;
  const void* residual;
  void* y;
  int M, N, K;
  int n_out;        // output columns (N, or N/2 with the SwiGLU epilogue)
  int group_size;
  int scale_dtype;
  int epilogue;
  int split_k;      // CTAs per cluster along K (1 = no split)
  int tiled;        // weights in 128x128 tile order (see cacheir_b200_pack_relayout)
  const uint8_t* w_tiled;   // the tile-ordered codes when tiled != 0
};

__device__ __forceinline__ float load_scale(const void* scales, int scale_dtype, size_t idx) {
  return scale_dtype == CACHEIR_B200_F16 ? __half2float(static_cast<const __half*>(scales)[idx])
                                         : static_cast<const float*>(scales)[idx];
}

__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// 8 int8 codes (two 32-bit words) -> 8 fp16 (four registers, k order), zero point removed exactly.
__device__ __forceinline__ void unpack8_int8(uint32_t w0, uint32_t w1, __half2 sub, bool scaled, __half2 gscale, uint32_t* o) {
  __half2 v[4];
  v[0] = __hsub2(bits_h2(__byte_perm(w0, 0x64646464u, 0x5140)), sub);   // (1024+b0, 1024+b1) - (1024+z)
  v[1] = __hsub2(bits_h2(__byte_perm(w0, 0x64646464u, 0x5342)), sub);
  v[2] = __hsub2(bits_h2(__byte_perm(w1, 0x64646464u, 0x5140)), sub);
  v[3] = __hsub2(bits_h2(__byte_perm(w1, 0x64646464u, 0x5342)), sub);
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = h2_bits(scaled ? __hmul2(v[i], gscale) : v[i]);
}
// 8 int4 codes (one 32-bit word) -> 8 fp16: byte q -> (0x6400 | low nibble, 0x6400 | high nibble << 4)
// = (1024 + n0, 1024 + 16*n1); one fma maps both to (n0 - z, n1 - z) exactly.
__device__ __forceinline__ void unpack8_int4(uint32_t w, __half2 mul, __half2 sub, bool scaled, __half2 gscale, uint32_t* o) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t t = __byte_perm(w, 0x64646464u, 0x4040 + 0x101 * q) & 0x64F0640Fu;
    const __half2 v = __hfma2(bits_h2(t), mul, sub);
    o[q] = h2_bits(scaled ? __hmul2(v, gscale) : v);
  }
}
// Rows whose zero point is not a small integer: plain fp32 arithmetic, scale folded in.
template <int BITS>
__device__ __forceinline__ void unpack8_slow(const uint8_t* bytes, int first, float zero, float scale, uint32_t* o) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float f[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int idx = first + 2 * e + h;
      const float code = BITS == 8 ? static_cast<float>(bytes[idx])
                                   : static_cast<float>((bytes[idx >> 1] >> ((idx & 1) * 4)) & 0xF);
      f[h] = (code - zero) * scale;
    }
    o[e] = h2_bits(__floats2half2_rn(f[0], f[1]));
  }
}

// GROUPED: group-wise scales (no zero-point array, codes centred on 2^(BITS-1)): the conversion loop then has
// neither the per-row "exact offset or not" branch nor the "scaled or not" select.
template <int BITS, int MP, bool GROUPED>
__global__ void __launch_bounds__(kThreads, 1)
qgemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const TcParams p) {
  constexpr int kStages = num_stages(BITS, MP);
  constexpr int kRawBytes = BITS == 8 ? kBlockN * 128 : kBlockN * 64;   // per stage
  constexpr int kXBytes = MP * kBlockK * 2;
  constexpr int kRawRow = BITS == 8 ? 128 : 64;                          // bytes of one row per stage
  constexpr int kChunksPerThread = kRawRow / 16 / 4;                     // 16-byte chunks per converter thread (a quarter row)
  constexpr int kAStages = a_stages(BITS, MP);
  constexpr bool kWide = MP == 128;                                      // activations are the 128-row operand

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* s_raw = smem;                                   // kStages x kRawBytes
  uint8_t* s_x = s_raw + kStages * kRawBytes;              // kStages x kXBytes (all sizes are multiples of 1024)
  uint8_t* s_a = s_x + kStages * kXBytes;                  // kAStages x kABytes: the dequantised fp16 weight tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_a + kAStages * kABytes);
  uint64_t* full = bars;                                   // [kStages]   TMA landed
  uint64_t* empty = bars + kStages;                        // [kStages]   converters (256) + MMA commit (1)
  uint64_t* a_full = bars + 2 * kStages;                   // [kAStages]  converters (256)
  uint64_t* a_empty = a_full + kAStages;                   // [kAStages]  MMA commit (1)
  uint64_t* acc_full = a_empty + kAStages;                 // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  uint64_t* xch_bar = bars + 40;                              // [1] 128-row batches: the other ranks' partials have landed
  float* s_rowscale = reinterpret_cast<float*>(bars + 64);   // [2 passes][128 tile rows], used when MP == 128
  float* s_partial = reinterpret_cast<float*>(smem);       // split-K partials reuse the ring once it has drained

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool swiglu = p.epilogue == CACHEIR_B200_EPI_SWIGLU;
  const int passes = swiglu ? 2 : 1;
  const int split = p.split_k;
  const int krank = split > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int kblocks_all = p.K / kBlockK;
  const int kb_begin = (kblocks_all * krank) / split;
  const int kb_end = (kblocks_all * (krank + 1)) / split;
  const int kblocks = kb_end - kb_begin;
  const int total = kblocks * passes;
  const int n0 = blockIdx.x * kBlockN;
  // Back-to-back MMAs into one accumulator serialise on it; k steps rotate over `nacc`
  // independent accumulators (summed in a fixed order in the epilogue).
  const int nacc = (kAColBase / (passes * MP)) > 4 ? 4 : (kAColBase / (passes * MP));

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&full[s]), 1); mbar_init(smem_u32(&empty[s]), kConvThreads + 1); }
    for (int t = 0; t < kAStages; ++t) { mbar_init(smem_u32(&a_full[t]), kConvThreads); mbar_init(smem_u32(&a_empty[t]), 1); }
    mbar_init(smem_u32(acc_full), 1);
    mbar_init(smem_u32(xch_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {   // TMEM allocation is a warp-wide operation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      for (int i = 0; i < total; ++i) {
        const int s = i % kStages;
        const uint32_t ph = (i / kStages) & 1;
        if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1, 1)) break;
        const int pass = i / kblocks;
        const int kb = kb_begin + i % kblocks;
        const int row0 = n0 + pass * (p.N / 2);
        const uint32_t bar = smem_u32(&full[s]);
        mbar_expect_tx(bar, kRawBytes + kXBytes);
        if (p.tiled) {   // one contiguous tile, stored with its 16-byte chunks already in swizzled order
          const size_t band = blockIdx.x + pass * (p.N / 2 / kBlockN);
          const uint8_t* src = p.w_tiled + (band * kblocks_all + kb) * kRawBytes;
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       :: "r"(smem_u32(s_raw + s * kRawBytes)), "l"(src), "r"(static_cast<uint32_t>(kRawBytes)), "r"(bar) : "memory");
        } else {
          tma_load_2d(smem_u32(s_raw + s * kRawBytes), &tmap_w, bar, kb * kRawRow, row0);
        }
        // x viewed as [K/64 spans][M rows][64 elements]: both 64-element halves of the k block in one copy
        tma_load_3d(smem_u32(s_x + s * kXBytes), &tmap_x, bar, 0, 0, kb * 2);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      // instruction descriptor: D=f32, A=B=f16, both K-major, N=MP, M=128
      const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(MP >> 3) << 17) | (static_cast<uint32_t>(kBlockN >> 4) << 24);
      for (int i = 0; i < total; ++i) {
        const int s = i % kStages;
        const int t = i % kAStages;
        if (!mbar_wait(smem_u32(&full[s]), (i / kStages) & 1, 2)) break;
        if (!mbar_wait(smem_u32(&a_full[t]), (i / kAStages) & 1, 3)) break;
        tc_fence_after();
        const int pass = i / kblocks;
        const int kb = i % kblocks;
        const uint32_t d = tmem_base + pass * nacc * MP;
        const uint32_t a_base = smem_u32(s_a + t * kABytes);
        const uint32_t x_base = smem_u32(s_x + s * kXBytes);
#pragma unroll
        for (int j = 0; j < kBlockK / 16; ++j) {
          // A (dequantised weights) and B (x): 128-byte swizzled rows, 8-row groups 1024 B apart; 32 B per k step
          // inside a 64-element span, the second span one half tile further.
          const uint64_t a_desc = smem_desc(a_base + (j / 4) * (kBlockN * 128) + (j % 4) * 32, 16, 1024, 2);
          const uint64_t b_desc = smem_desc(x_base + (j / 4) * (MP * 128) + (j % 4) * 32, 16, 1024, 2);
          if (kWide) tc_mma_f16_ss(d + (j & (nacc - 1)) * MP, b_desc, a_desc, idesc, (kb > 0 || j >= nacc) ? 1u : 0u);
          else tc_mma_f16_ss(d + (j & (nacc - 1)) * MP, a_desc, b_desc, idesc, (kb > 0 || j >= nacc) ? 1u : 0u);
        }
        tc_commit(smem_u32(&a_empty[t]));   // operand columns and the x stage are free once these MMAs retire
        tc_commit(smem_u32(&empty[s]));
      }
      tc_commit(smem_u32(acc_full));
    }
  } else if (warp >= 4) {
    // ---------------- converters, then epilogue ----------------
    const int cw = warp - 4;                      // 0..15
    const int q = cw & 3;                         // TMEM lane quarter this warp may access (= warp % 4)
    const int hsel = cw >> 2;                     // converting: which quarter of the row's k range; epilogue (warps 4..11): which half of the output columns
    const int r = q * 32 + lane;                  // row of the tile owned by this thread (= TMEM lane)
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const int swz = BITS == 8 ? (r & 7) : ((r >> 1) & 3);
    bool ok = true;
    float row_scale[2] = {1.f, 1.f};
    for (int pass = 0; pass < passes && ok; ++pass) {
      const int n = n0 + pass * (p.N / 2) + r;
      const bool row_valid = n < (swiglu ? (pass + 1) * (p.N / 2) : p.N);
      float zero = static_cast<float>(1 << (BITS - 1));
      float scale = 1.f;
      if (!GROUPED && row_valid) {
        scale = load_scale(p.scales, p.scale_dtype, n);
        if (p.zero_points) zero = p.zero_points[n];
      }
      // exact in-register zero-point removal needs an integer zero point that fp16 can offset exactly
      const bool fast = GROUPED || ((zero == rintf(zero)) && fabsf(zero) <= 960.f);
      row_scale[pass] = (!GROUPED && fast) ? scale : 1.f;
      if (kWide && hsel == 0) s_rowscale[pass * kBlockN + r] = row_scale[pass];
      const __half2 sub8 = __float2half2_rn(1024.f + zero);
      const __half2 mul4 = __floats2half2_rn(1.f, 0.0625f);
      const __half2 sub4 = __floats2half2_rn(-(1024.f + zero), -(64.f + zero));
      constexpr bool scaled = GROUPED;
      // group scales are fetched one k block ahead: the load must not sit between the barrier and the unpacking
      const int groups_per_row = scaled ? p.K / p.group_size : 1;
      const size_t scale_row = static_cast<size_t>(n) * groups_per_row;
      const int kb_per_group = scaled ? p.group_size / kBlockK : 1;       // the group size is a multiple of the k block
      auto group_scale = [&](int kbi) {
        const int kb = kb_begin + kbi;
        return (scaled && row_valid && kbi < kblocks)
                   ? load_scale(p.scales, p.scale_dtype, scale_row + (kb_per_group == 1 ? kb : kb / kb_per_group))
                   : 1.f;
      };
      float next_scale = group_scale(0);
      for (int kbi = 0; kbi < kblocks; ++kbi) {
        const int i = pass * kblocks + kbi;
        const int s = i % kStages;
        const int t = i % kAStages;
        ok = mbar_wait(smem_u32(&full[s]), (i / kStages) & 1, 4);
        ok = ok && mbar_wait(smem_u32(&a_empty[t]), ((i / kAStages) & 1) ^ 1, 5);
        if (!ok) break;
        tc_fence_after();
        const uint8_t* raw_row = s_raw + s * kRawBytes + r * kRawRow;
        uint8_t* a_tile = s_a + t * kABytes;
        const __half2 gscale = __float2half2_rn(next_scale);
        next_scale = group_scale(kbi + 1);
        uint4 raw[kChunksPerThread];
#pragma unroll
        for (int cc = 0; cc < kChunksPerThread; ++cc) {
          const int c = hsel * kChunksPerThread + cc;
          raw[cc] = *reinterpret_cast<const uint4*>(raw_row + ((c ^ swz) * 16));
        }
#pragma unroll
        for (int cc = 0; cc < kChunksPerThread; ++cc) {
          const int c = hsel * kChunksPerThread + cc;
          const uint32_t w[4] = {raw[cc].x, raw[cc].y, raw[cc].z, raw[cc].w};
          if (BITS == 8) {      // 16 codes -> 8 columns starting at 8c
            uint32_t o[8];
            if (fast) {
              unpack8_int8(w[0], w[1], sub8, scaled, gscale, o);
              unpack8_int8(w[2], w[3], sub8, scaled, gscale, o + 4);
            } else {
              unpack8_slow<8>(reinterpret_cast<const uint8_t*>(w), 0, zero, scale, o);
              unpack8_slow<8>(reinterpret_cast<const uint8_t*>(w), 8, zero, scale, o + 4);
            }
            st_operand16(a_tile, r, 16 * c, reinterpret_cast<const uint32_t(&)[8]>(o));
          } else {              // 32 codes -> 16 columns starting at 16c
#pragma unroll
            for (int hw = 0; hw < 2; ++hw) {
              uint32_t o[8];
              if (fast) {
                unpack8_int4(w[2 * hw], mul4, sub4, scaled, gscale, o);
                unpack8_int4(w[2 * hw + 1], mul4, sub4, scaled, gscale, o + 4);
              } else {
                unpack8_slow<4>(reinterpret_cast<const uint8_t*>(w), 16 * hw, zero, scale, o);
                unpack8_slow<4>(reinterpret_cast<const uint8_t*>(w), 16 * hw + 8, zero, scale, o + 4);
              }
              st_operand16(a_tile, r, 32 * c + 16 * hw, reinterpret_cast<const uint32_t(&)[8]>(o));
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads the tile through the async proxy
        mbar_arrive(smem_u32(&a_full[t]));
        mbar_arrive(smem_u32(&empty[s]));
      }
    }
    if constexpr (kWide) {
      // ---- epilogue, 128-row batches: this warp owns batch rows [32q, 32q+32) (its TMEM lanes) and
      //      tile rows [32 hsel, 32 hsel + 32) (accumulator columns) ----
      asm volatile("bar.sync 3, %0;" ::"n"(kConvThreads) : "memory");   // the row-scale table is complete
      constexpr int kCols = 32;
      ok = ok && mbar_wait(smem_u32(acc_full), 0, 6);
      tc_fence_after();
      const bool have = ok && total > 0;
      __half* y = static_cast<__half*>(p.y);
      const __half* res = static_cast<const __half*>(p.residual);
      // The epilogue runs once per CTA from a cold instruction cache, so its loops stay rolled: straight-line
      // code of a few thousand instructions costs more in fetches than the work it does.
      // eight columns (c0 .. c0+7 of this warp's 32) of accumulator a: the rotating accumulators added in a fixed order
      auto ld8 = [&](int a, int c0, float (&v8)[8]) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v8[j] = 0.f;
        if (have) {
#pragma unroll 1
          for (int part = 0; part < nacc; ++part) {
            uint32_t v[8];
            tc_ld_x8(tmem_base + lane_addr + (a * nacc + part) * MP + hsel * kCols + c0, v);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) v8[j] += __uint_as_float(v[j]);
          }
        }
      };
      const bool vec = (p.n_out % 4) == 0 && (reinterpret_cast<uintptr_t>(y) & 7) == 0 && (reinterpret_cast<uintptr_t>(res) & 7) == 0;
      // four finished outputs of row r, tile columns col0 .. col0+3
      auto store4 = [&](int col0, const float* v4) {
        const int n_idx = n0 + col0;
        if (n_idx >= p.n_out || !ok || r >= p.M) return;
        float out[4] = {v4[0], v4[1], v4[2], v4[3]};
        const size_t o = static_cast<size_t>(r) * p.n_out + n_idx;
        if (vec) {
          if (p.epilogue == CACHEIR_B200_EPI_RESIDUAL) {
            const uint2 rv = *reinterpret_cast<const uint2*>(res + o);
            const __half2* rh = reinterpret_cast<const __half2*>(&rv);
            const float2 f0 = __half22float2(rh[0]), f1 = __half22float2(rh[1]);
            out[0] += f0.x; out[1] += f0.y; out[2] += f1.x; out[3] += f1.y;
          }
          uint2 ov;
          __half2* oh = reinterpret_cast<__half2*>(&ov);
          oh[0] = __floats2half2_rn(out[0], out[1]);
          oh[1] = __floats2half2_rn(out[2], out[3]);
          *reinterpret_cast<uint2*>(y + o) = ov;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (n_idx + j < p.n_out) {
              float v = out[j];
              if (p.epilogue == CACHEIR_B200_EPI_RESIDUAL) v += __half2float(res[o + j]);
              y[o + j] = __float2half_rn(v);
            }
          }
        }
      };
      if (split == 1) {
#pragma unroll 1
        for (int c0 = 0; c0 < kCols; c0 += 8) {
          float g[8], u[8];
          ld8(0, c0, g);
          if (swiglu) ld8(1, c0, u);
          const int col = hsel * kCols + c0;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float v = g[j] * s_rowscale[col + j];
            g[j] = swiglu ? silu_fast(v) * (u[j] * s_rowscale[kBlockN + col + j]) : v;
          }
          store4(col, g);
          store4(col + 4, g + 4);
        }
      } else {
        // Split-K (2, 4 or 8 ranks) as a reduce-scatter: rank d finishes columns [d W, (d+1) W) of the tile,
        // W = 128 / split. Every rank stages its partial by destination in its drained ring, one bulk copy
        // per destination moves a slot into that rank's receive area, and each rank adds the `split`
        // partials of its own columns in rank order (deterministic). The two SwiGLU accumulators go one
        // after the other through the same 64 KB + 64 KB; the gate sums wait in a third area.
        const int W = kBlockN / split;                 // columns this rank finishes (64, 32 or 16)
        const int log_w = 31 - __clz(W);
        const int cnt = W / 4;                         // ... of which this thread handles cnt (4 column groups per row)
        const int slot_floats = W * 128;
        float* s_stage = s_partial;                    // [dest][W][128 rows]
        float* s_recv = s_partial + kBlockN * 128;     // [src][W][128 rows]
        float* s_keep = s_partial + 2 * kBlockN * 128; // [W][128 rows]: each thread parks its own gate sums here
#pragma unroll 1
        for (int a = 0; a < passes; ++a) {
          if (threadIdx.x == 128) mbar_expect_tx(smem_u32(xch_bar), (split - 1) * slot_floats * 4);
          cluster_sync_all();                          // every rank has drained its ring (and read the previous exchange) and armed its barrier
#pragma unroll 1
          for (int c0 = 0; c0 < kCols; c0 += 8) {
            float v8[8];
            ld8(a, c0, v8);
            const int c = hsel * kCols + c0;           // eight consecutive columns share a destination (W >= 16)
            float* dst = s_stage + (c >> log_w) * slot_floats + (c & (W - 1)) * 128 + r;
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j * 128] = v8[j];
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync 3, %0;" ::"n"(kConvThreads) : "memory");
          if (cw == 0 && lane < split - 1) {           // one lane per destination
            const int dest = (krank + 1 + lane) % split;
            bulk_copy_to_rank(smem_u32(s_recv + krank * slot_floats), smem_u32(s_stage + dest * slot_floats),
                              slot_floats * 4, smem_u32(xch_bar), dest);
          }
          __syncwarp();
          ok = mbar_wait(smem_u32(xch_bar), a & 1, 7) && ok;
#pragma unroll 1
          for (int i0 = 0; i0 < cnt; i0 += 4) {
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            const int mine = (hsel * cnt + i0) * 128 + r;
#pragma unroll 1
            for (int k = 0; k < split; ++k) {
              const float* src = (k == krank ? s_stage : s_recv) + k * slot_floats + mine;
#pragma unroll
              for (int j = 0; j < 4; ++j) sum[j] += src[j * 128];
            }
            const int col = krank * W + hsel * cnt + i0;
            if (swiglu && a == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) s_keep[mine + j * 128] = sum[j];
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float v = sum[j] * s_rowscale[a * kBlockN + col + j];
                sum[j] = swiglu ? silu_fast(s_keep[mine + j * 128] * s_rowscale[col + j]) * v : v;
              }
              store4(col, sum);
            }
          }
        }
        cluster_sync_all();                            // all copies out of this CTA's shared memory have landed
      }
    } else if (cw >= 8) {   // the second eight converter warps have no epilogue share; they only join the cluster barriers
      if (split > 1) {
        __syncwarp();
        cluster_sync_all();
        cluster_sync_all();
      }
    } else {
    // ---- epilogue: this warp owns rows [32q, 32q+32) and output columns [hsel*MP/2, (hsel+1)*MP/2) ----
    constexpr int kColsPerWarp = MP / 2;
    float acc[2][kColsPerWarp];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int j = 0; j < kColsPerWarp; ++j) acc[a][j] = 0.f;
    ok = ok && mbar_wait(smem_u32(acc_full), 0, 6);
    if (ok && total > 0) {
      tc_fence_after();
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        if (a == 1 && !swiglu) break;
        for (int part = 0; part < nacc; ++part) {
#pragma unroll
          for (int c0 = 0; c0 < kColsPerWarp; c0 += 8) {
            uint32_t v[8];
            tc_ld_x8(tmem_base + lane_addr + (a * nacc + part) * MP + hsel * kColsPerWarp + c0, v);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[a][c0 + j] += __uint_as_float(v[j]);
          }
        }
      }
    }
    if (split > 1) {
      // Deterministic split-K: ranks 1.. send their partial rows to rank 0's shared memory
      // (the pipeline ring, idle by now), rank 0 adds them in rank order.
      cluster_sync_all();
      if (krank != 0) {
#pragma unroll
        for (int a = 0; a < 2; ++a) {
          if (a == 1 && !swiglu) break;
#pragma unroll
          for (int j = 0; j < kColsPerWarp; ++j) {
            const int col = hsel * kColsPerWarp + j;
            st_cluster_f32(smem_u32(s_partial + ((static_cast<size_t>(krank - 1) * passes + a) * MP + col) * kBlockN + r), 0, acc[a][j]);
          }
        }
      }
      cluster_sync_all();
      if (krank == 0) {
        for (int k = 1; k < split; ++k)
#pragma unroll
          for (int a = 0; a < 2; ++a) {
            if (a == 1 && !swiglu) break;
#pragma unroll
            for (int j = 0; j < kColsPerWarp; ++j)
              acc[a][j] += s_partial[((static_cast<size_t>(k - 1) * passes + a) * MP + hsel * kColsPerWarp + j) * kBlockN + r];
          }
      }
    }
    if (ok && krank == 0) {
      const int n_out_idx = n0 + r;
      const bool store = n_out_idx < p.n_out;
      __half* y = static_cast<__half*>(p.y);
      const __half* res = static_cast<const __half*>(p.residual);
#pragma unroll
      for (int j = 0; j < kColsPerWarp; ++j) {
        const int m = hsel * kColsPerWarp + j;
        if (m < p.M && store) {
          float v = acc[0][j] * row_scale[0];
          const size_t o = static_cast<size_t>(m) * p.n_out + n_out_idx;
          if (swiglu) {
            const float u = acc[1][j] * row_scale[1];
            v = silu_fast(v) * u;
          } else if (p.epilogue == CACHEIR_B200_EPI_RESIDUAL) {
            v += __half2float(res[o]);
          }
          y[o] = __float2half_rn(v);
        }
      }
    }
    }   // cw < 8
  } 
  if (warp < 4 && split > 1) {   // warps without an epilogue still take part in the cluster barriers of the exchange
    __syncwarp();
    const int syncs = kWide ? passes + 1 : 2;
    for (int k = 0; k < syncs; ++k) cluster_sync_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  }
  return fn;
}

bool encode_2d(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t inner, uint64_t outer,
               uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem_strides[2] = {1, 1};
  return fn(map, type, 2, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
            swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// x[M, K] fp16 as a 3-D tensor [K/64][M][64]: a box {64, MP, 2} brings both 128-byte-swizzled
// halves of a 128-element k block in one copy, laid out as [half][row][64].
bool encode_x_3d(CUtensorMap* map, const void* base, uint64_t K, uint64_t M, uint64_t row_stride_bytes, uint32_t mp) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {64, M, K / 64};
  const cuuint64_t strides[2] = {row_stride_bytes, 128};
  const cuuint32_t box[3] = {64, mp, 2};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem_strides,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// CTAs per cluster along K: enough to put about one CTA on every SM. The SwiGLU form exchanges two
// accumulators per rank, so it splits at most in two (what fits in the drained ring).
int choose_split_k(int n_tiles, int kblocks, int epilogue) {
  int s = kNumSMs / n_tiles;
  if (s > kMaxSplitK) s = kMaxSplitK;
  if (epilogue == CACHEIR_B200_EPI_SWIGLU && s > 2) s = 2;
  if (s > kblocks / 4) s = kblocks / 4;     // keep at least four k blocks per CTA
  return s < 1 ? 1 : s;
}

template <int BITS, int MP, bool GROUPED>
int launch_tc(const QGemvParams& q, cudaStream_t stream) {
  constexpr int kStages = num_stages(BITS, MP);
  constexpr int kAStages = a_stages(BITS, MP);
  constexpr size_t kSmem = 1024 + static_cast<size_t>(kStages) * stage_bytes(BITS, MP) + kAStages * kABytes + 512 + 1024;
  static_assert(kSmem <= 227 * 1024, "ring + operand tiles must fit the shared memory of one SM");
  static_assert(MP == 128 ||
                    (static_cast<size_t>(kMaxSplitK - 1) * MP * kBlockN * 4 <= static_cast<size_t>(kStages) * stage_bytes(BITS, MP) &&
                     static_cast<size_t>(2) * MP * kBlockN * 4 <= static_cast<size_t>(kStages) * stage_bytes(BITS, MP)),
                "split-K partials must fit in the pipeline ring");
  static_assert(MP != 128 || static_cast<size_t>(2) * 128 * kBlockN * 4 + 64 * kBlockN * 4 <=
                                 static_cast<size_t>(kStages) * stage_bytes(BITS, MP) + kAStages * kABytes,
                "128-row batches: staging, receive and gate areas of the split-K exchange must fit in the ring plus the operand tiles");
  CUtensorMap tmap_w, tmap_x;
  const uint64_t row_bytes = BITS == 8 ? static_cast<uint64_t>(q.K) : static_cast<uint64_t>(q.K / 2);
  constexpr uint32_t kTileRowBytes = BITS == 8 ? 128 : 64;
  const uint64_t tiled_rows = static_cast<uint64_t>((q.N + kBlockN - 1) / kBlockN) * (q.K / kBlockK) * kBlockN;
  // (the tiled layout is fetched with plain bulk copies; the map is then only a valid placeholder)
  const bool w_ok = q.tiled
      ? encode_2d(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, q.packed, kTileRowBytes, tiled_rows, kTileRowBytes, kTileRowBytes, kBlockN,
                  BITS == 8 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B)
      : encode_2d(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, q.packed, row_bytes, static_cast<uint64_t>(q.N), row_bytes, kTileRowBytes,
                  kBlockN, BITS == 8 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
  if (!w_ok) return CACHEIR_B200_EUNSUPPORTED;
  if (!encode_x_3d(&tmap_x, q.x, static_cast<uint64_t>(q.K), static_cast<uint64_t>(q.M),
                   static_cast<uint64_t>(q.x_stride) * 2, MP))
    return CACHEIR_B200_EUNSUPPORTED;
  TcParams p{};
  p.scales = q.scales; p.zero_points = q.zero_points; p.residual = q.residual; p.y = q.y;
  p.M = q.M; p.N = q.N; p.K = q.K;
  p.n_out = q.epilogue == CACHEIR_B200_EPI_SWIGLU ? q.N / 2 : q.N;
  p.group_size = q.group_size; p.scale_dtype = q.scale_dtype; p.epilogue = q.epilogue; p.tiled = q.tiled ? 1 : 0;
  p.w_tiled = static_cast<const uint8_t*>(q.packed);
  const int n_tiles = (p.n_out + kBlockN - 1) / kBlockN;
  p.split_k = choose_split_k(n_tiles, q.K / kBlockK, q.epilogue);
  if (MP == 128) {   // reduce-scatter exchange: 2, 4 or 8 ranks, the SwiGLU form as far as the plain one; few tiles split further
    int want = kNumSMs / n_tiles;
    if (want > q.K / kBlockK / 4) want = q.K / kBlockK / 4;
    const int cap = n_tiles <= 16 ? 8 : kMaxSplitK;
    int s = 1;
    while (s * 2 <= want && s * 2 <= cap) s *= 2;
    p.split_k = s;
  }
  auto kern = qgemm_tc_kernel<BITS, MP, GROUPED>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmem));
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(n_tiles, p.split_k, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = p.split_k;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, tmap_w, tmap_x, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  return launch_status();
}

template <int BITS, bool GROUPED>
int launch_tc_mp(const QGemvParams& q, cudaStream_t stream) {
  if (q.M <= 16) return launch_tc<BITS, 16, GROUPED>(q, stream);
  if (q.M <= 32) return launch_tc<BITS, 32, GROUPED>(q, stream);
  if (q.M <= 64) return launch_tc<BITS, 64, GROUPED>(q, stream);
  return launch_tc<BITS, 128, GROUPED>(q, stream);
}

}  // namespace

bool qgemm_tc_supported(const QGemvParams& q) {
  if (q.x_dtype != CACHEIR_B200_F16) return false;
  if (q.bits != 4 && q.bits != 8) return false;
  if (q.M < 1 || q.M > 128) return false;
  if (q.K % kBlockK != 0 || q.K < kBlockK) return false;
  if (q.group_size != 0 && q.group_size % kBlockK != 0) return false;   // one scale per row and k block
  if (q.epilogue == CACHEIR_B200_EPI_SWIGLU && (q.N / 2) % kBlockN != 0) return false;
  if (!aligned_to(q.packed, 16) || !aligned_to(q.x, 16) || (q.x_stride * 2) % 16 != 0) return false;
  return get_encode_fn() != nullptr;
}

int launch_qgemm_tc(const QGemvParams& q, cudaStream_t stream) {
  if (q.group_size > 0) return q.bits == 8 ? launch_tc_mp<8, true>(q, stream) : launch_tc_mp<4, true>(q, stream);
  return q.bits == 8 ? launch_tc_mp<8, false>(q, stream) : launch_tc_mp<4, false>(q, stream);
}

int qgemm_tc_device_status(bool reset) {
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_qgemm_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_qgemm_status, &zero, sizeof(int));
  }
  return status;
}

}  // namespace cb200
