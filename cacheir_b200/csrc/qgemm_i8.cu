// int8 dequant-GEMM on the integer tensor cores (tcgen05.mma kind::i8), sm_100a.
//
//   y[M, N] = x[M, K] . ((code[N, K] - zero[N]) * scale[N])^T      M <= 64, fp16 x/y
//
// The packed uint8 codes go from HBM through TMA into shared memory and from there
// straight into the tensor core: nothing unpacks, converts or re-stores a weight.
// Activations are made integer instead. A pre-pass turns every row of x into 16-bit
// fixed point with its own scale, x[m,k] ~= sx[m] * q[m,k], |q| <= 32639 (2^-15 of the
// row maximum: far below fp16's own resolution), and splits q into two signed bytes,
// q = 256*hi + lo. With the weight tile as the 128-row operand and the [hi; lo] rows
// as the other one, a single accumulator row holds, for weight row n,
//   D[n, m] = sum_k code[n,k]*hi[m,k]      D[n, MP+m] = sum_k code[n,k]*lo[m,k]
// exactly (int32). The epilogue recombines in double precision:
//   y[m,n] = scale[n] * sx[m] * (256*D[n,m] + D[n,MP+m] - zero[n] * sum_k q[m,k]).
//
// One CTA owns 128 weight rows and a K range: warp 0 issues the TMA copies, warp 1 the
// MMAs (K = 32 per instruction, 4 per 128-column stage), warps 2-5 run the epilogue.
// K ranges of one row tile form a thread-block cluster. Their partial sums are integers, so
// the order of addition cannot matter; they are exchanged all-to-all through distributed
// shared memory, each CTA of the cluster finishing the outputs of its own slice of the batch.
#include "common.cuh"
#include "qgemv_common.cuh"
#include "tc_ptx.cuh"

namespace cb200 {
namespace {

using namespace ptx;

constexpr int kBlockN = 128;          // weight rows per CTA (UMMA M)
constexpr int kBlockK = 128;          // bytes of a weight row per stage
constexpr int kThreads = 192;         // producer, MMA, four epilogue warps
constexpr int kTmemCols = 256;
constexpr int kRingBudget = 96 * 1024;   // two CTAs per SM: one issues MMAs while the other waits on a barrier
constexpr int kMaxSplitK = 8;
constexpr float kQMax = 32639.f;      // 127*256 + 127: every value splits into two signed bytes

__device__ int g_i8_status = 0;

#ifdef CB200_QGEMM_TRACE
__device__ long long g_i8_trace[4][256][4];
#define CB200_TRACE(role, i, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (i) < 256) g_i8_trace[role][i][slot] = clock64(); } while (0)
#else
#define CB200_TRACE(role, i, slot) do { } while (0)
#endif

__host__ __device__ constexpr int stage_bytes(int mp) { return kBlockN * kBlockK + 2 * mp * kBlockK; }
__host__ __device__ constexpr int num_stages(int mp) { return kRingBudget / stage_bytes(mp) > 8 ? 8 : kRingBudget / stage_bytes(mp); }

// ---- pre-pass: rows of x -> two planes of signed bytes + scale + sum ------------------
// planes: [2*mp rows][K] int8 (rows [0,mp): high bytes, [mp,2mp): low bytes; rows >= M are zero)
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const __half* __restrict__ x, long long x_stride, int M, int K, int mp,
                     int8_t* __restrict__ planes, float* __restrict__ sx, int* __restrict__ qsum) {
  __shared__ float s_red[8];
  __shared__ int s_sum[8];
  const int m = blockIdx.x;
  int8_t* hi_row = planes + static_cast<size_t>(m) * K;
  int8_t* lo_row = planes + static_cast<size_t>(mp + m) * K;
  const int nvec = K / 8;
  if (m >= M) {
    for (int c = threadIdx.x; c < nvec; c += 256) {
      *reinterpret_cast<uint2*>(hi_row + c * 8) = make_uint2(0u, 0u);
      *reinterpret_cast<uint2*>(lo_row + c * 8) = make_uint2(0u, 0u);
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
    uint32_t hi_w[2] = {0u, 0u}, lo_w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int q = __float2int_rn(v[i] * inv);
      q = max(-32639, min(32639, q));
      const int hi = (q + 128) >> 8;            // arithmetic shift: floor((q+128)/256)
      const int lo = q - (hi << 8);             // in [-128, 127]
      sum += q;
      hi_w[i >> 2] |= static_cast<uint32_t>(hi & 0xFF) << (8 * (i & 3));
      lo_w[i >> 2] |= static_cast<uint32_t>(lo & 0xFF) << (8 * (i & 3));
    }
    *reinterpret_cast<uint2*>(hi_row + c * 8) = make_uint2(hi_w[0], hi_w[1]);
    *reinterpret_cast<uint2*>(lo_row + c * 8) = make_uint2(lo_w[0], lo_w[1]);
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

struct I8Params {
  const void* scales;
  const float* zero_points;
  const void* residual;
  void* y;
  const float* sx;
  const int* qsum;
  int M, N, K;
  int n_out;
  int scale_dtype;
  int epilogue;
  int split_k;
  int tiled;        // weights in 128x128 tile order: tile (band, kb) starts at row (band*KB + kb)*128 of a 128-byte-wide tensor
};

template <int MP>
__global__ void __launch_bounds__(kThreads, 2)
qgemm_i8_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const I8Params p) {
  constexpr int kStages = num_stages(MP);
  constexpr int kWBytes = kBlockN * kBlockK;          // 16 KB of codes per stage
  constexpr int kXBytes = 2 * MP * kBlockK;           // [hi; lo] rows per stage
  constexpr int kAccCols = 2 * MP;                    // one accumulator: MP high + MP low columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* s_w = smem;
  uint8_t* s_x = s_w + kStages * kWBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_x + kStages * kXBytes);
  uint64_t* full = bars;                  // [kStages] TMA landed
  uint64_t* empty = bars + kStages;       // [kStages] MMAs that read the stage have retired
  uint64_t* acc_full = empty + kStages;   // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  float* s_sx = reinterpret_cast<float*>(tmem_slot + 2);     // [MP]
  int* s_qsum = reinterpret_cast<int*>(s_sx + MP);           // [MP]
  int32_t* s_partial = reinterpret_cast<int32_t*>(smem);     // split-K partials reuse the drained ring

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 64) CB200_TRACE(3, 0, 0);
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

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&full[s]), 1); mbar_init(smem_u32(&empty[s]), 1); }
    mbar_init(smem_u32(acc_full), 1);
    mbar_fence_init();
  }
  if (threadIdx.x >= 64 && threadIdx.x < 64 + MP) {
    s_sx[threadIdx.x - 64] = p.sx[threadIdx.x - 64];
    s_qsum[threadIdx.x - 64] = p.qsum[threadIdx.x - 64];
  }
  if (warp == 1) tc_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 64) CB200_TRACE(3, 0, 1);

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      for (int i = 0; i < total; ++i) {
        const int s = i % kStages;
        CB200_TRACE(0, i, 0);
        if (!mbar_wait(smem_u32(&empty[s]), ((i / kStages) & 1) ^ 1, &g_i8_status, (3 << 8) | 1)) break;
        CB200_TRACE(0, i, 1);
        const int pass = i / kblocks;
        const int kb = kb_begin + i % kblocks;
        const uint32_t bar = smem_u32(&full[s]);
        mbar_expect_tx(bar, kWBytes + kXBytes);
        if (p.tiled) {
          const int band = blockIdx.x + pass * (p.N / 2 / kBlockN);
          tma_load_2d(smem_u32(s_w + s * kWBytes), &tmap_w, bar, 0, (band * kblocks_all + kb) * kBlockN);
        } else {
          tma_load_2d(smem_u32(s_w + s * kWBytes), &tmap_w, bar, kb * kBlockK, n0 + pass * (p.N / 2));
        }
        tma_load_2d(smem_u32(s_x + s * kXBytes), &tmap_x, bar, kb * kBlockK, 0);
        CB200_TRACE(0, i, 2);
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
        CB200_TRACE(1, i, 0);
        if (!mbar_wait(smem_u32(&full[s]), (i / kStages) & 1, &g_i8_status, (3 << 8) | 2)) break;
        CB200_TRACE(1, i, 1);
        tc_fence_after();
        const int pass = i / kblocks;
        const int kb = i % kblocks;
        const uint32_t d = tmem_base + pass * kAccCols;
        const uint32_t w_base = smem_u32(s_w + s * kWBytes);
        const uint32_t x_base = smem_u32(s_x + s * kXBytes);
#pragma unroll
        for (int j = 0; j < kBlockK / 32; ++j)   // 32 bytes of k per instruction inside the 128-byte swizzle span
          tc_mma_i8_ss(d, smem_desc_sw128(w_base + j * 32), smem_desc_sw128(x_base + j * 32), idesc, (kb > 0 || j > 0) ? 1u : 0u);
        CB200_TRACE(1, i, 2);
        tc_commit(smem_u32(&empty[s]));
        CB200_TRACE(1, i, 3);
      }
      tc_commit(smem_u32(acc_full));
    }
  } else {
    // ---------------- epilogue warps: lane quarter = warp % 4 ----------------
    const int q = warp & 3;
    const int r = q * 32 + lane;                 // weight row of the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    bool ok = mbar_wait(smem_u32(acc_full), 0, &g_i8_status, (3 << 8) | 3);
    tc_fence_after();
    if (threadIdx.x == 64) CB200_TRACE(3, 0, 2);
    const int n_out_idx = n0 + r;
    const bool store = ok && n_out_idx < p.n_out;
    double scale[2] = {0.0, 0.0}, zero[2] = {128.0, 128.0};
    for (int pass = 0; pass < passes; ++pass) {
      const int n = n0 + pass * (p.N / 2) + r;
      if (n < p.N) {
        scale[pass] = p.scale_dtype == CACHEIR_B200_F16 ? static_cast<double>(__half2float(static_cast<const __half*>(p.scales)[n]))
                                                        : static_cast<double>(static_cast<const float*>(p.scales)[n]);
        if (p.zero_points) zero[pass] = static_cast<double>(p.zero_points[n]);
      }
    }
    __half* y = static_cast<__half*>(p.y);
    const __half* res = static_cast<const __half*>(p.residual);
    if (split > 1) {
      // All-to-all over the cluster: rank j finishes batch rows [j*MS, (j+1)*MS). Every rank
      // sends, for each of those rows, its high and low partial sums to rank j's buffer
      // s_partial[sender][2*MS columns][128 weight rows].
      const int MS = MP / split;
      cluster_sync_all();                        // #1: every ring of the cluster has drained
      if (threadIdx.x == 64) CB200_TRACE(3, 0, 3);
#pragma unroll 1
      for (int c0 = 0; c0 < kAccCols; c0 += 8) {
        uint32_t v[8];
        if (total > 0) {
          tc_ld_x8(tmem_base + lane_addr + c0, v);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = c0 + j;
          const int m = c % MP;                  // batch row; c / MP selects high (0) or low (1) bytes
          const int dest = m / MS;
          const int lc = (c / MP) * MS + (m % MS);
          st_cluster_u32(smem_u32(s_partial + (static_cast<size_t>(krank) * 2 * MS + lc) * kBlockN + r), dest, v[j]);
        }
      }
      if (threadIdx.x == 64) CB200_TRACE(3, 1, 0);
      cluster_sync_all();                        // #2: all partials have arrived
      if (threadIdx.x == 64) CB200_TRACE(3, 1, 1);
      for (int ml = 0; ml < MS; ++ml) {
        const int m = krank * MS + ml;
        int32_t hi = 0, lo = 0;
        for (int k = 0; k < split; ++k) {
          hi += s_partial[(static_cast<size_t>(k) * 2 * MS + ml) * kBlockN + r];
          lo += s_partial[(static_cast<size_t>(k) * 2 * MS + MS + ml) * kBlockN + r];
        }
        if (m < p.M && store) {
          const double v = 256.0 * static_cast<double>(hi) + static_cast<double>(lo) - zero[0] * static_cast<double>(s_qsum[m]);
          float out = static_cast<float>(v * scale[0] * static_cast<double>(s_sx[m]));
          const size_t o = static_cast<size_t>(m) * p.n_out + n_out_idx;
          if (p.epilogue == CACHEIR_B200_EPI_RESIDUAL) out += __half2float(res[o]);
          y[o] = __float2half_rn(out);
        }
      }
    } else {
#pragma unroll 1
      for (int c0 = 0; c0 < MP; c0 += 8) {
        uint32_t hi[2][8], lo[2][8];
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          if (pass < passes && total > 0) {
            tc_ld_x8(tmem_base + lane_addr + pass * kAccCols + c0, hi[pass]);
            tc_ld_x8(tmem_base + lane_addr + pass * kAccCols + MP + c0, lo[pass]);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) { hi[pass][j] = 0u; lo[pass][j] = 0u; }
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int m = c0 + j;
          if (m < p.M && store) {
            const double sxm = static_cast<double>(s_sx[m]);
            const double qs = static_cast<double>(s_qsum[m]);
            const double v = 256.0 * static_cast<double>(static_cast<int32_t>(hi[0][j])) +
                             static_cast<double>(static_cast<int32_t>(lo[0][j])) - zero[0] * qs;
            float out = static_cast<float>(v * scale[0] * sxm);
            const size_t o = static_cast<size_t>(m) * p.n_out + n_out_idx;
            if (swiglu) {
              const double u = 256.0 * static_cast<double>(static_cast<int32_t>(hi[1][j])) +
                               static_cast<double>(static_cast<int32_t>(lo[1][j])) - zero[1] * qs;
              out = (out / (1.f + __expf(-out))) * static_cast<float>(u * scale[1] * sxm);
            } else if (p.epilogue == CACHEIR_B200_EPI_RESIDUAL) {
              out += __half2float(res[o]);
            }
            y[o] = __float2half_rn(out);
          }
        }
      }
    }
  }
  if (warp < 2 && split > 1) {   // warps without an epilogue still take part in the two cluster barriers
    __syncwarp();
    cluster_sync_all();
    cluster_sync_all();
  }
  if (threadIdx.x == 64) CB200_TRACE(3, 1, 2);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tc_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 64) CB200_TRACE(3, 1, 3);
}

// CTAs per cluster along K: enough to put about two CTAs on every SM; a power of two that
// divides the padded batch (each rank finishes MP/split batch rows). Never for SwiGLU.
int choose_split_k(int n_tiles, int kblocks, int epilogue, int mp) {
  if (epilogue == CACHEIR_B200_EPI_SWIGLU) return 1;
  int s = 1;
  while (s * 2 <= kMaxSplitK && n_tiles * s * 2 <= 2 * kNumSMs && kblocks / (s * 2) >= 4 && mp % (s * 2) == 0) s *= 2;
  return s;
}

template <int MP>
int launch_i8(const QGemvParams& q, void* workspace, cudaStream_t stream) {
  int8_t* planes = static_cast<int8_t*>(workspace);
  float* sx = reinterpret_cast<float*>(planes + static_cast<size_t>(2 * MP) * q.K);
  int* qsum = reinterpret_cast<int*>(sx + 64);
  quantize_rows_kernel<<<MP, 256, 0, stream>>>(static_cast<const __half*>(q.x), q.x_stride, q.M, q.K, MP, planes, sx, qsum);
  int rc = launch_status();
  if (rc != 0) return rc;

  CUtensorMap tmap_w, tmap_x;
  const uint64_t bands = static_cast<uint64_t>((q.N + kBlockN - 1) / kBlockN);
  const bool w_ok = q.tiled
      ? encode_u8_rows_sw128(&tmap_w, q.packed, kBlockK, bands * (q.K / kBlockK) * kBlockN, kBlockK, kBlockN)
      : encode_u8_rows_sw128(&tmap_w, q.packed, static_cast<uint64_t>(q.K), static_cast<uint64_t>(q.N), static_cast<uint64_t>(q.K), kBlockN);
  if (!w_ok) return CACHEIR_B200_EUNSUPPORTED;
  if (!encode_u8_rows_sw128(&tmap_x, planes, static_cast<uint64_t>(q.K), static_cast<uint64_t>(2 * MP), static_cast<uint64_t>(q.K), 2 * MP))
    return CACHEIR_B200_EUNSUPPORTED;
  I8Params p{};
  p.scales = q.scales; p.zero_points = q.zero_points; p.residual = q.residual; p.y = q.y;
  p.sx = sx; p.qsum = qsum;
  p.M = q.M; p.N = q.N; p.K = q.K;
  p.n_out = q.epilogue == CACHEIR_B200_EPI_SWIGLU ? q.N / 2 : q.N;
  p.scale_dtype = q.scale_dtype; p.epilogue = q.epilogue; p.tiled = q.tiled ? 1 : 0;
  const int n_tiles = (p.n_out + kBlockN - 1) / kBlockN;
  p.split_k = choose_split_k(n_tiles, q.K / kBlockK, q.epilogue, MP);
  constexpr size_t kSmem = 1024 + static_cast<size_t>(num_stages(MP)) * stage_bytes(MP) + 1024;
  auto kern = qgemm_i8_kernel<MP>;
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

}  // namespace

size_t qgemm_i8_workspace_bytes(int M, int K) {
  if (M <= 0 || K <= 0) return 0;
  return static_cast<size_t>(128) * K + 1024;   // two planes of up to 64 rows, then scales and sums
}

bool qgemm_i8_supported(const QGemvParams& q, const void* workspace, size_t workspace_bytes) {
  if (q.x_dtype != CACHEIR_B200_F16 || q.bits != 8 || q.group_size != 0) return false;
  if (q.M < 1 || q.M > 64) return false;
  if (q.K % kBlockK != 0 || q.K < kBlockK) return false;
  if (q.epilogue == CACHEIR_B200_EPI_SWIGLU && (q.N / 2) % kBlockN != 0) return false;
  if (!workspace || workspace_bytes < qgemm_i8_workspace_bytes(q.M, q.K) || !aligned_to(workspace, 128)) return false;
  if (!aligned_to(q.packed, 16) || !aligned_to(q.x, 16) || (q.x_stride * 2) % 16 != 0) return false;
  return tensor_map_encoder() != nullptr;
}

int launch_qgemm_i8(const QGemvParams& q, void* workspace, cudaStream_t stream) {
  if (q.M <= 16) return launch_i8<16>(q, workspace, stream);
  if (q.M <= 32) return launch_i8<32>(q, workspace, stream);
  return launch_i8<64>(q, workspace, stream);
}

#ifdef CB200_QGEMM_TRACE
extern "C" int cacheir_b200_debug_trace_i8(long long* out) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, g_i8_trace, sizeof(long long) * 4 * 256 * 4));
}
#endif

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
