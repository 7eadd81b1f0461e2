// One-shot collectives over NVLink peer memory for the tensor-parallel decode step.
//
// Every rank (one process per GPU) owns a data buffer and a small flag array allocated here
// and opened by its peers through CUDA IPC. A collective is one kernel per rank:
//   1. announce: write this call's epoch into slot [my rank] of every peer's flag array
//      (system-scope release: the producer kernel's writes to my buffer are visible first);
//   2. wait, bounded, until every peer's slot in my own flag array shows the epoch;
//   3. read all ranks' buffers with plain peer loads and combine them in rank order, so every
//      rank computes bit-identical results (all-reduce), or copy the peers' slices (all-gather).
// Large all-reduces take two steps inside one kernel (reduce-scatter, then all-gather): rank r adds only
// slice r of every rank's buffer and pushes the finished slice into a gather buffer on every rank; a second
// round of flags (raised by the last CTA of a rank to finish its slice) tells the peers that the slice has
// landed, and each rank copies its gather buffer to the output. Every rank moves 2 (world-1)/world of the
// message over NVLink instead of world-1 times the message, and the bits are identical everywhere because
// one rank computes each slice.
// Callers alternate between two data buffers from call to call: a rank may refill buffer A
// only after the call that used buffer B, whose wait proves every peer has left buffer A.
// The epoch lives on the device and advances with every call, so a captured CUDA graph can be
// replayed. Only plain peer loads and stores, no library collective. A wait that
// runs out of polls (about a second by default; state[3] > 0 sets the number of polls) records a code in the
// status word and the kernel returns (output undefined). While the status word is non-zero every later
// collective returns at once without waiting, so a lost peer costs one time-out, not one per call of a replayed
// graph; the host reads and clears the word with cacheir_b200_device_status.
#include <string.h>

#include "common.cuh"

namespace cb200 {
namespace {

constexpr int kMaxRanks = 8;
constexpr uint32_t kPeerPollLimit = 500u * 1000u;  // with the 2 us sleep below: about a second, then give up

__device__ int g_peer_status = 0;

struct PeerParams {
  const void* data[kMaxRanks];    // every rank's data buffer (index = rank), mapped into this process
  int* flags[kMaxRanks];          // every rank's flag array [kMaxRanks]
  void* gather[kMaxRanks];        // two-step all-reduce: every rank's gather buffer
  unsigned long long* ll_rs[kMaxRanks];   // flagged-word all-reduce: every rank's receive area of the reduce-scatter step
  unsigned long long* ll_ag[kMaxRanks];   // and of the all-gather step; each [2 parities][world senders][words per slice]
  void* out;
  size_t count;                   // all-reduce: elements; all-gather: elements of one rank's slice row
  int rows;                       // all-gather only: rows of the [rows, count] slices
  int rank, world;
  int* state;                     // local: {epoch, CTAs finished, CTAs that finished their slice, poll limit (0 = default)}
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Steps 1 and 2 for one CTA. Returns false when a peer never showed up.
__device__ __forceinline__ uint32_t poll_limit(const PeerParams& p) {
  const int configured = p.state[3];
  return configured > 0 ? static_cast<uint32_t>(configured) : kPeerPollLimit;
}
__device__ __forceinline__ bool peer_already_lost() { return *reinterpret_cast<volatile int*>(&g_peer_status) != 0; }

__device__ __forceinline__ bool announce_and_wait(const PeerParams& p, int epoch) {
  __shared__ int s_ok, s_lost;
  if (threadIdx.x == 0) { s_ok = 1; s_lost = peer_already_lost() ? 1 : 0; }   // one reader: the whole CTA takes the same branch
  __syncthreads();
  if (s_lost != 0) return false;                 // an earlier wait gave up and the host has not cleared the word yet
  const uint32_t limit = poll_limit(p);
  if (blockIdx.x == 0 && threadIdx.x < p.world && threadIdx.x != p.rank)
    st_release_sys(p.flags[threadIdx.x] + p.rank, epoch);   // (a release store carries its own system-scope fence)
  if (threadIdx.x < p.world && threadIdx.x != p.rank) {
    const int* slot = p.flags[p.rank] + threadIdx.x;
    bool seen = false;
    // Relaxed polls (an acquire load carries a system-scope fence: microseconds per poll), one acquire once the epoch shows.
    for (uint32_t i = 0; i < limit; ++i) {
      if (ld_relaxed_sys(slot) - epoch >= 0) { seen = ld_acquire_sys(slot) - epoch >= 0; break; }   // (difference: survives wrap-around)
      if (i > 256) __nanosleep(i > 16384 ? 2000 : 100);
    }
    if (!seen) {
      s_ok = 0;
      atomicCAS(&g_peer_status, 0, (4 << 8) | 1);
    }
  }
  __syncthreads();
  return s_ok != 0;
}

__device__ __forceinline__ void finish(const PeerParams& p, int epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(p.state + 1, 1) == static_cast<int>(gridDim.x) - 1) {   // last CTA: publish the epoch for the next call
      p.state[1] = 0;
      p.state[0] = epoch;
      __threadfence();
    }
  }
}

// acc = sum over ranks (in rank order) of 16-byte vector `i` of their data buffers. All loads are issued
// before the first add: a load from a peer takes microseconds, eight in a row would take eight times that.
template <typename T>
__device__ __forceinline__ void gather_sum(const PeerParams& p, size_t i, float (&acc)[16 / sizeof(T)]) {
  constexpr int VEC = 16 / sizeof(T);
  float v[kMaxRanks][VEC];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r)
    if (r < p.world) VecIO<T, VEC>::ld(static_cast<const T*>(p.data[r]) + i * VEC, v[r]);
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r)
    if (r < p.world) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] += v[r][j];
    }
}

template <typename T>
__global__ void __launch_bounds__(256) all_reduce_kernel(const PeerParams p) {
  const int epoch = p.state[0] + 1;
  if (announce_and_wait(p, epoch)) {
    constexpr int VEC = 16 / sizeof(T);
    const size_t nvec = p.count / VEC;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
      float acc[VEC];
      gather_sum<T>(p, i, acc);                  // rank order: the same sum, bit for bit, on every rank
      VecIO<T, VEC>::st(static_cast<T*>(p.out) + i * VEC, acc);
    }
  }
  finish(p, epoch);
}

// Reduce-scatter + all-gather in one launch; count is a multiple of world * (16 / sizeof(T)). Every CTA of
// a rank must be resident at once (the grid has at most one CTA per SM and the kernel owns the GPU when it
// runs): CTAs that have finished their slice wait for the peers' second flags while the others still add.
template <typename T>
__global__ void __launch_bounds__(256) all_reduce_two_step_kernel(const PeerParams p) {
  const int epoch = p.state[0] + 1;
  constexpr int VEC = 16 / sizeof(T);
  const size_t nvec = p.count / VEC;
  const size_t per = nvec / p.world;             // vectors of one slice
  __shared__ int s_ok2;
  bool ok = announce_and_wait(p, epoch);
  if (ok) {
    const size_t base = per * p.rank;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < per;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
      float acc[VEC];
      gather_sum<T>(p, base + i, acc);           // rank order
      for (int r = 0; r < p.world; ++r) VecIO<T, VEC>::st(static_cast<T*>(p.gather[r]) + (base + i) * VEC, acc);
    }
  }
  __shared__ int s_last;
  if (threadIdx.x == 0) s_ok2 = 1;
  __syncthreads();                               // every thread of the CTA has issued its pushes
  if (threadIdx.x == 0) {
    // One system-scope fence per CTA, after the barrier: it orders the whole CTA's pushes (fences are cumulative over
    // what the barrier made visible to this thread) before the counter, and through the counter before the flag that
    // the last CTA raises.
    __threadfence_system();
    s_last = atomicAdd(p.state + 2, 1) == static_cast<int>(gridDim.x) - 1 ? 1 : 0;
    __threadfence();                             // (acquire side of the counter: what the other CTAs fenced is ordered before the flag)
  }
  __syncthreads();
  if (s_last != 0) {                             // last CTA of this rank: the whole slice has been pushed
    if (threadIdx.x == 0) p.state[2] = 0;
    if (ok && threadIdx.x < p.world)             // one thread per peer: the system-scope releases run side by side
      st_release_sys(p.flags[threadIdx.x] + kMaxRanks + p.rank, epoch);
  }
  if (ok && threadIdx.x < p.world) {
    const int* slot = p.flags[p.rank] + kMaxRanks + threadIdx.x;
    const uint32_t limit = poll_limit(p);
    bool seen = false;
    for (uint32_t i = 0; i < limit; ++i) {
      if (ld_relaxed_sys(slot) - epoch >= 0) { seen = ld_acquire_sys(slot) - epoch >= 0; break; }
      if (i > 256) __nanosleep(i > 16384 ? 2000 : 100);
    }
    if (!seen) {
      s_ok2 = 0;
      atomicCAS(&g_peer_status, 0, (4 << 8) | 2);
    }
  }
  __syncthreads();
  if (ok && s_ok2 != 0) {
    const uint4* src = static_cast<const uint4*>(p.gather[p.rank]);
    uint4* dst = static_cast<uint4*>(p.out);
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {   // four loads in flight per thread; written by the peers: read past this SM's L1
      const uint4 a = __ldcg(src + i), b = __ldcg(src + i + stride), c = __ldcg(src + i + 2 * stride), d = __ldcg(src + i + 3 * stride);
      dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
    }
    for (; i < nvec; i += stride) dst[i] = __ldcg(src + i);
  }
  finish(p, epoch);
}

// ---- all-reduce with the flag inside every word ("low latency" protocol) --------------------------------------
// No flag rounds and no fences: a 32-bit data word travels as one 64-bit store {data, epoch}, which is single-copy
// atomic, so a receiver that reads the epoch of this call in the upper half holds valid data in the lower half.
//   A. every rank pushes slice j of its own buffer into rank j's reduce-scatter area [parity][sender];
//   B. rank r adds slice r of all ranks in rank order (its own from local memory, the others as they arrive),
//      writes the result to its output and pushes it into every rank's all-gather area [parity][owner];
//   C. every rank copies the other owners' slices from its all-gather area to its output as they arrive.
// Twice the bytes of the two-step form on the wire, about half its latency for the messages of a decode step.
// The areas alternate with the parity of the epoch: a sender can reach call k + 2 only after this rank has taken
// part in call k + 1, i.e. after it has read everything of call k. Stale words carry an older epoch and never match.
__device__ __forceinline__ void st_word_sys(unsigned long long* p, uint32_t data, uint32_t epoch) {
  const unsigned long long v = (static_cast<unsigned long long>(epoch) << 32) | data;
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Bounded wait for a flagged word; on time-out records the status and returns 0 with *ok cleared.
__device__ __forceinline__ uint32_t wait_word_sys(const unsigned long long* p, uint32_t epoch, uint32_t limit, bool* ok) {
  for (uint32_t i = 0; i < limit; ++i) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    if (static_cast<uint32_t>(v >> 32) == epoch) return static_cast<uint32_t>(v);
    if (i > 1024) __nanosleep(i > 16384 ? 2000 : 100);
  }
  *ok = false;
  atomicCAS(&g_peer_status, 0, (4 << 8) | 3);
  return 0u;
}
template <typename T>
__device__ __forceinline__ void add_word(uint32_t w, float (&acc)[2]);
template <>
__device__ __forceinline__ void add_word<float>(uint32_t w, float (&acc)[2]) { acc[0] += __uint_as_float(w); }
template <>
__device__ __forceinline__ void add_word<__half>(uint32_t w, float (&acc)[2]) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
  acc[0] += f.x; acc[1] += f.y;
}
template <>
__device__ __forceinline__ void add_word<__nv_bfloat16>(uint32_t w, float (&acc)[2]) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  acc[0] += f.x; acc[1] += f.y;
}
template <typename T>
__device__ __forceinline__ uint32_t pack_word(const float (&acc)[2]);
template <>
__device__ __forceinline__ uint32_t pack_word<float>(const float (&acc)[2]) { return __float_as_uint(acc[0]); }
template <>
__device__ __forceinline__ uint32_t pack_word<__half>(const float (&acc)[2]) {
  const __half2 h = __floats2half2_rn(acc[0], acc[1]);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack_word<__nv_bfloat16>(const float (&acc)[2]) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(acc[0], acc[1]);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// count * sizeof(T) is a multiple of 4 * world; every CTA of the grid is resident (at most one per SM).
template <typename T>
__global__ void __launch_bounds__(256) all_reduce_ll_kernel(const PeerParams p) {
  const int epoch_i = p.state[0] + 1;
  const uint32_t epoch = static_cast<uint32_t>(epoch_i);
  __shared__ int s_lost;
  if (threadIdx.x == 0) s_lost = peer_already_lost() ? 1 : 0;     // one reader: the whole CTA takes the same branch
  __syncthreads();
  if (s_lost == 0) {
    const uint32_t limit = poll_limit(p);
    const size_t words = p.count * sizeof(T) / 4;
    const size_t wps = words / p.world;                            // words per slice
    const size_t area = (static_cast<size_t>(epoch & 1u) * p.world) * wps;      // this call's parity half of an area
    const uint32_t* local = static_cast<const uint32_t*>(p.data[p.rank]);
    uint32_t* out = static_cast<uint32_t*>(p.out);
    const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
    bool ok = true;
    // A: my contribution to every other owner's slice
    for (int d = 1; d < p.world; ++d) {
      const int j = (p.rank + d) % p.world;                        // (each rank starts with a different peer)
      unsigned long long* dst = p.ll_rs[j] + area + static_cast<size_t>(p.rank) * wps;
      const uint32_t* src = local + static_cast<size_t>(j) * wps;
      for (size_t o = tid; o < wps; o += nthreads) st_word_sys(dst + o, src[o], epoch);
    }
    // B: my slice, summed in rank order, to my output and to everybody's all-gather area
    const unsigned long long* rs = p.ll_rs[p.rank] + area;
    for (size_t o = tid; o < wps; o += nthreads) {
      float acc[2] = {0.f, 0.f};
      for (int r = 0; r < p.world; ++r) {
        const uint32_t w = r == p.rank ? local[static_cast<size_t>(p.rank) * wps + o]
                                       : wait_word_sys(rs + static_cast<size_t>(r) * wps + o, epoch, limit, &ok);
        add_word<T>(w, acc);
      }
      const uint32_t res = pack_word<T>(acc);
      out[static_cast<size_t>(p.rank) * wps + o] = res;
      for (int d = 1; d < p.world; ++d) {
        const int j = (p.rank + d) % p.world;
        st_word_sys(p.ll_ag[j] + area + static_cast<size_t>(p.rank) * wps + o, res, epoch);
      }
    }
    // C: the other owners' slices
    const unsigned long long* ag = p.ll_ag[p.rank] + area;
    for (int d = 1; d < p.world && ok; ++d) {
      const int j = (p.rank + d) % p.world;
      for (size_t o = tid; o < wps && ok; o += nthreads)
        out[static_cast<size_t>(j) * wps + o] = wait_word_sys(ag + static_cast<size_t>(j) * wps + o, epoch, limit, &ok);
    }
  }
  finish(p, epoch_i);
}

// out[rows, world*count]: rank r's [rows, count] slice lands in columns [r*count, (r+1)*count)
template <typename T>
__global__ void __launch_bounds__(256) all_gather_kernel(const PeerParams p) {
  const int epoch = p.state[0] + 1;
  if (announce_and_wait(p, epoch)) {
    constexpr int VEC = 16 / sizeof(T);
    const size_t vec_per_row = p.count / VEC;
    const size_t total = static_cast<size_t>(p.world) * p.rows * vec_per_row;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
      const size_t c = i % vec_per_row;
      const size_t row = (i / vec_per_row) % p.rows;
      const int r = static_cast<int>(i / (vec_per_row * p.rows));
      const uint4 v = reinterpret_cast<const uint4*>(p.data[r])[row * vec_per_row + c];
      reinterpret_cast<uint4*>(p.out)[(row * p.world + r) * vec_per_row + c] = v;
    }
  }
  finish(p, epoch);
}

int fill(PeerParams& p, void* const* data, void* const* flags, void* out, int rank, int world, int* state) {
  if (!data || !flags || !out || !state || world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return CACHEIR_B200_EINVAL;
  for (int r = 0; r < world; ++r) {
    if (!data[r] || !flags[r] || !aligned_to(data[r], 16)) return CACHEIR_B200_EINVAL;
    p.data[r] = data[r];
    p.flags[r] = static_cast<int*>(flags[r]);
  }
  if (!aligned_to(out, 16)) return CACHEIR_B200_EALIGN;
  p.out = out; p.rank = rank; p.world = world; p.state = state;
  return 0;
}

}  // namespace
}  // namespace cb200

using namespace cb200;

extern "C" int cacheir_b200_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  if (!ptr || !handle64 || bytes == 0) return CACHEIR_B200_EINVAL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are exchanged as 64-byte blobs");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); return static_cast<int>(e); }
  memcpy(handle64, &h, 64);
  *ptr = p;
  return 0;
}

extern "C" int cacheir_b200_peer_open(const unsigned char* handle64, void** ptr) {
  if (!handle64 || !ptr) return CACHEIR_B200_EINVAL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}

extern "C" int cacheir_b200_peer_close(void* ptr) { return ptr ? static_cast<int>(cudaIpcCloseMemHandle(ptr)) : 0; }
extern "C" int cacheir_b200_peer_free(void* ptr) { return ptr ? static_cast<int>(cudaFree(ptr)) : 0; }

extern "C" int cacheir_b200_peer_all_reduce(void* const* data, void* const* flags, void* out, size_t count, int dtype,
                                            int rank, int world, int* state, void* stream) {
  if (count == 0) return 0;
  PeerParams p{};
  const int rc = fill(p, data, flags, out, rank, world, state);
  if (rc != 0) return rc;
  const int esize = dtype_size(dtype);
  if (esize == 0) return CACHEIR_B200_EINVAL;
  if ((count * esize) % 16 != 0) return CACHEIR_B200_EALIGN;
  p.count = count;
  const size_t nvec = count * esize / 16;
  const unsigned grid = static_cast<unsigned>(nvec / 256 < 1 ? 1 : (nvec / 256 > kNumSMs ? kNumSMs : nvec / 256));
  cudaStream_t st = as_stream(stream);
  switch (dtype) {
    case CACHEIR_B200_F32: all_reduce_kernel<float><<<grid, 256, 0, st>>>(p); break;
    case CACHEIR_B200_F16: all_reduce_kernel<__half><<<grid, 256, 0, st>>>(p); break;
    default: all_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p); break;
  }
  return launch_status();
}

extern "C" int cacheir_b200_peer_all_reduce_two_step(void* const* data, void* const* gather, void* const* flags, void* out,
                                                     size_t count, int dtype, int rank, int world, int* state, void* stream) {
  if (count == 0) return 0;
  PeerParams p{};
  const int rc = fill(p, data, flags, out, rank, world, state);
  if (rc != 0) return rc;
  if (!gather) return CACHEIR_B200_EINVAL;
  for (int r = 0; r < world; ++r) {
    if (!gather[r] || !aligned_to(gather[r], 16)) return CACHEIR_B200_EINVAL;
    p.gather[r] = gather[r];
  }
  const int esize = dtype_size(dtype);
  if (esize == 0) return CACHEIR_B200_EINVAL;
  if ((count * esize) % (16 * static_cast<size_t>(world)) != 0) return CACHEIR_B200_EALIGN;
  p.count = count;
  const size_t nvec = count * esize / 16;          // the copy to `out` covers the whole message: size the grid for it
  const unsigned grid = static_cast<unsigned>(nvec / 1024 < 1 ? 1 : (nvec / 1024 > kNumSMs ? kNumSMs : nvec / 1024));
  cudaStream_t st = as_stream(stream);
  switch (dtype) {
    case CACHEIR_B200_F32: all_reduce_two_step_kernel<float><<<grid, 256, 0, st>>>(p); break;
    case CACHEIR_B200_F16: all_reduce_two_step_kernel<__half><<<grid, 256, 0, st>>>(p); break;
    default: all_reduce_two_step_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p); break;
  }
  return launch_status();
}

extern "C" int cacheir_b200_peer_all_reduce_ll(const void* local_data, void* const* ll_rs, void* const* ll_ag, void* out,
                                               size_t count, int dtype, int rank, int world, int* state, void* stream) {
  if (count == 0) return 0;
  if (!local_data || !ll_rs || !ll_ag || !out || !state || world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return CACHEIR_B200_EINVAL;
  PeerParams p{};
  for (int r = 0; r < world; ++r) {
    if (!ll_rs[r] || !ll_ag[r] || !aligned_to(ll_rs[r], 8) || !aligned_to(ll_ag[r], 8)) return CACHEIR_B200_EINVAL;
    p.ll_rs[r] = static_cast<unsigned long long*>(ll_rs[r]);
    p.ll_ag[r] = static_cast<unsigned long long*>(ll_ag[r]);
  }
  if (!aligned_to(local_data, 4) || !aligned_to(out, 4)) return CACHEIR_B200_EALIGN;
  p.data[rank] = local_data;
  p.out = out; p.rank = rank; p.world = world; p.state = state;
  const int esize = dtype_size(dtype);
  if (esize == 0) return CACHEIR_B200_EINVAL;
  if ((count * esize) % (4 * static_cast<size_t>(world)) != 0) return CACHEIR_B200_EALIGN;
  p.count = count;
  const size_t words = count * esize / 4;
  const unsigned grid = static_cast<unsigned>(words / 1024 < 1 ? 1 : (words / 1024 > kNumSMs ? kNumSMs : words / 1024));
  cudaStream_t st = as_stream(stream);
  switch (dtype) {
    case CACHEIR_B200_F32: all_reduce_ll_kernel<float><<<grid, 256, 0, st>>>(p); break;
    case CACHEIR_B200_F16: all_reduce_ll_kernel<__half><<<grid, 256, 0, st>>>(p); break;
    default: all_reduce_ll_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p); break;
  }
  return launch_status();
}

extern "C" int cacheir_b200_peer_all_gather(void* const* data, void* const* flags, void* out, int rows, size_t cols, int dtype,
                                            int rank, int world, int* state, void* stream) {
  if (rows <= 0 || cols == 0) return 0;
  PeerParams p{};
  const int rc = fill(p, data, flags, out, rank, world, state);
  if (rc != 0) return rc;
  const int esize = dtype_size(dtype);
  if (esize == 0) return CACHEIR_B200_EINVAL;
  if ((cols * esize) % 16 != 0) return CACHEIR_B200_EALIGN;
  p.count = cols; p.rows = rows;
  const size_t nvec = static_cast<size_t>(world) * rows * cols * esize / 16;
  const unsigned grid = static_cast<unsigned>(nvec / 256 < 1 ? 1 : (nvec / 256 > kNumSMs ? kNumSMs : nvec / 256));
  cudaStream_t st = as_stream(stream);
  switch (dtype) {
    case CACHEIR_B200_F32: all_gather_kernel<float><<<grid, 256, 0, st>>>(p); break;
    case CACHEIR_B200_F16: all_gather_kernel<__half><<<grid, 256, 0, st>>>(p); break;
    default: all_gather_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p); break;
  }
  return launch_status();
}

namespace cb200 {
int peer_collectives_device_status(bool reset);
}
int cb200::peer_collectives_device_status(bool reset) {
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_peer_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int));
  }
  return status;
}
