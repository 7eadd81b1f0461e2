/*
 * cacheir_b200.h -- C ABI of libcacheir_b200.so: the batched decode step of
 * CacheIR (paged decode attention + packed int4/int8 dequant-GEMV and the
 * glue ops between them) as hand-written CUDA for sm_100a.
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer owned
 *     by the caller for the duration of the launch, `stream` is a
 *     cudaStream_t passed as void*;
 *   - nothing here allocates, frees or synchronises, except where an entry point's
 *     comment says so (cacheir_b200_peer_alloc / _free, cacheir_b200_device_status);
 *   - return value: 0 on success, a positive cudaError_t value when the CUDA
 *     runtime reported one, or a negative CACHEIR_B200_E* validation code.
 *     Non-positive extents return 0 without launching, exactly like the
 *     reference launchers (cpp/src/cacheir_cuda_kernels.cu:370-372);
 *   - `dtype` arguments use the CACHEIR_B200_F32/F16/BF16 codes below.
 *
 * Each declaration cites the interface of the reference project
 * (AhanBhatt/CacheIR, paths relative to its root) that it stands in for.
 */
#ifndef CACHEIR_B200_H_
#define CACHEIR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define CACHEIR_B200_F32 0
#define CACHEIR_B200_F16 1
#define CACHEIR_B200_BF16 2

/* validation errors (negative so they never collide with cudaError_t) */
#define CACHEIR_B200_EINVAL (-1)      /* bad extent, dtype or flag            */
#define CACHEIR_B200_EALIGN (-2)      /* pointer/stride alignment unusable    */
#define CACHEIR_B200_EWORKSPACE (-3)  /* workspace missing or too small       */
#define CACHEIR_B200_EUNSUPPORTED (-4)/* shape outside what the kernels cover */
#define CACHEIR_B200_ELIMIT (-5)      /* beyond a documented fixed maximum    */

/* `weight_layout` flags of cacheir_b200_qgemv_ex (may be OR-ed) */
#define CACHEIR_B200_LAYOUT_ROWS 0     /* the reference's row-major packed_values   */
#define CACHEIR_B200_LAYOUT_TILED 1    /* cacheir_b200_pack_relayout's tile order   */
#define CACHEIR_B200_X_PREQUANTIZED 2  /* workspace already holds x in integer form */
#define CACHEIR_B200_LAYOUT_PAIRED 4   /* tiled with `paired` != 0 (SwiGLU weights only)  */

/* qgemv epilogues */
#define CACHEIR_B200_EPI_NONE 0       /* y = x W^T                            */
#define CACHEIR_B200_EPI_RESIDUAL 1   /* y = residual + x W^T                 */
#define CACHEIR_B200_EPI_SWIGLU 2     /* W = [gate; up], y = silu(xWg^T)*xWu^T */

/* Library/ABI version (major*100 + minor) and a human readable build line. */
int cacheir_b200_version(void);
const char* cacheir_b200_build_info(void);
/* Text for any return code of this library (never NULL). */
const char* cacheir_b200_error_string(int code);

/* ------------------------------------------------------------------------
 * Paged decode attention over a shared page pool.
 *
 * Replaces: Triton `paged_attention_decode_batch_kernel`
 *   (cacheir/backends/triton_kernels.py:174-217, launched from
 *   cacheir/runtime/cuda.py:1238-1251 and :1166-1179) and its CUDA twin
 *   `cacheir_cuda_paged_attention_decode_batch`
 *   (cpp/src/cacheir_cuda_kernels.cu:357-411). Same argument order and
 *   meaning; the additions are dtype, q/out row strides, softmax_scale,
 *   and the split-K workspace.
 *
 *   out[b,h,:] = sum_t softmax_t(scale * q[b,h,:].K[b,t,kvh(h),:]) V[b,t,kvh(h),:]
 *   for t < seq_lens[b], kvh(h) = h / (num_heads/num_kv_heads); row t of
 *   sequence b lives at pool element
 *   ((page_table[b,t/page_size]*num_kv_heads + kvh)*page_size + t%page_size)*head_dim
 *   (triton_kernels.py:206). Page-table entries may alias between sequences
 *   (prefix-shared pages); entries past ceil(seq_len/page_size) are never read.
 *   A sequence with seq_lens[b] <= 0 produces zeros.
 *
 *   q, out:      [batch, num_heads, head_dim], row b at q + b*q_batch_stride
 *                elements (0 = dense, i.e. num_heads*head_dim)
 *   k/v_cache:   [slots, num_kv_heads, page_size, head_dim], same dtype as q
 *   page_table:  int32 [batch, max_pages_per_seq]; seq_lens: int32 [batch]
 *   softmax_scale: <= 0 selects rsqrt(head_dim) (the reference's constant)
 *   num_splits:  context splits per sequence (flash-decoding); 0 = choose.
 *                Partials are merged in split order, so the result is
 *                bit-identical from run to run for a given num_splits.
 *   workspace:   fp32 scratch of at least
 *                cacheir_b200_paged_attention_workspace_bytes(...) bytes;
 *                may be NULL only when that size is 0 (num_splits == 1).
 */
size_t cacheir_b200_paged_attention_workspace_bytes(int batch_size, int num_heads,
                                                    int head_dim, int num_splits);
/* The split count that num_splits == 0 resolves to for these extents. */
int cacheir_b200_paged_attention_auto_splits(int batch_size, int num_heads,
                                             int num_kv_heads, int max_pages_per_seq,
                                             int page_size, int head_dim);
int cacheir_b200_paged_attention_decode_batch(
    const void* q, const void* k_cache, const void* v_cache,
    const int32_t* page_table, const int32_t* seq_lens, void* out,
    int batch_size, int num_heads, int num_kv_heads, int max_pages_per_seq,
    int page_size, int head_dim, int dtype, long long q_batch_stride,
    long long out_batch_stride, float softmax_scale, int num_splits,
    void* workspace, size_t workspace_bytes, void* stream);

/* The same with two more inputs.
 *   num_slots: slots of the pool (k_cache.shape[0]); 0 = unknown. With it the tensor maps of the fast kernel carry
 *     the pool's true extent, so a page id outside the pool reads zeros instead of memory past the pool.
 *   kv_dtype / kv_scales: CACHEIR_B200_KV_INT8 selects pools of unsigned bytes, half the bytes of an fp16 pool:
 *     value = (byte - 128) * kv_scales[slot][kv_head][0 (K) | 1 (V)][token % page_size], fp16 scales, one per cached
 *     row, written by cacheir_b200_kv_append_q8. q and out keep `dtype`. CACHEIR_B200_KV_SAME: pools of `dtype`.
 * The reference only models the byte cost of a smaller cache (cacheir/runtime/kv_cache.py:138-259); its kernels
 * read pools of the activation type. */
#define CACHEIR_B200_KV_SAME 0
#define CACHEIR_B200_KV_INT8 1
int cacheir_b200_paged_attention_decode_batch_ex(
    const void* q, const void* k_cache, const void* v_cache,
    const int32_t* page_table, const int32_t* seq_lens, void* out,
    int batch_size, int num_heads, int num_kv_heads, int max_pages_per_seq,
    int page_size, int head_dim, int dtype, long long q_batch_stride,
    long long out_batch_stride, float softmax_scale, int num_splits,
    void* workspace, size_t workspace_bytes, int num_slots, int kv_dtype,
    const void* kv_scales, void* stream);

/* Decode attention that also hands its output to the projection behind it: besides `out` ([batch][num_heads*head_dim],
 * dense rows) the launch fills `gemm_workspace` with what cacheir_b200_quantize_activations would make of `out`
 * (fixed-point byte planes, scale and sum per row, bit for bit), so that cacheir_b200_qgemv_ex can follow with
 * CACHEIR_B200_X_PREQUANTIZED and no pre-pass launch of its own. One split; the kv heads of a sequence run as one
 * thread-block cluster and exchange the row maximum and sum through distributed shared memory.
 * Needs: fp16 q/out and fp16 pools, head_dim 128, pages of 16, at most 8 kv heads, num_heads / num_kv_heads <= 5,
 * batch_size <= 64, gemm_workspace of cacheir_b200_qgemv_workspace_bytes(batch_size, num_heads*head_dim) bytes,
 * 128-byte aligned; CACHEIR_B200_EUNSUPPORTED otherwise (cacheir_b200_paged_attention_quantize_supported tells
 * beforehand: 1 or 0). In the reference the two steps are separate ops of the decode graph
 * (cacheir/runtime/cuda.py:1238-1251 the attention launch, :932-954 the quantized matmul). */
int cacheir_b200_paged_attention_decode_batch_quantize(
    const void* q, const void* k_cache, const void* v_cache,
    const int32_t* page_table, const int32_t* seq_lens, void* out,
    int batch_size, int num_heads, int num_kv_heads, int max_pages_per_seq,
    int page_size, int head_dim, int dtype, long long q_batch_stride,
    float softmax_scale, int num_slots, void* gemm_workspace,
    size_t gemm_workspace_bytes, void* stream);
int cacheir_b200_paged_attention_quantize_supported(int batch_size, int num_heads, int num_kv_heads,
                                                    int max_pages_per_seq, int page_size, int head_dim, int dtype);

/* Allocation-free variant of cacheir_b200_paged_attention_decode_batch. It has no
 * counterpart in the reference; it exists for callers that have inputs and outputs
 * but no way to get scratch memory on the device: code bound to the reference's own
 * launcher signature (cpp/src/cacheir_cuda_kernels.cu:357-369 carries no workspace
 * argument), plug-ins of a serving process that handed all of HBM to its weight and
 * KV arenas at start-up, and hosts that run under a fixed device-memory budget and
 * treat any later cudaMalloc as an error. Same arguments and results as the entry
 * point above, minus the workspace: the split-K partials go to a 16 MiB array that is
 * part of the library image (every GPU that loads the library holds those 16 MiB
 * until the process exits). The call performs no cudaMalloc/cudaFree and calls no
 * allocating routine.
 *   - Limit: extents whose partials need more than
 *     cacheir_b200_paged_attention_noalloc_max_workspace_bytes() return
 *     CACHEIR_B200_ELIMIT and launch nothing; pass a smaller num_splits (1 needs no
 *     scratch at all) or use the workspace entry point.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call before
 *     any stream capture begins.
 *   - All calls share the one array. It keeps whatever the previous call left in it;
 *     nothing in it has to start at zero, because every partial that the combine step
 *     reads is written earlier in the same call. Two calls that overlap on the GPU
 *     (different streams, or different threads without ordering) race on it: issue
 *     them on one stream or order them with events. */
size_t cacheir_b200_paged_attention_noalloc_max_workspace_bytes(void);
int cacheir_b200_paged_attention_decode_batch_noalloc(
    const void* q, const void* k_cache, const void* v_cache,
    const int32_t* page_table, const int32_t* seq_lens, void* out,
    int batch_size, int num_heads, int num_kv_heads, int max_pages_per_seq,
    int page_size, int head_dim, int dtype, long long q_batch_stride,
    long long out_batch_stride, float softmax_scale, int num_splits, void* stream);

/* ------------------------------------------------------------------------
 * Packed int4/int8 dequant-GEMV / small-M GEMM:  y[M,N] = x[M,K] . deq(W)[N,K]^T
 *
 * Replaces: `CudaRuntime._quantized_matmul` + `_dequantize_cuda_weight`
 *   (cacheir/runtime/cuda.py:932-954; CPU twin cacheir/runtime/cpu.py:306-312),
 *   which materialise the dense weight on every call, and the fused ops built
 *   on it (cuda.py:812-820 QKV, :867-871 SwiGLU, :795-796 O/Down/lm_head).
 *   Pack format is the reference's (cacheir/quantization.py:96-139):
 *     bits 8: packed[n,k] = code;  bits 4: packed[n,j] = code[2j] | code[2j+1]<<4
 *     (row stride ceil(K/2) bytes, odd K zero padded);
 *     per-row affine (group_size 0): w = (code - zero_points[n]) * scales[n];
 *     zero_points are fp32 as uploaded by CudaWeightStore (cuda.py:83), NULL
 *     means the midpoint 2^(bits-1);
 *     group-wise symmetric (group_size > 0, a multiple of 32 dividing K):
 *     w = (code - 2^(bits-1)) * scales[n, k/group_size], zero_points NULL.
 *   bits 0 selects dense weights W[N,K] of x's dtype (`_matmul`, cuda.py:920-930).
 *
 *   x: [M,K] row stride x_stride elements (0 = K); y: [M,N_out] dense,
 *   N_out = N, or N/2 for EPI_SWIGLU where rows [0,N/2) are gate and
 *   [N/2,N) are up; residual: [M,N_out] dense, EPI_RESIDUAL only.
 *   x, y and residual share x_dtype; scales are fp32 or fp16 (scale_dtype).
 */
int cacheir_b200_qgemv(const void* x, const void* packed, const void* scales,
                       const float* zero_points, const void* residual, void* y,
                       int M, int N, int K, int bits, int group_size,
                       int x_dtype, int scale_dtype, long long x_stride,
                       int epilogue, void* stream);

/* Same operation with caller-provided scratch. With at least
 * cacheir_b200_qgemv_workspace_bytes(M, K) bytes of 128-byte aligned workspace, int8 and
 * int4 per-row weights with fp16 activations (K % 128 == 0, K <= 32768) run on the integer
 * tensor cores: the uint8 codes are fed to the MMA as they are (int4 nibbles are widened to
 * bytes in shared memory), and x is first turned into 16-bit fixed point per row (two
 * signed bytes, 2^-15 of the row maximum) in the workspace by a pre-pass kernel. Batches above 64 rows run as
 * 64-row chunks (128-row chunks on the fp16 tensor-core kernel, which takes 65..128 rows in
 * one launch with the activations as the 128-row operand). Other shapes ignore the
 * workspace. workspace may be NULL (then this is cacheir_b200_qgemv). The workspace is only used during the call's own kernels; two
 * calls that may overlap on the GPU need separate workspaces. */
size_t cacheir_b200_qgemv_workspace_bytes(int M, int K);
int cacheir_b200_qgemv_ex(const void* x, const void* packed, const void* scales,
                          const float* zero_points, const void* residual, void* y,
                          int M, int N, int K, int bits, int group_size,
                          int x_dtype, int scale_dtype, long long x_stride,
                          int epilogue, int weight_layout, void* workspace,
                          size_t workspace_bytes, void* stream);

/* RMSNorm in front of the projection: y = epilogue(rmsnorm(x; norm_weight, eps) . deq(W)^T), fp16 activations
 * with dense rows, K <= 8192, int8 / int4 per-row weights on the integer tensor-core path only (the conditions of
 * cacheir_b200_qgemv_ex with a workspace; otherwise CACHEIR_B200_EUNSUPPORTED: run cacheir_b200_rms_norm first).
 *
 * Replaces: `_rms_norm` (cacheir/runtime/cuda.py:889-895) followed by `_quantized_matmul` (:932-940) /
 *   the quantized fused SwiGLU (:867-871), i.e. the body of the reference's fused_rmsnorm_* ops.
 * Two launches: cacheir_b200_rms_norm_quantize into the workspace, then the GEMM on the quantized rows; the same
 * results as those two calls, bit for bit. */
int cacheir_b200_rmsnorm_qgemv(const void* x, const void* norm_weight, float eps, const void* packed,
                               const void* scales, const float* zero_points, const void* residual,
                               void* y, int M, int N, int K, int bits, int scale_dtype,
                               long long x_stride, int epilogue, int weight_layout, void* workspace,
                               size_t workspace_bytes, void* stream);

/* Which kernel cacheir_b200_qgemv_ex would launch for these extents and flags (fp16 activations, aligned
 * pointers): (family << 8) | detail, family 1 = integer tensor core with detail = its split-K factor,
 * 2 = fp16 tensor core, 3 = CUDA cores, 4 = streaming int4 GEMV (up to 8 rows); epilogue 3 asks about
 * cacheir_b200_qkv_rope_append. Negative:
 * the validation code the call would return. Launches nothing. No counterpart in the reference (its
 * kernel choice is the declarative `attrs["kernel"]`, cacheir/passes/transformer.py:391-424). */
int cacheir_b200_qgemv_plan(int M, int N, int K, int bits, int group_size, int epilogue,
                            int weight_layout, int with_workspace);

/* The fused QKV projection of a decode step on int8 weights (fp16 activations, M <= 64):
 * qkv[M, N] = x W^T with W = [Wq; Wk; Wv] (N = q_dim + 2*k_dim), then, in the same kernel,
 * interleaved-pair RoPE on the q and k heads at positions[m] and the new k / v rows written
 * into the page pool at (page_table[m][pos / page_size], kv head, pos % page_size).
 *
 * Replaces: the matmul of `fused_rmsnorm_qkv_rope` / `quantized_matmul`
 *   (cacheir/runtime/cuda.py:932-954), `_rope_with_offsets` (:1072-1102) and the cache
 *   append that opens `_try_triton_decode_attention_batch` (:1183-1229) for the batched
 *   decode step; results are bit-identical to cacheir_b200_qgemv_ex followed by
 *   cacheir_b200_rope_inplace and cacheir_b200_kv_append.
 * `rope_table` holds (cos, sin) float pairs [rope_table_positions][head_dim/2] written by
 * cacheir_b200_rope_table and must cover every position in use: a position outside it is
 * left unrotated and recorded in cacheir_b200_device_status.
 * `weight_layout`: CACHEIR_B200_LAYOUT_TILED and/or CACHEIR_B200_X_PREQUANTIZED. Needs the
 * workspace of cacheir_b200_qgemv_workspace_bytes(M, K). Returns CACHEIR_B200_EUNSUPPORTED
 * for shapes outside the integer tensor-core kernel (call the three separate entry points). */
int cacheir_b200_qkv_rope_append(const void* x, const void* packed, const void* scales,
                                 const float* zero_points, void* qkv, int M, int N, int K,
                                 int scale_dtype, long long x_stride, int weight_layout, int q_dim,
                                 int k_dim, int head_dim, float theta, const float* rope_table,
                                 int rope_table_positions, const int32_t* positions,
                                 const int32_t* page_table, int max_pages_per_seq, int page_size,
                                 void* k_cache, void* v_cache, void* workspace,
                                 size_t workspace_bytes, void* stream);
/* The same with the RMSNorm of the reference's `quantized_fused_rmsnorm_qkv_rope` op
 * (cacheir/runtime/cuda.py:812-820) in front, as in cacheir_b200_rmsnorm_qgemv (norm + pre-pass kernel, then this kernel). */
int cacheir_b200_rmsnorm_qkv_rope_append(const void* x, const void* norm_weight, float eps,
                                         const void* packed, const void* scales,
                                         const float* zero_points, void* qkv, int M, int N, int K,
                                         int scale_dtype, long long x_stride, int weight_layout,
                                         int q_dim, int k_dim, int head_dim, float theta,
                                         const float* rope_table, int rope_table_positions,
                                         const int32_t* positions, const int32_t* page_table,
                                         int max_pages_per_seq, int page_size, void* k_cache,
                                         void* v_cache, void* workspace, size_t workspace_bytes,
                                         void* stream);
/* table[pos][i] = (cos, sin)(pos * theta^(-2i/head_dim)) in fp32 for pos < positions, the
 * values cacheir_b200_rope_inplace evaluates on the fly. 8 * positions * head_dim/2 bytes. */
int cacheir_b200_rope_table(float* table, int positions, int head_dim, float theta, void* stream);

/* The activation pre-pass of the integer tensor-core path on its own, and fused with RMSNorm
 * (`_rms_norm`, cacheir/runtime/cuda.py:889-895, followed by `_quantized_matmul`, :932-940):
 * both leave x as 16-bit fixed point per row in `workspace` (>= cacheir_b200_qgemv_workspace_bytes
 * bytes, 128-byte aligned, fp16 only, rows <= 64, width a multiple of 128). A following
 * cacheir_b200_qgemv_ex with the same M, K and workspace and CACHEIR_B200_X_PREQUANTIZED set skips
 * its own pre-pass (x is then not read). rms_norm_quantize normalises x (+ residual, the rounded
 * sum going to sum_out) exactly like cacheir_b200_rms_norm, rounds to fp16, optionally stores the
 * fp16 row to `out` (may be NULL) and quantises it; width <= 8192. */
int cacheir_b200_quantize_activations(const void* x, int M, int K, long long x_stride, int x_dtype,
                                      void* workspace, size_t workspace_bytes, void* stream);
int cacheir_b200_rms_norm_quantize(const void* x, const void* residual, const void* weight,
                                   void* sum_out, void* out, int rows, int hidden, float eps,
                                   int dtype, void* workspace, size_t workspace_bytes, void* stream);

/* Device pack layout of the quantization loader. The codes of the reference format
 * (`packed_values`, cacheir/quantization.py:107-120; uploaded row-major by
 * CudaWeightStore.get_quantized, cacheir/runtime/cuda.py:77-94) are permuted into
 * tiles of 128 rows x 128 k elements stored contiguously (16 KB for int8, 8 KB for int4),
 * the tiles of one 128-row band following each other along K, so that a tensor-core CTA
 * streams one contiguous span of HBM instead of 128 strided 128-byte pieces per step.
 * Pure byte permutation (rows past N are zero padding): `unrelayout` restores the
 * reference bytes exactly. K must be a multiple of 128; `tiled` holds
 * cacheir_b200_pack_tiled_bytes(N, K, bits) bytes. Scales and zero points are not
 * touched. Pass CACHEIR_B200_LAYOUT_TILED to cacheir_b200_qgemv_ex for such weights
 * (tensor-core shapes only: fp16 x, M <= 64).
 * `paired` != 0 (N a multiple of 128) is the form for W = [gate; up] used with
 * CACHEIR_B200_EPI_SWIGLU on int8 weights: tile t holds gate rows 64t..64t+63 followed by
 * up rows N/2+64t..N/2+64t+63, so one CTA owns both factors of 64 output columns. Pass
 * CACHEIR_B200_LAYOUT_TILED | CACHEIR_B200_LAYOUT_PAIRED for such weights. */
size_t cacheir_b200_pack_tiled_bytes(int N, int K, int bits);
int cacheir_b200_pack_relayout(const uint8_t* packed, uint8_t* tiled, int N, int K, int bits, int paired, void* stream);
int cacheir_b200_pack_unrelayout(const uint8_t* tiled, uint8_t* packed, int N, int K, int bits, int paired, void* stream);

/* ------------------------------------------------------------------------
 * Collectives of the tensor-parallel decode step over NVLink peer memory (one process per
 * GPU, up to 8 ranks). No reference counterpart: the reference runs on one device.
 *
 * peer_alloc: device memory (zero-filled) that other processes can map; `handle64` receives
 * the 64-byte CUDA IPC handle to send them. peer_open maps a peer's allocation from its
 * handle; peer_close / peer_free undo the two. Each rank needs data buffers and one flag
 * array of 16 ints, all from peer_alloc, and a local `state` of 4 zero ints.
 *
 * peer_all_reduce: out[i] = sum over ranks r = 0..world-1 (in that order, fp32 accumulation,
 * so every rank gets the same bits) of data[r][i]. peer_all_gather: out[rows, world*cols]
 * with rank r's [rows, cols] slice in columns [r*cols, (r+1)*cols). `data` and `flags` are
 * host arrays of `world` device pointers (entry [rank] = the local buffers). One kernel per
 * rank; it announces itself to the peers, waits (bounded; a peer that never arrives is
 * recorded in cacheir_b200_device_status and the output is then undefined) and reads the
 * peers' buffers with plain loads. All ranks must issue the same sequence of calls, and a
 * data buffer may be refilled only after a later call that used a different buffer (alternate
 * between two). Safe to capture in a CUDA graph: the call counter lives in `state`.
 *
 * peer_all_reduce_two_step: the same result for large messages (count * element size a
 * multiple of 16 * world) in two steps inside one launch: rank r adds slice r of every
 * rank's buffer and pushes it into every rank's `gather` buffer (another peer_alloc buffer of
 * the message size, `gather[r]` = rank r's), then every rank copies its gather buffer to
 * `out`. Each rank moves 2 (world-1)/world of the message over NVLink instead of world-1
 * messages. The kernel must own the GPU while it runs (its CTAs wait for one another).
 * peer_all_reduce_ll: the same result again with the flag inside every word (count * element size a multiple of
 * 4 * world): each 32-bit word travels as one 64-bit store {word, epoch}; rank r receives slice r of every rank in
 * its `ll_rs` area, adds in rank order, and pushes the sum into every rank's `ll_ag` area; no flag rounds, no fences,
 * twice the bytes on the wire: the fastest form for the messages of a decode step. `ll_rs[r]` / `ll_ag[r]` are rank
 * r's areas (peer_alloc, zero-filled, 4 x the largest message each); `local_data` is this rank's own buffer and
 * needs no peer mapping. */
int cacheir_b200_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64);
int cacheir_b200_peer_open(const unsigned char* handle64, void** ptr);
int cacheir_b200_peer_close(void* ptr);
int cacheir_b200_peer_free(void* ptr);
int cacheir_b200_peer_all_reduce(void* const* data, void* const* flags, void* out, size_t count,
                                 int dtype, int rank, int world, int* state, void* stream);
int cacheir_b200_peer_all_reduce_two_step(void* const* data, void* const* gather, void* const* flags,
                                          void* out, size_t count, int dtype, int rank, int world,
                                          int* state, void* stream);
int cacheir_b200_peer_all_reduce_ll(const void* local_data, void* const* ll_rs, void* const* ll_ag, void* out,
                                    size_t count, int dtype, int rank, int world, int* state, void* stream);
int cacheir_b200_peer_all_gather(void* const* data, void* const* flags, void* out, int rows,
                                 size_t cols, int dtype, int rank, int world, int* state,
                                 void* stream);

/* Status word of the kernels that wait on hardware barriers (the tensor-core GEMM):
 * 0, or a non-zero code recorded by the first wait that ran out of its poll budget
 * (the kernel then drains and returns instead of hanging; its output is undefined).
 * Synchronises with the device. `reset` != 0 clears the word after reading it. */
int cacheir_b200_device_status(int reset);

/* ------------------------------------------------------------------------
 * Quantization loader on the device.
 *
 * Replaces: `_asymmetric_pack` / `_pack_int4` (cacheir/quantization.py:96-130)
 *   as called by `WeightStore._pack_value` (cacheir/runtime/cpu.py:47-58) and
 *   `dequantize_packed_weight` (quantization.py:74-84). Results are bit-exact
 *   with the NumPy code: scale = max((max-min)/qmax, 1e-8) in fp32,
 *   zero = rint(0 - min/scale) (not clipped), code = clip(rint((double)(w/scale)
 *   + zero), 0, qmax).
 *   weight: fp32 [N,K]; packed: uint8 [N,K] or [N,ceil(K/2)]; scales: fp32 [N];
 *   zero_points_i32: int32 [N] (may be NULL); zero_points_f32: fp32 [N] (may be
 *   NULL) -- the form the GEMV consumes.
 */
int cacheir_b200_pack_rows(const float* weight, uint8_t* packed, float* scales,
                           int32_t* zero_points_i32, float* zero_points_f32,
                           int N, int K, int bits, void* stream);
/* out[n,k] = (code - zero_points[n]) * scales[n]   (fp32 math, cast to out_dtype) */
int cacheir_b200_dequantize_rows(const uint8_t* packed, const float* scales,
                                 const float* zero_points, void* out, int N, int K,
                                 int bits, int out_dtype, void* stream);

/* ------------------------------------------------------------------------
 * Glue ops of the decode graph (one row per request).
 */

/* Replaces `cacheir_cuda_rms_norm` (cpp/src/cacheir_cuda_kernels.cu:273-284),
 * Triton `rms_norm_kernel` (triton_kernels.py:40-49), `_rms_norm`
 * (cuda.py:889-895): out = x * rsqrt(mean(x^2)+eps) * weight, statistics in
 * fp32. x/out/weight share `dtype`. When `residual` is non-NULL the row that
 * is normalised is x+residual and that sum is also stored to `sum_out`
 * (the graph's `add` node, cuda.py:851-852, fused with the following norm). */
int cacheir_b200_rms_norm(const void* x, const void* residual, const void* weight,
                          void* sum_out, void* out, int rows, int hidden, float eps,
                          int dtype, void* stream);

/* Replaces `_rope_with_offsets` / `_rope_offsets_one` (cuda.py:1072-1102; CPU
 * `_rope_one`, cpu.py:324-340): interleaved even/odd pair rotation in place,
 * angle = positions[b] * theta^(-2i/head_dim). x: [batch, num_heads, head_dim]
 * with row stride x_batch_stride elements (0 = dense). */
int cacheir_b200_rope_inplace(void* x, const int32_t* positions, int batch_size,
                              int num_heads, int head_dim, float theta, int dtype,
                              long long x_batch_stride, void* stream);

/* Replaces `TorchPagedKVCache.append` + `TorchKVPageAllocator.write_page`
 * (cuda.py:322-334, :172-199) for one new token per request: writes
 * k[b,kvh,:], v[b,kvh,:] to pool row
 * ((page_table[b,pos/page]*num_kv_heads + kvh)*page + pos%page) with
 * pos = positions[b]. No contiguous per-session copy is kept. */
int cacheir_b200_kv_append(const void* k, const void* v, void* k_cache, void* v_cache,
                           const int32_t* page_table, const int32_t* positions,
                           int batch_size, int num_kv_heads, int max_pages_per_seq,
                           int page_size, int head_dim, int dtype,
                           long long k_batch_stride, long long v_batch_stride,
                           void* stream);

/* `_rope_with_offsets` on the q and k heads of a fused row [q | k | v] (in place) and the append of the new k / v rows
 * (cacheir_b200_rope_inplace followed by cacheir_b200_kv_append, bit for bit) in one launch: qkv is
 * [batch][q_dim + 2*k_dim] with `qkv_batch_stride` elements between rows (0 = dense), pools of the same dtype. */
int cacheir_b200_rope_append(void* qkv, const int32_t* positions, const int32_t* page_table, void* k_cache,
                             void* v_cache, int batch_size, int q_dim, int k_dim, int head_dim, float theta,
                             int max_pages_per_seq, int page_size, int dtype, long long qkv_batch_stride,
                             void* stream);

/* The same into 8-bit pools (see cacheir_b200_paged_attention_decode_batch_ex): every new row is quantised with its
 * own scale, scale = fp16(max|row| / 127) (1 for an all-zero row), byte = clamp(rint(value / scale), -127, 127) + 128;
 * the scale goes to kv_scales[slot][kv_head][0 (K) | 1 (V)][pos % page_size] (fp16). head_dim <= 256.
 * No counterpart in the reference beyond the cost model of cacheir/runtime/kv_cache.py:138-259. */
int cacheir_b200_kv_append_q8(const void* k, const void* v, void* k_cache, void* v_cache, void* kv_scales,
                              const int32_t* page_table, const int32_t* positions, int batch_size,
                              int num_kv_heads, int max_pages_per_seq, int page_size, int head_dim,
                              int dtype, long long k_batch_stride, long long v_batch_stride,
                              void* stream);

/* Replaces `cacheir_cuda_fused_swiglu` (cacheir_cuda_kernels.cu:286-295),
 * Triton `silu_mul_kernel` (triton_kernels.py:51-59), `_silu_mul`
 * (cuda.py:1025-1030): out = gate/(1+exp(-gate)) * up. */
int cacheir_b200_silu_mul(const void* gate, const void* up, void* out, size_t total,
                          int dtype, void* stream);
/* The graph's `add` node (cuda.py:851-852). */
int cacheir_b200_add(const void* a, const void* b, void* out, size_t total, int dtype,
                     void* stream);
/* The graph's `token_embedding` node (cuda.py:789): out[r,:] = table[ids[r],:]. */
int cacheir_b200_embedding_gather(const void* table, const int64_t* ids, void* out,
                                  int rows, int hidden, int vocab, int dtype,
                                  void* stream);
/* Replaces `_argmax_tokens` (cacheir/runtime/scheduler.py:535-543) for
 * device-side greedy feedback: out_ids[r] = first index of the row maximum. */
int cacheir_b200_argmax_rows(const void* logits, int64_t* out_ids, int rows, int vocab,
                             int dtype, void* stream);
/* Per-step request bookkeeping kept on the device (no counterpart kernel in
 * the reference, which recomputes `_position_offset` on the host each step,
 * cuda.py:1064-1067): positions[b] = seq_lens[b]; seq_lens[b] += 1. */
int cacheir_b200_advance_positions(int32_t* positions, int32_t* seq_lens, int batch_size,
                                   void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CACHEIR_B200_H_ */
