// Arguments shared by the dequant-GEMV kernels and their launchers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace cb200 {

// Fused QKV epilogue: RoPE on the q and k heads, new k/v rows written into the page pool.
struct RopeAppendParams {
  const float* table;          // [table_positions][head_dim/2] (cos, sin) pairs, or null: evaluate on the fly
  int table_positions;
  const int32_t* positions;    // [M] position of the token of each batch row
  const int32_t* page_table;   // [M][max_pages]
  void* k_cache;               // [slots][kv_heads][page_size][head_dim], fp16
  void* v_cache;
  int q_dim, k_dim, head_dim, kv_heads, max_pages, page_size;
  float theta;
};
constexpr int kEpiQkvRopeAppend = 3;   // internal epilogue code (cacheir_b200_qkv_rope_append)

struct QGemvParams {
  const void* x;
  const void* packed;
  const void* scales;
  const float* zero_points;
  const void* residual;
  void* y;
  int M, N, K;
  int bits;        // 8, 4, or 0 for dense weights of x's type
  int group_size;  // 0: one (scale, zero) per row; >0: symmetric groups along K
  int x_dtype, scale_dtype;
  long long x_stride;
  int epilogue;
  bool vector_ok;  // rows of x and of the packed weight can be read in 16-byte units
  bool tiled;      // codes are in the 128x128 tile order of cacheir_b200_pack_relayout
  bool paired;     // tiled, and every tile pairs 64 rows of the first half of W with the matching 64 of the second half
  bool x_prequantized;  // the workspace already holds the integer form of x (see cacheir_b200_quantize_activations)
  const void* norm_weight;  // non-null: y = epilogue(rmsnorm(x; norm_weight, norm_eps) . W^T): the norm runs inside the activation pre-pass (integer tensor-core path only)
  float norm_eps;
  RopeAppendParams rope;  // epilogue == kEpiQkvRopeAppend only
};

int launch_qgemv_cuda_core(const QGemvParams& p, cudaStream_t stream);
// Streaming int4 GEMV for up to 8 batch rows (mma.sync on nibbles unpacked in registers, row-major codes).
bool qgemv_mma_supported(const QGemvParams& p);
int launch_qgemv_mma(const QGemvParams& p, cudaStream_t stream);

// Tensor-core (tcgen05) small-M GEMM: weights are the 128-row MMA operand.
bool qgemm_tc_supported(const QGemvParams& p);
int launch_qgemm_tc(const QGemvParams& p, cudaStream_t stream);
// Integer tensor-core path (int8 per-row weights, fp16 activations turned into 16-bit fixed point).
// Needs `qgemm_i8_workspace_bytes` of caller scratch for the activation bytes.
size_t qgemm_i8_workspace_bytes(int M, int K);
bool qgemm_i8_supported(const QGemvParams& p, const void* workspace, size_t workspace_bytes);
int launch_qgemm_i8(const QGemvParams& p, void* workspace, cudaStream_t stream);
int qgemm_i8_plan(const QGemvParams& p);   // the split-K factor the launcher would use
int qgemm_i8_device_status(bool reset);
int qgemv_mma_device_status(bool reset);
int qgemm_i8_quantize_activations(const void* x, long long x_stride, int M, int K, void* workspace, cudaStream_t stream);
int qgemm_i8_rms_norm_quantize(const void* x, const void* residual, const void* weight, void* sum_out, void* out, int M,
                               int hidden, float eps, void* workspace, cudaStream_t stream);
// Device-side status word of the tensor-core kernel (0 = no bounded wait ever gave up).
int qgemm_tc_device_status(bool reset);

}  // namespace cb200
