// Arguments shared by the dequant-GEMV kernels and their launchers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace cb200 {

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
};

int launch_qgemv_cuda_core(const QGemvParams& p, cudaStream_t stream);

// Tensor-core (tcgen05) small-M GEMM: weights are the 128-row MMA operand.
bool qgemm_tc_supported(const QGemvParams& p);
int launch_qgemm_tc(const QGemvParams& p, cudaStream_t stream);
// Device-side status word of the tensor-core kernel (0 = no bounded wait ever gave up).
int qgemm_tc_device_status(bool reset);

}  // namespace cb200
