// Tensor-core small-M dequant-GEMM (placeholder until the tcgen05 kernel lands).
#include "common.cuh"
#include "qgemv_common.cuh"

namespace cb200 {
bool qgemm_tc_supported(const QGemvParams&) { return false; }
int launch_qgemm_tc(const QGemvParams&, cudaStream_t) { return CACHEIR_B200_EUNSUPPORTED; }
}  // namespace cb200
