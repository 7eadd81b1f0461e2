// extern "C" doorway into the reference project's own native CPU kernels
// (cpp/src/cacheir_backend.cpp, compiled unmodified from where it lies; see
// oracle/Makefile). TEST / BASELINE INFRASTRUCTURE ONLY: used to cross-check the
// NumPy oracle and to time the reference's OpenMP/AVX path on the host cores.
#include <array>
#include <cstddef>

#include "cacheir/cacheir_backend.hpp"

extern "C" {

const char* cacheir_ref_simd_backend() { return cacheir::simd_backend(); }

// x: [rows, hidden] viewed as rank 3 [1, rows, hidden] (the reference kernels require rank 3)
void cacheir_ref_rms_norm(const float* x, const float* weight, float* out, std::size_t rows,
                          std::size_t hidden, float eps) {
  const std::array<std::size_t, 3> xs{1, rows, hidden};
  const std::array<std::size_t, 1> ws{hidden};
  cacheir::rms_norm({x, xs}, {weight, ws}, {out, xs}, eps);
}

void cacheir_ref_silu_mul(const float* gate, const float* up, float* out, std::size_t total) {
  const std::array<std::size_t, 1> s{total};
  cacheir::silu_mul({gate, s}, {up, s}, {out, s});
}

// out[rows, out_features] = x[rows, in_features] . weight[out_features, in_features]^T
void cacheir_ref_matmul_out_in(const float* x, const float* weight, float* out, std::size_t rows,
                               std::size_t in_features, std::size_t out_features) {
  const std::array<std::size_t, 3> xs{1, rows, in_features};
  const std::array<std::size_t, 2> ws{out_features, in_features};
  const std::array<std::size_t, 3> os{1, rows, out_features};
  cacheir::matmul_out_in({x, xs}, {weight, ws}, {out, os});
}

}  // extern "C"
