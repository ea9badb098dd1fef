// Launch interface of the single-CTA tcgen05 self test.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace ditto_b200 {

struct SelftestParams {
  CUtensorMap map_a;     // A [128, K], box 64 x 128
  CUtensorMap map_b;     // B [N, K] (box 64 x N) or [K, N] (box 64 x K)
  const void* a_global;  // A again, for the TMEM-operand path
  float* c;              // C [128, N] fp32
  int N, K;              // multiples of 64, <= 256
  int b_mn, a_tmem, bf16;
  int* status;
};

cudaError_t launch_umma_selftest(const SelftestParams& p, cudaStream_t stream);
// CTA-pair variant: A has 256 rows (box 64 x 128 per CTA), B boxes cover half of N.
cudaError_t launch_umma_pair_selftest(const SelftestParams& p, cudaStream_t stream);

// One CTA runs the library's bounded wait on a barrier nobody signals and reports `code` through `status`.
cudaError_t launch_wait_limit_selftest(int code, int* status, cudaStream_t stream);

}  // namespace ditto_b200
