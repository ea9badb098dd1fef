// Launch interface of the fused GEMM -> activation -> GEMM kernel.
#pragma once
#include <cuda_runtime.h>

namespace ditto_b200 {

// Returns a DITTO_* status code (0 on success).
int launch_mlp_chain(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                     bool bf16, int w_layout, int epilogue, int* status, cudaStream_t stream,
                     long long* trace = nullptr);

}  // namespace ditto_b200
