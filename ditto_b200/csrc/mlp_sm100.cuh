// Launch interface of the fused GEMM -> activation -> GEMM kernel.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ditto_b200 {

// Returns a DITTO_* status code (0 on success).  epilogue: activation after the first GEMM (0 identity,
// 1 ReLU, 2 GELU; | 0x200 selects the CTA-pair variant); b1 / b2: optional 16-bit bias vectors
// [batch, L] / [batch, N]; act2: activation after the second GEMM.
int launch_mlp_chain(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                     bool bf16, int w_layout, int epilogue, int* status, cudaStream_t stream,
                     long long* trace = nullptr, const void* b1 = nullptr, const void* b2 = nullptr, int act2 = 0);

// 2-D row-major 16-bit tensor map with 128-byte-swizzled boxes; false if the driver entry point is missing
// or the encoding is rejected.
bool mlp_make_map(CUtensorMap* map, bool bf16, const void* base, uint64_t cols, uint64_t rows, uint32_t box_cols,
                  uint32_t box_rows);

// CTA-pair (cta_group::2) variant: M % 256 == 0, L % 512 == 0, K % 64 == 0, N in {512, 1024}.
bool mlp_pair_supported(int M, int N, int K, int L);
int launch_mlp_pair(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                    bool bf16, int w_layout, int epilogue, int* status, cudaStream_t stream, long long* trace = nullptr);

}  // namespace ditto_b200
