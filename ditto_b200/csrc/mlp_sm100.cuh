// Launch interface of the fused GEMM -> activation -> GEMM kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "host_util.cuh"

namespace ditto_b200 {

// Which kernel a call takes.
//   kMlpAuto    the four-CTA kernel where it covers the shape, else the CTA-pair kernel
//   kMlpQuad    four-CTA clusters, single-SM MMAs (mlp_sm100.cu): L % 128 == 0, K % 64 == 0, N in {256, ..., 1024}
//   kMlpPair    eight-CTA clusters of CTA pairs, 2-SM MMAs (mlp_pair_sm100.cu): L % 256 == 0, K % 16 == 0,
//               N in {512, 1024} ([in, out] weights) or {256, 512, 768, 1024} ([out, in])
//   kMlpWide    four-CTA clusters, single-SM MMAs, 256-wide hidden chunks (mlp_wide_sm100.cu): L % 256 == 0,
//               K % 16 == 0, N in {256, 512, 768, 1024}
enum MlpVariant { kMlpAuto = 0, kMlpQuad = 1, kMlpPair = 2, kMlpWide = 3 };

// Returns a DITTO_* status code (0 on success).  act1 / act2: activation after the first / second GEMM
// (0 identity, 1 ReLU, 2 GELU); b1 / b2: optional 16-bit bias vectors [batch, L] / [batch, N].
// workspace / ws_bytes: optional scratch for the hidden-split form of the pair kernel (see
// mlp_workspace_bytes); without it every row block is computed by one cluster.
int launch_mlp_chain(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                     bool bf16, int w_layout, int act1, int act2, const void* b1, const void* b2, int variant,
                     void* workspace, size_t ws_bytes, int* status, cudaStream_t stream, long long* trace = nullptr);

// Scratch bytes with which the chain runs fastest at this shape on the current device (0: none needed).
size_t mlp_workspace_bytes(int batch, int M, int N, int K, int L, bool bf16, int w_layout, int variant);

// The four-CTA kernel with the library's own scratch array in place of a caller-provided workspace
// (see ditto_b200_gemm_relu_gemm_static_scratch).  Allocates nothing.
int launch_mlp_static_scratch(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                              bool bf16, int w_layout, int act1, int* status, cudaStream_t stream);

// Clusters of four CTAs of the four-CTA kernel the current device holds at once (queried once per device).
int mlp_quad_cluster_slots(bool bf16, int* slots);

// ---- four-CTA kernel with 256-wide hidden chunks (mlp_wide_sm100.cu)
bool mlp_wide_supported(int N, int K, int L);
int mlp_wide_cluster_slots(bool bf16, int* slots);
RowBlockPlan mlp_wide_plan(int batch, int M, int L, int cluster_slots, bool allow_scratch);
size_t mlp_wide_workspace_bytes(int batch, int M, int N, const RowBlockPlan& plan);
int launch_mlp_wide(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                    bool bf16, int w_layout, int act1, int act2, const void* b1, const void* b2,
                    const RowBlockPlan& plan, void* workspace, int* status, cudaStream_t stream, long long* trace = nullptr);

// ---- CTA-pair kernel (mlp_pair_sm100.cu)
bool mlp_pair_supported(int N, int K, int L, int w_layout);
// Clusters of eight CTAs the current device holds at once (queried once per device).
int mlp_pair_cluster_slots(bool bf16, int* slots);
using PairPlan = RowBlockPlan;   // 256-row blocks, 256-wide hidden chunks
// The plan with the shortest modelled run time on a device that holds `cluster_slots` clusters at once;
// without scratch memory: every row block whole.
PairPlan mlp_pair_plan(int batch, int M, int L, int cluster_slots, bool allow_scratch);
size_t mlp_pair_workspace_bytes(int batch, int M, int N, const PairPlan& plan);
int launch_mlp_pair(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                    bool bf16, int w_layout, int act1, int act2, const void* b1, const void* b2,
                    const PairPlan& plan, void* workspace, int* status, cudaStream_t stream, long long* trace = nullptr);

}  // namespace ditto_b200
