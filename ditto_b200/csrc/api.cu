// C ABI of libditto_b200: argument checking, TMA tensor-map construction and
// kernel launch.  Declarations and the reference interfaces they stand in for
// are in include/ditto_b200.h.
#include "../../include/ditto_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "attention_sm100.cuh"
#include "host_util.cuh"
#include "mlp_sm100.cuh"
#include "selftest_sm100.cuh"

namespace {

using ditto_b200::cuda_fail;
using ditto_b200::set_error;

// Key/value rows up to which the persistent attention kernel is the faster one for head dims <= 64
// (measured: 469 vs 453 TFLOP/s at 512 keys, 656 vs 680 at 2048).
constexpr int kPersistentMaxKeys = 1024;

// 2-D row-major tensor [rows, cols] of 16-bit elements, 128-byte swizzled boxes.
int make_map_2d(CUtensorMap* map, bool bf16, const void* base, uint64_t cols, uint64_t rows, uint32_t box_cols,
                uint32_t box_rows) {
  const uint64_t dims[2] = {cols, rows}, strides[1] = {cols * 2};
  const uint32_t box[2] = {box_cols, box_rows};
  return ditto_b200::make_tensor_map(map, bf16, base, 2, dims, strides, box);
}

// 3-D tensor [slices, rows, cols] of 16-bit elements: coordinates (col, row, slice), boxes of
// box_cols x box_rows x 1.  Rows beyond `rows` inside a slice are out of bounds and read as zero,
// which is what makes partial tiles at the end of a sequence safe.
int make_map_3d(CUtensorMap* map, bool bf16, const void* base, uint64_t cols, uint64_t rows, uint64_t slices,
                uint64_t row_stride_elems, uint64_t slice_stride_elems, uint32_t box_cols, uint32_t box_rows) {
  const uint64_t dims[3] = {cols, rows, slices}, strides[2] = {row_stride_elems * 2, slice_stride_elems * 2};
  const uint32_t box[3] = {box_cols, box_rows, 1};
  return ditto_b200::make_tensor_map(map, bf16, base, 3, dims, strides, box);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" {

int ditto_b200_bmm_softmax_bmm(const void* q, const void* k, const void* v, void* out, int batch, int M, int N,
                               int K, int L, int dtype, int k_layout, float scale, int flags, void* workspace,
                               size_t ws_bytes, int* status_word, void* stream) {
  (void)workspace;
  (void)ws_bytes;
  if (!q || !k || !v || !out) return DITTO_ERR_INVALID_ARG;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0 || L <= 0) return DITTO_ERR_INVALID_ARG;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return DITTO_ERR_INVALID_ARG;
  if (!(scale > 0.f) || !std::isfinite(scale)) return DITTO_ERR_INVALID_ARG;
  if (dtype != DITTO_DTYPE_FP16 && dtype != DITTO_DTYPE_BF16) return DITTO_ERR_UNSUPPORTED;
  if (k_layout != 0 && k_layout != 1) return DITTO_ERR_INVALID_ARG;
  // The reference asserts multiples of 16 (bmm_chain.py:34-38); so does this entry point.  Partial
  // 128-row tiles are handled by TMA zero fill, masked scores and predicated stores.
  if (M % 16 || N % 16 || K % 16 || L % 16) return DITTO_ERR_INVALID_ARG;
  if (K > 128 || N > 128) return DITTO_ERR_UNSUPPORTED;
  if (static_cast<long long>(batch) * ((M + 127) / 128) > 0x7fffffffLL) return DITTO_ERR_UNSUPPORTED;

  const bool bf16 = dtype == DITTO_DTYPE_BF16;
  // kernel variant by the wider of the two widths; K (the reduction of Q K^T) and N (the width of V and of the
  // output) may differ and be any multiples of 16 below it, as in the reference's definition (bmm_chain.py:28-38)
  const int d = (K <= 64 && N <= 64) ? 64 : 128;
  int nt = (M > 128 && !(flags & DITTO_FLAG_ONE_TILE)) ? 2 : 1;
  // d <= 64: one tile per CTA with separate S / P columns, two CTAs per SM (see attention_sm100.cu)
  if (d == 64 && !(flags & (DITTO_FLAG_TWO_TILES | DITTO_FLAG_P_VIA_SMEM))) nt = 1;
  const bool psmem = (flags & DITTO_FLAG_P_VIA_SMEM) != 0;

  ditto_b200::AttnParams p;
  std::memset(&p, 0, sizeof(p));
  const uint64_t uK = K, uM = M, uL = L, ub = batch;
  int rc = make_map_3d(&p.map_q, bf16, q, uK, uM, ub, uK, uM * uK, 64, 128);
  if (rc) return rc;
  if (k_layout == 0)
    rc = make_map_3d(&p.map_k, bf16, k, uL, uK, ub, uL, uK * uL, 64, d);
  else
    rc = make_map_3d(&p.map_k, bf16, k, uK, uL, ub, uK, uL * uK, 64, 128);
  if (rc) return rc;
  const uint64_t uN = N;
  rc = make_map_3d(&p.map_v, bf16, v, uN, uL, ub, uN, uL * uN, 64, 128);
  if (rc) return rc;
  p.out = out;
  p.M = M;
  p.L = L;
  p.k_transposed = (k_layout == 0);
  p.d = K;
  p.dv = N;
  p.heads = 1;
  p.out_ld = N;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_word;
#ifdef DITTO_TRACE
  p.trace = ws_bytes >= 1280 * sizeof(long long) ? static_cast<long long*>(workspace) : nullptr;
#endif
  // head dimensions up to 64 with few key blocks per item take the persistent kernel (it hides the
  // per-item start-up, which long sequences amortise anyway) unless a flag asks for a specific tiling
  const bool persistent = d == 64 && L <= kPersistentMaxKeys &&
                          !(flags & (DITTO_FLAG_ONE_TILE | DITTO_FLAG_TWO_TILES | DITTO_FLAG_P_VIA_SMEM));
  cudaError_t e = persistent
                      ? ditto_b200::launch_attention_persistent(p, batch, bf16, 0, static_cast<cudaStream_t>(stream))
                      : ditto_b200::launch_attention(p, batch, d, bf16, nt, psmem, 0, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("bmm_softmax_bmm launch", e);
  return DITTO_OK;
}

int ditto_b200_multi_head_attention(const void* qkv, void* out, int batch, int M, int heads, int head_dim, int dtype,
                                    float scale, int flags, int* status_word, void* stream) {
  if (!qkv || !out) return DITTO_ERR_INVALID_ARG;
  if (batch <= 0 || M <= 0 || heads <= 0 || head_dim <= 0) return DITTO_ERR_INVALID_ARG;
  if (!aligned16(qkv) || !aligned16(out)) return DITTO_ERR_INVALID_ARG;
  if (!(scale > 0.f) || !std::isfinite(scale)) return DITTO_ERR_INVALID_ARG;
  if (dtype != DITTO_DTYPE_FP16 && dtype != DITTO_DTYPE_BF16) return DITTO_ERR_UNSUPPORTED;
  if (head_dim % 16 || head_dim > 128 || M % 16) return DITTO_ERR_UNSUPPORTED;
  if (static_cast<long long>(batch) * heads * ((M + 127) / 128) > 0x7fffffffLL) return DITTO_ERR_UNSUPPORTED;
  const bool bf16 = dtype == DITTO_DTYPE_BF16;
  const int d = head_dim <= 64 ? 64 : 128, hidden = heads * head_dim;
  int nt = (M > 128 && !(flags & DITTO_FLAG_ONE_TILE)) ? 2 : 1;
  if (d == 64 && !(flags & DITTO_FLAG_TWO_TILES)) nt = 1;
  ditto_b200::AttnParams p;
  std::memset(&p, 0, sizeof(p));
  // one tensor map over the packed [batch*M, 3*hidden] matrix serves Q, K and V: the head split and
  // the [b, M, h, d] -> [b*h, M, d] permutes become TMA coordinates
  int rc = make_map_3d(&p.map_q, bf16, qkv, 3ull * hidden, M, batch, 3ull * hidden, 3ull * hidden * M, 64, 128);
  if (rc) return rc;
  p.map_k = p.map_q;
  p.map_v = p.map_q;
  p.out = out;
  p.M = M;
  p.L = M;
  p.k_transposed = 0;
  p.d = head_dim;
  p.dv = head_dim;
  p.heads = heads;
  p.q_col0 = 0;
  p.k_col0 = hidden;
  p.v_col0 = 2 * hidden;
  p.out_ld = hidden;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status_word;
  const bool persistent = d == 64 && M <= kPersistentMaxKeys && !(flags & (DITTO_FLAG_ONE_TILE | DITTO_FLAG_TWO_TILES));
  cudaError_t e = persistent ? ditto_b200::launch_attention_persistent(p, batch * heads, bf16, 0,
                                                                       static_cast<cudaStream_t>(stream))
                             : ditto_b200::launch_attention(p, batch * heads, d, bf16, nt, false, 0,
                                                            static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("multi_head_attention launch", e);
  return DITTO_OK;
}

int ditto_b200_gemm_relu_gemm(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N,
                              int K, int L, int dtype, int w_layout, int epilogue, void* workspace,
                              size_t ws_bytes, int* status_word, void* stream) {
  if (!x || !w1 || !w2 || !y) return DITTO_ERR_INVALID_ARG;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0 || L <= 0) return DITTO_ERR_INVALID_ARG;
  if (!aligned16(x) || !aligned16(w1) || !aligned16(w2) || !aligned16(y)) return DITTO_ERR_INVALID_ARG;
  if (dtype != DITTO_DTYPE_FP16 && dtype != DITTO_DTYPE_BF16) return DITTO_ERR_UNSUPPORTED;
  if (w_layout != 0 && w_layout != 1) return DITTO_ERR_INVALID_ARG;
  constexpr int kVariantMask = DITTO_EPILOGUE_PAIR_MMA | DITTO_EPILOGUE_QUAD_MMA | DITTO_EPILOGUE_WIDE_MMA;
  const int variant_bits = epilogue & kVariantMask;
  const int act = epilogue & ~kVariantMask;
  if (act != 0 && act != 1) return DITTO_ERR_INVALID_ARG;
  if (variant_bits & (variant_bits - 1)) return DITTO_ERR_INVALID_ARG;   // at most one kernel can be named
  if (M % 16 || N % 16 || K % 16 || L % 16) return DITTO_ERR_INVALID_ARG;
  if (N <= 128 && K <= 128) {
    // Small-N chains (the reference's shape family: N = K = 64, L = 512 ...): the result tile
    // [128, N] fits TMEM next to the intermediate, so the chain runs on the attention kernel with
    // the activation in place of the softmax: A = x, B = w1, C = w2.
    if (static_cast<long long>(batch) * ((M + 127) / 128) > 0x7fffffffLL) return DITTO_ERR_UNSUPPORTED;
    const bool bf16 = dtype == DITTO_DTYPE_BF16;
    const int dk = (K <= 64 && N <= 64) ? 64 : 128;
    ditto_b200::AttnParams p;
    std::memset(&p, 0, sizeof(p));
    const uint64_t uK = K, uM = M, uL = L, ub = batch;
    int rc = make_map_3d(&p.map_q, bf16, x, uK, uM, ub, uK, uM * uK, 64, 128);
    if (rc) return rc;
    const uint64_t uN = N;
    if (w_layout == 0) {
      // [in, out] weights: w1 [K, L] is the reference's transposed-K form, w2 [L, N] the usual V
      rc = make_map_3d(&p.map_k, bf16, w1, uL, uK, ub, uL, uK * uL, 64, dk);
      if (rc) return rc;
      rc = make_map_3d(&p.map_v, bf16, w2, uN, uL, ub, uN, uL * uN, 64, 128);
    } else {
      // [out, in] weights: w1 [L, K] is K in rows-of-keys form, w2 [N, L] a transposed V (K-major operand of GEMM2)
      rc = make_map_3d(&p.map_k, bf16, w1, uK, uL, ub, uK, uL * uK, 64, 128);
      if (rc) return rc;
      rc = make_map_3d(&p.map_v, bf16, w2, uL, uN, ub, uL, uN * uL, 64, dk);
    }
    if (rc) return rc;
    p.out = y;
    p.M = M;
    p.L = L;
    p.k_transposed = w_layout == 0;
    p.v_transposed = w_layout != 0;
    p.d = K;
    p.dv = N;
    p.heads = 1;
    p.out_ld = N;
    p.scale_log2 = 1.0f;
    p.status = status_word;
    const int nt = (dk == 64 || M <= 128) ? 1 : 2;
    const int mode = act == 1 ? 1 : 2;
    cudaError_t e = (dk == 64 && L <= kPersistentMaxKeys) ? ditto_b200::launch_attention_persistent(p, batch, bf16, mode, static_cast<cudaStream_t>(stream))
                             : ditto_b200::launch_attention(p, batch, dk, bf16, nt, false, mode,
                                                            static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail("gemm_relu_gemm launch", e);
    return DITTO_OK;
  }
  long long* trace = nullptr;
#ifdef DITTO_TRACE
  if (ws_bytes >= 512 * sizeof(long long)) trace = static_cast<long long*>(workspace);
#endif
#ifdef DITTO_TRACE
  workspace = nullptr;   // the buffer is the timeline, not scratch
  ws_bytes = 0;
#endif
  const int variant = variant_bits == DITTO_EPILOGUE_PAIR_MMA   ? ditto_b200::kMlpPair
                      : variant_bits == DITTO_EPILOGUE_QUAD_MMA ? ditto_b200::kMlpQuad
                      : variant_bits == DITTO_EPILOGUE_WIDE_MMA ? ditto_b200::kMlpWide
                                                                : ditto_b200::kMlpAuto;
  return ditto_b200::launch_mlp_chain(x, w1, w2, y, batch, M, N, K, L, dtype == DITTO_DTYPE_BF16, w_layout, act, 0,
                                      nullptr, nullptr, variant, workspace, ws_bytes, status_word,
                                      static_cast<cudaStream_t>(stream), trace);
}

int ditto_b200_gemm_relu_gemm_static_scratch(const void* x, const void* w1, const void* w2, void* y, int batch, int M,
                                             int N, int K, int L, int dtype, int w_layout, int epilogue,
                                             int* status_word, void* stream) {
  if (!x || !w1 || !w2 || !y) return DITTO_ERR_INVALID_ARG;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0 || L <= 0) return DITTO_ERR_INVALID_ARG;
  if (!aligned16(x) || !aligned16(w1) || !aligned16(w2) || !aligned16(y)) return DITTO_ERR_INVALID_ARG;
  if (dtype != DITTO_DTYPE_FP16 && dtype != DITTO_DTYPE_BF16) return DITTO_ERR_UNSUPPORTED;
  if (w_layout != 0 && w_layout != 1) return DITTO_ERR_INVALID_ARG;
  if (epilogue != 0 && epilogue != 1) return DITTO_ERR_INVALID_ARG;
  if (M % 16 || N % 16 || K % 16 || L % 16) return DITTO_ERR_INVALID_ARG;
  return ditto_b200::launch_mlp_static_scratch(x, w1, w2, y, batch, M, N, K, L, dtype == DITTO_DTYPE_BF16, w_layout,
                                               epilogue, status_word, static_cast<cudaStream_t>(stream));
}

int ditto_b200_ffn(const void* x, const void* w1, const void* b1, const void* w2, const void* b2, void* y, int batch,
                   int M, int N, int K, int L, int dtype, int w_layout, int act1, int act2, int* status_word,
                   void* stream) {
  if (!x || !w1 || !w2 || !y) return DITTO_ERR_INVALID_ARG;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0 || L <= 0) return DITTO_ERR_INVALID_ARG;
  if (!aligned16(x) || !aligned16(w1) || !aligned16(w2) || !aligned16(y)) return DITTO_ERR_INVALID_ARG;
  if ((b1 && (reinterpret_cast<uintptr_t>(b1) & 3)) || (b2 && (reinterpret_cast<uintptr_t>(b2) & 3))) return DITTO_ERR_INVALID_ARG;
  if (dtype != DITTO_DTYPE_FP16 && dtype != DITTO_DTYPE_BF16) return DITTO_ERR_UNSUPPORTED;
  if (w_layout != 0 && w_layout != 1) return DITTO_ERR_INVALID_ARG;
  if (act1 < 0 || act1 > 2 || act2 < 0 || act2 > 2) return DITTO_ERR_INVALID_ARG;
  if (M % 16 || N % 16 || K % 16 || L % 16) return DITTO_ERR_INVALID_ARG;
  return ditto_b200::launch_mlp_chain(x, w1, w2, y, batch, M, N, K, L, dtype == DITTO_DTYPE_BF16, w_layout, act1, act2,
                                      b1, b2, ditto_b200::kMlpAuto, nullptr, 0, status_word,
                                      static_cast<cudaStream_t>(stream));
}

size_t ditto_b200_workspace_bytes(int op, int batch, int M, int N, int K, int L, int dtype) {
  // The attention chain keeps everything on chip.  The MLP chain does too, except that with few row blocks
  // it runs faster when several clusters share a row block and combine fp32 partials of Y through scratch
  // memory (the hidden activations still never leave the chip); the call works without it.
  if ((op & 0xff) != DITTO_OP_GEMM_RELU_GEMM || batch <= 0 || M <= 0 || N <= 0 || K <= 0 || L <= 0) return 0;
  if (N <= 128 && K <= 128) return 0;
  // `op` may carry DITTO_EPILOGUE_PAIR_MMA / DITTO_EPILOGUE_QUAD_MMA like the call's `epilogue` argument
  const int variant = (op & DITTO_EPILOGUE_PAIR_MMA)   ? ditto_b200::kMlpPair
                      : (op & DITTO_EPILOGUE_QUAD_MMA) ? ditto_b200::kMlpQuad
                      : (op & DITTO_EPILOGUE_WIDE_MMA) ? ditto_b200::kMlpWide
                                                       : ditto_b200::kMlpAuto;
  size_t a = ditto_b200::mlp_workspace_bytes(batch, M, N, K, L, dtype == DITTO_DTYPE_BF16, 0, variant);
  size_t b = ditto_b200::mlp_workspace_bytes(batch, M, N, K, L, dtype == DITTO_DTYPE_BF16, 1, variant);
  return a > b ? a : b;
}

int ditto_b200_mlp_cluster_slots(int dtype, int variant) {
  if (dtype != DITTO_DTYPE_FP16 && dtype != DITTO_DTYPE_BF16) return DITTO_ERR_UNSUPPORTED;
  int slots = 0;
  int rc = variant == DITTO_EPILOGUE_PAIR_MMA   ? ditto_b200::mlp_pair_cluster_slots(dtype == DITTO_DTYPE_BF16, &slots)
           : variant == DITTO_EPILOGUE_QUAD_MMA ? ditto_b200::mlp_quad_cluster_slots(dtype == DITTO_DTYPE_BF16, &slots)
           : variant == DITTO_EPILOGUE_WIDE_MMA ? ditto_b200::mlp_wide_cluster_slots(dtype == DITTO_DTYPE_BF16, &slots)
                                                : DITTO_ERR_INVALID_ARG;
  return rc ? rc : slots;
}

int ditto_b200_selftest_umma(const void* a, const void* b, float* c, int N, int K, int dtype, int b_mn, int a_tmem,
                             int* status_word, void* stream) {
  if (!a || !b || !c) return DITTO_ERR_INVALID_ARG;
  if (N <= 0 || K <= 0 || N % 64 || K % 64 || N > 256 || K > 256) return DITTO_ERR_UNSUPPORTED;
  if (dtype != DITTO_DTYPE_FP16 && dtype != DITTO_DTYPE_BF16) return DITTO_ERR_UNSUPPORTED;
  const bool bf16 = dtype == DITTO_DTYPE_BF16;
  ditto_b200::SelftestParams p;
  std::memset(&p, 0, sizeof(p));
  int rc = make_map_2d(&p.map_a, bf16, a, K, 128, 64, 128);
  if (rc) return rc;
  rc = b_mn ? make_map_2d(&p.map_b, bf16, b, N, K, 64, K) : make_map_2d(&p.map_b, bf16, b, K, N, 64, N);
  if (rc) return rc;
  p.a_global = a;
  p.c = c;
  p.N = N;
  p.K = K;
  p.b_mn = b_mn ? 1 : 0;
  p.a_tmem = a_tmem ? 1 : 0;
  p.bf16 = bf16 ? 1 : 0;
  p.status = status_word;
  cudaError_t e = ditto_b200::launch_umma_selftest(p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("selftest launch", e);
  return DITTO_OK;
}

int ditto_b200_selftest_umma_pair(const void* a, const void* b, float* c, int N, int K, int dtype, int b_mn,
                                  int* status_word, void* stream) {
  if (!a || !b || !c) return DITTO_ERR_INVALID_ARG;
  if (N <= 0 || K <= 0 || N % 128 || K % 64 || N > 256 || K > 256) return DITTO_ERR_UNSUPPORTED;
  if (dtype != DITTO_DTYPE_FP16 && dtype != DITTO_DTYPE_BF16) return DITTO_ERR_UNSUPPORTED;
  const bool bf16 = dtype == DITTO_DTYPE_BF16;
  ditto_b200::SelftestParams p;
  std::memset(&p, 0, sizeof(p));
  int rc = make_map_2d(&p.map_a, bf16, a, K, 256, 64, 128);
  if (rc) return rc;
  rc = b_mn ? make_map_2d(&p.map_b, bf16, b, N, K, 64, K) : make_map_2d(&p.map_b, bf16, b, K, N, 64, N / 2);
  if (rc) return rc;
  p.a_global = a;
  p.c = c;
  p.N = N;
  p.K = K;
  p.b_mn = b_mn ? 1 : 0;
  p.bf16 = bf16 ? 1 : 0;
  p.status = status_word;
  cudaError_t e = ditto_b200::launch_umma_pair_selftest(p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("pair selftest launch", e);
  return DITTO_OK;
}

int ditto_b200_selftest_wait_limit(int code, int* status_word, void* stream) {
  if (code <= 0 || status_word == nullptr) return DITTO_ERR_INVALID_ARG;
  cudaError_t e = ditto_b200::launch_wait_limit_selftest(code, status_word, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail("selftest_wait_limit launch", e);
  return DITTO_OK;
}

int ditto_b200_check_status(int* status_word, void* stream, int* code_out) {
  if (status_word == nullptr) return DITTO_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int value = 0;
  cudaError_t e = cudaMemcpyAsync(&value, status_word, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail("check_status", e);
  if (code_out != nullptr) *code_out = value;
  if (value == 0) return DITTO_OK;
  e = cudaMemsetAsync(status_word, 0, sizeof(int), st);       // ready for the next calls
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail("check_status", e);
  return DITTO_ERR_TIMEOUT;
}

const char* ditto_b200_strerror(int code) {
  switch (code) {
    case DITTO_OK: return "ok";
    case DITTO_ERR_INVALID_ARG: return "invalid argument";
    case DITTO_ERR_UNSUPPORTED: return "shape, dtype or layout not supported by the sm_100a kernels";
    case DITTO_ERR_CUDA: return "CUDA error";
    case DITTO_ERR_TIMEOUT: return "device-side wait timed out";
    case DITTO_ERR_WORKSPACE: return "workspace too small";
    case DITTO_ERR_DRIVER: return "driver entry point missing";
    default: return "unknown error";
  }
}

const char* ditto_b200_last_cuda_error(void) { return ditto_b200::last_error_text(); }

int ditto_b200_version(void) { return 100; }

}  // extern "C"
