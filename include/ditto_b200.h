/* ditto_b200 -- C ABI of the B200 (sm_100a) fused GEMM-chain kernels.
 *
 * The reference (KnowingNothing/Ditto) has no C plugin interface of its own: a
 * fused chain is compiled by TVM into a runtime.Module whose entry
 * "default_function" is called with positional DLTensor arguments -- inputs,
 * weights, then outputs, all caller-allocated, compact row-major
 * (src/runtime/graph_runtime.cc:133-204, python/ditto/auto_compute/graph.py:90-102,
 * benchmark/chimera/cuda/bmm_softmax_bmm_cuda.py:239-256).  The entry points
 * below take the place of those generated modules for the two chains; the
 * shape tuple (batch, M, N, K, L) is the reference's:
 *     A/query [batch, M, K]   B/key [batch, K, L]   C/value [batch, L, N]   out [batch, M, N]
 *
 * Conventions: every pointer is a device pointer owned by the caller; nothing
 * is allocated per call; launches are asynchronous on `stream` (a
 * cudaStream_t passed as void*); argument errors are reported synchronously by
 * the return value; no entry point throws, aborts or traps.  A device-side
 * bounded wait that expires stores a non-zero code in *status_word (device
 * memory, optional) -- read it after synchronising the stream.
 */
#ifndef DITTO_B200_H_
#define DITTO_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DITTO_OK 0
#define DITTO_ERR_INVALID_ARG (-1) /* null pointer, non-positive size, misaligned buffer */
#define DITTO_ERR_UNSUPPORTED (-2) /* shape / dtype / layout outside what the kernels cover */
#define DITTO_ERR_CUDA (-3)        /* a CUDA runtime call failed; see ditto_b200_last_cuda_error() */
#define DITTO_ERR_TIMEOUT (-4)     /* a device-side bounded wait expired */
#define DITTO_ERR_WORKSPACE (-5)   /* workspace smaller than ditto_b200_workspace_bytes() */
#define DITTO_ERR_DRIVER (-6)      /* the driver does not export cuTensorMapEncodeTiled */

#define DITTO_DTYPE_FP16 0
#define DITTO_DTYPE_BF16 1

/* or-ed into `epilogue` of ditto_b200_gemm_relu_gemm: force one of the two kernels (default: chosen by shape) */
#define DITTO_EPILOGUE_PAIR_MMA 0x200 /* eight-CTA clusters of CTA pairs, 2-SM MMAs */
#define DITTO_EPILOGUE_QUAD_MMA 0x400 /* four-CTA clusters, single-SM MMAs, 128-wide hidden chunks */
#define DITTO_EPILOGUE_WIDE_MMA 0x800 /* four-CTA clusters, single-SM MMAs, 256-wide hidden chunks */

#define DITTO_OP_BMM_SOFTMAX_BMM 0
#define DITTO_OP_GEMM_RELU_GEMM 1

/* flags of ditto_b200_bmm_softmax_bmm */
#define DITTO_FLAG_P_VIA_SMEM 1   /* stage the probabilities through shared memory instead of TMEM */
#define DITTO_FLAG_ONE_TILE 2     /* one 128-row query tile per CTA, one CTA per tile (no persistent work loop) */
#define DITTO_FLAG_TWO_TILES 4    /* two query tiles per CTA even where one is the default (N = K = 64) */

/* Fused attention chain  out = softmax(scale * Q K^T) V, replacing the module TVM builds from
 * BatchGemmSoftmaxGemmMMA (python/ditto/auto_compute/nn/functional/bmm_chain.py:5-104) under
 * TensorizeCUDA (src/auto_tensorize/hyper_fusion.cc:1494-1603).
 *   k_layout 0: key is [batch, K, L] (the reference's pre-transposed layout,
 *               python/ditto/auto_compute/nn/module/self_attention.py:55-57)
 *   k_layout 1: key is [batch, L, K]
 *   scale 1.0 reproduces the reference's exp(QK^T)/sum semantics; the softmax is evaluated in the
 *   max-subtracted form, which is the same function without the overflow.
 * Supported: K <= 128 and N <= 128 (they may differ, as in the reference's definition); M, N, K, L multiples of 16 like the reference asserts (partial 128-row tiles are
 * zero-filled by TMA, masked and not stored); fp16 or bf16 in/out, fp32 accumulate. */
int ditto_b200_bmm_softmax_bmm(const void* q, const void* k, const void* v, void* out, int batch, int M, int N,
                               int K, int L, int dtype, int k_layout, float scale, int flags, void* workspace,
                               size_t ws_bytes, int* status_word, void* stream);

/* Multi-head self-attention over a packed tensor, replacing the layer "multi_head_attention_mma_layer"
 * that MultiHeadAttentionMMA builds (python/ditto/auto_compute/nn/module/self_attention.py:15-82):
 *   qkv [batch, M, 3 * heads * head_dim] = [Q | K | V] per row; out [batch, M, heads * head_dim].
 * The reference splits, reshapes to [batch*heads, M, d], transposes K and reshapes the result back in
 * six extra passes; here the head split is done by the TMA coordinates and the result is written in
 * place.  scale 1.0 = the reference's semantics.  head_dim and M multiples of 16, head_dim <= 128. */
int ditto_b200_multi_head_attention(const void* qkv, void* out, int batch, int M, int heads, int head_dim, int dtype,
                                    float scale, int flags, int* status_word, void* stream);

/* Fused MLP chain  y = act(X W1) W2 with the hidden activations kept on chip, replacing the
 * module built from BatchGemmReluGemm (python_test/auto_tensorize/test_hyper_fusion_cpu.py:24-96,
 * evaluation/cpu/bmm_relu_bmm.py:56-125) and, with epilogue 0, BatchGemmGemm
 * (benchmark/chimera/cuda/bmm_bmm_cuda.py:69-150).
 *   x [batch, M, K]; w1 [batch, K, L]; w2 [batch, L, N]; y [batch, M, N]
 *   w_layout 0: weights as above ([in, out]); 1: [out, in] as in nn/functional/linear.py:4-41
 *   epilogue 0: identity between the GEMMs; 1: ReLU; | DITTO_EPILOGUE_PAIR_MMA / _QUAD_MMA / _WIDE_MMA
 *   forces one of the kernels (same results up to fp32 summation order; default: by shape)
 *   workspace / ws_bytes: optional scratch memory (ditto_b200_workspace_bytes; contents irrelevant on entry,
 *   undefined on return).  With few row blocks several clusters share a row block, each takes a range of the
 *   hidden dimension and the fp32 partials of Y are added through the scratch memory in a fixed order (the
 *   hidden activations still never leave the chip).  NULL or too small: one cluster per row block.
 * Shapes: N <= 128 and K <= 128 (any multiples of 16, either weight layout): the reference's own shape family;
 * otherwise L % 128 == 0, K % 64 == 0, N in {256, 512, 768, 1024}, or -- on the default kernel -- L % 64 == 0,
 * K % 16 == 0 and N any multiple of 256 up to 16384 (results wider than 1024 columns are computed in column
 * groups of at most 1024, one launch each in stream order, GEMM1 recomputed per group); M any multiple of 16. */
int ditto_b200_gemm_relu_gemm(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N,
                              int K, int L, int dtype, int w_layout, int epilogue, void* workspace,
                              size_t ws_bytes, int* status_word, void* stream);

/* The MLP chain for callers that cannot allocate device memory.  No counterpart in the reference.
 *
 * ditto_b200_gemm_relu_gemm runs fastest on few row blocks when it is handed scratch memory, and somebody has
 * to own that memory.  Some callers cannot: code that runs while a CUDA graph is being captured or inside a
 * library's callback, where cudaMalloc is forbidden or would synchronise the device; plugins whose host hands
 * them input and output buffers and nothing else; services with a fixed memory budget decided at start-up.
 * For them the scratch memory is part of the library image: a 12 MiB array in device memory, which every GPU
 * that loads the library holds until the process exits.  This entry point and everything under it call no
 * cudaMalloc, cudaFree or other allocating routine.
 *
 *   Arguments as ditto_b200_gemm_relu_gemm without workspace / ws_bytes; epilogue 0 or 1 (no kernel bits: the
 *   four-CTA kernel is used).  Shapes: L % 128 == 0, K % 64 == 0, N in {256, 512, 768, 1024}, M % 16 == 0.
 *   Results are those of ditto_b200_gemm_relu_gemm | DITTO_EPILOGUE_QUAD_MMA with a workspace, bit for bit.
 *   Limit: a shape whose plan needs more than the 12 MiB returns DITTO_ERR_WORKSPACE (text in
 *   ditto_b200_last_cuda_error()) and launches nothing; use the entry point with a caller workspace then.
 *   First call on a device: looks up the array's device address (cudaGetSymbolAddress, with that device
 *   current) and the kernel's attributes, and keeps them.  Make that first call outside any stream capture.
 *   Every call on a device uses the same array.  The part that must start at zero (a few counters) is cleared
 *   on `stream` in front of the kernel; the rest is written before it is read.  Two calls that overlap on the
 *   GPU (different streams, no dependency) race on it: order them, or give one of them its own workspace. */
int ditto_b200_gemm_relu_gemm_static_scratch(const void* x, const void* w1, const void* w2, void* y, int batch, int M,
                                             int N, int K, int L, int dtype, int w_layout, int epilogue,
                                             int* status_word, void* stream);

/* Position-wise feed-forward block  y = act2(act1(X W1 + b1) W2 + b2)  with the hidden layer on chip, the
 * fused form of PositionwiseFeedForward (python/ditto/auto_compute/nn/model/transformer.py:21-34:
 * linear -> ReLU -> linear -> ReLU, linear with bias as in nn/functional/linear.py:4-41; GELU as in
 * nn/functional/activation.py:29-39).
 *   b1 [batch, L], b2 [batch, N]: bias vectors in the input type, either may be NULL
 *   act1 / act2: 0 identity, 1 ReLU, 2 GELU (tanh form)
 * Shapes as for the large-N form of ditto_b200_gemm_relu_gemm (L % 128 == 0 with K % 64 == 0 and N in {256, 512,
 * 768, 1024}; L % 64 == 0 with K % 16 == 0 and N any multiple of 256; M any multiple of 16). */
int ditto_b200_ffn(const void* x, const void* w1, const void* b1, const void* w2, const void* b2, void* y, int batch,
                   int M, int N, int K, int L, int dtype, int w_layout, int act1, int act2, int* status_word,
                   void* stream);

/* Scratch bytes with which the op runs fastest at this shape on the current device (0 when none; every call
 * also works without).  `op` may be or-ed with DITTO_EPILOGUE_PAIR_MMA / DITTO_EPILOGUE_QUAD_MMA / DITTO_EPILOGUE_WIDE_MMA to ask for the
 * kernel that the same bits in `epilogue` select. */
size_t ditto_b200_workspace_bytes(int op, int batch, int M, int N, int K, int L, int dtype);

/* How many thread-block clusters of the MLP chain kernel the current device holds at once
 * (cudaOccupancyMaxActiveClusters): the number of row blocks -- or, for the pair kernel, (row block,
 * hidden range) items -- that run concurrently; a launch takes ceil(items / slots) waves.
 * variant: DITTO_EPILOGUE_PAIR_MMA (clusters of eight), DITTO_EPILOGUE_QUAD_MMA or DITTO_EPILOGUE_WIDE_MMA
 * (clusters of four).
 * Returns the count, or a negative DITTO_ERR_* code.  No counterpart in the reference (its schedules are
 * sized by the hardware table of python/ditto/hardware/__init__.py:43-54). */
int ditto_b200_mlp_cluster_slots(int dtype, int variant);

/* Single-CTA check of one tcgen05 MMA chain: c[128, N] (fp32) = a[128, K] * b.
 *   b_mn 0: b is [N, K]; 1: b is [K, N].  a_tmem 1: the A operand is read from tensor memory.
 * N, K multiples of 64, at most 256.  Exists so the descriptor encodings the fused kernels depend
 * on can be verified one at a time; it has no counterpart in the reference. */
int ditto_b200_selftest_umma(const void* a, const void* b, float* c, int N, int K, int dtype, int b_mn,
                             int a_tmem, int* status_word, void* stream);

/* The same check for a CTA pair (cta_group::2): c[256, N] = a[256, K] * b, N in {128, 256}.
 * No counterpart in the reference. */
int ditto_b200_selftest_umma_pair(const void* a, const void* b, float* c, int N, int K, int dtype, int b_mn,
                                  int* status_word, void* stream);

/* Exercises the failure path of the device-side waits without faulting anything: one CTA waits, with the
 * same bounded wait every kernel here uses, on a barrier that nothing ever signals; when the limit is
 * reached the wait gives up, the kernel writes `code` to *status_word and ends normally, and the context
 * stays usable.  Takes about a second.  No counterpart in the reference. */
int ditto_b200_selftest_wait_limit(int code, int* status_word, void* stream);

/* Waits for `stream`, reads the status word the calls on it were given and returns DITTO_OK if it is zero,
 * else DITTO_ERR_TIMEOUT (a device-side bounded wait expired in one of them: their outputs are not valid);
 * the word is cleared again and its value -- which wait gave up -- is stored in *code_out (may be NULL).
 * The reference reports a failed kernel as a tvm::Error out of the module call
 * (src/runtime/graph_runtime.cc:212-226 synchronises the same way); no counterpart for the code itself. */
int ditto_b200_check_status(int* status_word, void* stream, int* code_out);

const char* ditto_b200_strerror(int code);
/* Text of the last CUDA / driver error seen by the calling thread ("" if none). */
const char* ditto_b200_last_cuda_error(void);
int ditto_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DITTO_B200_H_ */
