// Host-visible launch interface of the fused bmm -> softmax -> bmm kernel.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace ditto_b200 {

// Tensor maps are 3-D (column, row inside the sequence, sequence) so that a partial tile at the end
// of a sequence is zero-filled by TMA instead of reading the next sequence's rows.
struct AttnParams {
  CUtensorMap map_q;  // [batch, M, d] (or the packed [batch, M, 3*hidden]), box 64 x 128 x 1, 128B swizzle
  CUtensorMap map_k;  // [batch, L, d] (box 64 x 128 x 1) or, transposed, [batch, d, L] (box 64 x D x 1)
  CUtensorMap map_v;  // [batch, L, dv], box 64 x 128 x 1
  void* out;          // [batch, M, dv] fp16 / bf16
  int M;              // query rows per sequence (any multiple of 16)
  int L;              // key/value rows per sequence (any multiple of 16)
  int d;              // width of Q and K in use: the reduction length of S = Q K^T (multiple of 16, <= the kernel's D)
  int dv;             // width of V and of the output (multiple of 16, <= the kernel's D); columns beyond it are zero-filled / not stored
  int k_transposed;   // 1: K stored [batch, D, L] (the reference's layout)
  int v_transposed;   // 1: V stored [batch, dv, L] (map_v: box 64 x D x 1; the [out, in] second weight of a small-N chain)
  int heads;          // 1, or heads folded into the slice index of a packed [sequences, rows, cols] input
  int q_col0, k_col0, v_col0;  // first column of Q / K / V inside the packed row (0 when not packed)
  int out_ld;         // elements between output rows (D when not packed)
  int items;          // work items of the launch: slices x tiles of NT x 128 query rows (filled in by the launcher)
  float scale_log2;   // softmax scale * log2(e)
  int* status;        // device word receiving a non-zero code if a bounded wait expired; may be null
  long long* trace;   // timeline buffer of -DDITTO_TRACE builds (null otherwise)
};

// d in {64,128}; nt in {1,2} query tiles per CTA; psmem: stage P through shared memory instead of TMEM
// (softmax mode only); mode 0 softmax, 1 ReLU, 2 identity between the two GEMMs.
cudaError_t launch_attention(const AttnParams& p, int batch, int d, bool bf16, int nt, bool psmem, int mode,
                             cudaStream_t stream);

// Persistent variant for head dimensions up to 64 (attention_persistent_sm100.cu): two CTAs per SM walk the
// (slice, tile) work items.  mode as above.
cudaError_t launch_attention_persistent(const AttnParams& p, int batch, bool bf16, int mode, cudaStream_t stream);

}  // namespace ditto_b200
