// Device helpers shared by the cluster kernels of the GEMM -> activation -> GEMM chain.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

namespace ditto_b200 {

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (BF16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
  }
}

// Activation codes of the chain: 0 identity, 1 ReLU, 2 GELU (tanh form).
template <int ACT>
__device__ __forceinline__ float act_apply(float v) {
  if constexpr (ACT == 1) {
    return v > 0.f ? v : 0.f;                      // if_then_else(x > 0, x, 0) as in the reference's ReLU
  } else if constexpr (ACT == 2) {                 // the reference's GELU: 0.5 x (1 + tanh(0.79788456 x (1 + 0.044715 x^2)))
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(v * 0.7978845608f * (1.0f + 0.044715f * v * v)));
    return 0.5f * v * (1.0f + t);
  } else {
    return v;
  }
}

// N fp32 accumulator values of one row (+ a 16-bit bias vector, the same address in every lane: broadcast
// loads) -> activation -> N / 2 packed 16-bit pairs.  The activation and the presence of a bias are
// compile-time here: a run-time test per element costs a branch per element, which made this loop the
// longest step of the hidden-chunk hand-over.
// VEC: the bias pointer is 16-byte aligned and is read eight values at a time (a load per pair of columns is
// 64 load instructions per thread and hidden chunk).
template <bool BF16, int ACT, bool BIAS, int N, bool VEC = false>
__device__ __forceinline__ void act_pack_fixed(const uint32_t (&acc)[N], const uint32_t* bias, uint32_t (&out)[N / 2]) {
  uint32_t bw[BIAS ? N / 2 : 1];
  if constexpr (BIAS) {
    if constexpr (VEC) {
#pragma unroll
      for (int j4 = 0; j4 < N / 8; ++j4) {
        const uint4 t = __ldg(reinterpret_cast<const uint4*>(bias) + j4);
        bw[4 * j4] = t.x; bw[4 * j4 + 1] = t.y; bw[4 * j4 + 2] = t.z; bw[4 * j4 + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < N / 2; ++j) bw[j] = __ldg(bias + j);
    }
  }
#pragma unroll
  for (int j = 0; j < N / 2; ++j) {
    float v0 = __uint_as_float(acc[2 * j]), v1 = __uint_as_float(acc[2 * j + 1]);
    if constexpr (BIAS) {
      const float2 bb = unpack2<BF16>(bw[j]);
      v0 += bb.x;
      v1 += bb.y;
    }
    out[j] = pack2<BF16>(act_apply<ACT>(v0), act_apply<ACT>(v1));
  }
}
// The same with the bias values already in registers (two 16-bit values per word).
template <bool BF16, int ACT, int N>
__device__ __forceinline__ void act_pack_words(const uint32_t (&acc)[N], const uint32_t (&bw)[N / 2], uint32_t (&out)[N / 2]) {
#pragma unroll
  for (int j = 0; j < N / 2; ++j) {
    const float2 bb = unpack2<BF16>(bw[j]);
    out[j] = pack2<BF16>(act_apply<ACT>(__uint_as_float(acc[2 * j]) + bb.x), act_apply<ACT>(__uint_as_float(acc[2 * j + 1]) + bb.y));
  }
}
// One warp-uniform dispatch per call instead of one per element.
template <bool BF16, int N>
__device__ __forceinline__ void act_pack(const uint32_t (&acc)[N], const uint32_t* bias, int act, uint32_t (&out)[N / 2]) {
  if (bias == nullptr) {
    if (act == 1) act_pack_fixed<BF16, 1, false, N>(acc, bias, out);
    else if (act == 2) act_pack_fixed<BF16, 2, false, N>(acc, bias, out);
    else act_pack_fixed<BF16, 0, false, N>(acc, bias, out);
  } else {
    if (act == 1) act_pack_fixed<BF16, 1, true, N>(acc, bias, out);
    else if (act == 2) act_pack_fixed<BF16, 2, true, N>(acc, bias, out);
    else act_pack_fixed<BF16, 0, true, N>(acc, bias, out);
  }
}
__device__ __forceinline__ float act_apply_rt(float v, int act) {
  return act == 1 ? act_apply<1>(v) : act == 2 ? act_apply<2>(v) : v;
}

// Four consecutive lanes (a = lane & 3) each hold four 16-byte pieces v[b][0..3], b = 0 .. 3, of their own row:
// afterwards lane a holds piece a of row b of the group in v[b] -- a 4 x 4 transpose by two rounds of pairwise
// exchanges -- so that one store instruction writes 64 contiguous bytes of a row instead of 16.
__device__ __forceinline__ void quad_transpose(uint32_t (&v)[4][4], int a) {
#pragma unroll
  for (int b = 0; b < 4; b += 2) {              // lanes a ^ 1 exchange pieces b / b + 1
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t give = (a & 1) ? v[b][j] : v[b + 1][j];
      const uint32_t got = __shfl_xor_sync(0xffffffffu, give, 1);
      if (a & 1) v[b][j] = got; else v[b + 1][j] = got;
    }
  }
#pragma unroll
  for (int b = 0; b < 2; ++b) {                 // lanes a ^ 2 exchange pieces b / b + 2
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t give = (a & 2) ? v[b][j] : v[b + 2][j];
      const uint32_t got = __shfl_xor_sync(0xffffffffu, give, 2);
      if (a & 2) v[b][j] = got; else v[b + 2][j] = got;
    }
  }
}

// Last step of a row block that several clusters shared: add the clusters' fp32 partials of a
// rows x cols region of Y (one slab per cluster, `slab_stride` floats apart, row pitch `ld` floats) in
// slab order, apply bias and activation, write the 16-bit result.  `nthreads` threads of one CTA call it with
// tid = 0 .. nthreads - 1.  Every thread issues the loads of J float4 positions in all P slabs before the
// first add: with one load in flight at a time this pass is bound by L2 latency (measured 100 us for
// 128 x 256 x 8 slabs), with J x P = 16 in flight it takes a few microseconds.
constexpr int kMaxSlabs = 8;
template <bool BF16, int J, int P>
__device__ __forceinline__ void combine_slabs_fixed(const float* slab0, size_t slab_stride, int parts, int rows, int cols,
                                                    size_t ld, const uint32_t* bias, int act, uint8_t* y,
                                                    size_t y_pitch_bytes, int tid, int nthreads) {
  const int per_row = cols / 4;
  const int total = rows * per_row;
  for (int base = 0; base < total; base += J * nthreads) {
    float4 v[J][P];
    int r[J], c[J];
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int idx = base + j * nthreads + tid;
      r[j] = idx / per_row;
      c[j] = (idx - r[j] * per_row) * 4;
#pragma unroll
      for (int s = 0; s < P; ++s)
        if (idx < total && s < parts)
          v[j][s] = __ldcg(reinterpret_cast<const float4*>(slab0 + static_cast<size_t>(s) * slab_stride + static_cast<size_t>(r[j]) * ld + c[j]));
    }
#pragma unroll
    for (int j = 0; j < J; ++j) {
      if (base + j * nthreads + tid >= total) continue;
      float4 acc = v[j][0];
#pragma unroll
      for (int s = 1; s < P; ++s)
        if (s < parts) {
          acc.x += v[j][s].x; acc.y += v[j][s].y; acc.z += v[j][s].z; acc.w += v[j][s].w;
        }
      if (bias != nullptr) {
        const float2 b01 = unpack2<BF16>(__ldg(bias + c[j] / 2)), b23 = unpack2<BF16>(__ldg(bias + c[j] / 2 + 1));
        acc.x += b01.x; acc.y += b01.y; acc.z += b23.x; acc.w += b23.y;
      }
      const uint2 out = make_uint2(pack2<BF16>(act_apply_rt(acc.x, act), act_apply_rt(acc.y, act)),
                                   pack2<BF16>(act_apply_rt(acc.z, act), act_apply_rt(acc.w, act)));
      *reinterpret_cast<uint2*>(y + static_cast<size_t>(r[j]) * y_pitch_bytes + c[j] * 2) = out;
    }
  }
}
template <bool BF16>
__device__ __forceinline__ void combine_slabs(const float* slab0, size_t slab_stride, int parts, int rows, int cols,
                                              size_t ld, const uint32_t* bias, int act, uint8_t* y, size_t y_pitch_bytes,
                                              int tid, int nthreads) {
  if (parts <= 2)
    combine_slabs_fixed<BF16, 8, 2>(slab0, slab_stride, parts, rows, cols, ld, bias, act, y, y_pitch_bytes, tid, nthreads);
  else if (parts <= 4)
    combine_slabs_fixed<BF16, 4, 4>(slab0, slab_stride, parts, rows, cols, ld, bias, act, y, y_pitch_bytes, tid, nthreads);
  else
    combine_slabs_fixed<BF16, 2, kMaxSlabs>(slab0, slab_stride, parts, rows, cols, ld, bias, act, y, y_pitch_bytes, tid, nthreads);
}

// Bulk copy from this CTA's shared memory into a peer's; completion (bytes) on the peer's mbarrier.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster_addr, const void* src, uint32_t bytes,
                                                  uint32_t mbar_cluster_addr) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster_addr), "r"(smem_u32(src)), "r"(bytes), "r"(mbar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_word,
                                                  uint32_t code) {
  for (uint32_t spin = 0; spin < (1u << 22); ++spin) {   // unhinted polls: the default limit
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (*abort_word != 0u) return false;
    if (spin > 4096u) __nanosleep(64);
  }
  atomicCAS(const_cast<uint32_t*>(abort_word), 0u, code);
  return false;
}


}  // namespace ditto_b200
