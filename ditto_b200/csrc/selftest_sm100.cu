// Single-CTA unit test of the tcgen05 building blocks: C[128, N] = A[128, K] * B
// with one MMA chain, so that every operand form the fused kernels rely on can be
// checked in isolation against a CPU product:
//   b_mn = 0 : B stored [N, K] (K contiguous, "K-major"), as K in S = Q * K^T
//   b_mn = 1 : B stored [K, N] (N contiguous, "MN-major"), as V in O = P * V
//   a_tmem = 1 : A is first copied into TMEM (two 16-bit values per column) and
//               the MMA reads it from there, as P in O = P * V
#include "selftest_sm100.cuh"

#include "sm100_ptx.cuh"

namespace ditto_b200 {

namespace {
struct TestBars {
  uint64_t full;
  uint64_t done;
  uint32_t tmem_base;
  uint32_t abort_word;
};
}  // namespace

__global__ void __launch_bounds__(128, 1) umma_selftest_kernel(const __grid_constant__ SelftestParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int a_bytes = 128 * p.K * 2;
  const int b_bytes = p.N * p.K * 2;
  uint8_t* sa = smem;
  uint8_t* sb = smem + a_bytes;
  TestBars* bar = reinterpret_cast<TestBars*>(sb + b_bytes);
  volatile uint32_t* abort_word = &bar->abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&bar->full, 1);
    mbar_init(&bar->done, 1);
    bar->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&bar->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bar->tmem_base;

  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(&bar->full, a_bytes + b_bytes);
    for (int a = 0; a < p.K / 64; ++a) tma_load_2d(sa + a * (128 * 128), &p.map_a, &bar->full, a * 64, 0);
    if (p.b_mn) {
      for (int a = 0; a < p.N / 64; ++a) tma_load_2d(sb + a * (p.K * 128), &p.map_b, &bar->full, a * 64, 0);
    } else {
      for (int a = 0; a < p.K / 64; ++a) tma_load_2d(sb + a * (p.N * 128), &p.map_b, &bar->full, a * 64, 0);
    }
  }
  bool ok = mbar_wait(&bar->full, 0, abort_word, 0x10);
  ok = __syncthreads_and(ok);

  const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  if (ok && p.a_tmem) {
    // Row r of A (K 16-bit values) -> TMEM lane r, columns [256, 256 + K/2).
    const uint32_t* arow = reinterpret_cast<const uint32_t*>(p.a_global) + static_cast<size_t>(threadIdx.x) * (p.K / 2);
    for (int c = 0; c < p.K / 2; c += 8) {
      uint32_t r[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) r[i] = arow[c + i];
      tmem_st_x8(lane_base + 256 + c, r);
    }
    tmem_wait_st();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  if (ok && threadIdx.x == 0) {
    const uint32_t idesc = umma_idesc_f16(p.bf16 != 0, 128, p.N, false, p.b_mn != 0);
    const uint32_t a_addr = smem_u32(sa), b_addr = smem_u32(sb);
    for (int i = 0; i < p.K / 16; ++i) {
      uint64_t db;
      if (p.b_mn)
        db = umma_desc_sw128(b_addr + i * 2048, p.K * 128, 1024);
      else
        db = umma_desc_sw128(b_addr + (i / 4) * (p.N * 128) + (i % 4) * 32, 16, 1024);
      if (p.a_tmem) {
        umma_ts(tmem_base, tmem_base + 256 + i * 8, db, idesc, i > 0);
      } else {
        const uint64_t da = umma_desc_sw128(a_addr + (i / 4) * (128 * 128) + (i % 4) * 32, 16, 1024);
        umma_ss(tmem_base, da, db, idesc, i > 0);
      }
    }
    umma_commit(&bar->done);
  }
  __syncwarp();
  if (ok) ok = mbar_wait(&bar->done, 0, abort_word, 0x20);
  ok = __all_sync(0xffffffffu, ok);
  if (ok) {
    tc_fence_after_sync();
    float* crow = p.c + static_cast<size_t>(threadIdx.x) * p.N;
    for (int c = 0; c < p.N; c += 8) {
      uint32_t r[8];
      tmem_ld_x8_wait(lane_base + c, r);
#pragma unroll
      for (int i = 0; i < 8; ++i) crow[c + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tmem_dealloc(tmem_base, 512);
    if (lane == 0 && bar->abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, static_cast<int>(bar->abort_word));
  }
}

cudaError_t launch_umma_selftest(const SelftestParams& p, cudaStream_t stream) {
  const int smem = 128 * p.K * 2 + p.N * p.K * 2 + 64 + 1024;
  cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  umma_selftest_kernel<<<1, 128, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace ditto_b200

// ------------------------------------------------------------------ CTA-pair self test
// C[256, N] = A[256, K] * B with one cta_group::2 MMA chain: cluster of two CTAs, each holding its
// 128 rows of A and half of B's N extent, the leader (rank 0) issuing.  Checks the pair mechanics
// (2-CTA TMEM allocation, TMA byte counts reported to the leader's barrier, operand split,
// completion signalled to both CTAs) in isolation.
namespace ditto_b200 {

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1)
    umma_pair_selftest_kernel(const __grid_constant__ SelftestParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int half_n = p.N / 2;
  const int a_bytes = 128 * p.K * 2;
  const int b_bytes = half_n * p.K * 2;
  uint8_t* sa = smem;
  uint8_t* sb = smem + a_bytes;
  TestBars* bar = reinterpret_cast<TestBars*>(sb + b_bytes);
  volatile uint32_t* abort_word = &bar->abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();

  if (threadIdx.x == 0) {
    mbar_init(&bar->full, 1);
    mbar_init(&bar->done, 1);
    bar->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc_pair(&bar->tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = bar->tmem_base;

  if (threadIdx.x == 0) {
    const uint32_t leader_full = map_to_cta(smem_u32(&bar->full), 0);
    if (rank == 0) mbar_arrive_expect_tx(&bar->full, 2 * (a_bytes + b_bytes));
    for (int a = 0; a < p.K / 64; ++a)
      tma_load_2d_pair(sa + a * (128 * 128), &p.map_a, leader_full, a * 64, static_cast<int>(rank) * 128);
    if (p.b_mn) {
      for (int a = 0; a < half_n / 64; ++a)
        tma_load_2d_pair(sb + a * (p.K * 128), &p.map_b, leader_full, static_cast<int>(rank) * half_n + a * 64, 0);
    } else {
      for (int a = 0; a < p.K / 64; ++a)
        tma_load_2d_pair(sb + a * (half_n * 128), &p.map_b, leader_full, a * 64, static_cast<int>(rank) * half_n);
    }
  }
  bool ok = true;
  if (warp == 0 && rank == 0) {
    const uint32_t issuer = elect_one();
    ok = mbar_wait(&bar->full, 0, abort_word, 0x10);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after_sync();
    if (ok) {
      const uint32_t idesc = umma_idesc_f16(p.bf16 != 0, 256, p.N, false, p.b_mn != 0);
      const uint32_t a_addr = smem_u32(sa), b_addr = smem_u32(sb);
      for (int i = 0; i < p.K / 16; ++i) {
        const uint64_t da = umma_desc_sw128(a_addr + (i / 4) * (128 * 128) + (i % 4) * 32, 16, 1024);
        const uint64_t db = p.b_mn ? umma_desc_sw128(b_addr + i * 2048, p.K * 128, 1024)
                                   : umma_desc_sw128(b_addr + (i / 4) * (half_n * 128) + (i % 4) * 32, 16, 1024);
        umma_ss_pair_elected(tmem_base, da, db, idesc, i > 0, issuer);
      }
      umma_commit_pair_elected(&bar->done, 0x3, issuer);
    }
  }
  __syncwarp();
  ok = mbar_wait(&bar->done, 0, abort_word, 0x20);
  ok = __all_sync(0xffffffffu, ok);
  if (ok) {
    tc_fence_after_sync();
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    float* crow = p.c + (static_cast<size_t>(rank) * 128 + threadIdx.x) * p.N;
    for (int c = 0; c < p.N; c += 8) {
      uint32_t r[8];
      tmem_ld_x8_wait(lane_base + c, r);
#pragma unroll
      for (int i = 0; i < 8; ++i) crow[c + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 0) {
    tmem_dealloc_pair(tmem_base, 512);
    if (lane == 0 && bar->abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, static_cast<int>(bar->abort_word));
  }
}

cudaError_t launch_umma_pair_selftest(const SelftestParams& p, cudaStream_t stream) {
  const int smem = 128 * p.K * 2 + (p.N / 2) * p.K * 2 + 64 + 1024;
  cudaError_t e = cudaFuncSetAttribute(umma_pair_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  umma_pair_selftest_kernel<<<2, 128, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace ditto_b200

// ------------------------------------------------------------------ bounded-wait self test
// The failure path every kernel of the library relies on, run on purpose and harmlessly: a barrier
// that is never signalled, the shared bounded wait, the abort word, the host-visible status word.
namespace ditto_b200 {

__global__ void __launch_bounds__(64, 1) wait_limit_selftest_kernel(int code, int* status) {
  __shared__ uint64_t never;
  __shared__ uint32_t abort_word_storage;
  volatile uint32_t* abort_word = &abort_word_storage;
  if (threadIdx.x == 0) {
    mbar_init(&never, 1);
    abort_word_storage = 0;
    fence_mbar_init();
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait(&never, 0, abort_word, static_cast<uint32_t>(code));   // gives up at the limit
  // the other waiter sees the abort word the first one set and returns at once, as the kernels' warps do
  __syncthreads();
  if (threadIdx.x == 32) ok = mbar_wait(&never, 0, abort_word, 0x7fffffffu);
  __syncthreads();
  if (threadIdx.x == 0 && status != nullptr && abort_word_storage != 0) atomicCAS(status, 0, static_cast<int>(abort_word_storage));
  (void)ok;
}

cudaError_t launch_wait_limit_selftest(int code, int* status, cudaStream_t stream) {
  wait_limit_selftest_kernel<<<1, 64, 0, stream>>>(code, status);
  return cudaGetLastError();
}

}  // namespace ditto_b200
