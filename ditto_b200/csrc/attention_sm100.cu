// Fused bmm -> softmax -> bmm for sm_100a.
//
// Replaces the two kernels the reference generates for this chain
// (src/auto_tensorize/hyper_fusion.cc:1494-1603 schedules a WMMA kernel that
// writes fp32 partial results plus a separate divide kernel; the arithmetic is
// python/ditto/auto_compute/nn/functional/bmm_chain.py:40-103) by ONE kernel:
//
//   S = Q * K^T           tcgen05.mma, fp32 accumulator in TMEM
//   P = exp2((S - m)*c)   online softmax, one thread per query row
//   O += P * V            tcgen05.mma, P read from TMEM (or swizzled smem)
//   out = O / rowsum(P)   epilogue, written once as fp16 / bf16
//
// The score tile never leaves the SM.  One CTA owns NT (1 or 2) tiles of 128
// query rows of one slice (batch x head) and streams the slice's K/V in blocks
// of 128 rows through a TMA-fed ring of 128B-swizzled shared-memory stages.
//
// Warp roles (320 threads):
//   warps 0-3   softmax + epilogue for query tile 0  (thread i <-> row i, TMEM lane i)
//   warps 4-7   softmax + epilogue for query tile 1
//   warp  8     TMA producer (one lane issues)
//   warp  9     MMA issuer   (one lane issues)
// With two tiles the tensor pipe works on one tile while the other tile's
// softmax runs, so the exponentials overlap the MMAs.
//
// TMEM columns (512 allocated): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).
// P (16-bit, two values per 32-bit column) overwrites the first 64 columns of
// its own S tile; the next S MMA for that tile is issued after the P*V MMA
// that reads it, and the tensor pipe executes one thread's MMAs in order.
#include "attention_sm100.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

namespace ditto_b200 {

namespace {

constexpr int kBM = 128;   // query rows per tile
constexpr int kBN = 128;   // K/V rows per block
constexpr int kThreads = 320;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units; P stays <= 2^8 with a stale max

template <int D, int NT, bool PSMEM>
struct Smem {
  static constexpr int kTileQ = kBM * D * 2;
  static constexpr int kTileKV = kBN * D * 2;
  static constexpr int kTileP = kBM * kBN * 2;
  static constexpr int kStages = PSMEM ? (D == 64 ? 3 : 1) : (D == 64 ? 4 : 2);
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + NT * kTileQ;
  static constexpr int kOffV = kOffK + kStages * kTileKV;
  static constexpr int kOffP = kOffV + kStages * kTileKV;
  static constexpr int kOffBar = kOffP + (PSMEM ? NT * kTileP : 0);
  static constexpr int kBytes = kOffBar + 512 + 1024;  // barriers + slack for 1024-byte alignment
};

struct Barriers {
  uint64_t q_full;
  uint64_t k_full[4], k_empty[4], v_full[4], v_empty[4];
  uint64_t s_full[2], p_full[2], o_done[2];
  uint32_t tmem_base;
  uint32_t abort_word;
};
static_assert(sizeof(Barriers) <= 512, "barrier block too large");

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

}  // namespace

template <bool BF16, int D, int NT, bool PSMEM>
__global__ void __launch_bounds__(kThreads, 1) attention_kernel(const __grid_constant__ AttnParams p) {
  using SM = Smem<D, NT, PSMEM>;
  constexpr int kStages = SM::kStages;
  constexpr int kAtoms = D / 64;  // 64-element (128-byte) chunks along the head dimension

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Barriers* bar = reinterpret_cast<Barriers*>(smem + SM::kOffBar);
  volatile uint32_t* abort_word = &bar->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slice = blockIdx.y;
  const int m0 = blockIdx.x * (NT * kBM);
  const int nkv = p.L / kBN;

  if (threadIdx.x == 0) {
    mbar_init(&bar->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bar->k_full[s], 1);
      mbar_init(&bar->k_empty[s], 1);
      mbar_init(&bar->v_full[s], 1);
      mbar_init(&bar->v_empty[s], 1);
    }
    for (int t = 0; t < NT; ++t) {
      mbar_init(&bar->s_full[t], 1);
      mbar_init(&bar->p_full[t], kBM);
      mbar_init(&bar->o_done[t], 1);
    }
    bar->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&bar->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bar->tmem_base;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&p.map_q);
      tma_prefetch_desc(&p.map_k);
      tma_prefetch_desc(&p.map_v);
      mbar_arrive_expect_tx(&bar->q_full, NT * SM::kTileQ);
      for (int t = 0; t < NT; ++t)
        for (int a = 0; a < kAtoms; ++a)
          tma_load_2d(smem + SM::kOffQ + t * SM::kTileQ + a * (kBM * 128), &p.map_q, &bar->q_full, a * 64,
                      slice * p.M + m0 + t * kBM);
    }
    bool ok = true;
    int armed_k[4] = {-1, -1, -1, -1}, armed_v[4] = {-1, -1, -1, -1};  // parity of the newest armed phase
    for (int j = 0; j < nkv; ++j) {
      const int s = j % kStages;
      const uint32_t ph = (j / kStages) & 1;
      ok = mbar_wait(&bar->k_empty[s], ph ^ 1, abort_word, 0x100 + j);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        uint8_t* dst = smem + SM::kOffK + s * SM::kTileKV;
        mbar_arrive_expect_tx(&bar->k_full[s], SM::kTileKV);
        armed_k[s] = static_cast<int>(ph);
        if (p.k_transposed) {
          // K given as [slice, D, L]: boxes of 64 kv-columns x D rows (MN-major operand)
          for (int a = 0; a < kBN / 64; ++a)
            tma_load_2d(dst + a * (D * 128), &p.map_k, &bar->k_full[s], j * kBN + a * 64, slice * D);
        } else {
          for (int a = 0; a < kAtoms; ++a)
            tma_load_2d(dst + a * (kBN * 128), &p.map_k, &bar->k_full[s], a * 64, slice * p.L + j * kBN);
        }
      }
      ok = mbar_wait(&bar->v_empty[s], ph ^ 1, abort_word, 0x200 + j);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        uint8_t* dst = smem + SM::kOffV + s * SM::kTileKV;
        mbar_arrive_expect_tx(&bar->v_full[s], SM::kTileKV);
        armed_v[s] = static_cast<int>(ph);
        for (int a = 0; a < kAtoms; ++a)
          tma_load_2d(dst + a * (kBN * 128), &p.map_v, &bar->v_full[s], a * 64, slice * p.L + j * kBN);
      }
    }
    if (!ok && lane == 0) {
      // Drain: let copies that were already issued land before the CTA exits.
      for (int s = 0; s < kStages; ++s) {
        if (armed_k[s] >= 0)
          for (uint32_t spin = 0; spin < (1u << 20) && !mbar_try_wait(&bar->k_full[s], armed_k[s]); ++spin) {}
        if (armed_v[s] >= 0)
          for (uint32_t spin = 0; spin < (1u << 20) && !mbar_try_wait(&bar->v_full[s], armed_v[s]); ++spin) {}
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    const uint32_t idesc_s = umma_idesc_f16(BF16, kBM, kBN, false, p.k_transposed != 0);
    const uint32_t idesc_o = umma_idesc_f16(BF16, kBM, D, false, true);
    const uint32_t q_addr = smem_u32(smem + SM::kOffQ);
    const uint32_t k_addr = smem_u32(smem + SM::kOffK);
    const uint32_t v_addr = smem_u32(smem + SM::kOffV);
    const uint32_t p_addr = smem_u32(smem + SM::kOffP);

    auto issue_s = [&](int t, int stage) {
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
          const uint64_t da =
              umma_desc_sw128(q_addr + t * SM::kTileQ + (i / 4) * (kBM * 128) + (i % 4) * 32, 16, 1024);
          uint64_t db;
          if (p.k_transposed)
            db = umma_desc_sw128(k_addr + stage * SM::kTileKV + i * 2048, D * 128, 1024);
          else
            db = umma_desc_sw128(k_addr + stage * SM::kTileKV + (i / 4) * (kBN * 128) + (i % 4) * 32, 16, 1024);
          umma_ss(tmem_base + t * kBN, da, db, idesc_s, i > 0 ? 1u : 0u);
        }
        umma_commit(&bar->s_full[t]);
      }
      __syncwarp();
    };
    auto issue_pv = [&](int t, int stage, bool accumulate) {
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < kBN / 16; ++i) {
          const uint64_t db = umma_desc_sw128(v_addr + stage * SM::kTileKV + i * 2048, kBN * 128, 1024);
          const uint32_t acc = (accumulate || i > 0) ? 1u : 0u;
          if constexpr (PSMEM) {
            const uint64_t da =
                umma_desc_sw128(p_addr + t * SM::kTileP + (i / 4) * (kBM * 128) + (i % 4) * 32, 16, 1024);
            umma_ss(tmem_base + 256 + t * D, da, db, idesc_o, acc);
          } else {
            umma_ts(tmem_base + 256 + t * D, tmem_base + t * kBN + i * 8, db, idesc_o, acc);
          }
        }
        umma_commit(&bar->o_done[t]);
      }
      __syncwarp();
    };
    auto commit_to = [&](uint64_t* b) {
      if (lane == 0) umma_commit(b);
      __syncwarp();
    };
    auto wait_all = [&](uint64_t* b, uint32_t parity, uint32_t code) {
      bool ok = mbar_wait(b, parity, abort_word, code);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
      return ok;
    };

    bool ok = wait_all(&bar->q_full, 0, 0x300);
    ok = ok && wait_all(&bar->k_full[0], 0, 0x301);
    if (ok) {
      issue_s(0, 0);
      if (NT == 2) issue_s(1, 0);
      commit_to(&bar->k_empty[0]);
    }
    for (int j = 0; j < nkv && ok; ++j) {
      const int sv = j % kStages;
      const int sk = (j + 1) % kStages;
      const bool more = (j + 1 < nkv);
      ok = wait_all(&bar->v_full[sv], (j / kStages) & 1, 0x400 + j);
      if (!ok) break;
      ok = wait_all(&bar->p_full[0], j & 1, 0x500 + j);
      if (!ok) break;
      issue_pv(0, sv, j > 0);
      if (NT == 1) commit_to(&bar->v_empty[sv]);
      if (more) {
        ok = wait_all(&bar->k_full[sk], ((j + 1) / kStages) & 1, 0x600 + j);
        if (!ok) break;
        issue_s(0, sk);
        if (NT == 1) commit_to(&bar->k_empty[sk]);
      }
      if (NT == 2) {
        ok = wait_all(&bar->p_full[1], j & 1, 0x700 + j);
        if (!ok) break;
        issue_pv(1, sv, j > 0);
        commit_to(&bar->v_empty[sv]);
        if (more) {
          issue_s(1, sk);
          commit_to(&bar->k_empty[sk]);
        }
      }
    }
  } else if (warp < 4 * NT) {
    // ------------------------------------------------------------ softmax + epilogue
    const int t = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t s_col = lane_base + t * kBN;
    const uint32_t o_col = lane_base + 256 + t * D;
    const float c = p.scale_log2;
    float m = -INFINITY, l = 0.f;
    bool ok = true;

    for (int j = 0; j < nkv; ++j) {
      ok = mbar_wait(&bar->s_full[t], j & 1, abort_word, 0x800 + j);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();

      uint32_t sv[kBN];
      tmem_ld_x128_wait(s_col, sv);

      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < kBN; i += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(sv[i + 0]));
        mx1 = fmaxf(mx1, __uint_as_float(sv[i + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(sv[i + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(sv[i + 3]));
      }
      const float m_new = fmaxf(m, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)));
      // Lazy rescale: keep the stale maximum while the true one is within
      // 2^kRescaleThreshold of it; the final division by l cancels the difference.
      const bool need = (m_new - m) * c > kRescaleThreshold;
      if (__any_sync(0xffffffffu, need)) {
        const float f = ex2_approx((m - m_new) * c);
        if (j > 0) {
          ok = mbar_wait(&bar->o_done[t], (j - 1) & 1, abort_word, 0x900 + j);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int cc = 0; cc < D; cc += 32) {
            uint32_t o[32];
            tmem_ld_x32_wait(o_col + cc, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
            tmem_st_x32(o_col + cc, o);
          }
          tmem_wait_st();
        }
        l *= f;
        m = m_new;
      }

      const float mc = m * c;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pk[kBN / 2];
#pragma unroll
      for (int i = 0; i < kBN / 2; ++i) {
        const float p0 = ex2_approx(fmaf(__uint_as_float(sv[2 * i]), c, -mc));
        const float p1 = ex2_approx(fmaf(__uint_as_float(sv[2 * i + 1]), c, -mc));
        sum0 += p0;
        sum1 += p1;
        pk[i] = pack2<BF16>(p0, p1);
      }
      l += sum0 + sum1;

      if constexpr (PSMEM) {
        // K-major, 128B-swizzled A operand: two 64-column atoms of 128 rows x 128 bytes.
        uint8_t* pt = smem + SM::kOffP + t * SM::kTileP;
#pragma unroll
        for (int ch = 0; ch < 16; ++ch) {
          const int atom = ch >> 3, cidx = ch & 7;
          uint4 v = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
          *reinterpret_cast<uint4*>(pt + atom * (kBM * 128) + row * 128 + ((cidx ^ (row & 7)) << 4)) = v;
        }
        fence_proxy_async_smem();
      } else {
        tmem_st_x64(s_col, pk);
        tmem_wait_st();
      }
      tc_fence_before_sync();
      mbar_arrive(&bar->p_full[t]);
    }

    if (ok) {
      ok = mbar_wait(&bar->o_done[t], (nkv - 1) & 1, abort_word, 0xA00);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.0f / l;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) +
                      (static_cast<size_t>(slice) * p.M + m0 + t * kBM + row) * (D * 2);
#pragma unroll
      for (int cc = 0; cc < D; cc += 32) {
        uint32_t o[32];
        tmem_ld_x32_wait(o_col + cc, o);
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          w[i] = pack2<BF16>(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(orow + cc * 2 + i * 16) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tmem_dealloc(tmem_base, kTmemCols);
    if (lane == 0 && bar->abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, static_cast<int>(bar->abort_word));
  }
}

// ------------------------------------------------------------------ launcher
template <bool BF16, int D, int NT, bool PSMEM>
static cudaError_t launch_one(const AttnParams& p, int batch, cudaStream_t stream) {
  using SM = Smem<D, NT, PSMEM>;
  auto kern = attention_kernel<BF16, D, NT, PSMEM>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kBytes);
  if (e != cudaSuccess) return e;
  dim3 grid(p.M / (NT * kBM), batch, 1);
  kern<<<grid, kThreads, SM::kBytes, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_attention(const AttnParams& p, int batch, int d, bool bf16, int nt, bool psmem,
                             cudaStream_t stream) {
#define DITTO_DISPATCH(BF, DD, NN, PS) \
  if (bf16 == BF && d == DD && nt == NN && psmem == PS) return launch_one<BF, DD, NN, PS>(p, batch, stream);
  DITTO_DISPATCH(false, 64, 1, false)
  DITTO_DISPATCH(false, 64, 2, false)
  DITTO_DISPATCH(false, 128, 1, false)
  DITTO_DISPATCH(false, 128, 2, false)
  DITTO_DISPATCH(true, 64, 1, false)
  DITTO_DISPATCH(true, 64, 2, false)
  DITTO_DISPATCH(true, 128, 1, false)
  DITTO_DISPATCH(true, 128, 2, false)
  DITTO_DISPATCH(false, 64, 1, true)
  DITTO_DISPATCH(false, 64, 2, true)
  DITTO_DISPATCH(false, 128, 1, true)
  DITTO_DISPATCH(false, 128, 2, true)
  DITTO_DISPATCH(true, 64, 1, true)
  DITTO_DISPATCH(true, 64, 2, true)
  DITTO_DISPATCH(true, 128, 1, true)
  DITTO_DISPATCH(true, 128, 2, true)
#undef DITTO_DISPATCH
  return cudaErrorInvalidValue;
}

}  // namespace ditto_b200
