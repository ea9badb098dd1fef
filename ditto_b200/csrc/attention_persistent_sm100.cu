// Persistent form of the fused bmm -> softmax -> bmm kernel for head dimensions up to 64.
//
// Same arithmetic and warp roles as the separate-P variant in attention_sm100.cu (one 128-row query
// tile in flight per CTA; S, O and P in their own TMEM columns; S(j+1) issued while the softmax of
// block j runs; two CTAs per SM), but a CTA does not end with its tile: the grid has two CTAs per SM
// and each CTA walks a list of work items (slice, tile).  Short sequences -- config 3 has four K/V
// blocks per tile -- otherwise spend a third of every CTA's life in the prologue (barrier and TMEM
// set-up, first Q/K/V loads) and the epilogue.  Here the producer runs ahead into the next item's
// Q and K/V while the current one is still being multiplied, the MMA warp issues the next item's
// first S behind the current item's last P*V, and the output of one item is written while the next
// one's scores are being computed.
//
// All mbarrier phases are driven by global counters (items, K/V blocks) that every role advances
// identically.  Every wait is bounded as everywhere else in this library.
#include "attention_sm100.cuh"

#include <atomic>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

// 1: the softmax evaluates its exponentials two at a time on packed 16-bit arguments (see ex2_packed)
#ifndef DITTO_PACKED_EX2
#define DITTO_PACKED_EX2 0
#endif

#ifdef DITTO_TRACE
#define DITTO_STAMP(idx)                                                                         \
  do {                                                                                           \
    if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && (idx) < 1280) p.trace[idx] = clock64(); \
  } while (0)
#define DITTO_STAMP_T(tid, idx)                                                                  \
  do {                                                                                           \
    if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == (tid) && (idx) < 1280) p.trace[idx] = clock64(); \
  } while (0)
#else
#define DITTO_STAMP(idx) do {} while (0)
#define DITTO_STAMP_T(tid, idx) do {} while (0)
#endif

namespace ditto_b200 {

namespace {

constexpr int kBM = 128, kBN = 128, kD = 64;
constexpr int kMaxDevices = 64;
constexpr int kStages = 2;
constexpr int kTileQ = kBM * kD * 2;     // 16 KB
constexpr int kTileKV = kBN * kD * 2;    // 16 KB
constexpr int kOffQ = 0;               // two Q buffers: the next item's Q is loaded while the current one is in use
constexpr int kOffK = kOffQ + 2 * kTileQ;
constexpr int kOffV = kOffK + kStages * kTileKV;
constexpr int kOffBar = kOffV + kStages * kTileKV;
constexpr int kSmemBytes = kOffBar + 256 + 1024;
constexpr int kThreads = 192;            // 4 softmax warps, producer, MMA issuer
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColO = 128, kColP = 192;
constexpr int kSplit = 96;               // K/V rows in the first part of P
constexpr float kRescaleThreshold = 8.0f;
constexpr int kModeSoftmax = 0, kModeRelu = 1;

struct PBars {
  uint64_t q_full[2], q_empty[2];
  uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t s_full, s_taken, p_part[2], o_done, o_free;
  uint32_t tmem_base;
  uint32_t abort_word;
};
static_assert(sizeof(PBars) <= 256, "barrier block too large");

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

template <bool BF16, int MODE>
__global__ void __launch_bounds__(kThreads, 2) attention_persistent_kernel(const __grid_constant__ AttnParams p,
                                                                           const int total_items) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  PBars* bar = reinterpret_cast<PBars*>(smem + kOffBar);
  volatile uint32_t* abort_word = &bar->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles = (p.M + kBM - 1) / kBM;
  const int nkv = (p.L + kBN - 1) / kBN;
  const int ksteps_d = p.d / 16;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->q_full[i], 1);
      mbar_init(&bar->q_empty[i], 1 + 4);     // the item's last S MMA has read Q, and the four softmax warps are done
                                              // with the buffer as the staging area of the item's write-out
    }
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bar->k_full[s], 1);
      mbar_init(&bar->k_empty[s], 1);
      mbar_init(&bar->v_full[s], 1);
      mbar_init(&bar->v_empty[s], 1);
    }
    mbar_init(&bar->s_full, 1);
    mbar_init(&bar->s_taken, kBM);
    mbar_init(&bar->p_part[0], kBM);
    mbar_init(&bar->p_part[1], kBM);
    mbar_init(&bar->o_done, 1);
    mbar_init(&bar->o_free, kBM);
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
  // Programmatic dependent launch: everything above touches no global memory, so it may run while the
  // kernel ahead of this one in the stream is still finishing; from here on its results are needed.
  // The kernel behind this one may start its own set-up right away (it waits at the same point).
  grid_dependency_wait();
  grid_launch_dependents();

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer (one thread)
    if (lane == 0) {
      tma_prefetch_desc(&p.map_q);
      tma_prefetch_desc(&p.map_k);
      tma_prefetch_desc(&p.map_v);
      bool ok = true;
      int g = 0;                                   // K/V blocks loaded so far, over all items
      int it = 0;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++it) {
        const int slice = item / tiles;
        const int seq = slice / p.heads;
        const int head_col = (slice % p.heads) * p.d;
        const int m0 = (item % tiles) * kBM;
        const int qb = it & 1;                       // Q buffer of this item; its previous user was item it - 2
        ok = mbar_wait(&bar->q_empty[qb], ((it >> 1) & 1) ^ 1, abort_word, 0x100);
        if (!ok) break;
        DITTO_STAMP_T(128, 768 + it * 16 + 15);
        mbar_arrive_expect_tx(&bar->q_full[qb], kTileQ);
        tma_load_3d(smem + kOffQ + qb * kTileQ, &p.map_q, &bar->q_full[qb], p.q_col0 + head_col, m0, seq);
        for (int j = 0; j < nkv; ++j, ++g) {
          const int s = g % kStages;
          const uint32_t ph = (g / kStages) & 1;
          ok = mbar_wait(&bar->k_empty[s], ph ^ 1, abort_word, 0x110);
          if (!ok) break;
          DITTO_STAMP_T(128, 768 + it * 16 + j);
          mbar_arrive_expect_tx(&bar->k_full[s], kTileKV);
          if (p.k_transposed) {
            for (int a = 0; a < kBN / 64; ++a)
              tma_load_3d(smem + kOffK + s * kTileKV + a * (kD * 128), &p.map_k, &bar->k_full[s], j * kBN + a * 64, 0,
                          slice);
          } else {
            tma_load_3d(smem + kOffK + s * kTileKV, &p.map_k, &bar->k_full[s], p.k_col0 + head_col, j * kBN, seq);
          }
          ok = mbar_wait(&bar->v_empty[s], ph ^ 1, abort_word, 0x120);
          if (!ok) break;
          DITTO_STAMP_T(128, 768 + it * 16 + 8 + j);
          mbar_arrive_expect_tx(&bar->v_full[s], kTileKV);
          if (p.v_transposed) {
            for (int a = 0; a < kBN / 64; ++a)
              tma_load_3d(smem + kOffV + s * kTileKV + a * (kD * 128), &p.map_v, &bar->v_full[s], j * kBN + a * 64, 0,
                          slice);
          } else {
            tma_load_3d(smem + kOffV + s * kTileKV, &p.map_v, &bar->v_full[s], p.v_col0 + head_col, j * kBN, seq);
          }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer (converged warp, elected lane issues)
    const uint32_t issuer = elect_one();
    const bool kt = p.k_transposed != 0;
    const uint32_t idesc_s = umma_idesc_f16(BF16, kBM, kBN, false, kt);
    const bool vt = p.v_transposed != 0;           // V stored [slice, dv, L]: K-major operand of P*V
    const uint32_t idesc_o = umma_idesc_f16(BF16, kBM, kD, false, !vt);
    const uint64_t dq0 = umma_desc_sw128(smem_u32(smem + kOffQ), 16, 1024);
    const uint64_t dk0 = kt ? umma_desc_sw128(smem_u32(smem + kOffK), kD * 128, 1024)
                            : umma_desc_sw128(smem_u32(smem + kOffK), 16, 1024);
    const uint64_t dv0 = vt ? umma_desc_sw128(smem_u32(smem + kOffV), 16, 1024)
                            : umma_desc_sw128(smem_u32(smem + kOffV), kBN * 128, 1024);
    auto wait = [&](uint64_t* b, uint32_t parity, uint32_t code) {
      bool r = mbar_wait(b, parity, abort_word, code);
      r = __all_sync(0xffffffffu, r);
      tc_fence_after_sync();
      return r;
    };
    auto issue_s = [&](int stage, int qb) {
      const uint64_t dq = dq0 + ((qb * kTileQ) >> 4);
      const uint64_t db = dk0 + ((stage * kTileKV) >> 4);
#pragma unroll
      for (int i = 0; i < kD / 16; ++i) {
        const uint32_t off_k = (i * 32) >> 4;
        const uint32_t off_b = kt ? static_cast<uint32_t>((i * 2048) >> 4) : off_k;
        if (i < ksteps_d) umma_ss_elected(tmem_base + kColS, dq + off_k, db + off_b, idesc_s, i > 0 ? 1u : 0u, issuer);
      }
      umma_commit_elected(&bar->s_full, issuer);
      umma_commit_elected(&bar->k_empty[stage], issuer);
    };
    auto issue_pv = [&](int stage, int part, uint32_t accumulate) {
      const uint64_t db = dv0 + ((stage * kTileKV) >> 4);
#pragma unroll
      for (int i = (part == 0 ? 0 : kSplit / 16); i < (part == 0 ? kSplit / 16 : kBN / 16); ++i)
        umma_ts_elected(tmem_base + kColO, tmem_base + kColP + i * 8,
                        db + (vt ? static_cast<uint32_t>(((i / 4) * (kD * 128) + (i % 4) * 32) >> 4)
                                 : static_cast<uint32_t>((i * 2048) >> 4)),
                        idesc_o, i > 0 ? 1u : accumulate, issuer);
    };
    bool ok = true;
    int g = 0, it = 0;                             // g: K/V blocks multiplied so far, over all items
    // The scores of block g + 1 are always issued ahead of P*V(g), across item boundaries too, so
    // that the softmax warps find the next item's first scores ready when they leave the epilogue.
    if (static_cast<int>(blockIdx.x) < total_items) {
      ok = wait(&bar->q_full[0], 0, 0x300) && wait(&bar->k_full[0], 0, 0x320);
      if (ok) {
        issue_s(0, 0);
        if (nkv == 1) umma_commit_elected(&bar->q_empty[0], issuer);
      }
    }
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++it) {
      const int qb = it & 1;
      const bool next_item = item + static_cast<int>(gridDim.x) < total_items;
      for (int j = 0; j < nkv && ok; ++j, ++g) {
        const int st = g % kStages;
        const bool more = j + 1 < nkv;
        if (more || next_item) {
          const int sn = (g + 1) % kStages;
          const int nqb = more ? qb : qb ^ 1;
          if (!more) ok = wait(&bar->q_full[nqb], ((it + 1) >> 1) & 1, 0x300);
          // the softmax warps must have taken S(g) out of TMEM before S(g + 1) lands there
          ok = ok && wait(&bar->s_taken, g & 1, 0x330) && wait(&bar->k_full[sn], ((g + 1) / kStages) & 1, 0x340);
          if (!ok) break;
          issue_s(sn, nqb);
          // release Q after the last scores of its item
          if ((more ? j + 2 : 1) == nkv) umma_commit_elected(&bar->q_empty[nqb], issuer);
        }
        ok = wait(&bar->v_full[st], (g / kStages) & 1, 0x350);
        // the first P*V of an item overwrites O: the previous item's epilogue must have read it
        if (ok && j == 0 && it > 0) ok = wait(&bar->o_free, (it - 1) & 1, 0x360);
        ok = ok && wait(&bar->p_part[0], g & 1, 0x370);
        if (!ok) break;
        issue_pv(st, 0, j > 0 ? 1u : 0u);
        ok = wait(&bar->p_part[1], g & 1, 0x380);
        if (!ok) break;
        issue_pv(st, 1, 1u);
        umma_commit_elected(&bar->v_empty[st], issuer);     // also tells the softmax warps that P*V(g) is done
        if (!more) umma_commit_elected(&bar->o_done, issuer);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue (warps 0-3, thread r <-> row r)
    const int row = warp * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const uint32_t s_col = lane_base + kColS, o_col = lane_base + kColO, p_col = lane_base + kColP;
    const float c = p.scale_log2;
    bool ok = true;
    int g = 0, it = 0;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++it) {
      const int slice = item / tiles;
      const int seq = slice / p.heads;
      const int head_col = (slice % p.heads) * p.d;
      const int m0 = (item % tiles) * kBM;
      float m = -INFINITY, l = 0.f;
      for (int j = 0; j < nkv; ++j, ++g) {
        ok = mbar_wait(&bar->s_full, g & 1, abort_word, 0x800);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        DITTO_STAMP(it * 16 + j * 2);
        uint32_t sv[kBN];
        tmem_ld_x128_wait(s_col, sv);
        tc_fence_before_sync();
        mbar_arrive(&bar->s_taken);                // the S columns may be overwritten by the next S

        float m_new = m;
        if constexpr (MODE == kModeSoftmax) {
          if (j == nkv - 1 && (p.L % kBN) != 0) {
            const int valid = p.L % kBN;           // partial last block: zero-filled K rows must not count
#pragma unroll
            for (int i = 0; i < kBN; ++i)
              if (i >= valid) sv[i] = __float_as_uint(-INFINITY);
          }
          float mx[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) mx[u] = __uint_as_float(sv[u]);
#pragma unroll
          for (int i = 16; i < kBN; i += 16) {
#pragma unroll
            for (int u = 0; u < 16; ++u) mx[u] = fmaxf(mx[u], __uint_as_float(sv[i + u]));
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) mx[u] = fmaxf(mx[u], mx[u + 8]);
#pragma unroll
          for (int u = 0; u < 4; ++u) mx[u] = fmaxf(mx[u], mx[u + 4]);
          m_new = fmaxf(fmaxf(m, mx[0]), fmaxf(fmaxf(mx[1], mx[2]), mx[3]));
        }
        DITTO_STAMP(1024 + it * 16 + j);
        if (g > 0) {
          // P*V(g-1) must have finished before P is overwritten or O is rescaled (S(g) was issued ahead of it)
          ok = mbar_wait(&bar->v_empty[(g - 1) % kStages], ((g - 1) / kStages) & 1, abort_word, 0x900);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
        }
        DITTO_STAMP(it * 16 + 8 + j);
        const bool need = MODE == kModeSoftmax && (m_new - m) * c > kRescaleThreshold;
        if (MODE == kModeSoftmax && __any_sync(0xffffffffu, need)) {
          const float f = ex2_approx((m - m_new) * c);
          if (j > 0) {
#pragma unroll
            for (int cc = 0; cc < kD; cc += 32) {
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
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          constexpr int kFirst = kSplit / 2;
          const int w0 = part == 0 ? 0 : kFirst;
          const int w1 = part == 0 ? kFirst : kBN / 2;
          uint32_t pk[kFirst];
#pragma unroll
          for (int i = 0; i < kFirst; ++i) {
            if (w0 + i < w1) {
              float p0 = __uint_as_float(sv[2 * (w0 + i)]), p1 = __uint_as_float(sv[2 * (w0 + i) + 1]);
              if constexpr (MODE == kModeSoftmax && DITTO_PACKED_EX2 != 0) {
                // one special-function instruction for the pair; the sum takes the rounded values the MMA will see
                pk[i] = ex2_packed<BF16>(fmaf(p0, c, -mc), fmaf(p1, c, -mc));
                const float2 pf = BF16 ? unpack_bf16x2(pk[i]) : unpack_f16x2(pk[i]);
                sum0 += pf.x;
                sum1 += pf.y;
                continue;
              } else if constexpr (MODE == kModeSoftmax) {
                p0 = ex2_approx(fmaf(p0, c, -mc));
                p1 = ex2_approx(fmaf(p1, c, -mc));
              } else if constexpr (MODE == kModeRelu) {
                p0 = p0 > 0.f ? p0 : 0.f;
                p1 = p1 > 0.f ? p1 : 0.f;
              }
              sum0 += p0;
              sum1 += p1;
              pk[i] = pack2<BF16>(p0, p1);
            }
          }
          if (part == 0) {
            uint32_t lo[32], hi[16];
#pragma unroll
            for (int i = 0; i < 32; ++i) lo[i] = pk[i];
#pragma unroll
            for (int i = 0; i < 16; ++i) hi[i] = pk[32 + i];
            tmem_st_x32(p_col, lo);
            tmem_st_x16(p_col + 32, hi);
          } else {
            uint32_t lo[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) lo[i] = pk[i];
            tmem_st_x16(p_col + kFirst, lo);
          }
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(&bar->p_part[part]);
          DITTO_STAMP(1024 + it * 16 + 4 + j * 2 + part);
        }
        l += sum0 + sum1;
        DITTO_STAMP(it * 16 + j * 2 + 1);
      }
      if (!ok) break;
      DITTO_STAMP(it * 16 + 12);

      // epilogue of the item: O / l, written once
      ok = mbar_wait(&bar->o_done, it & 1, abort_word, 0xA00);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      DITTO_STAMP(it * 16 + 13);
      uint32_t o[kD];
      tmem_ld_x64_wait(o_col, o);
      tc_fence_before_sync();
      mbar_arrive(&bar->o_free);                   // the next item's first P*V may overwrite O
      const float inv = MODE == kModeSoftmax ? 1.0f / l : 1.0f;
      // Written straight from the registers a store instruction would touch 32 rows, 16 bytes each; the
      // requests back up the load/store path and delay the barrier operations behind them.  Every warp turns
      // its 32 rows x 128 bytes around in 4 KB of shared memory of its own (16-byte pieces swizzled by row) and
      // writes 4 rows x 128 contiguous bytes per instruction.
      // The staging area is the item's own Q buffer: every MMA of the item has retired (o_done), and the
      // producer refills the buffer -- for the item after next -- only when these warps have arrived on
      // q_empty as well.
      uint8_t* stage = smem + kOffQ + (it & 1) * kTileQ + warp * 4096;
#pragma unroll
      for (int i = 0; i < kD / 8; ++i) {
        uint32_t w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          w[u] = pack2<BF16>(__uint_as_float(o[8 * i + 2 * u]) * inv, __uint_as_float(o[8 * i + 2 * u + 1]) * inv);
        *reinterpret_cast<uint4*>(stage + lane * 128 + ((i ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      __syncwarp();
      const size_t out_row0 = static_cast<size_t>(seq) * p.M + m0 + warp * 32;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + (lane >> 3), piece = lane & 7;
        const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((piece ^ (rr & 7)) << 4));
        if (m0 + warp * 32 + rr < p.M && piece * 8 < p.dv)
          *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.out) + ((out_row0 + rr) * p.out_ld + head_col + piece * 8) * 2) = v;
      }
      fence_proxy_async_smem();                    // these generic-proxy accesses precede the TMA write of the next Q
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->q_empty[it & 1]);
      DITTO_STAMP(it * 16 + 14);
    }
  }

  // After a wait has given up, TMA loads this CTA has armed may still be in flight; they complete within
  // microseconds.  Give them that time before the shared memory they target is released.
  if (bar->abort_word != 0u) {
    for (int t = 0; t < 64; ++t) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tmem_dealloc(tmem_base, kTmemCols);
    if (lane == 0 && bar->abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, static_cast<int>(bar->abort_word));
  }
}

// ------------------------------------------------------------------ launcher
template <bool BF16, int MODE>
static cudaError_t launch_p(const AttnParams& p, long long total_items, cudaStream_t stream) {
  auto kern = attention_persistent_kernel<BF16, MODE>;
  // function attributes and the SM count are looked up once per device (this instantiation's statics):
  // the launches of short sequences are a few microseconds long and every runtime call shows
  static std::atomic<int> sm_count[kMaxDevices];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  int sms = sm_count[dev].load(std::memory_order_acquire);
  if (sms == 0) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    sm_count[dev].store(sms, std::memory_order_release);
  }
  const long long slots = 2LL * sms;                 // two CTAs per SM (TMEM: 2 x 256 columns)
  const unsigned grid = static_cast<unsigned>(total_items < slots ? total_items : slots);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see grid_dependency_wait in the kernel
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p, static_cast<int>(total_items));
}

cudaError_t launch_attention_persistent(const AttnParams& p, int batch, bool bf16, int mode, cudaStream_t stream) {
  const long long total = static_cast<long long>((p.M + kBM - 1) / kBM) * batch;
  if (total > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (mode == 0) return bf16 ? launch_p<true, 0>(p, total, stream) : launch_p<false, 0>(p, total, stream);
  if (mode == 1) return bf16 ? launch_p<true, 1>(p, total, stream) : launch_p<false, 1>(p, total, stream);
  return bf16 ? launch_p<true, 2>(p, total, stream) : launch_p<false, 2>(p, total, stream);
}

}  // namespace ditto_b200
