// Fused GEMM -> activation -> GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a.
//
// Same decomposition as mlp_sm100.cu (Y columns split four ways, hidden chunks exchanged through
// distributed shared memory), but every MMA is a 2-SM MMA of M = 256: a cluster of eight CTAs =
// four pairs shares a 256-row block of X / Y.  Pair p (CTAs 2p, 2p+1) owns the Y columns
// [p N/4, (p+1) N/4) and every fourth hidden chunk; inside a pair CTA h holds rows
// [128 h, 128 h + 128) and half of each B operand's N extent, so a weight byte fetched from L2
// now serves 256 rows instead of 128: per CTA the chain streams 4 MB instead of 6 MB.
// (The single-CTA kernel is bound by how many operand bytes its shared-memory ring can keep in
// flight, not by the tensor pipe.)
//
// Who talks to whom:
//   * TMA: each CTA loads its own X rows and its half of W1 / W2 tiles; byte counts go to the
//     pair leader's `full` barrier (cp.async.bulk.tensor ... cta_group::2, no multicast).
//   * MMA: only the leader's warp 5 issues; commits are delivered to both CTAs of the pair.
//   * Hidden chunks travel in units of 64 columns (16 KB per CTA); unit u = 2 chunk + half lives in slot
//     u % 6 of every CTA.  CTA (p, h) drains its 128 rows of its pair's chunk from TMEM, writes the two
//     units into its own slots and pushes them to the CTAs (p', h) of the other pairs.
//   * Each CTA's ready-relay thread takes the units in order, arms the slot's barrier for units a peer
//     pushes, waits until the unit is present and tells the pair leader (h_pair, 2 arrivals): the pair's
//     GEMM2 on a unit needs it in both CTAs.
//   * A slot may be refilled when all four pairs have finished GEMM2 on the unit in it: each CTA's
//     free-relay thread forwards the leader's g2_done to the CTA of its half that writes the slot next.
//   * Tensor-pipe order on the leader: GEMM1 of the pair's first two chunks, then per unit
//     GEMM2(unit) | an eighth of GEMM1 of the chunk two rounds ahead.
#include <cuda.h>

#include <cstring>

#include "../../include/ditto_b200.h"
#include "mlp_common.cuh"
#include "mlp_sm100.cuh"
#include "sm100_ptx.cuh"

#ifdef DITTO_TRACE
#define DITTO_STAMP(i, k)                                                                   \
  do {                                                                                      \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (i) < 8) p.trace[(i) * 16 + (k)] = clock64(); \
  } while (0)
#else
#define DITTO_STAMP(i, k) do {} while (0)
#endif

namespace ditto_b200 {

namespace {

constexpr int kCluster = 8;
constexpr int kPairs = 4;
constexpr int kRows = 128;            // rows per CTA (256 per pair / cluster)
constexpr int kChunk = 128;           // hidden columns per chunk
constexpr int kStageBytes = 24 * 1024;
constexpr int kUnitBytes = kRows * 64 * 2;   // 64 hidden columns of this CTA's 128 rows: one 128-byte-row atom, 16 KB
#ifndef DITTO_PAIR_UNITS
#define DITTO_PAIR_UNITS 6
#endif
#ifndef DITTO_PAIR_STAGES
#define DITTO_PAIR_STAGES 5
#endif
constexpr int kUnits = DITTO_PAIR_UNITS;    // unit slots per CTA
constexpr int kStages = DITTO_PAIR_STAGES;
constexpr int kThreads = 288;
constexpr uint32_t kProducers = 2;      // TMA-issuing threads (warps 4 and 7), alternate ring stages
constexpr int kOffSlots = 0;
constexpr int kOffRing = kOffSlots + kUnits * kUnitBytes;
constexpr int kOffBar = kOffRing + kStages * kStageBytes;
constexpr int kSmemBytes = kOffBar + 512 + 1024;

struct PairParams {
  CUtensorMap map_x;   // X  [batch*M, K], box 64 x 128
  CUtensorMap map_w1;  // IO: W1 [batch*K, L], box 64 x 64;  OI: W1 [batch*L, K], box 64 x 64
  CUtensorMap map_w2;  // IO: W2 [batch*L, N], box 64 x 64;  OI: W2 [batch*N, L], box 64 x N/8
  void* y;
  int M, N, K, L;
  int w_oi;
  int relu;
  int* status;
  long long* trace;    // timeline buffer of -DDITTO_TRACE builds (null otherwise)
};

struct PairBars {
  uint64_t full[kStages];      // leader: operands of both CTAs have landed
  uint64_t empty[kStages];     // each CTA: the pair's MMAs have finished with the stage
  uint64_t h_tmem_full[2];     // each CTA: GEMM1 of the chunk is in TMEM
  uint64_t h_tmem_empty[2];    // leader: both CTAs' epilogues have read the TMEM buffer (8 warp arrivals)
  uint64_t h_ready[kUnits];    // each CTA: the unit of the slot's current use is present (own: local arrive; peer's: pushed bytes)
  uint64_t h_pair[kUnits];     // leader: ... in both CTAs of the pair (2 arrivals)
  uint64_t g2_done[kUnits];    // each CTA: the pair's GEMM2 has finished reading the slot
  uint64_t slot_free[kUnits];  // all four pairs have (4 arrivals); kept at the CTA that writes the slot next
  uint64_t y_done;
  uint64_t epi_sync;
  uint32_t tmem_base;
  uint32_t abort_word;
};
static_assert(sizeof(PairBars) <= 512, "barrier block too large");

}  // namespace

template <bool BF16>
__global__ void __cluster_dims__(kCluster, 1, 1) __launch_bounds__(kThreads, 1)
    mlp_pair_kernel(const __grid_constant__ PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  PairBars* bar = reinterpret_cast<PairBars*>(smem + kOffBar);
  volatile uint32_t* abort_word = &bar->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t pair = rank >> 1;        // owns Y columns [pair NS, (pair+1) NS) and chunks pair, pair+4, ...
  const uint32_t half = rank & 1;         // 0 = leader of the pair
  const uint32_t leader = rank & ~1u;
  const int row0 = (blockIdx.x / kCluster) * (2 * kRows) + static_cast<int>(half) * kRows;
  const int b = blockIdx.y;
  const int NS = p.N / kPairs;            // the pair's Y columns
  const int NH = NS / 2;                  // this CTA's share of the W2 tile's N extent
  const int rounds = p.L / (kPairs * kChunk);
  const int units = 2 * kPairs * rounds;  // 64-column units of hidden chunks in all
  const int ksteps1 = p.K / 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bar->full[s], 1);
      mbar_init(&bar->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->h_tmem_full[i], 1);
      mbar_init(&bar->h_tmem_empty[i], 8);
    }
    for (int x = 0; x < kUnits; ++x) {
      mbar_init(&bar->h_ready[x], 1);
      mbar_init(&bar->h_pair[x], 2);
      mbar_init(&bar->g2_done[x], 1);
      mbar_init(&bar->slot_free[x], kPairs);
    }
    mbar_init(&bar->y_done, 1);
    mbar_init(&bar->epi_sync, kRows);
    bar->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc_pair(&bar->tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                     // every CTA's barriers exist before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = bar->tmem_base;
  const uint32_t tmem_y = tmem_base;
  const uint32_t tmem_h = tmem_base + 256;

  if (warp == 4 || warp == 7) {
    // ------------------------------------------------------------ TMA producers (one thread each, alternate stages)
    if (lane == 0) {
      const uint32_t pw = warp == 4 ? 0u : 1u;
      uint32_t cnt = 0;
      tma_prefetch_desc(&p.map_x);
      tma_prefetch_desc(&p.map_w1);
      tma_prefetch_desc(&p.map_w2);
      int ps = 0;
      uint32_t pph = 0;
      bool ok = true;
      uint32_t full_addr = 0;             // the leader's full[ps] as a cluster address
      // `pair_bytes`: what both CTAs of the pair put into the stage (armed by the leader only)
      auto acquire = [&](uint32_t pair_bytes, uint32_t code) -> uint8_t* {
        if ((cnt++ & (kProducers - 1)) != pw) return nullptr;
        ok = mbar_wait(&bar->empty[ps], pph ^ 1, abort_word, code);
        if (!ok) return nullptr;
        if (half == 0) mbar_arrive_expect_tx(&bar->full[ps], pair_bytes);
        full_addr = map_to_cta(smem_u32(&bar->full[ps]), leader);
        return smem + kOffRing + ps * kStageBytes;
      };
      auto advance = [&]() {
        if (++ps == kStages) { ps = 0; pph ^= 1; }
      };
      auto load_g1 = [&](int i, int ks0, int ks1) {   // X rows of this CTA and its half of the W1 chunk tile, k-steps [ks0, ks1)
        const int g = i * kPairs + static_cast<int>(pair);
        for (int ks = ks0; ks < ks1 && ok; ++ks) {
          uint8_t* dst = acquire(2 * (16384 + 8192), 0x100 + i);
          if (dst != nullptr) {
            tma_load_2d_pair(dst, &p.map_x, full_addr, ks * 64, b * p.M + row0);
            if (p.w_oi)
              tma_load_2d_pair(dst + 16384, &p.map_w1, full_addr, ks * 64, b * p.L + g * kChunk + half * 64);
            else
              tma_load_2d_pair(dst + 16384, &p.map_w1, full_addr, g * kChunk + half * 64, b * p.K + ks * 64);
          }
          advance();
        }
      };
      auto load_g2 = [&](int u) {         // this CTA's half of the pair's W2 slice for hidden unit u
        const int g = u >> 1, kk = u & 1;
        uint8_t* dst = acquire(2 * 64 * NH * 2, 0x200 + (u >> 3));
        if (dst != nullptr) {
          if (p.w_oi) {
            tma_load_2d_pair(dst, &p.map_w2, full_addr, g * kChunk + kk * 64, b * p.N + pair * NS + half * NH);
          } else {
            for (int a = 0; a < NH / 64; ++a)
              tma_load_2d_pair(dst + a * 8192, &p.map_w2, full_addr, pair * NS + half * NH + a * 64,
                               b * p.L + g * kChunk + kk * 64);
          }
        }
        advance();
      };
      // the order the leader's MMA warp consumes the ring in
      load_g1(0, 0, ksteps1);
      if (rounds > 1) load_g1(1, 0, ksteps1);
      for (int u = 0; u < units && ok; ++u) {
        const int i = u >> 3, e = u & 7;
        load_g2(u);
        if (i + 2 < rounds) load_g1(i + 2, e * ksteps1 / 8, (e + 1) * ksteps1 / 8);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (half == 0) {
      const uint32_t issuer = elect_one();
      const uint32_t pair_mask = 0x3u << leader;
      const uint32_t idesc1 = umma_idesc_f16(BF16, 2 * kRows, kChunk, false, p.w_oi == 0);
      const uint32_t idesc2 = umma_idesc_f16(BF16, 2 * kRows, NS, false, p.w_oi == 0);
      const uint32_t ring = smem_u32(smem + kOffRing);
      const uint32_t slots = smem_u32(smem + kOffSlots);
      int cs = 0;
      uint32_t cph = 0;
      bool ok = true;
      auto wait = [&](uint64_t* bp, uint32_t parity, uint32_t code) {
        bool r = mbar_wait(bp, parity, abort_word, code);
        r = __all_sync(0xffffffffu, r);
        tc_fence_after_sync();
        return r;
      };
      auto wait_cluster = [&](uint64_t* bp, uint32_t parity, uint32_t code) {
        bool r = mbar_wait_cluster(bp, parity, abort_word, code);
        r = __all_sync(0xffffffffu, r);
        tc_fence_after_sync();
        return r;
      };
      auto advance = [&]() {
        if (++cs == kStages) { cs = 0; cph ^= 1; }
      };
      auto g1 = [&](int i, int ks0, int ks1, bool first, bool last) {
        const int hb = i & 1;
        if (first && i >= 2) ok = wait_cluster(&bar->h_tmem_empty[hb], ((i >> 1) - 1) & 1, 0x300 + i);
        if (first && lane == 0) DITTO_STAMP(i, 0);
        for (int ks = ks0; ks < ks1 && ok; ++ks) {
          ok = wait(&bar->full[cs], cph, 0x310 + i);
          if (!ok) break;
          const uint32_t st = ring + cs * kStageBytes;
          const uint64_t da = umma_desc_sw128(st, 16, 1024);
          const uint64_t db = p.w_oi ? umma_desc_sw128(st + 16384, 16, 1024) : umma_desc_sw128(st + 16384, 8192, 1024);
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4) {
            const uint32_t offb = p.w_oi ? (s4 * 32) >> 4 : (s4 * 2048) >> 4;
            umma_ss_pair_elected(tmem_h + hb * kChunk, da + ((s4 * 32) >> 4), db + offb, idesc1, (ks | s4) ? 1u : 0u,
                                 issuer);
          }
          umma_commit_pair_elected(&bar->empty[cs], pair_mask, issuer);
          advance();
        }
        if (last && ok) umma_commit_pair_elected(&bar->h_tmem_full[hb], pair_mask, issuer);
        if (last && lane == 0) DITTO_STAMP(i, 1);
      };
      auto g2 = [&](int u) {              // GEMM2 on hidden unit u: needs it in both CTAs' slots
        const int sl = u % kUnits;
        if (lane == 0 && (u & 7) == 0) DITTO_STAMP(u >> 3, 2);
        ok = wait_cluster(&bar->h_pair[sl], (u / kUnits) & 1, 0x400 + (u >> 3));
        if (lane == 0 && (u & 7) == 0) DITTO_STAMP(u >> 3, 3);
        if (ok) ok = wait(&bar->full[cs], cph, 0x410 + (u >> 3));
        if (ok) {
          const uint32_t st = ring + cs * kStageBytes;
          const uint64_t da = umma_desc_sw128(slots + sl * kUnitBytes, 16, 1024);
          const uint64_t db = p.w_oi ? umma_desc_sw128(st, 16, 1024) : umma_desc_sw128(st, 8192, 1024);
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4) {
            const uint32_t offb = p.w_oi ? (s4 * 32) >> 4 : (s4 * 2048) >> 4;
            umma_ss_pair_elected(tmem_y, da + ((s4 * 32) >> 4), db + offb, idesc2, (u | s4) ? 1u : 0u, issuer);
          }
          umma_commit_pair_elected(&bar->empty[cs], pair_mask, issuer);
          advance();
          umma_commit_pair_elected(&bar->g2_done[sl], pair_mask, issuer);
        }
        if (lane == 0 && (u & 7) == 7) DITTO_STAMP(u >> 3, 4);
      };
      g1(0, 0, ksteps1, true, true);
      if (rounds > 1 && ok) g1(1, 0, ksteps1, true, true);
      for (int u = 0; u < units && ok; ++u) {
        const int i = u >> 3, e = u & 7;
        g2(u);
        if (i + 2 < rounds && ok) g1(i + 2, e * ksteps1 / 8, (e + 1) * ksteps1 / 8, e == 0, e == 7);
      }
      if (ok) umma_commit_pair_elected(&bar->y_done, pair_mask, issuer);
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------ ready relay (one thread)
    if (lane == 0) {
      for (int u = 0; u < units; ++u) {
        const int sl = u % kUnits;
        // a peer pushes this unit: arm the slot's barrier for its bytes (the own pair's units arrive locally)
        if (static_cast<uint32_t>((u >> 1) & 3) != pair) mbar_arrive_expect_tx(&bar->h_ready[sl], kUnitBytes);
        if (!mbar_wait(&bar->h_ready[sl], (u / kUnits) & 1, abort_word, 0x500 + (u >> 3))) break;
        mbar_arrive_cluster(&bar->h_pair[sl], leader);
      }
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------ free relay (one thread)
    if (lane == 0) {
      for (int u = 0; u < units; ++u) {
        const int sl = u % kUnits;
        if (!mbar_wait(&bar->g2_done[sl], (u / kUnits) & 1, abort_word, 0x580 + (u >> 3))) break;
        if ((u & 7) == 7) DITTO_STAMP(u >> 3, 5);
        // tell the CTA of this half that writes the slot next (the pair that owns unit u + kUnits)
        if (u + kUnits < units)
          mbar_arrive_cluster(&bar->slot_free[sl], 2 * static_cast<uint32_t>(((u + kUnits) >> 1) & 3) + half);
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------ epilogue
    const int row = warp * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    bool ok = true;
    uint32_t free_waits[kUnits] = {};       // completed waits per slot: the parity of the next one
    for (int i = 0; i < rounds; ++i) {
      const int hb = i & 1;
      ok = mbar_wait(&bar->h_tmem_full[hb], (i >> 1) & 1, abort_word, 0x600 + i);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      if (threadIdx.x == 0) DITTO_STAMP(i, 6);
      uint32_t h[kChunk];
      tmem_ld_x128_wait(tmem_h + hb * kChunk + lane_base, h);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(&bar->h_tmem_empty[hb], leader);   // one arrival per warp, 8 per pair
      uint32_t pk[kChunk / 2];
#pragma unroll
      for (int j = 0; j < kChunk / 2; ++j) {
        float v0 = __uint_as_float(h[2 * j]), v1 = __uint_as_float(h[2 * j + 1]);
        if (p.relu) {
          v0 = v0 > 0.f ? v0 : 0.f;       // if_then_else(D > 0, D, 0) as in the reference
          v1 = v1 > 0.f ? v1 : 0.f;
        }
        pk[j] = pack2<BF16>(v0, v1);
      }
      const int g = i * kPairs + static_cast<int>(pair);   // this pair's chunk of the round
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const int u = 2 * g + kk;
        const int sl = u % kUnits;
        if (u >= kUnits) {
          // every pair has finished GEMM2 on the slot's previous unit: it may be overwritten
          uint32_t par = 0;
#pragma unroll
          for (int t = 0; t < kUnits; ++t)
            if (t == sl) par = free_waits[t]++ & 1;
          ok = mbar_wait_cluster(&bar->slot_free[sl], par, abort_word, 0x700 + i);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        if (threadIdx.x == 0 && kk == 0) DITTO_STAMP(i, 7);
        uint8_t* slot = smem + kOffSlots + sl * kUnitBytes;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const int w = kk * 32 + 4 * ch;
          const uint4 v = make_uint4(pk[w], pk[w + 1], pk[w + 2], pk[w + 3]);
          *reinterpret_cast<uint4*>(slot + row * 128 + ((ch ^ (row & 7)) << 4)) = v;
        }
        fence_proxy_async_smem();
        mbar_arrive(&bar->epi_sync);
        ok = mbar_wait(&bar->epi_sync, kk, abort_word, 0x780 + i);   // two phases per round
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (threadIdx.x == 0) {
          const uint32_t slot_addr = smem_u32(slot);
          const uint32_t bar_addr = smem_u32(&bar->h_ready[sl]);
          for (uint32_t d = 1; d < kPairs; ++d) {
            const uint32_t peer = 2 * ((pair + d) % kPairs) + half;   // same rows, other pairs
            bulk_copy_to_peer(map_to_cta(slot_addr, peer), slot, kUnitBytes, map_to_cta(bar_addr, peer));
          }
          mbar_arrive(&bar->h_ready[sl]);    // the local copy is in place
          if (kk == 1) DITTO_STAMP(i, 8);
        }
      }
      if (!ok) break;
    }
    if (ok) {
      ok = mbar_wait(&bar->y_done, 0, abort_word, 0x800);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      uint8_t* yrow = reinterpret_cast<uint8_t*>(p.y) +
                      ((static_cast<size_t>(b) * p.M + row0 + row) * p.N + static_cast<size_t>(pair) * NS) * 2;
      for (int cc = 0; cc < NS; cc += 32) {
        uint32_t o[32];
        tmem_ld_x32_wait(tmem_y + lane_base + cc, o);
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) w[j] = pack2<BF16>(__uint_as_float(o[2 * j]), __uint_as_float(o[2 * j + 1]));
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(yrow + cc * 2 + j * 16) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                     // no CTA leaves while a peer may still write to it or use its operands
  if (warp == 0) {
    tmem_dealloc_pair(tmem_base, 512);
    if (lane == 0 && bar->abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, static_cast<int>(bar->abort_word));
  }
}

// ------------------------------------------------------------------ host side
bool mlp_pair_supported(int M, int N, int K, int L) {
  return M % (2 * kRows) == 0 && L % (kPairs * kChunk) == 0 && K % 64 == 0 && N % (kPairs * 128) == 0 &&
         N <= kPairs * 256;
}

int launch_mlp_pair(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                    bool bf16, int w_layout, int epilogue, int* status, cudaStream_t stream, long long* trace) {
  if (!mlp_pair_supported(M, N, K, L) || batch > 65535) return DITTO_ERR_UNSUPPORTED;
  const int NH = N / kPairs / 2;
  PairParams p;
  std::memset(&p, 0, sizeof(p));
  bool ok = mlp_make_map(&p.map_x, bf16, x, K, static_cast<uint64_t>(batch) * M, 64, 128);
  if (w_layout == 1) {
    ok = ok && mlp_make_map(&p.map_w1, bf16, w1, K, static_cast<uint64_t>(batch) * L, 64, 64);
    ok = ok && mlp_make_map(&p.map_w2, bf16, w2, L, static_cast<uint64_t>(batch) * N, 64, NH);
  } else {
    ok = ok && mlp_make_map(&p.map_w1, bf16, w1, L, static_cast<uint64_t>(batch) * K, 64, 64);
    ok = ok && mlp_make_map(&p.map_w2, bf16, w2, N, static_cast<uint64_t>(batch) * L, 64, 64);
  }
  if (!ok) return DITTO_ERR_DRIVER;
  p.y = y;
  p.M = M;
  p.N = N;
  p.K = K;
  p.L = L;
  p.w_oi = w_layout == 1;
  p.relu = epilogue == 1;
  p.status = status;
  p.trace = trace;
  dim3 grid(kCluster * (M / (2 * kRows)), batch, 1);
  cudaError_t e;
  if (bf16) {
    e = cudaFuncSetAttribute(mlp_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess) mlp_pair_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(p);
  } else {
    e = cudaFuncSetAttribute(mlp_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess) mlp_pair_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(p);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? DITTO_OK : DITTO_ERR_CUDA;
}

}  // namespace ditto_b200
