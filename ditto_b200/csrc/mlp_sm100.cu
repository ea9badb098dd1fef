// Fused GEMM -> activation -> GEMM for sm_100a:  Y = act(X W1) W2, hidden activations on chip.
//
// Replaces what the reference would build from BatchGemmReluGemm / BatchGemmGemm
// (python_test/auto_tensorize/test_hyper_fusion_cpu.py:24-96, benchmark/chimera/cuda/
// bmm_bmm_cuda.py:69-150): first GEMM, element-wise stage cast to the input type, second GEMM.
//
// Why a cluster.  One 128-row block of Y with N up to 1024 fp32 columns does not fit the 512
// TMEM columns of an SM, and its hidden row block (128 x L 16-bit) does not fit shared memory.
// So four CTAs (a cluster, one SM each) share a row block:
//   * CTA q owns the Y columns [q N/4, (q+1) N/4) -- N/4 <= 256 TMEM columns, resident for the
//     whole kernel -- and every fourth 128-wide chunk of the hidden dimension;
//   * for its own chunks it runs GEMM1 (X block x W1 chunk -> 128 x 128 fp32 in TMEM), applies
//     the activation, rounds to the 16-bit type, writes the tile into its shared memory in the
//     K-major 128B-swizzled operand layout, and pushes a copy to the three peers with a
//     shared::cta -> shared::cluster bulk copy that signals the peer's mbarrier;
//   * for every chunk (its own and the peers') it runs GEMM2 (H chunk x its W2 slice) into Y.
// The hidden activations therefore exist only in TMEM and (distributed) shared memory.
// No TMA load in this file uses cluster multicast; every CTA fetches its own operands.
//
// Warp roles (256 threads): warps 0-3 epilogue (thread r <-> row r / TMEM lane r), warps 4 and 7 TMA
// producers (alternate ring stages), warp 5 MMA issuer (converged, one elected lane issues),
// warp 6 relay (after this CTA's GEMM2 has finished with a slot, tells the CTA that fills it next).
//
// Hand-over of hidden chunks: in units of 64 columns (16 KB), six unit slots per CTA; unit u goes to
// slot u % 6 of all four CTAs.  The owner refills a slot as soon as all four CTAs have consumed the
// previous unit in it (slot_free, count 4), so the copy of unit u + 6 runs under GEMM2 of units
// u + 1 .. u + 5.  Tensor-pipe order on every CTA: GEMM1 of its first two chunks, then per unit
//   GEMM2(unit u)  |  an eighth of GEMM1 of the own chunk two rounds ahead
// while the epilogue warps drain GEMM1's accumulator (two TMEM buffers, ping-pong).
#define DITTO_TRY_WAIT_HINT_NS 5000   // see mbar_try_wait
#include "mlp_sm100.cuh"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstdio>
#include <cstring>

#include "../../include/ditto_b200.h"
#include "host_util.cuh"
#include "mlp_common.cuh"
#include "sm100_ptx.cuh"

// Optional timeline capture for tuning (compiled in only with -DDITTO_TRACE): the first CTA stores
// clock64() stamps of its rounds into the buffer passed as the call's workspace.
#ifdef DITTO_TRACE
#define DITTO_STAMP(i, k)                                                                   \
  do {                                                                                      \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (i) < 8) p.trace[(i) * 16 + (k)] = clock64(); \
  } while (0)
#define DITTO_TIMED(acc, expr)          \
  do {                                 \
    const long long t_ = clock64();    \
    expr;                              \
    acc += clock64() - t_;             \
  } while (0)
#else
#define DITTO_STAMP(i, k) do {} while (0)
#define DITTO_TIMED(acc, expr) do { expr; } while (0)
#endif

// 1: calls that do not name a kernel take the 256-wide-chunk kernel where it covers the shape
#ifndef DITTO_MLP_DEFAULT_WIDE
#define DITTO_MLP_DEFAULT_WIDE 1
#endif

#ifndef DITTO_MLP_UNITS
#define DITTO_MLP_UNITS 6
#endif

namespace ditto_b200 {

namespace {

constexpr int kCluster = 4;
constexpr int kRows = 128;            // rows of X / Y per cluster
constexpr int kChunk = 128;           // hidden columns per chunk
constexpr int kStageBytes = 32 * 1024;
// Hidden chunks travel and are consumed in units of 64 columns (128 rows x 64 x 16 bit = 16 KB, one
// swizzle atom column = one GEMM2 k-step group).  Unit u = 2 * chunk + half lives in slot u % kUnits of
// every CTA; a slot is handed on unit by unit, so the exchange of unit u + kUnits overlaps GEMM2 on the
// units in between.  Small units keep the hand-over loop (GEMM2 done everywhere -> owner refills ->
// copies land) short relative to the work that hides it.  Slots and operand ring share 224 KB.
constexpr int kUnitBytes = kRows * 64 * 2;
constexpr int kUnits = DITTO_MLP_UNITS;
constexpr int kStages = (14 - kUnits) / 2;
constexpr int kThreads = 256;
constexpr uint32_t kProducers = 2;         // TMA-issuing threads (warps 4 and 7)
constexpr int kOffSlots = 0;
constexpr int kOffRing = kOffSlots + kUnits * kUnitBytes;
constexpr int kOffBar = kOffRing + kStages * kStageBytes;
constexpr int kSmemBytes = kOffBar + 512 + 1024;

struct MlpParams {
  CUtensorMap map_x;   // X  [batch, M, K] (3-D: a partial last row block is zero-filled), box 64 x 128 x 1
  CUtensorMap map_w1;  // IO: W1 [batch*K, L], box 64 x 64;  OI: W1 [batch*L, K], box 64 x 128
  CUtensorMap map_w2;  // IO: W2 [batch*L, N], box 64 x 64;  OI: W2 [batch*N, L], box 64 x N/4
  void* y;             // Y  [batch, M, N]
  float* slabs;        // shared row blocks: fp32 partials [part][batch][shared row blocks * 128][N]
  int* counters;       // shared row blocks: one per (batch, shared row block, CTA rank), zero at launch
  int M, N, K, L;
  int row_blocks;      // ceil(M / 128)
  int whole_blocks;    // the first row blocks are computed by one cluster each ...
  int parts;           // ... the others by `parts` clusters, each taking a range of the hidden chunks
  int w_oi;            // 1: weights stored [out, in] (K-major B operands)
  int w_atoms;         // [in, out] weights: maps are 3-D atom views, one box per operand tile
  int act1, act2;      // 0 identity, 1 ReLU, 2 GELU (tanh form) after the first / second GEMM
  const void* b1;      // optional bias [batch, L] added before act1 (16-bit, same type as X); may be null
  const void* b2;      // optional bias [batch, N] added before act2; may be null
  int* status;
  long long* trace;    // timeline buffer of -DDITTO_TRACE builds (null otherwise)
};

struct Bars {
  uint64_t full[kStages], empty[kStages];
  uint64_t h_tmem_full[2], h_tmem_empty[2];
  uint64_t h_ready[kUnits];    // the unit of the slot's current use is present (own: local arrive; peer's: pushed bytes)
  uint64_t g2_done[kUnits];    // this CTA's GEMM2 has finished reading the slot
  uint64_t slot_free[kUnits];  // all four CTAs have (count 4, remote arrivals); kept at the CTA that writes the slot next
  uint64_t y_done;
  uint64_t epi_sync;     // the 128 epilogue threads, once per round (bounded, unlike bar.sync)
  uint32_t tmem_base;
  uint32_t abort_word;
  uint32_t last_flag;    // shared row blocks: this CTA is the last of its rank to finish the row block
};
static_assert(sizeof(Bars) <= 512, "barrier block too large");

}  // namespace

template <bool BF16>
__global__ void __cluster_dims__(kCluster, 1, 1) __launch_bounds__(kThreads, 1)
    mlp_chain_kernel(const __grid_constant__ MlpParams p) {
  extern __shared__ uint8_t smem_raw[];
  // Every CTA of the cluster rounds its dynamic shared memory up by the same amount (the base
  // offset is identical across CTAs of a launch), so slot and barrier offsets match across peers.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bar = reinterpret_cast<Bars*>(smem + kOffBar);
  volatile uint32_t* abort_word = &bar->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t q = cluster_ctarank();
  // Work item = (row block, range of hidden chunks).  The first whole_blocks row blocks of a batch entry are
  // computed by one cluster each; each of the others is shared by `parts` clusters, whose fp32 partials of Y
  // meet in the caller's scratch memory (the hidden activations themselves never leave the chip).
  const int item = blockIdx.x / kCluster;
  const bool shared = item >= p.whole_blocks;
  const int nparts = shared ? p.parts : 1;
  const int rb = shared ? p.whole_blocks + (item - p.whole_blocks) / p.parts : item;
  const int sp = shared ? (item - p.whole_blocks) % p.parts : 0;
  const int row0 = rb * kRows;
  const int b = blockIdx.y;
  const int NS = p.N / kCluster;          // this CTA's Y columns
  const int all_chunks = p.L / kChunk;
  const int c0 = static_cast<int>(static_cast<long long>(sp) * all_chunks / nparts);           // first hidden chunk of the item
  const int chunks = static_cast<int>(static_cast<long long>(sp + 1) * all_chunks / nparts) - c0;  // any count; chunk n of the item belongs to CTA n % 4
  const int units = 2 * chunks;           // 64-column halves of them
  // this CTA owns chunk 4 i + q for i < rounds: one round fewer than its peers if the last round is partial
  const int rounds = (chunks - static_cast<int>(q) + kCluster - 1) / kCluster;
  const int ksteps1 = p.K / 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bar->full[s], 1);
      mbar_init(&bar->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->h_tmem_full[i], 1);
      mbar_init(&bar->h_tmem_empty[i], kRows);
    }
    for (int i = 0; i < kUnits; ++i) {
      mbar_init(&bar->h_ready[i], 1);
      mbar_init(&bar->g2_done[i], 1);
      mbar_init(&bar->slot_free[i], kCluster);
    }
    mbar_init(&bar->y_done, 1);
    mbar_init(&bar->epi_sync, kRows);
    bar->abort_word = 0;
    bar->last_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&bar->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                     // peers' barriers exist before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = bar->tmem_base;
  // Programmatic dependent launch: the set-up above touches no global memory and may overlap the end of
  // the kernel ahead in the stream; from here on its results are needed.
  grid_dependency_wait();
  grid_launch_dependents();
  const uint32_t tmem_y = tmem_base;
  const uint32_t tmem_h = tmem_base + 256;

  if (warp == 4 || warp == 7) {
    // ------------------------------------------------------------ TMA producers (one thread each)
    // One thread gets a ring stage out per ~350-700 clocks (barrier wait + expect_tx + the copies),
    // i.e. at most ~46 B/clk of operands; two threads taking alternate stages lift that limit.
    if (lane == 0) {
      const uint32_t pw = warp == 4 ? 0u : 1u;
      tma_prefetch_desc(&p.map_x);
      tma_prefetch_desc(&p.map_w1);
      tma_prefetch_desc(&p.map_w2);
      int ps = 0;
      uint32_t pph = 0, cnt = 0;
      bool ok = true;
      // Both producers walk the same sequence of stages; each fills the ones of its parity.
      auto acquire = [&](uint32_t bytes, uint32_t code) -> uint8_t* {
        if ((cnt++ & (kProducers - 1)) != pw) return nullptr;
        ok = mbar_wait(&bar->empty[ps], pph ^ 1, abort_word, code);
        if (!ok) return nullptr;
        mbar_arrive_expect_tx(&bar->full[ps], bytes);
        return smem + kOffRing + ps * kStageBytes;
      };
      auto advance = [&]() {
        if (++ps == kStages) { ps = 0; pph ^= 1; }
      };
      auto load_g1 = [&](int i, int ks0, int ks1) {   // operands of k-steps [ks0, ks1) of GEMM1 for this CTA's chunk of round i
        const int g = c0 + i * kCluster + static_cast<int>(q);   // hidden chunk
        for (int ks = ks0; ks < ks1 && ok; ++ks) {
          uint8_t* dst = acquire(2 * 16384, 0x100 + i);
          if (dst != nullptr) {
            tma_load_3d(dst, &p.map_x, &bar->full[ps], ks * 64, row0, b);
            if (p.w_oi) {
              tma_load_2d(dst + 16384, &p.map_w1, &bar->full[ps], ks * 64, b * p.L + g * kChunk);
            } else if (p.w_atoms) {
              tma_load_3d(dst + 16384, &p.map_w1, &bar->full[ps], 0, b * p.K + ks * 64, g * (kChunk / 64));
            } else {
              tma_load_2d(dst + 16384, &p.map_w1, &bar->full[ps], g * kChunk, b * p.K + ks * 64);
              tma_load_2d(dst + 16384 + 8192, &p.map_w1, &bar->full[ps], g * kChunk + 64, b * p.K + ks * 64);
            }
          }
          advance();
        }
      };
      auto load_g2 = [&](int u) {         // this CTA's W2 slice for hidden unit u (64 hidden columns)
        const int g = c0 + (u >> 1), kk = u & 1;             // hidden chunk and its half
        uint8_t* dst = acquire(64 * NS * 2, 0x200 + (u >> 3));
        if (dst != nullptr) {
          if (p.w_oi) {
            tma_load_2d(dst, &p.map_w2, &bar->full[ps], g * kChunk + kk * 64, b * p.N + q * NS);
          } else if (p.w_atoms) {
            tma_load_3d(dst, &p.map_w2, &bar->full[ps], 0, b * p.L + g * kChunk + kk * 64, q * (NS / 64));
          } else {
            for (int a = 0; a < NS / 64; ++a)
              tma_load_2d(dst + a * 8192, &p.map_w2, &bar->full[ps], q * NS + a * 64, b * p.L + g * kChunk + kk * 64);
          }
        }
        advance();
      };
      // the order the MMA warp consumes the ring in: see there
      if (rounds > 0) load_g1(0, 0, ksteps1);
      if (rounds > 1) load_g1(1, 0, ksteps1);
      for (int u = 0; u < units && ok; ++u) {
        const int i = u >> 3, e = u & 7;
        load_g2(u);
        if (i + 2 < rounds) load_g1(i + 2, e * ksteps1 / 8, (e + 1) * ksteps1 / 8);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer (converged warp)
    const uint32_t issuer = elect_one();
    const uint32_t idesc1 = umma_idesc_f16(BF16, kRows, kChunk, false, p.w_oi == 0);
    const uint32_t idesc2 = umma_idesc_f16(BF16, kRows, NS, false, p.w_oi == 0);
    const uint32_t ring = smem_u32(smem + kOffRing);
    const uint32_t slots = smem_u32(smem + kOffSlots);
    int cs = 0;
    uint32_t cph = 0;
    bool ok = true;
    long long w_acc = 0, w_g1 = 0, w_unit = 0, w_g2 = 0;   // clocks spent waiting (timeline builds only)
    (void)w_acc; (void)w_g1; (void)w_unit; (void)w_g2;
    auto wait = [&](uint64_t* bp, uint32_t parity, uint32_t code) {
      bool r = mbar_wait(bp, parity, abort_word, code);
      r = __all_sync(0xffffffffu, r);
      tc_fence_after_sync();
      return r;
    };
    auto advance = [&]() {
      if (++cs == kStages) { cs = 0; cph ^= 1; }
    };
    // GEMM1 of this CTA's chunk of round i, k-steps [ks0, ks1); `first` / `last`: the part that starts / ends the chunk
    auto g1 = [&](int i, int ks0, int ks1, bool first, bool last) {
      const int hb = i & 1;
      if (first && i >= 2) DITTO_TIMED(w_acc, ok = wait(&bar->h_tmem_empty[hb], ((i >> 1) - 1) & 1, 0x300 + i));
      if (first && lane == 0) DITTO_STAMP(i, 0);
      for (int ks = ks0; ks < ks1 && ok; ++ks) {
        DITTO_TIMED(w_g1, ok = wait(&bar->full[cs], cph, 0x310 + i));
        if (!ok) break;
        const uint32_t st = ring + cs * kStageBytes;
        const uint64_t da = umma_desc_sw128(st, 16, 1024);
        const uint64_t db = p.w_oi ? umma_desc_sw128(st + 16384, 16, 1024) : umma_desc_sw128(st + 16384, 8192, 1024);
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) {
          const uint32_t offb = p.w_oi ? (s4 * 32) >> 4 : (s4 * 2048) >> 4;
          umma_ss_elected(tmem_h + hb * kChunk, da + ((s4 * 32) >> 4), db + offb, idesc1, (ks | s4) ? 1u : 0u, issuer);
        }
        umma_commit_elected(&bar->empty[cs], issuer);
        advance();
      }
      if (last && ok) umma_commit_elected(&bar->h_tmem_full[hb], issuer);
      if (last && lane == 0) DITTO_STAMP(i, 1);
    };
    // GEMM2 on hidden unit u (64 hidden columns of any CTA's chunk), accumulated into Y
    auto g2 = [&](int u) {
      const int sl = u % kUnits;
      const int owner = (u >> 1) & 3;
      if (owner != static_cast<int>(q) && lane == 0)
        mbar_arrive_expect_tx(&bar->h_ready[sl], kUnitBytes);   // a peer pushes this unit; the owner's own copy arrives locally
      __syncwarp();
      if (lane == 0 && (u & 7) == 0) DITTO_STAMP(u >> 3, 2);
      DITTO_TIMED(w_unit, ok = wait(&bar->h_ready[sl], (u / kUnits) & 1, 0x400 + (u >> 3)));
      if (lane == 0 && (u & 1) == 0) DITTO_STAMP(u >> 3, 9 + ((u >> 1) & 3));
      if (ok) DITTO_TIMED(w_g2, ok = wait(&bar->full[cs], cph, 0x410 + (u >> 3)));
      if (ok) {
        const uint32_t st = ring + cs * kStageBytes;
        const uint64_t da = umma_desc_sw128(slots + sl * kUnitBytes, 16, 1024);
        const uint64_t db = p.w_oi ? umma_desc_sw128(st, 16, 1024) : umma_desc_sw128(st, 8192, 1024);
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) {
          const uint32_t offb = p.w_oi ? (s4 * 32) >> 4 : (s4 * 2048) >> 4;
          umma_ss_elected(tmem_y, da + ((s4 * 32) >> 4), db + offb, idesc2, (u | s4) ? 1u : 0u, issuer);
        }
        umma_commit_elected(&bar->empty[cs], issuer);
        advance();
        umma_commit_elected(&bar->g2_done[sl], issuer);
      }
      if (lane == 0 && (u & 7) == 7) DITTO_STAMP(u >> 3, 4);
    };
    // Tensor-pipe order: GEMM1 of the first two own chunks, then unit by unit GEMM2(unit u) followed by an
    // eighth of GEMM1 of the own chunk two rounds ahead, so that a unit that arrives late stalls little.
    if (rounds > 0) g1(0, 0, ksteps1, true, true);
    if (rounds > 1 && ok) g1(1, 0, ksteps1, true, true);
    for (int u = 0; u < units && ok; ++u) {
      const int i = u >> 3, e = u & 7;
      g2(u);
      if (i + 2 < rounds && ok) g1(i + 2, e * ksteps1 / 8, (e + 1) * ksteps1 / 8, e == 0, e == 7);
    }
    if (ok) umma_commit_elected(&bar->y_done, issuer);
#ifdef DITTO_TRACE
    if (lane == 0 && p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0) {
      p.trace[200] = w_acc; p.trace[201] = w_g1; p.trace[202] = w_unit; p.trace[203] = w_g2; p.trace[204] = clock64();
    }
#endif
  } else if (warp == 6) {
    // ------------------------------------------------------------ relay (one thread)
    if (lane == 0) {
      for (int u = 0; u < units; ++u) {
        const int sl = u % kUnits;
        if (!mbar_wait(&bar->g2_done[sl], (u / kUnits) & 1, abort_word, 0x500 + (u >> 3))) break;
        if ((u & 7) == 7) DITTO_STAMP(u >> 3, 5);
        // tell the CTA that writes this slot next (the owner of unit u + kUnits)
        if (u + kUnits < units) mbar_arrive_cluster(&bar->slot_free[sl], static_cast<uint32_t>(((u + kUnits) >> 1) & 3));
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
      const int g = i * kCluster + static_cast<int>(q);   // this CTA's chunk of the round
      ok = mbar_wait(&bar->h_tmem_full[hb], (i >> 1) & 1, abort_word, 0x600 + i);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      if (threadIdx.x == 0) DITTO_STAMP(i, 6);
      uint32_t h[kChunk];
      tmem_ld_x128_wait(tmem_h + hb * kChunk + lane_base, h);
      tc_fence_before_sync();
      mbar_arrive(&bar->h_tmem_empty[hb]);
      uint32_t pk[kChunk / 2];
      const uint32_t* bias1 = p.b1 == nullptr ? nullptr
                                              : reinterpret_cast<const uint32_t*>(p.b1) +
                                                    (static_cast<size_t>(b) * p.L + (c0 + i * kCluster + q) * kChunk) / 2;
      act_pack<BF16>(h, bias1, p.act1, pk);
      // the chunk leaves as two units of 64 columns
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const int u = 2 * g + kk;
        const int sl = u % kUnits;
        uint8_t* my_slot = smem + kOffSlots + sl * kUnitBytes;
        if (u >= kUnits) {
          // every CTA of the cluster has finished GEMM2 on the slot's previous unit: it may be overwritten
          uint32_t par = 0;
#pragma unroll
          for (int t = 0; t < kUnits; ++t)
            if (t == sl) par = free_waits[t]++ & 1;
          ok = mbar_wait_cluster(&bar->slot_free[sl], par, abort_word, 0x700 + i);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        if (threadIdx.x == 0 && kk == 0) DITTO_STAMP(i, 7);
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
          const int ch = kk * 8 + c8;
          const uint4 v = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
          *reinterpret_cast<uint4*>(my_slot + row * 128 + ((c8 ^ (row & 7)) << 4)) = v;
        }
        fence_proxy_async_smem();
        mbar_arrive(&bar->epi_sync);                        // all 128 rows of the unit are written
        ok = mbar_wait(&bar->epi_sync, kk, abort_word, 0x780 + i);   // two phases per round
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (threadIdx.x == 0) {
          const uint32_t slot_addr = smem_u32(my_slot);
          const uint32_t bar_addr = smem_u32(&bar->h_ready[sl]);
          for (uint32_t d = 1; d < kCluster; ++d) {
            const uint32_t c = (q + d) % kCluster;
            bulk_copy_to_peer(map_to_cta(slot_addr, c), my_slot, kUnitBytes, map_to_cta(bar_addr, c));
          }
          mbar_arrive(&bar->h_ready[sl]);      // the local copy is in place
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
      const uint32_t* bias2 = p.b2 == nullptr ? nullptr
                                              : reinterpret_cast<const uint32_t*>(p.b2) +
                                                    (static_cast<size_t>(b) * p.N + static_cast<size_t>(q) * NS) / 2;
      if (!shared) {
        uint8_t* yrow = reinterpret_cast<uint8_t*>(p.y) +
                        ((static_cast<size_t>(b) * p.M + row0 + row) * p.N + static_cast<size_t>(q) * NS) * 2;
        for (int cc = 0; cc < NS; cc += 32) {
          uint32_t o[32];
          tmem_ld_x32_wait(tmem_y + lane_base + cc, o);
          uint32_t w[16];
          act_pack<BF16>(o, bias2 == nullptr ? nullptr : bias2 + cc / 2, p.act2, w);
          if (row0 + row < p.M) {               // rows >= M of a partial last block were computed on zero-filled X
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(yrow + cc * 2 + j * 16) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          }
        }
      } else {
        // this cluster's fp32 partial goes to its slab; the last cluster to finish the row block (a counter per
        // CTA rank) adds the slabs in slab order -- the result does not depend on which one came last -- and
        // applies bias and activation
        const size_t mpad = static_cast<size_t>(p.row_blocks - p.whole_blocks) * kRows;   // rows of the shared blocks
        const size_t slab = static_cast<size_t>(gridDim.y) * mpad * p.N;
        const int srow0 = row0 - p.whole_blocks * kRows;
        float* region = p.slabs + (static_cast<size_t>(b) * mpad + srow0) * p.N + static_cast<size_t>(q) * NS;
        float* prow = region + static_cast<size_t>(sp) * slab + static_cast<size_t>(row) * p.N;
        for (int cc = 0; cc < NS; cc += 32) {
          uint32_t o[32];
          tmem_ld_x32_wait(tmem_y + lane_base + cc, o);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            __stcg(reinterpret_cast<uint4*>(prow + cc) + j, make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]));
        }
        __threadfence();
        // epi_sync has completed two phases per round: its next phase has parity 0
        mbar_arrive(&bar->epi_sync);
        ok = mbar_wait(&bar->epi_sync, 0, abort_word, 0x810);
        ok = __all_sync(0xffffffffu, ok);
        if (ok && threadIdx.x == 0) {
          int* ctr = p.counters + (static_cast<size_t>(b) * (p.row_blocks - p.whole_blocks) + (rb - p.whole_blocks)) * kCluster + q;
          const int seen = atomicAdd(ctr, 1);
          __threadfence();
          bar->last_flag = (seen == p.parts - 1) ? 1u : 0u;
        }
        // (the combining pass runs below, on all threads of the CTA, once the other warps are done too)
      }
    }
  }

  // After a wait has given up, copies this CTA issued (TMA loads into its ring, pushes into its peers'
  // slots) may still be in flight; they complete within microseconds.  Give them that time before the
  // shared memory they target is released.
  if (*abort_word != 0u) {
    for (int t = 0; t < 64; ++t) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (shared && bar->last_flag != 0u && bar->abort_word == 0u) {
    // Every part of this CTA's (rows, columns) region of a shared row block is in its slab, and this
    // cluster was the last to get there: add the slabs in slab order, apply bias and activation, write Y.
    // All warps take part -- the pass is bound by how many loads the CTA keeps in flight.
    __threadfence();
    const size_t mpad = static_cast<size_t>(p.row_blocks - p.whole_blocks) * kRows;
    const size_t slab = static_cast<size_t>(gridDim.y) * mpad * p.N;
    const size_t col0 = static_cast<size_t>(q) * NS;
    const uint32_t* bias2 = p.b2 == nullptr ? nullptr
                                            : reinterpret_cast<const uint32_t*>(p.b2) + (static_cast<size_t>(b) * p.N + col0) / 2;
    combine_slabs<BF16>(p.slabs + (static_cast<size_t>(b) * mpad + (row0 - p.whole_blocks * kRows)) * p.N + col0, slab, p.parts,
                        min(kRows, p.M - row0), NS, static_cast<size_t>(p.N), bias2, p.act2,
                        reinterpret_cast<uint8_t*>(p.y) + ((static_cast<size_t>(b) * p.M + row0) * p.N + col0) * 2,
                        static_cast<size_t>(p.N) * 2, static_cast<int>(threadIdx.x), kThreads);
  }
  cluster_sync_all();                     // no CTA leaves while a peer may still write to it
  if (warp == 0) {
    tmem_dealloc(tmem_base, 512);
    if (lane == 0 && bar->abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, static_cast<int>(bar->abort_word));
  }
}

// ------------------------------------------------------------------ host side
namespace {

// [batch, rows, cols] row-major, boxes of box_cols x box_rows inside one batch entry: rows past the end of
// an entry are zero-filled instead of running into the next entry.
int quad_map_3d(CUtensorMap* map, bool bf16, const void* base, uint64_t cols, uint64_t rows, uint64_t batch,
                uint32_t box_cols, uint32_t box_rows) {
  const uint64_t dims[3] = {cols, rows, batch}, strides[2] = {cols * 2, rows * cols * 2};
  const uint32_t box[3] = {box_cols, box_rows, 1};
  return make_tensor_map(map, bf16, base, 3, dims, strides, box);
}
int quad_map_2d(CUtensorMap* map, bool bf16, const void* base, uint64_t cols, uint64_t rows, uint32_t box_cols,
                uint32_t box_rows) {
  const uint64_t dims[2] = {cols, rows}, strides[1] = {cols * 2};
  const uint32_t box[2] = {box_cols, box_rows};
  return make_tensor_map(map, bf16, base, 2, dims, strides, box);
}
// [rows, cols] row-major seen as (64 columns, rows, cols / 64): one box of 64 x box_rows x box_atoms
// brings box_atoms 64-column swizzle atoms of an MN-major operand tile with a single TMA operation
// (atom a lands at a * box_rows * 128 bytes, exactly the operand layout).
int quad_atom_map(CUtensorMap* map, bool bf16, const void* base, uint64_t cols, uint64_t rows, uint32_t box_rows,
                  uint32_t box_atoms) {
  const uint64_t dims[3] = {64, rows, cols / 64}, strides[2] = {cols * 2, 128};
  const uint32_t box[3] = {64, box_rows, box_atoms};
  return make_tensor_map(map, bf16, base, 3, dims, strides, box);
}

template <bool BF16>
cudaError_t quad_launch(const cudaLaunchConfig_t& cfg, const MlpParams& p) {
  // the function attribute is set once per device (this instantiation's static)
  static std::atomic<unsigned long long> configured{0};
  int dev = 0;
  cudaError_t e = current_device_checked(&dev);
  if (e != cudaSuccess) return e;
  if (!device_configured(configured, dev)) {
    e = cudaFuncSetAttribute(mlp_chain_kernel<BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    mark_device_configured(configured, dev);
  }
  return cudaLaunchKernelEx(&cfg, mlp_chain_kernel<BF16>, p);
}

bool quad_supported(int N, int K, int L) {
  // 128-row blocks (the last one may be partial); hidden size a multiple of the 128-wide chunk (the last
  // round of four chunks may be partial); N/4 Y columns per CTA (<= 256 TMEM columns, whole 64-column
  // swizzle atoms); K in 64-wide steps.
  return L % kChunk == 0 && K % 64 == 0 && N % (kCluster * 64) == 0 && N <= kCluster * 256;
}

// in units of a 128-wide chunk: an item takes about 14 us + 2.1 us per chunk, sharing adds about 17 us
constexpr double kQuadFixedCost = 6.5, kQuadSharedCost = 8.0;

RowBlockPlan quad_plan(int batch, int M, int L, int cluster_slots, bool allow_scratch) {
  const int rbs = (M + kRows - 1) / kRows;
  if (!allow_scratch) return {rbs, 1};
  return plan_row_blocks(batch, rbs, L / kChunk, kCluster, kMaxSlabs, cluster_slots, kQuadFixedCost, kQuadSharedCost);
}

int launch_mlp_quad(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                    bool bf16, int w_layout, int act1, int act2, const void* b1, const void* b2, const RowBlockPlan& plan,
                    void* workspace, int* status, cudaStream_t stream, long long* trace) {
  if (!quad_supported(N, K, L) || batch > 65535) return DITTO_ERR_UNSUPPORTED;
  const int rbs = (M + kRows - 1) / kRows;
  const int shared_blocks = rbs - plan.whole_blocks;
  if (plan.whole_blocks < 0 || shared_blocks < 0 || plan.parts < 1 || plan.parts > L / kChunk || plan.parts > kMaxSlabs)
    return DITTO_ERR_INVALID_ARG;
  const bool split = shared_blocks > 0 && plan.parts > 1;
  const int NS = N / kCluster;
  MlpParams p;
  std::memset(&p, 0, sizeof(p));
  int rc = quad_map_3d(&p.map_x, bf16, x, K, M, batch, 64, 128);
  if (rc) return rc;
  if (w_layout == 1) {
    rc = quad_map_2d(&p.map_w1, bf16, w1, K, static_cast<uint64_t>(batch) * L, 64, 128);
    if (rc) return rc;
    rc = quad_map_2d(&p.map_w2, bf16, w2, L, static_cast<uint64_t>(batch) * N, 64, NS);
    if (rc) return rc;
  } else {
    // one TMA operation per operand tile where the driver accepts the atom view, else one per atom
    p.w_atoms = quad_atom_map(&p.map_w1, bf16, w1, L, static_cast<uint64_t>(batch) * K, 64, 2) == DITTO_OK &&
                quad_atom_map(&p.map_w2, bf16, w2, N, static_cast<uint64_t>(batch) * L, 64, NS / 64) == DITTO_OK;
    if (!p.w_atoms) {
      rc = quad_map_2d(&p.map_w1, bf16, w1, L, static_cast<uint64_t>(batch) * K, 64, 64);
      if (rc) return rc;
      rc = quad_map_2d(&p.map_w2, bf16, w2, N, static_cast<uint64_t>(batch) * L, 64, 64);
      if (rc) return rc;
    }
  }
  p.y = y;
  p.M = M;
  p.N = N;
  p.K = K;
  p.L = L;
  p.w_oi = w_layout == 1;
  p.act1 = act1;
  p.act2 = act2;
  p.b1 = b1;
  p.b2 = b2;
  p.status = status;
  p.trace = trace;
  p.row_blocks = rbs;
  p.whole_blocks = split ? plan.whole_blocks : rbs;
  p.parts = split ? plan.parts : 1;
  if (split) {
    if (workspace == nullptr) return DITTO_ERR_WORKSPACE;
    const size_t slab_bytes = static_cast<size_t>(plan.parts) * batch * shared_blocks * kRows * N * sizeof(float);
    p.slabs = static_cast<float*>(workspace);
    p.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + slab_bytes);
    cudaError_t e = cudaMemsetAsync(p.counters, 0, static_cast<size_t>(batch) * shared_blocks * kCluster * sizeof(int), stream);
    if (e != cudaSuccess) return cuda_fail("mlp chain counters", e);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(kCluster * (p.whole_blocks + (rbs - p.whole_blocks) * p.parts)), batch, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see grid_dependency_wait in the kernel
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = split ? 0 : 1;           // a launch with shared row blocks follows its own counter reset: plain stream order
  const cudaError_t e = bf16 ? quad_launch<true>(cfg, p) : quad_launch<false>(cfg, p);
  return e == cudaSuccess ? DITTO_OK : cuda_fail("mlp chain kernel launch", e);
}

}  // namespace

int mlp_quad_cluster_slots(bool bf16, int* slots) {
  static std::atomic<int> cached[2][kMaxDevices];
  int dev = 0;
  cudaError_t e = current_device_checked(&dev);
  if (e != cudaSuccess) return cuda_fail("mlp chain kernel set-up", e);
  int n = cached[bf16 ? 1 : 0][dev].load(std::memory_order_relaxed);
  if (n == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kCluster * 64, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    if (bf16) {
      e = cudaFuncSetAttribute(mlp_chain_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
      if (e == cudaSuccess) e = cudaOccupancyMaxActiveClusters(&n, mlp_chain_kernel<true>, &cfg);
    } else {
      e = cudaFuncSetAttribute(mlp_chain_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
      if (e == cudaSuccess) e = cudaOccupancyMaxActiveClusters(&n, mlp_chain_kernel<false>, &cfg);
    }
    if (e != cudaSuccess) return cuda_fail("mlp chain kernel set-up", e);
    cached[bf16 ? 1 : 0][dev].store(n > 0 ? n : 1, std::memory_order_relaxed);
  }
  *slots = n > 0 ? n : 1;
  return DITTO_OK;
}

// ------------------------------------------------------------------ the chain without caller-provided scratch
// Scratch memory that belongs to the library image instead of the caller: a fixed array in device memory
// that every GPU holds from the moment it loads this library until the process exits.
constexpr size_t kStaticScratchBytes = 12u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int launch_mlp_static_scratch(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                              bool bf16, int w_layout, int act1, int* status, cudaStream_t stream) {
  if (!quad_supported(N, K, L)) return DITTO_ERR_UNSUPPORTED;
  // In host code `g_static_scratch` is only a handle for the symbol, not an address the GPU can use: the
  // array's device address is looked up once per device, with that device current, and kept.
  static std::atomic<unsigned char*> scratch_of_device[kMaxDevices];
  int dev = 0;
  cudaError_t e = current_device_checked(&dev);
  if (e != cudaSuccess) return cuda_fail("static-scratch set-up", e);
  unsigned char* scratch = scratch_of_device[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) return cuda_fail("static-scratch set-up (cudaGetSymbolAddress)", e);
    scratch = static_cast<unsigned char*>(ptr);
    scratch_of_device[dev].store(scratch, std::memory_order_release);
  }
  int slots = 0;
  int rc = mlp_quad_cluster_slots(bf16, &slots);
  if (rc) return rc;
  const RowBlockPlan plan = quad_plan(batch, M, L, slots, true);
  const size_t need = plan_workspace_bytes(plan, batch, (M + kRows - 1) / kRows, kRows, N, kCluster);
  if (need > kStaticScratchBytes) {
    char msg[160];
    std::snprintf(msg, sizeof(msg), "this shape needs %zu bytes of scratch memory, the built-in array holds %zu; "
                  "use ditto_b200_gemm_relu_gemm with a workspace", need, kStaticScratchBytes);
    set_error("ditto_b200_gemm_relu_gemm_static_scratch", msg);
    return DITTO_ERR_WORKSPACE;
  }
  // The counters at the end of the used part are cleared by the launch itself (cudaMemsetAsync on `stream`);
  // the partial-result slabs are written before they are read and need no clearing.
  return launch_mlp_quad(x, w1, w2, y, batch, M, N, K, L, bf16, w_layout, act1, 0, nullptr, nullptr, plan, scratch, status,
                         stream, nullptr);
}

// Which kernel an "auto" call takes: the 256-wide-chunk kernel where it covers the shape (measured fastest at
// the benchmark configuration), the 128-wide one for hidden sizes that are only multiples of 128, the pair
// kernel for what neither covers.
static int resolve_variant(int variant, int N, int K, int L, int w_layout) {
  if (variant != kMlpAuto) return variant;
  if (DITTO_MLP_DEFAULT_WIDE && mlp_wide_supported(N, K, L)) return kMlpWide;
  if (quad_supported(N, K, L)) return kMlpQuad;
  if (mlp_wide_supported(N, K, L)) return kMlpWide;
  if (mlp_pair_supported(N, K, L, w_layout)) return kMlpPair;
  return kMlpQuad;
}

size_t mlp_workspace_bytes(int batch, int M, int N, int K, int L, bool bf16, int w_layout, int variant) {
  int slots = 0;
  switch (resolve_variant(variant, N, K, L, w_layout)) {
    case kMlpWide:
      if (!mlp_wide_supported(N, K, L) || mlp_wide_cluster_slots(bf16, &slots) != DITTO_OK) return 0;
      return mlp_wide_workspace_bytes(batch, M, N, mlp_wide_plan(batch, M, L, slots, true));
    case kMlpPair:
      if (!mlp_pair_supported(N, K, L, w_layout) || mlp_pair_cluster_slots(bf16, &slots) != DITTO_OK) return 0;
      return mlp_pair_workspace_bytes(batch, M, N, mlp_pair_plan(batch, M, L, slots, true));
    default:
      if (!quad_supported(N, K, L) || mlp_quad_cluster_slots(bf16, &slots) != DITTO_OK) return 0;
      return plan_workspace_bytes(quad_plan(batch, M, L, slots, true), batch, (M + kRows - 1) / kRows, kRows, N, kCluster);
  }
}

int launch_mlp_chain(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                     bool bf16, int w_layout, int act1, int act2, const void* b1, const void* b2, int variant,
                     void* workspace, size_t ws_bytes, int* status, cudaStream_t stream, long long* trace) {
  // With few row blocks -- or a last wave that would leave most of the device idle -- some row blocks are
  // shared by several clusters, if the caller provided the scratch memory that form needs.
  int slots = 0, rc = 0;
  switch (resolve_variant(variant, N, K, L, w_layout)) {
    case kMlpWide: {
      if (!mlp_wide_supported(N, K, L)) return DITTO_ERR_UNSUPPORTED;
      if ((rc = mlp_wide_cluster_slots(bf16, &slots)) != DITTO_OK) return rc;
      RowBlockPlan plan = mlp_wide_plan(batch, M, L, slots, workspace != nullptr);
      if (ws_bytes < mlp_wide_workspace_bytes(batch, M, N, plan)) plan = mlp_wide_plan(batch, M, L, slots, false);
      return launch_mlp_wide(x, w1, w2, y, batch, M, N, K, L, bf16, w_layout, act1, act2, b1, b2, plan, workspace, status,
                             stream, trace);
    }
    case kMlpPair: {
      if (!mlp_pair_supported(N, K, L, w_layout)) return DITTO_ERR_UNSUPPORTED;
      if ((rc = mlp_pair_cluster_slots(bf16, &slots)) != DITTO_OK) return rc;
      PairPlan plan = mlp_pair_plan(batch, M, L, slots, workspace != nullptr);
      if (ws_bytes < mlp_pair_workspace_bytes(batch, M, N, plan)) plan = mlp_pair_plan(batch, M, L, slots, false);
      return launch_mlp_pair(x, w1, w2, y, batch, M, N, K, L, bf16, w_layout, act1, act2, b1, b2, plan, workspace, status,
                             stream, trace);
    }
    default: {
      if (!quad_supported(N, K, L)) return DITTO_ERR_UNSUPPORTED;
      if ((rc = mlp_quad_cluster_slots(bf16, &slots)) != DITTO_OK) return rc;
      RowBlockPlan plan = quad_plan(batch, M, L, slots, workspace != nullptr);
      if (ws_bytes < plan_workspace_bytes(plan, batch, (M + kRows - 1) / kRows, kRows, N, kCluster))
        plan = quad_plan(batch, M, L, slots, false);
      return launch_mlp_quad(x, w1, w2, y, batch, M, N, K, L, bf16, w_layout, act1, act2, b1, b2, plan, workspace, status,
                             stream, trace);
    }
  }
}

}  // namespace ditto_b200
