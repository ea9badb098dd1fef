// Fused GEMM -> activation -> GEMM for sm_100a with 256-wide hidden chunks:
//   Y = act2(act1(X W1 + b1) W2 + b2), hidden activations on chip.
//
// Replaces what the reference would build from BatchGemmReluGemm / BatchGemmGemm
// (python_test/auto_tensorize/test_hyper_fusion_cpu.py:24-96, benchmark/chimera/cuda/bmm_bmm_cuda.py:69-150)
// and the feed-forward block of nn/model/transformer.py:21-34.
//
// Four CTAs (a cluster, one SM each) share a 128-row block of X / Y, as in mlp_sm100.cu: CTA q keeps the Y
// columns [q N/4, (q+1) N/4) in tensor memory (<= 256 columns) and owns every fourth chunk of the hidden
// dimension.  What differs is the chunk: 256 hidden columns, so GEMM1 of a chunk is one 128 x 256 accumulator
// (the other 256 tensor-memory columns) built from 128 x 256 x 16 MMAs.  Why:
//   * a 128 x 128 x 16 MMA reads 8 KB of operands from shared memory in its 64 clocks -- the whole
//     128 B/clk the SM's shared memory delivers, while TMA, the hand-over copies and the epilogue write into
//     the same memory.  Timelines of the 128-wide kernel show its GEMM1 running well below the tensor
//     pipe's rate for that reason.  128 x 256 x 16 needs 12 KB per 128 clocks (96 B/clk);
//   * the X block is re-read once per 256 hidden columns instead of once per 128: 5 MB of operands per CTA
//     at config 4 instead of 6 MB.
// The price is a single GEMM1 accumulator: the next chunk's GEMM1 cannot start before the epilogue warps
// hold the previous chunk in registers (they drain the whole chunk before they wait for free slots).
//
// A chunk leaves tensor memory as four units of 64 hidden columns (128 rows x 64 x 16 bit = 16 KB): the
// eight epilogue warps apply bias / activation, round to 16 bit, write the unit into their CTA's shared
// memory in the K-major 128B-swizzled operand layout and push it to the three peers with
// shared::cta -> shared::cluster bulk copies.  Hidden activations exist only in tensor memory and
// (distributed) shared memory.  No TMA load in this file uses cluster multicast.
//
// Roles (12 warps -- registers are handed out to warps in fours, a thirteenth would cost every thread 40):
// 0-7 epilogue (warp w: TMEM lanes 32 (w % 4) ..., column half w / 4), 8 GEMM1 operand producer, 9 GEMM1
// issuer, 10 GEMM2 operand producer, 11 GEMM2 issuer (both issuers converged, one elected lane issues).
// A unit's slot is free when all four CTAs have multiplied the unit: each CTA's GEMM2 completion arrives, by a
// multicast tcgen05.commit, directly on the barrier of the CTA that writes the slot next.
// Operands: a GEMM1 stage holds one k-step (X 128 x 64 and the W1 tile 64 x 256, 48 KB); a GEMM2 stage one W2
// tile (64 x N/4, 32 KB); each GEMM has its own ring.
// One issuing warp per GEMM: an issuer pays a few hundred clocks per stage for the barrier wait, the four MMAs
// and the commits, about what the MMAs take to execute.  A single warp issuing both GEMMs spent 90 k clocks
// issuing 65 k clocks of tensor work; with two, the issue cost of one GEMM hides behind the other's tensor
// work and whichever GEMM has its operands is issued.
// Units are numbered n in the order GEMM2 consumes them -- round by round (four chunks, one per CTA),
// inside a round quarter by quarter across the CTAs, which is the order they arrive in -- and live in slot
// n % kUnits of every CTA.
//
// Work items.  An item is (batch entry, row block, hidden range).  Normally the range is the whole hidden
// dimension and the launch is persistent: one cluster per place the device has, each walking its items with
// rings, slots and barrier phases running on, so that the next item's GEMM1 and first hidden unit are under
// way while the finished item's Y leaves tensor memory.  Row blocks may instead be shared by several clusters
// (few row blocks, many SMs): each writes its fp32 partial of Y to its own slab of the caller's workspace, and
// the last cluster to finish a row block (a counter per CTA rank) adds the slabs in a fixed order and writes
// Y; such a launch has one item per cluster.
#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <cstring>

#include "../../include/ditto_b200.h"
#include "host_util.cuh"
#include "mlp_common.cuh"
#include "mlp_sm100.cuh"
#include "sm100_ptx.cuh"

// Optional timeline capture for tuning (compiled in only with -DDITTO_TRACE): the first CTA stores
// clock64() stamps into the buffer passed as the call's workspace.
#ifdef DITTO_TRACE
#define DITTO_STAMP(slot)                                                                          \
  do {                                                                                             \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (slot) < 512) p.trace[(slot)] = clock64(); \
  } while (0)
#define DITTO_TIMED(acc, expr)          \
  do {                                 \
    const long long t_ = clock64();    \
    expr;                              \
    acc += clock64() - t_;             \
  } while (0)
#else
#define DITTO_STAMP(slot) do {} while (0)
#define DITTO_TIMED(acc, expr) do { expr; } while (0)
#endif

#ifndef DITTO_WIDE_UNITS
#define DITTO_WIDE_UNITS 4
#endif
#ifndef DITTO_WIDE_G1STAGES
#define DITTO_WIDE_G1STAGES 2
#endif
#ifndef DITTO_WIDE_W2STAGES
#define DITTO_WIDE_W2STAGES 2
#endif

namespace ditto_b200 {

namespace {

constexpr int kCluster = 4;
constexpr int kRows = 128;            // rows of X / Y per cluster
constexpr int kChunk = 256;           // hidden columns per chunk = N of a GEMM1 MMA
constexpr int kUnitCols = 64;         // hidden columns per unit: one 128-byte-row swizzle atom
constexpr int kUnitBytes = kRows * kUnitCols * 2;
constexpr int kXTileBytes = 16 * 1024;    // one k-step of the X block: 128 rows x 64
constexpr int kG1StageBytes = kXTileBytes + 32 * 1024;   // ... plus the W1 tile of the k-step (64 x 256)
constexpr int kW2StageBytes = 32 * 1024;  // one W2 tile (64 x N/4 <= 256)
constexpr int kUnits = DITTO_WIDE_UNITS;
constexpr int kG1Stages = DITTO_WIDE_G1STAGES;
constexpr int kW2Stages = DITTO_WIDE_W2STAGES;
constexpr int kEpiWarps = 8;
static_assert(kW2Stages <= kUnits, "the W2 producer arms a slot's barrier: it must not run ahead of the slot's previous unit");
constexpr int kWarpProdG1 = 8, kWarpMmaG1 = 9, kWarpProdW2 = 10, kWarpMmaG2 = 11;
// Twelve warps: registers are handed out to warps in fours, so a thirteenth would cost every thread 40 of them
// (65536 / (16 x 32) = 128 against 65536 / (12 x 32) -> 168), and the epilogue warps hold a 128 x 256 tile.
constexpr int kThreads = 12 * 32;
constexpr int kOffSlots = 0;
constexpr int kOffG1Ring = kOffSlots + kUnits * kUnitBytes;
constexpr int kOffW2Ring = kOffG1Ring + kG1Stages * kG1StageBytes;
constexpr int kOffBar = kOffW2Ring + kW2Stages * kW2StageBytes;
constexpr int kSmemBytes = kOffBar + 512 + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

struct WideParams {
  CUtensorMap map_x;   // X (K, M, batch), box 64 x 128 x 1: partial row blocks and K tails read as zero
  CUtensorMap map_w1;  // IO: W1 as atoms (64, K, L/64, batch), box 64 x 64 x 4 x 1;  OI: (K, L, batch), box 64 x 256 x 1
  CUtensorMap map_w2;  // IO: W2 as atoms (64, L, N/64, batch), box 64 x 64 x N/256 x 1;  OI: (L, N, batch), box 64 x N/4 x 1
  void* y;             // Y [batch, M, N]
  float* slabs;        // shared row blocks: fp32 partials [part][batch][shared row blocks * 128][N]
  int* counters;       // shared row blocks: one per (batch, shared row block, CTA rank), zero at launch
  int M, N, K, L;
  int row_blocks;      // ceil(M / 128)
  int n0;              // first Y column of this launch's column group (a launch covers N <= 1024 columns of ldn)
  int ldn;             // columns of Y, W2 and b2 in memory
  int batch;
  int persistent;      // 1: no shared row blocks, a cluster walks several items (see the kernel)
  int whole_blocks;    // the first row blocks are computed by one cluster each ...
  int parts;           // ... the others by `parts` clusters, each taking a range of the hidden chunks
  int w_oi;            // 1: weights stored [out, in] (K-major B operands)
  int w_atoms;         // [in, out] weights: the maps are atom views (one box per tile); else (L | N, K | L, batch), box 64 x 64 x 1
  int act1, act2;      // 0 identity, 1 ReLU, 2 GELU (tanh form)
  const void* b1;      // optional bias [batch, L] (16-bit, the input type); may be null
  const void* b2;      // optional bias [batch, N]; may be null
  int* status;
  long long* trace;    // timeline buffer of -DDITTO_TRACE builds (null otherwise)
};

struct WideBars {
  uint64_t g1full[kG1Stages], g1empty[kG1Stages];   // GEMM1 operand ring
  uint64_t w2full[kW2Stages], w2empty[kW2Stages];   // GEMM2 operand ring
  uint64_t h_tmem_full;        // GEMM1 of the chunk is in tensor memory
  uint64_t h_tmem_empty;       // the epilogue warps hold the chunk in registers (8 warp arrivals)
  uint64_t h_ready[kUnits];    // the slot's unit is present (own: local arrive; a peer's: pushed bytes)
  uint64_t slot_free[kUnits];  // all four CTAs' GEMM2 have finished reading the slot (4 multicast-commit arrivals at the CTA that writes it next)
  uint64_t y_done;             // the item's last MMA has retired
  uint64_t y_free;             // the epilogue warps have read the item's Y out of tensor memory (8 warp arrivals)
  uint64_t epi_sync;           // all 256 epilogue threads, once per unit they write
  uint64_t y_sync;             // all 256 epilogue threads (shared row blocks only)
  uint32_t tmem_base;
  uint32_t abort_word;
  uint32_t last_flag;          // shared row blocks: this CTA is the last of its rank to finish the row block
};
static_assert(sizeof(WideBars) <= 512, "barrier block too large");

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

}  // namespace

// EPI names the two epilogues at compile time: 1 = ReLU after GEMM1, nothing after GEMM2, no bias (the chain as
// the reference defines it); 2 = bias + ReLU after both (the reference's feed-forward block); 3 = bias + GELU,
// then bias (the same block with the reference's GELU in the usual place); 4 = no activation, no bias (the plain
// GEMM -> GEMM chain); 0 = activations and biases picked at
// run time (one warp-uniform dispatch per accumulator piece).  The general form's six code paths per call site
// cost registers (1.5 KB of spills) and time -- config 4 with biases: 878 against 1030 TFLOP/s -- which the
// named forms do not pay.
template <int EPI> struct Epilogues;
template <> struct Epilogues<0> { static constexpr int act1 = 0, act2 = 0; static constexpr bool bias = false; };
template <> struct Epilogues<1> { static constexpr int act1 = 1, act2 = 0; static constexpr bool bias = false; };
template <> struct Epilogues<2> { static constexpr int act1 = 1, act2 = 1; static constexpr bool bias = true; };
template <> struct Epilogues<3> { static constexpr int act1 = 2, act2 = 0; static constexpr bool bias = true; };
template <> struct Epilogues<4> { static constexpr int act1 = 0, act2 = 0; static constexpr bool bias = false; };

template <bool BF16, int EPI>
__global__ void __cluster_dims__(kCluster, 1, 1) __launch_bounds__(kThreads, 1)
    mlp_wide_kernel(const __grid_constant__ WideParams p) {
  extern __shared__ uint8_t smem_raw[];
  // Every CTA of the cluster rounds its dynamic shared memory up by the same amount (the base offset is
  // identical across CTAs of a launch), so slot and barrier offsets match across peers.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  WideBars* bar = reinterpret_cast<WideBars*>(smem + kOffBar);
  volatile uint32_t* abort_word = &bar->abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t q = cluster_ctarank();   // owns Y columns [q NS, (q+1) NS) and chunks q, q + 4, ... of the item
  const int NS = p.N / kCluster;          // this CTA's Y columns
  const int all_chunks = (p.L + kChunk - 1) / kChunk;   // the last chunk may reach past L: TMA zero-fills W1 columns / W2 rows >= L
  const int ksteps1 = (p.K + 63) / 64;
  // Work items.  Without shared row blocks the launch is persistent: a cluster per place the device has
  // (cudaOccupancyMaxActiveClusters), cluster c taking the (batch entry, row block) items c, c + clusters, ...
  // Rings, slots, barrier phases and the unit numbering run on across items, so the next item's GEMM1 fills the
  // tensor pipe while the last hidden units of the current item are still on their way and Y is written out.
  // With shared row blocks every cluster has one item: grid.x numbers the items of a batch entry (whole row
  // blocks first, then the parts of the shared ones), grid.y the batch entries.
  const int cluster_id = blockIdx.x / kCluster;
  const int n_clusters = gridDim.x / kCluster;
  const int total_items = p.row_blocks * static_cast<int>(p.batch);
  const int my_items = p.persistent ? (total_items - cluster_id + n_clusters - 1) / n_clusters : 1;
  // What all items of a cluster have in common: which part of the hidden dimension they cover.
  const bool shared = !p.persistent && cluster_id >= p.whole_blocks;
  const int nparts = shared ? p.parts : 1;
  const int rb_one = shared ? p.whole_blocks + (cluster_id - p.whole_blocks) / p.parts : cluster_id;   // 128-row block (one-item launch)
  const int sp = shared ? (cluster_id - p.whole_blocks) % p.parts : 0;                                 // which part of the hidden dimension
  const int c0 = sp * all_chunks / nparts;               // (parts <= 8, chunks in the thousands at most: 32 bits are plenty)
  const int chunks = (sp + 1) * all_chunks / nparts - c0;
  const int units = 4 * chunks;            // 64-column units of an item, numbered in consumption order
  // this CTA owns chunks q, q + 4, ... of an item
  const int my_rounds = static_cast<int>(q) < chunks ? (chunks - static_cast<int>(q) + kCluster - 1) / kCluster : 0;
  struct Item {
    int b, row0;                           // batch entry, first row of the block
  };
  auto decode = [&](int k) -> Item {       // the k-th item of this cluster
    Item t;
    if (p.persistent) {
      const int id = cluster_id + k * n_clusters;
      t.b = id / p.row_blocks;
      t.row0 = (id - t.b * p.row_blocks) * kRows;
    } else {
      t.b = blockIdx.y;
      t.row0 = rb_one * kRows;
    }
    return t;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kG1Stages; ++s) {
      mbar_init(&bar->g1full[s], 1);
      mbar_init(&bar->g1empty[s], 1);
    }
    for (int s = 0; s < kW2Stages; ++s) {
      mbar_init(&bar->w2full[s], 1);
      mbar_init(&bar->w2empty[s], 1);
    }
    mbar_init(&bar->h_tmem_full, 1);
    mbar_init(&bar->h_tmem_empty, kEpiWarps);
    for (int x = 0; x < kUnits; ++x) {
      mbar_init(&bar->h_ready[x], 1);
      mbar_init(&bar->slot_free[x], kCluster);
    }
    mbar_init(&bar->y_done, 1);
    mbar_init(&bar->y_free, kEpiWarps);
    mbar_init(&bar->epi_sync, kEpiWarps * 32);
    mbar_init(&bar->y_sync, kEpiWarps * 32);
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
  cluster_sync_all();                     // every CTA's barriers exist before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = bar->tmem_base;
  const uint32_t tmem_y = tmem_base;
  const uint32_t tmem_h = tmem_base + 256;
  // Programmatic dependent launch: the set-up above touches no global memory and may overlap the end of
  // the kernel ahead in the stream; from here on its results are needed.
  grid_dependency_wait();
  grid_launch_dependents();

  if (warp == kWarpProdG1) {
    // ------------------------------------------------------------ GEMM1 operand producer (one thread)
    // A stage holds one k-step of GEMM1: this block's 128 x 64 piece of X and the 64 x 256 tile of W1, a TMA
    // box each (the atom view of [in, out] weights makes the W1 tile one box).  Operand delivery from L2 sets
    // the pace (a stage per 1.3 k clocks); one thread gets two boxes out in about 600.
    if (lane == 0) {
      tma_prefetch_desc(&p.map_x);
      tma_prefetch_desc(&p.map_w1);
      int ps = 0;
      uint32_t pph = 0;
      bool ok = true;
      for (int k = 0; k < my_items && ok; ++k) {
        const Item t = decode(k);
        for (int i = 0; i < my_rounds && ok; ++i) {
          const int hcol = (c0 + i * kCluster + static_cast<int>(q)) * kChunk;   // this CTA's chunk of round i
          for (int ks = 0; ks < ksteps1 && ok; ++ks) {
            {
              ok = mbar_wait(&bar->g1empty[ps], pph ^ 1, abort_word, 0x100 + i);
              if (!ok) break;
              uint8_t* dst = smem + kOffG1Ring + ps * kG1StageBytes;
              mbar_arrive_expect_tx(&bar->g1full[ps], kG1StageBytes);
              tma_load_3d(dst, &p.map_x, &bar->g1full[ps], ks * 64, t.row0, t.b);
              dst += kXTileBytes;
              if (p.w_oi) {
                tma_load_3d(dst, &p.map_w1, &bar->g1full[ps], ks * 64, hcol, t.b);
              } else if (p.w_atoms) {
                tma_load_4d(dst, &p.map_w1, &bar->g1full[ps], 0, ks * 64, hcol / 64, t.b);
              } else {
                for (int a = 0; a < kChunk / 64; ++a)
                  tma_load_3d(dst + a * 8192, &p.map_w1, &bar->g1full[ps], hcol + a * 64, ks * 64, t.b);
              }
            }
            if (++ps == kG1Stages) { ps = 0; pph ^= 1; }
          }
        }
      }
    }
  } else if (warp == kWarpProdW2) {
    // ------------------------------------------------------------ GEMM2 operand producer (one thread)
    // One W2 tile per hidden unit, in the order GEMM2 consumes the units: 64 hidden rows x this CTA's Y columns.
    if (lane == 0) {
      tma_prefetch_desc(&p.map_w2);
      int ps = 0;
      uint32_t pph = 0;
      const int ncol = p.n0 + static_cast<int>(q) * NS;   // W2 / Y column in memory
      bool ok = true;
      int g = 0;                              // units so far, over all items: slot g % kUnits
      for (int k = 0; k < my_items && ok; ++k) {
        const Item t = decode(k);
        for (int n = 0; n < units; ++n, ++g) {
          const int i = n / (4 * kCluster);
          const int cr = min(kCluster, chunks - kCluster * i);
          const int e = n - 4 * kCluster * i;
          const int hrow = (c0 + i * kCluster + e % cr) * kChunk + (e / cr) * kUnitCols;
          ok = mbar_wait(&bar->w2empty[ps], pph ^ 1, abort_word, 0x200 + i);
          if (!ok) break;
          // A peer pushes this unit: arm its slot's barrier for the bytes (own units arrive locally).  This thread
          // is at most kW2Stages units ahead of GEMM2, the slot's previous unit is kUnits back: its phase is over.
          if (e % cr != static_cast<int>(q)) mbar_arrive_expect_tx(&bar->h_ready[g % kUnits], kUnitBytes);
          uint8_t* dst = smem + kOffW2Ring + ps * kW2StageBytes;
          mbar_arrive_expect_tx(&bar->w2full[ps], static_cast<uint32_t>(64 * NS * 2));
          if (p.w_oi) {
            tma_load_3d(dst, &p.map_w2, &bar->w2full[ps], hrow, ncol, t.b);
          } else if (p.w_atoms) {
            tma_load_4d(dst, &p.map_w2, &bar->w2full[ps], 0, hrow, ncol / 64, t.b);
          } else {
            for (int a = 0; a < NS / 64; ++a)
              tma_load_3d(dst + a * 8192, &p.map_w2, &bar->w2full[ps], ncol + a * 64, hrow, t.b);
          }
          if (++ps == kW2Stages) { ps = 0; pph ^= 1; }
        }
      }
    }
  } else if (warp == kWarpMmaG1) {
    // ------------------------------------------------------------ GEMM1 issuer (converged warp)
    // Each issuing warp pays a few hundred clocks per stage for the barrier wait, the four MMAs and the
    // commits -- about what the stage's MMAs take to execute.  One warp issuing both GEMMs spent 90 k clocks
    // issuing 65 k clocks of tensor work; with a warp per GEMM the issue cost of one hides behind the other's
    // tensor work, and whichever GEMM has its operands is issued (no fixed interleaving).
    const uint32_t issuer = elect_one();
    const uint32_t idesc1 = umma_idesc_f16(BF16, kRows, kChunk, false, p.w_oi == 0);
    const uint32_t ring = smem_u32(smem + kOffG1Ring);
    int cs = 0;
    uint32_t cph = 0;
    bool ok = true;
    long long w_acc = 0, w_g1 = 0;        // clocks spent waiting (timeline builds only)
    (void)w_acc; (void)w_g1;
    auto wait = [&](uint64_t* bp, uint32_t parity, uint32_t code) {
      bool r = mbar_wait(bp, parity, abort_word, code);
      r = __all_sync(0xffffffffu, r);
      tc_fence_after_sync();
      return r;
    };
    int gc = 0;                           // chunks this CTA has multiplied so far, over all items
    for (int k = 0; k < my_items && ok; ++k) {
      const Item t = decode(k);
      const int tr = k < 6 ? 64 * k : 4096;   // timeline slot base (stamps past the buffer are dropped)
      (void)tr;
      for (int i = 0; i < my_rounds && ok; ++i, ++gc) {
        // the accumulator is single: the previous chunk must be in the epilogue warps' registers
        if (gc > 0) DITTO_TIMED(w_acc, ok = wait(&bar->h_tmem_empty, (gc - 1) & 1, 0x300 + i));
        if (lane == 0) DITTO_STAMP(tr + 16 * i + 0);
        for (int ks = 0; ks < ksteps1 && ok; ++ks) {
          DITTO_TIMED(w_g1, ok = wait(&bar->g1full[cs], cph, 0x310 + i));
          if (!ok) break;
          const uint32_t sx = ring + cs * kG1StageBytes, sw = sx + kXTileBytes;
          const uint64_t da = umma_desc_sw128(sx, 16, 1024);
          const uint64_t db = p.w_oi ? umma_desc_sw128(sw, 16, 1024) : umma_desc_sw128(sw, 8192, 1024);
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4) {
            const uint32_t offb = p.w_oi ? (s4 * 32) >> 4 : (s4 * 2048) >> 4;
            umma_ss_elected(tmem_h, da + ((s4 * 32) >> 4), db + offb, idesc1, (ks | s4) ? 1u : 0u, issuer);
          }
          umma_commit_elected(&bar->g1empty[cs], issuer);
          if (++cs == kG1Stages) { cs = 0; cph ^= 1; }
        }
        if (ok) umma_commit_elected(&bar->h_tmem_full, issuer);
        if (lane == 0) DITTO_STAMP(tr + 16 * i + 1);
      }
    }
#ifdef DITTO_TRACE
    if (lane == 0 && p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0) {
      p.trace[400] = w_acc; p.trace[401] = w_g1; p.trace[404] = clock64();
    }
#endif
  } else if (warp == kWarpMmaG2) {
    // ------------------------------------------------------------ GEMM2 issuer (converged warp)
    const uint32_t issuer = elect_one();
    const uint32_t idesc2 = umma_idesc_f16(BF16, kRows, NS, false, p.w_oi == 0);
    const uint32_t ring = smem_u32(smem + kOffW2Ring);
    const uint32_t slots = smem_u32(smem + kOffSlots);
    int cs = 0;
    uint32_t cph = 0;
    bool ok = true;
    long long w_unit = 0, w_g2 = 0;
    (void)w_unit; (void)w_g2;
    auto wait = [&](uint64_t* bp, uint32_t parity, uint32_t code) {
      bool r = mbar_wait(bp, parity, abort_word, code);
      r = __all_sync(0xffffffffu, r);
      tc_fence_after_sync();
      return r;
    };
    int gn = 0;                           // units consumed so far, over all items: slot gn % kUnits
    const int all_units = units * my_items;
    for (int k = 0; k < my_items && ok; ++k) {
      const Item t = decode(k);
      const int tr = k < 6 ? 64 * k : 4096;
      (void)tr;
      // the Y accumulator is single: the epilogue warps must have read the previous item's out
#ifdef DITTO_TRACE
      if (k == 1 && lane == 0 && p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0) p.trace[410] = clock64();
#endif
      if (k > 0) DITTO_TIMED(w_unit, ok = wait(&bar->y_free, (k - 1) & 1, 0x420));
#ifdef DITTO_TRACE
      if (k == 1 && lane == 0 && p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0) p.trace[411] = clock64();
#endif
      for (int n = 0; n < units && ok; ++n, ++gn) {
        // (This warp is the serial resource of GEMM2: no divergent region, no division in its loop.  The W2
        // producer thread arms h_ready for the units peers push.)
        const int sl = gn % kUnits;
        const int i = n / (4 * kCluster);
        if (lane == 0 && (n & 15) == 0) DITTO_STAMP(tr + 16 * i + 2);
        DITTO_TIMED(w_unit, ok = wait(&bar->h_ready[sl], (gn / kUnits) & 1, 0x400 + i));
        if (!ok) break;
        if (lane == 0 && (n & 15) == 0) DITTO_STAMP(tr + 16 * i + 3);
        DITTO_TIMED(w_g2, ok = wait(&bar->w2full[cs], cph, 0x410 + i));
        if (!ok) break;
#ifdef DITTO_TRACE
        if (k == 1 && n < 4 && lane == 0 && p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0) p.trace[412 + n] = clock64();
#endif
        const uint32_t sw = ring + cs * kW2StageBytes;
        const uint64_t da = umma_desc_sw128(slots + sl * kUnitBytes, 16, 1024);
        const uint64_t db = p.w_oi ? umma_desc_sw128(sw, 16, 1024) : umma_desc_sw128(sw, 8192, 1024);
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) {
          const uint32_t offb = p.w_oi ? (s4 * 32) >> 4 : (s4 * 2048) >> 4;
          umma_ss_elected(tmem_y, da + ((s4 * 32) >> 4), db + offb, idesc2, (n | s4) ? 1u : 0u, issuer);
        }
        umma_commit_elected(&bar->w2empty[cs], issuer);
        {
          // The slot is free once all four CTAs have multiplied the unit: each one's MMA completion arrives
          // directly on the barrier of the CTA that writes the slot next -- the owner of unit gn + kUnits, of
          // this item or the next (all items of a cluster have the same number of units).  The last units of
          // the CTA have no successor: their commit is predicated off.
          int m = n + kUnits;
          m -= m >= units ? units : 0;
          const int x = m & (4 * kCluster - 1);                      // position in its round
          const int mcr = min(kCluster, chunks - kCluster * (m / (4 * kCluster)));   // chunks of that round: 1 .. 4
          const int owner = mcr == 4 ? (x & 3) : mcr == 3 ? x - 3 * ((x * 11) >> 5) : mcr == 2 ? (x & 1) : 0;   // x % mcr, x < 16
          umma_commit_mcast_elected(&bar->slot_free[sl], 1u << owner, gn + kUnits < all_units ? issuer : 0u);
        }
        if (++cs == kW2Stages) { cs = 0; cph ^= 1; }
        if (lane == 0 && (n & 15) == 15) DITTO_STAMP(tr + 16 * i + 4);
      }
      if (ok) umma_commit_elected(&bar->y_done, issuer);
    }
#ifdef DITTO_TRACE
    if (lane == 0 && p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0) {
      p.trace[402] = w_unit; p.trace[403] = w_g2; p.trace[405] = clock64();
    }
#endif
  } else if (warp < kEpiWarps) {
    // ------------------------------------------------------------ epilogue: eight warps
    // Warp w: rows 32 (w % 4) ... + 31 (its TMEM lanes), column half w / 4 of every 64-column quarter.  All
    // eight warps work on one quarter at a time, so the units leave in the order GEMM2 consumes them and
    // each push has the whole outgoing bandwidth (about 16 B/clk per SM) instead of sharing it with a unit
    // that is needed later.
    const int grp = warp >> 2;            // column half of a quarter; half of the Y columns
    const int row = (warp & 3) * 32 + lane;              // row of the block = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    bool ok = true;
    uint32_t free_par = 0;                // bit s: parity of the next wait for slot s to be free
    uint32_t sync_uses = 0;               // completed phases of epi_sync
    int gc = 0;                           // chunks drained so far, over all items
    int ubase = 0;                        // units of the items before this one
    const int colg = grp * (NS / 2);      // this warp group's share of the CTA's NS accumulator columns
    const size_t ycol0 = static_cast<size_t>(q) * NS + colg;

    // Y of item t leaves tensor memory.  With `release` the accumulator is handed back to the GEMM2 warp as soon
    // as it is in registers (NS / 2 <= 128 columns per thread, rounded: 64 registers), before the stores.
    auto drain_y = [&](const Item& t, int k, bool release) __attribute__((always_inline)) -> bool {
      // (named forms with biases: lane l < NS / 16 loads piece l of its warp's NS / 2 bias values ahead of the wait)
      uint4 bq2 = make_uint4(0u, 0u, 0u, 0u);
      if constexpr (EPI != 0 && Epilogues<EPI>::bias) {
        if (!shared && lane * 8 < NS / 2)
          bq2 = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint32_t*>(p.b2) +
                                                     (static_cast<size_t>(t.b) * p.ldn + p.n0 + ycol0) / 2) + lane);
      }
      bool good = mbar_wait(&bar->y_done, k & 1, abort_word, 0x800);
      good = __all_sync(0xffffffffu, good);
      if (!good) return false;
      tc_fence_after_sync();
      if (threadIdx.x == 0) DITTO_STAMP(k < 6 ? 500 + 2 * k : 4096);
      if (!shared) {
        uint8_t* yrow = reinterpret_cast<uint8_t*>(p.y) + ((static_cast<size_t>(t.b) * p.M + t.row0 + row) * p.ldn + p.n0 + ycol0) * 2;
        const uint32_t* bias2 = p.b2 == nullptr ? nullptr
                                                : reinterpret_cast<const uint32_t*>(p.b2) + (static_cast<size_t>(t.b) * p.ldn + p.n0 + ycol0) / 2;
        uint32_t w[8][8];                       // 16 columns a piece
        auto pack_piece = [&](int c, const uint32_t (&o)[16]) __attribute__((always_inline)) {
          if constexpr (EPI != 0 && Epilogues<EPI>::bias) {
            uint32_t bw[8];
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) {
              bw[4 * pc] = __shfl_sync(0xffffffffu, bq2.x, 2 * c + pc);
              bw[4 * pc + 1] = __shfl_sync(0xffffffffu, bq2.y, 2 * c + pc);
              bw[4 * pc + 2] = __shfl_sync(0xffffffffu, bq2.z, 2 * c + pc);
              bw[4 * pc + 3] = __shfl_sync(0xffffffffu, bq2.w, 2 * c + pc);
            }
            act_pack_words<BF16, Epilogues<EPI>::act2>(o, bw, w[c]);
          } else if constexpr (EPI != 0) act_pack_fixed<BF16, Epilogues<EPI>::act2, false>(o, nullptr, w[c]);
          else act_pack<BF16>(o, bias2 == nullptr ? nullptr : bias2 + c * 8, p.act2, w[c]);
        };
        if (NS == 256) {
          // the full width: two loads of 64 columns -- the accumulator is handed back (below) two loads'
          // latencies after the item's last MMA instead of eight (one load of 128 would not fit the registers)
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            uint32_t o[64];
            tmem_ld_x64_wait(tmem_y + lane_base + colg + hf * 64, o);
#pragma unroll
            for (int c = 0; c < 4; ++c) pack_piece(4 * hf + c, *reinterpret_cast<const uint32_t(*)[16]>(&o[16 * c]));
          }
        } else {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            if (c * 16 < NS / 2) {
              uint32_t o[16];
              tmem_ld_x16_wait(tmem_y + lane_base + colg + c * 16, o);
              pack_piece(c, o);
            }
          }
        }
        if (release) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar->y_free);
        }
        // Stored as they are, a store instruction would touch 32 rows with 16 bytes each, and the 2048 requests of
        // a CTA back up the load/store path: the barrier operations of every other warp queue behind them (timeline:
        // the next item's first GEMM2 started when the stores ended, 5 k clocks late).  Shared memory has no room
        // for staging here, so groups of four lanes transpose 4 x 4 blocks of 16-byte pieces with shuffles: an
        // instruction then writes 64 contiguous bytes of each of 8 rows, a quarter of the requests.
        {
          const int a = lane & 3;
          (void)yrow;
          // rows of this lane's group of four: lane_row - a + b, b = 0 .. 3
          uint8_t* ygrp = reinterpret_cast<uint8_t*>(p.y) +
                          ((static_cast<size_t>(t.b) * p.M + t.row0 + row - a) * p.ldn + p.n0 + ycol0) * 2;
          const size_t pitch = static_cast<size_t>(p.ldn) * 2;
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            if (m * 32 < NS / 2) {
              // v[b][0..3]: piece 4 m + b of this lane's row  ->  piece 4 m + a of row b of the group
              uint32_t (&v0)[8] = w[2 * m];
              uint32_t (&v1)[8] = w[2 * m + 1];
              auto el = [&](int b, int j) -> uint32_t& { return b < 2 ? v0[4 * b + j] : v1[4 * (b - 2) + j]; };
#pragma unroll
              for (int b = 0; b < 4; b += 2) {            // lanes a ^ 1 exchange pieces b / b + 1
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint32_t give = (a & 1) ? el(b, j) : el(b + 1, j);
                  const uint32_t got = __shfl_xor_sync(0xffffffffu, give, 1);
                  if (a & 1) el(b, j) = got; else el(b + 1, j) = got;
                }
              }
#pragma unroll
              for (int b = 0; b < 2; ++b) {               // lanes a ^ 2 exchange pieces b / b + 2
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint32_t give = (a & 2) ? el(b, j) : el(b + 2, j);
                  const uint32_t got = __shfl_xor_sync(0xffffffffu, give, 2);
                  if (a & 2) el(b, j) = got; else el(b + 2, j) = got;
                }
              }
#pragma unroll
              for (int b = 0; b < 4; ++b)                 // rows >= M of a partial last block were computed on zero-filled X
                if (t.row0 + row - a + b < p.M)
                  *reinterpret_cast<uint4*>(ygrp + b * pitch + (4 * m + a) * 16) = make_uint4(el(b, 0), el(b, 1), el(b, 2), el(b, 3));
            }
          }
        }
      } else {
        // this cluster's fp32 partial goes to its slab; bias and activation are applied when the slabs are added
        const size_t mpad = static_cast<size_t>(p.row_blocks - p.whole_blocks) * kRows;   // rows of the shared blocks
        const size_t slab = static_cast<size_t>(gridDim.y) * mpad * p.N;
        const int srow0 = t.row0 - p.whole_blocks * kRows;
        // (64-byte runs per row, like Y: groups of four lanes transpose 4 x 4 blocks of 16-byte pieces)
        const int a = lane & 3;
        float* pgrp = p.slabs + static_cast<size_t>(sp) * slab + (static_cast<size_t>(t.b) * mpad + srow0 + row - a) * p.N + ycol0;
        for (int cc = 0; cc < NS / 2; cc += 32) {
          uint32_t o[32];
          tmem_ld_x32_wait(tmem_y + lane_base + colg + cc, o);
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            uint32_t v[4][4];
#pragma unroll
            for (int b = 0; b < 4; ++b)
#pragma unroll
              for (int j = 0; j < 4; ++j) v[b][j] = o[16 * m + 4 * b + j];
            quad_transpose(v, a);
#pragma unroll
            for (int b = 0; b < 4; ++b)
              __stcg(reinterpret_cast<uint4*>(pgrp + static_cast<size_t>(b) * p.N + cc + 16 * m) + a, make_uint4(v[b][0], v[b][1], v[b][2], v[b][3]));
          }
        }
        __threadfence();
        mbar_arrive(&bar->y_sync);
        good = mbar_wait(&bar->y_sync, 0, abort_word, 0x810);
        good = __all_sync(0xffffffffu, good);
        if (good && threadIdx.x == 0) {
          int* ctr = p.counters + (static_cast<size_t>(t.b) * (p.row_blocks - p.whole_blocks) + (rb_one - p.whole_blocks)) * kCluster + q;
          const int seen = atomicAdd(ctr, 1);
          __threadfence();
          bar->last_flag = (seen == p.parts - 1) ? 1u : 0u;
        }
        // (the combining pass runs after the roles, on all threads of the CTA)
      }
      if (threadIdx.x == 0) DITTO_STAMP(k < 6 ? 501 + 2 * k : 4096);
      return good;
    };

    // Order at an item boundary: the first unit of the next item's first chunk is pushed BEFORE the finished
    // item's Y is read out.  That unit only needs a slot the finished item's last GEMM2 steps release, and with
    // it (and Y handed back right after) the GEMM2 warp goes on almost without a gap; the Y stores and the rest
    // of the chunk's hand-over run behind it.
    int pending = -1;                     // item whose Y is still in tensor memory
    for (int k = 0; k < my_items && ok; ++k) {
      const Item t = decode(k);
      const int tr = k < 6 ? 64 * k : 4096;
      (void)tr;
      for (int i = 0; i < my_rounds; ++i, ++gc) {
        const int cr = min(kCluster, chunks - kCluster * i);
        const int hcol0 = (c0 + i * kCluster + static_cast<int>(q)) * kChunk;   // first hidden column of the chunk
        const uint32_t* bias1 = p.b1 == nullptr ? nullptr
                                                : reinterpret_cast<const uint32_t*>(p.b1) +
                                                      (static_cast<size_t>(t.b) * p.L + hcol0 + grp * 32) / 2;
        // The named forms with biases: a bias value is the same for all rows, so instead of every lane loading all
        // of its warp's 128 values (16 load instructions of 16 bytes per thread and chunk, each on the path
        // between "accumulator ready" and "unit pushed"), lane l < 16 loads one 16-byte piece -- piece l % 4 of
        // quarter l / 4 -- before the wait for the accumulator, and the values are handed round by shuffles.
        uint4 bq = make_uint4(0u, 0u, 0u, 0u);
        if constexpr (EPI != 0 && Epilogues<EPI>::bias) {
          if (lane < 16 && hcol0 + (lane >> 2) * kUnitCols + grp * 32 < p.L)
            bq = __ldg(reinterpret_cast<const uint4*>(bias1 + (lane >> 2) * (kUnitCols / 2)) + (lane & 3));
        }
        // quarter kk of the chunk: tensor memory -> bias, activation, rounding -> registers
        auto load_quarter = [&](int kk, uint32_t (&v)[16]) __attribute__((always_inline)) {
          uint32_t h[32];
          tmem_ld_x32_wait(tmem_h + lane_base + kk * kUnitCols + grp * 32, h);
          // (hidden columns >= L of a last partial chunk: GEMM1 gave zeros, the bias is not read, every
          // activation maps 0 to 0 and the W2 rows they meet are zero-filled)
          if constexpr (EPI != 0 && Epilogues<EPI>::bias) {
            // (pieces past L were loaded as zeros: 0 + 0 stays 0 under every activation)
            uint32_t bw[16];
#pragma unroll
            for (int pc = 0; pc < 4; ++pc) {
              bw[4 * pc] = __shfl_sync(0xffffffffu, bq.x, kk * 4 + pc);
              bw[4 * pc + 1] = __shfl_sync(0xffffffffu, bq.y, kk * 4 + pc);
              bw[4 * pc + 2] = __shfl_sync(0xffffffffu, bq.z, kk * 4 + pc);
              bw[4 * pc + 3] = __shfl_sync(0xffffffffu, bq.w, kk * 4 + pc);
            }
            act_pack_words<BF16, Epilogues<EPI>::act1>(h, bw, v);
          } else if constexpr (EPI != 0) {
            act_pack_fixed<BF16, Epilogues<EPI>::act1, false>(h, nullptr, v);
          } else act_pack<BF16>(h, (bias1 == nullptr || hcol0 + kk * kUnitCols + grp * 32 >= p.L) ? nullptr : bias1 + kk * (kUnitCols / 2),
                              p.act1, v);
        };
        auto release_h = [&]() __attribute__((always_inline)) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar->h_tmem_empty);   // one arrival per warp
          if (threadIdx.x == 0) DITTO_STAMP(tr + 16 * i + 7);
        };
        // quarter kk becomes a unit: into its slot once that is free, then to the three peers
        auto emit = [&](int kk, const uint32_t (&v)[16]) __attribute__((always_inline)) -> bool {
          const int gn = ubase + 4 * kCluster * i + cr * kk + static_cast<int>(q);
          const int sl = gn % kUnits;
          bool good = true;
          if (gn >= kUnits) {
            // every CTA has finished GEMM2 on the slot's previous unit: it may be overwritten
            const uint32_t par = (free_par >> sl) & 1u;
            free_par ^= 1u << sl;
            good = mbar_wait_cluster(&bar->slot_free[sl], par, abort_word, 0x700 + i);
            good = __all_sync(0xffffffffu, good);
            if (!good) return false;
          }
          uint8_t* slot = smem + kOffSlots + sl * kUnitBytes;
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const int ch = grp * 4 + c4;      // 16-byte piece of the 128-byte row
            *reinterpret_cast<uint4*>(slot + row * 128 + ((ch ^ (row & 7)) << 4)) =
                make_uint4(v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
          }
          fence_proxy_async_smem();
          mbar_arrive(&bar->epi_sync);
          good = mbar_wait(&bar->epi_sync, sync_uses++ & 1, abort_word, 0x780 + i);   // all 256 threads have written
          good = __all_sync(0xffffffffu, good);
          if (!good) return false;
          if (threadIdx.x == 0) {
            const uint32_t slot_addr = smem_u32(slot);
            const uint32_t bar_addr = smem_u32(&bar->h_ready[sl]);
            for (uint32_t d = 1; d < kCluster; ++d) {
              const uint32_t peer = (q + d) % kCluster;     // every CTA of the cluster consumes the unit
              bulk_copy_to_peer(map_to_cta(slot_addr, peer), slot, kUnitBytes, map_to_cta(bar_addr, peer));
            }
            mbar_arrive(&bar->h_ready[sl]);    // the local copy is in place
            DITTO_STAMP(tr + 16 * i + 8 + kk);
          }
          return true;
        };

        ok = mbar_wait(&bar->h_tmem_full, gc & 1, abort_word, 0x600 + i);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        if (threadIdx.x == 0) DITTO_STAMP(tr + 16 * i + 6);
        if (pending < 0) {
          // the whole chunk leaves tensor memory first, so that the accumulator is released without waiting
          // for a free slot (the next GEMM1 is ahead of this chunk's GEMM2 in the tensor-pipe order)
          uint32_t pk[4][16];
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) load_quarter(kk, pk[kk]);
          release_h();
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            ok = emit(kk, pk[kk]);
            if (!ok) break;
          }
        } else {
          // item boundary: first quarter, the finished item's Y, then the other three quarters
          {
            uint32_t p0[16];
            load_quarter(0, p0);
            ok = emit(0, p0);
          }
          if (ok) ok = drain_y(decode(pending), pending, true);
          if (!ok) break;
          pending = -1;
          uint32_t pk[3][16];
#pragma unroll
          for (int kk = 1; kk < 4; ++kk) load_quarter(kk, pk[kk - 1]);
          release_h();
#pragma unroll
          for (int kk = 1; kk < 4; ++kk) {
            ok = emit(kk, pk[kk - 1]);
            if (!ok) break;
          }
        }
        if (!ok) break;
      }
      if (!ok) break;
      ubase += units;
      if (pending >= 0) {                 // a CTA without a chunk in this item (fewer chunks than CTAs)
        ok = drain_y(decode(pending), pending, true);
        if (!ok) break;
      }
      pending = k;
    }
    if (ok && pending >= 0) drain_y(decode(pending), pending, false);
  }

  // After a wait has given up, copies this CTA issued (TMA loads into its rings, pushes into its peers'
  // slots) may still be in flight; they complete within microseconds.  Give them that time before the
  // shared memory and tensor memory they target are released.
  if (*abort_word != 0u) {
    for (int t = 0; t < 64; ++t) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  const Item t0 = decode(0);              // with shared row blocks a cluster has this one item
  if (shared && bar->last_flag != 0u && bar->abort_word == 0u) {
    // Every part of this CTA's (rows, columns) region of a shared row block is in its slab, and this
    // cluster was the last to get there: add the slabs in slab order, apply bias and activation, write Y.
    // All warps take part -- the pass is bound by how many loads the CTA keeps in flight.
    __threadfence();
    const size_t mpad = static_cast<size_t>(p.row_blocks - p.whole_blocks) * kRows;
    const size_t slab = static_cast<size_t>(gridDim.y) * mpad * p.N;
    const size_t col0 = static_cast<size_t>(q) * NS;
    const uint32_t* bias2 = p.b2 == nullptr ? nullptr
                                            : reinterpret_cast<const uint32_t*>(p.b2) + (static_cast<size_t>(t0.b) * p.ldn + p.n0 + col0) / 2;
    combine_slabs<BF16>(p.slabs + (static_cast<size_t>(t0.b) * mpad + (t0.row0 - p.whole_blocks * kRows)) * p.N + col0, slab, p.parts,
                        min(kRows, p.M - t0.row0), NS, static_cast<size_t>(p.N), bias2, p.act2,
                        reinterpret_cast<uint8_t*>(p.y) + ((static_cast<size_t>(t0.b) * p.M + t0.row0) * p.ldn + p.n0 + col0) * 2,
                        static_cast<size_t>(p.ldn) * 2, static_cast<int>(threadIdx.x), kThreads);
  }
  cluster_sync_all();                     // no CTA leaves while a peer may still write to it
  if (warp == 0) {
    tmem_dealloc(tmem_base, 512);
    if (lane == 0 && bar->abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, static_cast<int>(bar->abort_word));
  }
}

// ------------------------------------------------------------------ host side
bool mlp_wide_supported(int N, int K, int L) {
  // 256-wide hidden chunks, the last one possibly partial in whole 64-column groups (TMA zero-fills the rest); K
  // in 16-wide steps (a last partial 64-wide k-step is zero-filled as well); a launch covers up to 1024 Y columns
  // -- N/4 per CTA in whole 64-column groups, at most 256 -- and wider results are computed as several launches
  // over column groups (see mlp_wide_column_groups)
  return L % 64 == 0 && K % 16 == 0 && N % (kCluster * 64) == 0;
}

static int mlp_wide_column_groups(int N, int* first, int* width) {
  // N = 256 u columns in g = ceil(u / 4) groups of near-equal width (multiples of 256, at most 1024)
  const int u = N / 256, g = (u + 3) / 4;
  int c = 0;
  for (int i = 0; i < g; ++i) {
    const int w = (u / g + (i < u % g ? 1 : 0)) * 256;
    first[i] = c;
    width[i] = w;
    c += w;
  }
  return g;
}

namespace {

template <bool BF16>
cudaError_t wide_configure(int* slots_out) {
  static std::atomic<unsigned long long> configured{0};
  static std::atomic<int> cluster_slots[kMaxDevices];
  int dev = 0;
  cudaError_t e = current_device_checked(&dev);
  if (e != cudaSuccess) return e;
  if (!device_configured(configured, dev)) {
    auto kern = mlp_wide_kernel<BF16, 0>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(mlp_wide_kernel<BF16, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(mlp_wide_kernel<BF16, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(mlp_wide_kernel<BF16, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(mlp_wide_kernel<BF16, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    // how many clusters of four the device holds at once: the unit row-block sharing is sized against
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kCluster * 64, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess) return e;
    cluster_slots[dev].store(n > 0 ? n : 1, std::memory_order_relaxed);
    mark_device_configured(configured, dev);
  }
  *slots_out = cluster_slots[dev].load(std::memory_order_relaxed);
  return cudaSuccess;
}

}  // namespace

int mlp_wide_cluster_slots(bool bf16, int* slots) {
  cudaError_t e = bf16 ? wide_configure<true>(slots) : wide_configure<false>(slots);
  return e == cudaSuccess ? DITTO_OK : cuda_fail("mlp wide kernel set-up", e);
}

RowBlockPlan mlp_wide_plan(int batch, int M, int L, int cluster_slots, bool allow_scratch) {
  const int rbs = (M + kRows - 1) / kRows;
  if (!allow_scratch) return {rbs, 1};
  // in units of a 256-wide chunk: an item takes about 14 us + 3.5 us per chunk, sharing adds about 17 us
  return plan_row_blocks(batch, rbs, (L + kChunk - 1) / kChunk, kCluster, kMaxSlabs, cluster_slots, 4.0, 5.0);
}

size_t mlp_wide_workspace_bytes(int batch, int M, int N, const RowBlockPlan& plan) {
  int first[16], width[16];
  const int widest = (N % 256 == 0 && N <= 16 * kCluster * 256 && mlp_wide_column_groups(N, first, width) > 0) ? width[0] : N;
  return plan_workspace_bytes(plan, batch, (M + kRows - 1) / kRows, kRows, widest, kCluster);
}

namespace {

// One launch: the Y columns [n0, n0 + N) of a result that has ldn columns in memory (N <= 1024).
int launch_wide_group(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                      int n0, int ldn, bool bf16, int w_layout, int act1, int act2, const void* b1, const void* b2,
                      const RowBlockPlan& plan, void* workspace, int* status, cudaStream_t stream, long long* trace) {
  if (!mlp_wide_supported(N, K, L) || N > kCluster * 256 || batch > 65535) return DITTO_ERR_UNSUPPORTED;
  int slots = 0;
  int rc = mlp_wide_cluster_slots(bf16, &slots);
  if (rc) return rc;
  const int NS = N / kCluster;
  const int rbs = (M + kRows - 1) / kRows;
  const int shared_blocks = rbs - plan.whole_blocks;
  if (plan.whole_blocks < 0 || shared_blocks < 0 || plan.parts < 1 || plan.parts > (L + kChunk - 1) / kChunk || plan.parts > kMaxSlabs)
    return DITTO_ERR_INVALID_ARG;
  const bool split = shared_blocks > 0 && plan.parts > 1;
  WideParams p;
  std::memset(&p, 0, sizeof(p));
  const uint64_t uM = M, uN = ldn, uK = K, uL = L, ub = batch;   // uN: W2's extent along N in memory
  {
    const uint64_t dims[3] = {uK, uM, ub}, strides[2] = {uK * 2, uM * uK * 2};
    const uint32_t box[3] = {64, kRows, 1};
    rc = make_tensor_map(&p.map_x, bf16, x, 3, dims, strides, box);
    if (rc) return rc;
  }
  if (w_layout == 1) {
    const uint64_t d1[3] = {uK, uL, ub}, s1[2] = {uK * 2, uL * uK * 2};
    const uint32_t bx1[3] = {64, kChunk, 1};
    rc = make_tensor_map(&p.map_w1, bf16, w1, 3, d1, s1, bx1);
    if (rc) return rc;
    const uint64_t d2[3] = {uL, uN, ub}, s2[2] = {uL * 2, uN * uL * 2};
    const uint32_t bx2[3] = {64, static_cast<uint32_t>(NS), 1};
    rc = make_tensor_map(&p.map_w2, bf16, w2, 3, d2, s2, bx2);
    if (rc) return rc;
  } else {
    // [rows, cols] row-major seen as (64 columns, rows, cols / 64, batch): one box of 64 x 64 x atoms brings the
    // 64-column swizzle atoms of an MN-major operand tile with a single TMA operation (atom a lands at
    // a * 8 KB, exactly the operand layout)
    const uint64_t d1[4] = {64, uK, uL / 64, ub}, s1[3] = {uL * 2, 128, uK * uL * 2};
    const uint32_t bx1[4] = {64, 64, kChunk / 64, 1};
    const uint64_t d2[4] = {64, uL, uN / 64, ub}, s2[3] = {uN * 2, 128, uL * uN * 2};
    const uint32_t bx2[4] = {64, 64, static_cast<uint32_t>(NS / 64), 1};
    p.w_atoms = make_tensor_map(&p.map_w1, bf16, w1, 4, d1, s1, bx1) == DITTO_OK &&
                make_tensor_map(&p.map_w2, bf16, w2, 4, d2, s2, bx2) == DITTO_OK;
    if (!p.w_atoms) {
      // a driver that rejects the atom view: plain maps, one box per 64-column atom
      const uint64_t e1[3] = {uL, uK, ub}, t1[2] = {uL * 2, uK * uL * 2};
      const uint64_t e2[3] = {uN, uL, ub}, t2[2] = {uN * 2, uL * uN * 2};
      const uint32_t bx[3] = {64, 64, 1};
      rc = make_tensor_map(&p.map_w1, bf16, w1, 3, e1, t1, bx);
      if (rc) return rc;
      rc = make_tensor_map(&p.map_w2, bf16, w2, 3, e2, t2, bx);
      if (rc) return rc;
    }
  }
  p.y = y;
  p.M = M;
  p.N = N;
  p.n0 = n0;
  p.ldn = ldn;
  p.K = K;
  p.L = L;
  p.row_blocks = rbs;
  p.batch = batch;
  p.persistent = split ? 0 : 1;
  p.whole_blocks = split ? plan.whole_blocks : rbs;
  p.parts = split ? plan.parts : 1;
  p.w_oi = w_layout == 1;
  p.act1 = act1;
  p.act2 = act2;
  p.b1 = b1;
  p.b2 = b2;
  p.status = status;
  p.trace = trace;
  if (split) {
    if (workspace == nullptr) return DITTO_ERR_WORKSPACE;
    const size_t slab_bytes = static_cast<size_t>(plan.parts) * batch * shared_blocks * kRows * N * sizeof(float);
    p.slabs = static_cast<float*>(workspace);
    p.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + slab_bytes);
    cudaError_t e = cudaMemsetAsync(p.counters, 0, static_cast<size_t>(batch) * shared_blocks * kCluster * sizeof(int), stream);
    if (e != cudaSuccess) return cuda_fail("mlp wide counters", e);
  }
  cudaLaunchConfig_t cfg = {};
  if (p.persistent) {
    // one cluster per place the device has (fewer when there are fewer items); each walks its items
    const long long items = static_cast<long long>(rbs) * batch;
    cfg.gridDim = dim3(static_cast<unsigned>(kCluster * std::min<long long>(items, slots)), 1, 1);
  } else {
    cfg.gridDim = dim3(static_cast<unsigned>(kCluster * (p.whole_blocks + (rbs - p.whole_blocks) * p.parts)), static_cast<unsigned>(batch), 1);
  }
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see grid_dependency_wait in the kernel
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = split ? 0 : 1;           // a launch with shared row blocks follows its own counter reset: plain stream order
  // the named forms read their biases 16 bytes at a time
  const bool both = b1 != nullptr && b2 != nullptr && ((reinterpret_cast<uintptr_t>(b1) | reinterpret_cast<uintptr_t>(b2)) & 15) == 0;
  const bool none = b1 == nullptr && b2 == nullptr;
  const int epi = (act1 == 1 && act2 == 0 && none) ? 1 : (act1 == 1 && act2 == 1 && both) ? 2 : (act1 == 2 && act2 == 0 && both) ? 3
                  : (act1 == 0 && act2 == 0 && none) ? 4 : 0;
  cudaError_t e = cudaErrorInvalidValue;
  switch (epi * 2 + (bf16 ? 1 : 0)) {
    case 0: e = cudaLaunchKernelEx(&cfg, mlp_wide_kernel<false, 0>, p); break;
    case 1: e = cudaLaunchKernelEx(&cfg, mlp_wide_kernel<true, 0>, p); break;
    case 2: e = cudaLaunchKernelEx(&cfg, mlp_wide_kernel<false, 1>, p); break;
    case 3: e = cudaLaunchKernelEx(&cfg, mlp_wide_kernel<true, 1>, p); break;
    case 4: e = cudaLaunchKernelEx(&cfg, mlp_wide_kernel<false, 2>, p); break;
    case 5: e = cudaLaunchKernelEx(&cfg, mlp_wide_kernel<true, 2>, p); break;
    case 6: e = cudaLaunchKernelEx(&cfg, mlp_wide_kernel<false, 3>, p); break;
    case 7: e = cudaLaunchKernelEx(&cfg, mlp_wide_kernel<true, 3>, p); break;
    case 8: e = cudaLaunchKernelEx(&cfg, mlp_wide_kernel<false, 4>, p); break;
    default: e = cudaLaunchKernelEx(&cfg, mlp_wide_kernel<true, 4>, p); break;
  }
  return e == cudaSuccess ? DITTO_OK : cuda_fail("mlp wide kernel launch", e);
}

}  // namespace

int launch_mlp_wide(const void* x, const void* w1, const void* w2, void* y, int batch, int M, int N, int K, int L,
                    bool bf16, int w_layout, int act1, int act2, const void* b1, const void* b2, const RowBlockPlan& plan,
                    void* workspace, int* status, cudaStream_t stream, long long* trace) {
  if (!mlp_wide_supported(N, K, L) || N > 16 * kCluster * 256) return DITTO_ERR_UNSUPPORTED;
  // Results wider than 1024 columns do not fit the cluster's tensor memory next to a hidden chunk: they are
  // computed group of columns by group, one launch each, in stream order (the scratch memory of a plan with
  // shared row blocks is sized for the widest group and reused).  Every group recomputes GEMM1 -- the hidden
  // layer still never leaves the chip; the price is (groups - 1) x the FLOPs of GEMM1.
  int first[16], width[16];
  const int groups = mlp_wide_column_groups(N, first, width);
  for (int g = 0; g < groups; ++g) {
    const int rc = launch_wide_group(x, w1, w2, y, batch, M, width[g], K, L, first[g], N, bf16, w_layout, act1, act2, b1, b2,
                                     plan, workspace, status, stream, g == 0 ? trace : nullptr);
    if (rc != DITTO_OK) return rc;
  }
  return DITTO_OK;
}

}  // namespace ditto_b200
