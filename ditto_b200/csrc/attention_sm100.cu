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
// The score tile never leaves the SM.  A work item is NT (1 or 2) tiles of 128
// query rows of one slice (batch x head); its K/V stream in blocks of 128 rows
// through a TMA-fed ring of 128B-swizzled shared-memory stages.  At head
// dimension 128 a CTA per SM walks the items (ring, barrier phases and tensor
// memory run on across them); the other instances are launched with a CTA per
// item.  O leaves through 4 KB of shared memory per softmax warp, so that a
// store instruction writes whole rows.
//
// Warp roles (NT = 2: 320 threads):
//   warps 0-3   softmax + epilogue for query tile 0  (thread i <-> row i, TMEM lane i)
//   warps 4-7   softmax + epilogue for query tile 1
//   warp  8     TMA producer (one lane issues)
//   warp  9     MMA issuer (one elected lane issues)
// With two tiles the tensor pipe works on one tile while the other tile's
// softmax runs, so the exponentials overlap the MMAs.  A single issuing warp
// serving the tiles alternately is what keeps them half a period apart: with
// one issuing warp per tile the two softmax phases drift into step, fight for
// the exponential unit and leave the tensor pipe idle (measured: 18 % slower).
//
// TMEM columns (512 allocated): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).
// P (16-bit, two values per 32-bit column) overwrites the first 64 columns of
// its own S tile; the next S MMA for that tile is issued after the P*V MMA
// that reads it, and the tensor pipe executes one thread's MMAs in order.
#include "attention_sm100.cuh"

#include <algorithm>
#include <atomic>
#include <type_traits>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

// 1: the softmax evaluates its exponentials two at a time on packed 16-bit arguments (see ex2_packed)
#ifndef DITTO_PACKED_EX2
#define DITTO_PACKED_EX2 0
#endif

// Optional timeline capture for tuning (compiled in only with -DDITTO_TRACE): CTA (0,0) stores
// clock64() stamps of its first iterations into the buffer passed as the call's workspace.
#ifdef DITTO_TRACE
#define DITTO_STAMP(base, j, k)                                                                   \
  do {                                                                                            \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && (j) < 16)        \
      p.trace[(base) + (j) * 16 + (k)] = clock64();                                               \
  } while (0)
#else
#define DITTO_STAMP(base, j, k) do {} while (0)
#endif

namespace ditto_b200 {

namespace {

constexpr int kBM = 128;   // query rows per tile
constexpr int kBN = 128;   // K/V rows per block
// 1: the two-tile kernel runs with twelve warps (two of them idle) so that its third warp group can hand
// registers to the two softmax warp groups (setmaxnreg: 136 / 184 instead of 168 each; ptxas refuses a larger step with "register allocation failed" under this launch bound).  Measured: no gain
// (the softmax warps spill 20 bytes at 168 registers and are not bound by per-thread work), so it is off.
#ifndef DITTO_ATTN_SETMAXNREG
#define DITTO_ATTN_SETMAXNREG 0
#endif
constexpr int threads_for(int nt) { return (DITTO_ATTN_SETMAXNREG && nt == 2) ? 384 : 32 * (4 * nt + 2); }
constexpr int kModeSoftmax = 0, kModeRelu = 1, kModeIdentity = 2;
constexpr int kSplit = 96;  // K/V rows in the first part of P (the rest follows separately)
constexpr float kRescaleThreshold = 8.0f;  // log2 units; P stays <= 2^8 with a stale max

// "Separate-P" variant (one 128-row tile per CTA, D = 64, P through TMEM): S, O and P each get
// their own TMEM columns (128 + 64 + 64 = 256), so the next S MMA no longer has to wait for the
// P*V that reads P and runs while the softmax of the current block is still computing; with 256
// TMEM columns and 80 KB of shared memory two such CTAs share an SM and hide each other's
// prologue and epilogue.
template <int D, int NT, bool PSMEM>
constexpr bool kSeparateP = (NT == 1 && D == 64 && !PSMEM);

// Instances whose CTAs walk several work items (the others are launched with one CTA per item).
template <int D, int NT, bool PSMEM>
constexpr bool kLoopItems = (D == 128 && !kSeparateP<D, NT, PSMEM>);

template <int D, int NT, bool PSMEM>
struct Smem {
  static constexpr int kTileQ = kBM * D * 2;
  static constexpr int kTileKV = kBN * D * 2;
  static constexpr int kTileP = kBM * kBN * 2;
  static constexpr int kStages = kSeparateP<D, NT, PSMEM> ? 2 : PSMEM ? (D == 64 ? 3 : 1) : (D == 64 ? 4 : 2);
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + NT * kTileQ;
  static constexpr int kOffV = kOffK + kStages * kTileKV;
  static constexpr int kOffP = kOffV + kStages * kTileKV;
  static constexpr int kOffBar = kOffP + (PSMEM ? NT * kTileP : 0);
  static constexpr int kOffStage = kOffBar + 512;       // 4 KB per softmax warp: O rows on their way to global memory
  static constexpr int kBytes = kOffStage + NT * 4 * 4096 + 1024;  // ... + slack for 1024-byte alignment
};

struct Barriers {
  uint64_t q_full[2], q_empty[2];   // per query tile: Q has landed / the item's last S MMA has read it
  uint64_t k_full[4], k_empty[4], v_full[4], v_empty[4];
  uint64_t s_full[2], p_part[2][2], o_done[2];
  uint64_t o_free[2];    // the softmax warps have read the finished item's O out of tensor memory (4 warp arrivals)
  uint64_t s_taken[2];   // separate-P variant: the softmax warps hold S in registers
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

// MODE selects the element-wise stage between the two GEMMs: kModeSoftmax (online softmax and final
// normalisation), kModeRelu / kModeIdentity (P = act(S) rounded to the input type, no scale, no
// normalisation) -- the small-N form of the GEMM -> ReLU -> GEMM and plain GEMM -> GEMM chains.
template <bool BF16, int D, int NT, bool PSMEM, int MODE>
__global__ void __launch_bounds__(threads_for(NT), kSeparateP<D, NT, PSMEM> ? 2 : 1)
    attention_kernel(const __grid_constant__ AttnParams p) {
  using SM = Smem<D, NT, PSMEM>;
  constexpr bool kSep = kSeparateP<D, NT, PSMEM>;
  constexpr uint32_t kTmemCols = kSep ? 256 : 512;
  constexpr uint32_t kColO = kSep ? 128 : 256;       // first accumulator column
  constexpr uint32_t kColP = 192;                    // separate-P variant only
  constexpr int kStages = SM::kStages;
  constexpr int kAtoms = D / 64;  // 64-element (128-byte) chunks along the head dimension

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Barriers* bar = reinterpret_cast<Barriers*>(smem + SM::kOffBar);
  volatile uint32_t* abort_word = &bar->abort_word;

  constexpr int kProducerWarp = 4 * NT;
  constexpr int kMmaWarp = 4 * NT + 1;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Work items: (slice, tile of NT x 128 query rows), tile index fastest, so that the tiles of a slice are
  // worked on together (their K/V share L2) and the number of slices is not limited by the 65535 of the other
  // grid dimensions.  The grid is one CTA per place the device has and CTA b takes the items b, b + grid, ...:
  // the K/V ring, the barrier phases and the tensor-memory columns run on across items, the next item's Q and
  // first K/V blocks are loaded and its first scores computed under the current item's last blocks, and O is
  // written out while the other tile is still being multiplied.  A CTA's fixed cost -- launch, set-up, first
  // loads, pipeline fill, write-out, measured 9 us per item against 1.7 us per K/V block -- is paid once per
  // CTA instead of once per item.  (The separate-P variant has one item per CTA.)
  const int tiles = (p.M + NT * kBM - 1) / (NT * kBM);
  // The loop is a compile-time property of the instance (head dimension 128; see the launcher): with one item
  // per CTA known at compile time the other instances keep the code -- and the registers -- of a single pass.
  constexpr bool kLoop = kLoopItems<D, NT, PSMEM>;
  const int my_items = kLoop ? (p.items - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x) : 1;
  struct Item {
    int slice, seq, head_col, m0;
  };
  auto decode = [&](int k) -> Item {
    Item it;
    const int id = static_cast<int>(blockIdx.x) + k * static_cast<int>(gridDim.x);
    it.slice = id / tiles;
    // Packed multi-head input: slice = (sequence, head); rows come from the sequence, columns from
    // the head.  Plain batched input has heads == 1 and zero column offsets.
    it.seq = it.slice / p.heads;
    it.head_col = (it.slice % p.heads) * p.d;
    it.m0 = (id % tiles) * (NT * kBM);
    return it;
  };
  const int nkv = (p.L + kBN - 1) / kBN;        // the last block may be partial: TMA zero-fills rows >= L
  const int ksteps_d = p.d / 16;                // head dimension actually used by S = Q K^T (<= D / 16)

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bar->k_full[s], 1);
      mbar_init(&bar->k_empty[s], 1);
      mbar_init(&bar->v_full[s], 1);
      mbar_init(&bar->v_empty[s], 1);
    }
    for (int t = 0; t < NT; ++t) {
      mbar_init(&bar->q_full[t], 1);
      mbar_init(&bar->q_empty[t], 1);
      mbar_init(&bar->o_free[t], 4);
      mbar_init(&bar->s_full[t], 1);
      mbar_init(&bar->p_part[t][0], kBM);
      mbar_init(&bar->p_part[t][1], kBM);
      mbar_init(&bar->o_done[t], 1);
      mbar_init(&bar->s_taken[t], kBM);
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
  // Programmatic dependent launch: nothing above touches global memory, so it may overlap the end of the
  // kernel ahead in the stream; its results are needed from here on.  The kernel behind may begin its set-up.
  grid_dependency_wait();
  grid_launch_dependents();
  if (warp == 0) DITTO_STAMP(512, 0, 8);
#if DITTO_ATTN_SETMAXNREG
  if constexpr (NT == 2) {
    if (warp < 8) asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 136;");
  }
#endif

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA producer (one thread)
    if (lane == 0) {
      tma_prefetch_desc(&p.map_q);
      tma_prefetch_desc(&p.map_k);
      tma_prefetch_desc(&p.map_v);
      bool ok = true;
      int armed_k[4] = {-1, -1, -1, -1}, armed_v[4] = {-1, -1, -1, -1};  // parity of the newest armed phase
      int g = 0;                            // K/V blocks loaded so far, over all items: ring stage g % kStages
      for (int k = 0; k < my_items && ok; ++k) {
        const Item it = decode(k);
        auto load_q = [&]() {
          for (int t = 0; t < NT && ok; ++t) {
            // the tile's Q buffer is single: the previous item's last S MMA must have read it
            if (k > 0) ok = mbar_wait(&bar->q_empty[t], (k - 1) & 1, abort_word, 0x180 + t);
            if (!ok) break;
            mbar_arrive_expect_tx(&bar->q_full[t], SM::kTileQ);
            for (int a = 0; a < kAtoms; ++a)
              tma_load_3d(smem + SM::kOffQ + t * SM::kTileQ + a * (kBM * 128), &p.map_q, &bar->q_full[t],
                          p.q_col0 + it.head_col + a * 64, it.m0 + t * kBM, it.seq);
          }
        };
        // A later item's first K block goes out before its Q: the ring stage is free an iteration before the Q
        // buffers are, and the MMA warp looks two K blocks ahead.
        if (k == 0) load_q();
        for (int j = 0; j < nkv && ok; ++j, ++g) {
          const int s = g % kStages;
          const uint32_t ph = (g / kStages) & 1;
          ok = mbar_wait(&bar->k_empty[s], ph ^ 1, abort_word, 0x100 + j);
          if (!ok) break;
          {
            uint8_t* dst = smem + SM::kOffK + s * SM::kTileKV;
            mbar_arrive_expect_tx(&bar->k_full[s], SM::kTileKV);
            armed_k[s] = static_cast<int>(ph);
            if (p.k_transposed) {
              // K given as [slice, D, L]: boxes of 64 kv-columns x D rows (MN-major operand)
              for (int a = 0; a < kBN / 64; ++a)
                tma_load_3d(dst + a * (D * 128), &p.map_k, &bar->k_full[s], j * kBN + a * 64, 0, it.slice);
            } else {
              for (int a = 0; a < kAtoms; ++a)
                tma_load_3d(dst + a * (kBN * 128), &p.map_k, &bar->k_full[s], p.k_col0 + it.head_col + a * 64,
                            j * kBN, it.seq);
            }
          }
          if (j == 0 && k > 0) {
            load_q();
            if (!ok) break;
          }
          ok = mbar_wait(&bar->v_empty[s], ph ^ 1, abort_word, 0x200 + j);
          if (!ok) break;
          {
            uint8_t* dst = smem + SM::kOffV + s * SM::kTileKV;
            mbar_arrive_expect_tx(&bar->v_full[s], SM::kTileKV);
            armed_v[s] = static_cast<int>(ph);
            if (p.v_transposed) {
              // V given as [slice, dv, L]: boxes of 64 kv-columns x D rows (K-major operand of P*V)
              for (int a = 0; a < kBN / 64; ++a)
                tma_load_3d(dst + a * (D * 128), &p.map_v, &bar->v_full[s], j * kBN + a * 64, 0, it.slice);
            } else {
              for (int a = 0; a < kAtoms; ++a)
                tma_load_3d(dst + a * (kBN * 128), &p.map_v, &bar->v_full[s], p.v_col0 + it.head_col + a * 64,
                            j * kBN, it.seq);
            }
          }
        }
      }
      if (!ok) {
        // Drain: let copies that were already issued land before the CTA exits.
        for (int s = 0; s < kStages; ++s) {
          if (armed_k[s] >= 0)
            for (uint32_t spin = 0; spin < (1u << 20) && !mbar_try_wait(&bar->k_full[s], armed_k[s]); ++spin) {}
          if (armed_v[s] >= 0)
            for (uint32_t spin = 0; spin < (1u << 20) && !mbar_try_wait(&bar->v_full[s], armed_v[s]); ++spin) {}
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------ MMA issuer
    // The issuing warp is the serial resource of the CTA.  It stays converged: every lane
    // evaluates the (warp-uniform) waits and descriptor arithmetic, and one elected lane issues
    // the MMAs and commits.  Descriptors are built once and advanced by adding precomputed
    // (byte offset >> 4) constants to their low word.
    const uint32_t issuer = elect_one();
    const bool kt = p.k_transposed != 0;
    const uint32_t idesc_s = umma_idesc_f16(BF16, kBM, kBN, false, kt);
    const bool vt = p.v_transposed != 0;
    const uint32_t idesc_o = umma_idesc_f16(BF16, kBM, D, false, !vt);
    const uint64_t dq0 = umma_desc_sw128(smem_u32(smem + SM::kOffQ), 16, 1024);
    const uint64_t dk0 = kt ? umma_desc_sw128(smem_u32(smem + SM::kOffK), D * 128, 1024)
                            : umma_desc_sw128(smem_u32(smem + SM::kOffK), 16, 1024);
    const uint64_t dv0 = vt ? umma_desc_sw128(smem_u32(smem + SM::kOffV), 16, 1024)
                            : umma_desc_sw128(smem_u32(smem + SM::kOffV), kBN * 128, 1024);
    const uint64_t dp0 = umma_desc_sw128(smem_u32(smem + SM::kOffP), 16, 1024);

    auto issue_s = [&](int t, int stage) {
      const uint64_t da = dq0 + ((t * SM::kTileQ) >> 4);
      const uint64_t db = dk0 + ((stage * SM::kTileKV) >> 4);
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        // K-major operand: 32 bytes per k-step inside a 64-element atom, then the next atom;
        // MN-major (transposed K): 16 rows of 128 bytes per k-step
        const uint32_t off_k = ((i / 4) * (kBM * 128) + (i % 4) * 32) >> 4;
        const uint32_t off_b = kt ? static_cast<uint32_t>((i * 2048) >> 4) : off_k;
        if (i < ksteps_d)   // head dimensions below D use the first d / 16 k-steps only
          umma_ss_elected(tmem_base + t * kBN, da + off_k, db + off_b, idesc_s, i > 0 ? 1u : 0u, issuer);
      }
      umma_commit_elected(&bar->s_full[t], issuer);
    };
    // P arrives in two parts (the first kSplit K/V rows, then the rest); each part is multiplied
    // as soon as it is there, so the second part's exponentials overlap the first part's MMAs.
    auto issue_pv = [&](int t, int stage, int part, uint32_t accumulate) {
      const uint64_t db = dv0 + ((stage * SM::kTileKV) >> 4);
#pragma unroll
      for (int i = (part == 0 ? 0 : kSplit / 16); i < (part == 0 ? kSplit / 16 : kBN / 16); ++i) {
        const uint32_t acc = i > 0 ? 1u : accumulate;
        // MN-major V: 16 K/V rows of 128 bytes per k-step; K-major (transposed V): 32 bytes per k-step inside a
        // 64-column atom of D rows, then the next atom
        const uint32_t off_v = vt ? static_cast<uint32_t>(((i / 4) * (D * 128) + (i % 4) * 32) >> 4)
                                  : static_cast<uint32_t>((i * 2048) >> 4);
        if constexpr (PSMEM) {
          const uint64_t da = dp0 + ((t * SM::kTileP + (i / 4) * (kBM * 128) + (i % 4) * 32) >> 4);
          umma_ss_elected(tmem_base + kColO + t * D, da, db + off_v, idesc_o, acc, issuer);
        } else {
          umma_ts_elected(tmem_base + kColO + t * D, tmem_base + (kSep ? kColP : t * kBN) + i * 8,
                          db + off_v, idesc_o, acc, issuer);
        }
      }
    };
    auto wait = [&](uint64_t* b, uint32_t parity, uint32_t code) {
      bool ok = mbar_wait(b, parity, abort_word, code);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
      return ok;
    };

    // With a single K/V stage the release cannot wait for the next iteration's first MMA
    // (that MMA needs the very load the release unblocks).
    constexpr bool kDeferRelease = kStages >= 2;
    // The CTA's K/V blocks form one sequence G = 0 .. my_items * nkv - 1 (block j = G % nkv of item G / nkv):
    // ring stages, barrier phases and the look-ahead waits follow G, whatever item a block belongs to.
    const int total_blocks = my_items * nkv;
    bool ok = wait(&bar->k_full[0], 0, 0x301);
    for (int t = 0; t < NT && ok; ++t) {
      ok = wait(&bar->q_full[t], 0, 0x300 + t);
      if (!ok) break;
      issue_s(t, 0);
      if (nkv == 1) umma_commit_elected(&bar->q_empty[t], issuer);   // the item's only S: its Q may be replaced
    }
    if (ok) {
      umma_commit_elected(&bar->k_empty[0], issuer);
      // operands of the first iteration; later ones are checked one iteration ahead, off the
      // critical path (the loads land long before they are needed)
      ok = wait(&bar->v_full[0], 0, 0x400);
      if (ok && total_blocks > 1) ok = wait(&bar->k_full[1 % kStages], (1 / kStages) & 1, 0x600);
    }
    if constexpr (kSep) {
      // One item per CTA.  S(j+1) is issued as soon as the softmax warps have taken S(j) out of TMEM, ahead of
      // P*V(j): the tensor pipe computes the next scores while the exponentials run.
      for (int j = 0; j < nkv && ok; ++j) {
        const int sv = j % kStages;
        const int sk = (j + 1) % kStages;
        const bool more = (j + 1 < nkv);
        if (more) {
          ok = wait(&bar->s_taken[0], j & 1, 0x480 + j);
          if (!ok) break;
          issue_s(0, sk);
          umma_commit_elected(&bar->k_empty[sk], issuer);
        }
        ok = wait(&bar->p_part[0][0], j & 1, 0x500 + j);
        if (!ok) break;
        issue_pv(0, sv, 0, j > 0 ? 1u : 0u);
        ok = wait(&bar->p_part[0][1], j & 1, 0x580 + j);
        if (!ok) break;
        issue_pv(0, sv, 1, 1u);
        // v_empty doubles as "P*V(j) has finished" for the softmax warps (they overwrite P and may
        // rescale O in the next iteration)
        umma_commit_elected(&bar->v_empty[sv], issuer);
        if (!more) umma_commit_elected(&bar->o_done[0], issuer);
        if (more) {
          ok = wait(&bar->v_full[sk], ((j + 1) / kStages) & 1, 0x400 + j);
          if (ok && j + 2 < nkv) ok = wait(&bar->k_full[(j + 2) % kStages], ((j + 2) / kStages) & 1, 0x600 + j);
        }
      }
    }
    // The issuing warp has to stay converged, and every conditional region around an elected issue or a
    // warp-wide wait costs it a reconvergence: the iteration body therefore exists in three compile-time
    // forms -- a block inside an item, an item's second-to-last block (its S is the item's last: Q is
    // released) and an item's last block (O is complete; the next S is the next item's first) -- and the
    // loop over an item's inner blocks carries no item-boundary tests at all.
    int G = 0;                                 // the CTA's K/V blocks so far
    auto iteration = [&](auto kind_c, int j, int k) -> bool {
      constexpr int kind = decltype(kind_c)::value;     // 0 inner block, 1 second-to-last, 2 last of its item
      const int sv = G % kStages;
      const int sk = (G + 1) % kStages;
      auto tile_step = [&](auto tile) -> bool {
        constexpr int t = decltype(tile)::value;
        if (!wait(&bar->p_part[t][0], G & 1, 0x500 + j)) return false;
        DITTO_STAMP(512, G, 1 + 4 * t);
        issue_pv(t, sv, 0, j > 0 ? 1u : 0u);
        if (kDeferRelease && t == 0 && G > 0) {
          // Release the stages the previous iteration finished with.  Deferred to here so that
          // the two commits do not sit between "P is ready" and the first MMA that consumes it.
          umma_commit_elected(&bar->v_empty[(G - 1) % kStages], issuer);
          umma_commit_elected(&bar->k_empty[sv], issuer);
        }
        if (!wait(&bar->p_part[t][1], G & 1, 0x580 + j)) return false;
        DITTO_STAMP(512, G, 2 + 4 * t);
        issue_pv(t, sv, 1, 1u);
        // Same thread, in-order pipe: the next S overwrites the P it follows only after P*V has
        // read it, and its commit also covers that P*V (a commit tracks every earlier MMA).
        if constexpr (kind == 0) {
          issue_s(t, sk);
        } else if constexpr (kind == 1) {
          issue_s(t, sk);
          umma_commit_elected(&bar->q_empty[t], issuer);   // that was the item's last S: its Q may be replaced
        } else {
          umma_commit_elected(&bar->o_done[t], issuer);
          if (k + 1 < my_items) {
            // the next item's first S: its Q must have landed
            if (!wait(&bar->q_full[t], (k + 1) & 1, 0x300 + t)) return false;
            issue_s(t, sk);
            if (nkv == 1) umma_commit_elected(&bar->q_empty[t], issuer);
          }
        }
        DITTO_STAMP(512, G, 3 + 4 * t);
        return true;
      };
      if (!tile_step(std::integral_constant<int, 0>{})) return false;
      if constexpr (NT == 2) {
        if (!tile_step(std::integral_constant<int, 1>{})) return false;
      }
      const bool more = G + 1 < total_blocks;
      if (!kDeferRelease) {
        umma_commit_elected(&bar->v_empty[sv], issuer);
        if (more) umma_commit_elected(&bar->k_empty[sk], issuer);
      }
      if (more) {
        if (!wait(&bar->v_full[sk], ((G + 1) / kStages) & 1, 0x400 + j)) return false;
        if (G + 2 < total_blocks && !wait(&bar->k_full[(G + 2) % kStages], ((G + 2) / kStages) & 1, 0x600 + j)) return false;
      }
      DITTO_STAMP(512, G, 0);
      ++G;
      return true;
    };
    for (int k = 0; k < (kSep ? 0 : my_items) && ok; ++k) {
      if (k > 0) {
        // the first P*V of an item overwrites O: the finished item's O must be out of tensor memory
        for (int t = 0; t < NT && ok; ++t) ok = wait(&bar->o_free[t], (k - 1) & 1, 0x680 + t);
        if (!ok) break;
      }
      int j = 0;
      for (; j < nkv - 2 && ok; ++j) ok = iteration(std::integral_constant<int, 0>{}, j, k);
      if (ok && nkv >= 2) { ok = iteration(std::integral_constant<int, 1>{}, j, k); ++j; }
      if (ok) ok = iteration(std::integral_constant<int, 2>{}, j, k);
    }
  } else if (warp < 4 * NT) {
    // ------------------------------------------------------------ softmax + epilogue
    const int t = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t s_col = lane_base + t * kBN;
    const uint32_t o_col = lane_base + kColO + t * D;
    const uint32_t p_col = kSep ? lane_base + kColP : s_col;   // P overwrites S unless it has its own columns
    const float c = p.scale_log2;
    bool ok = true;

    uint32_t par = 0;                       // parity of the K/V blocks of all items so far: the phase of s_full / p_part

    for (int k = 0; k < my_items && ok; ++k) {
    float m = -INFINITY, l = 0.f;
    for (int j = 0; j < nkv; ++j, par ^= 1u) {
      ok = mbar_wait(&bar->s_full[t], par, abort_word, 0x800 + j);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      if ((warp & 3) == 0) DITTO_STAMP(t * 256, k * nkv + j, 0); else DITTO_STAMP(t * 256, k * nkv + j, 8 + (warp & 3));

      uint32_t sv[kBN];
      tmem_ld_x128_wait(s_col, sv);
      if constexpr (kSep) {
        tc_fence_before_sync();
        mbar_arrive(&bar->s_taken[t]);             // the S columns may be overwritten by S(j+1)
      }
      if ((warp & 3) == 0) DITTO_STAMP(t * 256, k * nkv + j, 1);

      float m_new = m;
      if constexpr (MODE == kModeSoftmax) {
        if (j == nkv - 1 && (p.L % kBN) != 0) {
          // partial last block: K rows >= L were zero-filled, their scores must not count
          const int valid = p.L % kBN;
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
      if constexpr (kSep) {
        if (j > 0) {
          // P*V(j-1) must have finished before P is overwritten or O is rescaled; here S(j) was
          // issued ahead of it, so s_full does not imply it.  Normally long complete.
          ok = mbar_wait(&bar->v_empty[(j - 1) % kStages], ((j - 1) / kStages) & 1, abort_word, 0x900 + j);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
        }
      }
      // Lazy rescale: keep the stale maximum while the true one is within
      // 2^kRescaleThreshold of it; the final division by l cancels the difference.
      const bool need = MODE == kModeSoftmax && (m_new - m) * c > kRescaleThreshold;
      if (MODE == kModeSoftmax && __any_sync(0xffffffffu, need)) {
        const float f = ex2_approx((m - m_new) * c);
        if (j > 0) {
          // s_full(j) was committed after P*V(j-1) by the same thread and a commit covers every
          // earlier MMA, so the accumulator is quiescent here.
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

      if ((warp & 3) == 0) DITTO_STAMP(t * 256, k * nkv + j, 2);
      const float mc = m * c;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        constexpr int kFirst = kSplit / 2;               // packed 32-bit words in part 0
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
              p0 = p0 > 0.f ? p0 : 0.f;                  // if_then_else(D > 0, D, 0) as in the reference
              p1 = p1 > 0.f ? p1 : 0.f;
            }
            sum0 += p0;
            sum1 += p1;
            pk[i] = pack2<BF16>(p0, p1);
          }
        }
        if (part == 0 && (warp & 3) == 0) DITTO_STAMP(t * 256, k * nkv + j, 3);
        if constexpr (PSMEM) {
          // K-major, 128B-swizzled A operand: 64-column atoms of 128 rows x 128 bytes, 16-byte chunks.
          uint8_t* pt = smem + SM::kOffP + t * SM::kTileP;
#pragma unroll
          for (int ch = 0; ch < kFirst / 4; ++ch) {
            const int gch = w0 / 4 + ch;                  // chunk index within the 128-column row
            if (gch < w1 / 4) {
              uint4 v = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
              *reinterpret_cast<uint4*>(pt + (gch >> 3) * (kBM * 128) + row * 128 + (((gch & 7) ^ (row & 7)) << 4)) = v;
            }
          }
          fence_proxy_async_smem();
        } else {
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
        }
        tc_fence_before_sync();
        mbar_arrive(&bar->p_part[t][part]);
        if (part == 0 && (warp & 3) == 0) DITTO_STAMP(t * 256, k * nkv + j, 4);
      }
      l += sum0 + sum1;
      if ((warp & 3) == 0) DITTO_STAMP(t * 256, k * nkv + j, 5); else DITTO_STAMP(t * 256, k * nkv + j, 5 + (warp & 3));
    }

    if (!ok) break;
    ok = mbar_wait(&bar->o_done[t], k & 1, abort_word, 0xA00);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    tc_fence_after_sync();
    if ((warp & 3) == 0) DITTO_STAMP(t * 256, k * nkv + nkv - 1, 12);
    {
      const Item it = decode(k);
      const float inv = MODE == kModeSoftmax ? 1.0f / l : 1.0f;
      // O leaves tensor memory whole (normalised and rounded: D / 2 registers), so that the accumulator is
      // handed back before the stores and the next item's first P*V never waits for them
      uint32_t w[D / 2];
      {
        uint32_t o[D];                                  // one load for the whole row (the scores' registers are free now)
        if constexpr (D == 128) tmem_ld_x128_wait(o_col, o); else tmem_ld_x64_wait(o_col, o);   // warp-collective
#pragma unroll
        for (int i = 0; i < D / 2; ++i)
          w[i] = pack2<BF16>(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->o_free[t]);
      if ((warp & 3) == 0) DITTO_STAMP(t * 256, k * nkv + nkv - 1, 13);
      // Written straight from the registers, a warp's store instruction would touch 32 rows (one 16-byte piece
      // each): 2048 partial-sector requests per tile that back up the load/store path and delay the barrier
      // operations behind them (measured: the next item's first block ran 6 k clocks late).  Instead every
      // warp turns its 32 rows x 128 bytes around in 4 KB of shared memory of its own (16-byte pieces swizzled
      // by row, no bank conflicts either way) and writes 4 rows x 128 contiguous bytes per instruction.
      uint8_t* stage = smem + SM::kOffStage + warp * 4096;
      const size_t out_row0 = static_cast<size_t>(it.seq) * p.M + it.m0 + t * kBM + (warp & 3) * 32;
#pragma unroll
      for (int pass = 0; pass < D / 64; ++pass) {
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8)
          *reinterpret_cast<uint4*>(stage + lane * 128 + ((c8 ^ (lane & 7)) << 4)) =
              make_uint4(w[pass * 32 + 4 * c8], w[pass * 32 + 4 * c8 + 1], w[pass * 32 + 4 * c8 + 2], w[pass * 32 + 4 * c8 + 3]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = 4 * i + (lane >> 3), piece = lane & 7;
          const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((piece ^ (rr & 7)) << 4));
          const int col = pass * 64 + piece * 8;        // widths are multiples of 16: whole 16-byte pieces
          if (it.m0 + t * kBM + (warp & 3) * 32 + rr < p.M && col < p.dv)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.out) + ((out_row0 + rr) * p.out_ld + it.head_col + col) * 2) = v;
        }
        __syncwarp();
      }
      if ((warp & 3) == 0) DITTO_STAMP(t * 256, k * nkv + nkv - 1, 14);
    }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) DITTO_STAMP(512, 0, 9);
  if (warp == 0) {
    tmem_dealloc(tmem_base, kTmemCols);
    if (lane == 0 && bar->abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, static_cast<int>(bar->abort_word));
  }
}

// ------------------------------------------------------------------ launcher
template <bool BF16, int D, int NT, bool PSMEM, int MODE>
static cudaError_t launch_one(const AttnParams& p, int batch, cudaStream_t stream) {
  using SM = Smem<D, NT, PSMEM>;
  auto kern = attention_kernel<BF16, D, NT, PSMEM, MODE>;
  // the function attributes are set once per device (this instantiation's static)
  static std::atomic<unsigned long long> configured{0};
  static std::atomic<int> places[64];      // CTAs of this kernel the device holds at once
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!((configured.load(std::memory_order_acquire) >> dev) & 1ull)) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    int per_sm = 0, sms = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads_for(NT), SM::kBytes);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    // the looped variants allocate all 512 tensor-memory columns: one CTA per SM whatever shared memory allows
    if (!kSeparateP<D, NT, PSMEM>) per_sm = std::min(per_sm, 1);
    places[dev].store(std::max(1, per_sm * sms), std::memory_order_relaxed);
    configured.fetch_or(1ull << dev, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg = {};
  // one CTA per place the device has (or per item, if there are fewer), or one CTA per item
  AttnParams q = p;
  q.items = ((p.M + NT * kBM - 1) / (NT * kBM)) * batch;
  // The work loop pays where an item is long enough for its fixed cost to show and short enough for it to
  // matter: measured at head dimension 128 (S = 512: -5 %, 2048: -1 % per item); at 64, where the exponentials
  // set the pace, one CTA per item was faster (S = 2048: 109 against 119 us), so those launches keep it.
  constexpr bool loop = kLoopItems<D, NT, PSMEM>;
  const int grid = loop ? std::min(q.items, places[dev].load(std::memory_order_relaxed)) : q.items;
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(threads_for(NT), 1, 1);
  cfg.dynamicSmemBytes = SM::kBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see grid_dependency_wait in the kernel
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, q);
}

cudaError_t launch_attention(const AttnParams& p, int batch, int d, bool bf16, int nt, bool psmem, int mode,
                             cudaStream_t stream) {
#define DITTO_DISPATCH(BF, DD, NN, PS, MO) \
  if (bf16 == BF && d == DD && nt == NN && psmem == PS && mode == MO) \
    return launch_one<BF, DD, NN, PS, MO>(p, batch, stream);
#define DITTO_DISPATCH_SHAPES(PS, MO)  \
  DITTO_DISPATCH(false, 64, 1, PS, MO) \
  DITTO_DISPATCH(false, 64, 2, PS, MO) \
  DITTO_DISPATCH(false, 128, 1, PS, MO) \
  DITTO_DISPATCH(false, 128, 2, PS, MO) \
  DITTO_DISPATCH(true, 64, 1, PS, MO)  \
  DITTO_DISPATCH(true, 64, 2, PS, MO)  \
  DITTO_DISPATCH(true, 128, 1, PS, MO) \
  DITTO_DISPATCH(true, 128, 2, PS, MO)
  DITTO_DISPATCH_SHAPES(false, kModeSoftmax)
  DITTO_DISPATCH_SHAPES(true, kModeSoftmax)
  DITTO_DISPATCH_SHAPES(false, kModeRelu)
  DITTO_DISPATCH_SHAPES(false, kModeIdentity)
#undef DITTO_DISPATCH_SHAPES
#undef DITTO_DISPATCH
  return cudaErrorInvalidValue;
}

}  // namespace ditto_b200
