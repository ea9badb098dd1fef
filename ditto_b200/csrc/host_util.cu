// Error text, and the one encoder of TMA tensor maps every launcher goes through.
#include "host_util.cuh"

#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/ditto_b200.h"

namespace ditto_b200 {

namespace {

thread_local char g_last_error[256] = "";

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The encoder is a host-side driver function; it is resolved through the runtime, once, so the library
// has no link-time dependency on libcuda.
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

struct MapKey {
  const void* base;
  uint64_t dims[4], strides[3];
  uint32_t box[4];
  uint32_t rank, bf16;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapCache {
  static constexpr int kEntries = 16;
  MapKey key[kEntries];
  CUtensorMap map[kEntries];
  bool valid[kEntries] = {};
  int next = 0;
};
thread_local MapCache g_map_cache;

}  // namespace

void set_error(const char* what, const char* detail) {
  std::snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, detail ? detail : "");
}

const char* last_error_text() { return g_last_error; }

int cuda_fail(const char* what, cudaError_t e) {
  set_error(what, cudaGetErrorString(e));
  return DITTO_ERR_CUDA;
}

int make_tensor_map(CUtensorMap* map, bool bf16, const void* base, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box) {
  if (rank < 2 || rank > 4) return DITTO_ERR_INVALID_ARG;
  MapKey want;
  std::memset(&want, 0, sizeof(want));   // padding included: keys are compared bytewise
  want.base = base;
  want.rank = static_cast<uint32_t>(rank);
  want.bf16 = bf16 ? 1u : 0u;
  for (int r = 0; r < rank; ++r) {
    want.dims[r] = dims[r];
    want.box[r] = box[r];
    if (r + 1 < rank) want.strides[r] = strides_bytes[r];
  }
  MapCache& cache = g_map_cache;
  for (int i = 0; i < MapCache::kEntries; ++i)
    if (cache.valid[i] && cache.key[i] == want) {
      *map = cache.map[i];
      return DITTO_OK;
    }
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled", "entry point not found");
    return DITTO_ERR_DRIVER;
  }
  cuuint64_t d[4], s[3];
  cuuint32_t b[4], estr[4] = {1, 1, 1, 1};
  for (int r = 0; r < rank; ++r) {
    d[r] = dims[r];
    b[r] = box[r];
    if (r + 1 < rank) s[r] = strides_bytes[r];
  }
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, s, b, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[64];
    std::snprintf(buf, sizeof(buf), "CUresult %d", static_cast<int>(r));
    set_error("cuTensorMapEncodeTiled", buf);
    return DITTO_ERR_CUDA;
  }
  cache.key[cache.next] = want;
  cache.map[cache.next] = *map;
  cache.valid[cache.next] = true;
  cache.next = (cache.next + 1) % MapCache::kEntries;
  return DITTO_OK;
}

RowBlockPlan plan_row_blocks(int batch, int row_blocks, int chunks, int min_chunks, int max_parts, int cluster_slots,
                             double fixed_cost, double shared_cost) {
  RowBlockPlan best = {row_blocks, 1};
  if (cluster_slots <= 1 || chunks < 2 * min_chunks || max_parts < 2) return best;
  if (static_cast<long long>(batch) * row_blocks > 4096) return best;   // large problems: nothing to gain at the tail
  // The search costs tens of microseconds of host time, more than a launch: the answers for the last few
  // shapes are kept per thread (a plan is a pure function of the arguments).
  struct Memo {
    int batch, row_blocks, chunks, min_chunks, max_parts, slots;
    double fixed, shared;
    RowBlockPlan plan;
    bool valid;
  };
  constexpr int kMemo = 8;
  thread_local Memo memo[kMemo] = {};
  thread_local int memo_next = 0;
  for (int i = 0; i < kMemo; ++i) {
    const Memo& m = memo[i];
    if (m.valid && m.batch == batch && m.row_blocks == row_blocks && m.chunks == chunks && m.min_chunks == min_chunks &&
        m.max_parts == max_parts && m.slots == cluster_slots && m.fixed == fixed_cost && m.shared == shared_cost)
      return m.plan;
  }
  constexpr int kMaxSlots = 160;
  const int slots = cluster_slots < kMaxSlots ? cluster_slots : kMaxSlots;
  auto makespan = [&](int shared_blocks, int parts) {
    double free_at[kMaxSlots];
    for (int s = 0; s < slots; ++s) free_at[s] = 0.0;
    double end = 0.0;
    auto place = [&](double dur) {
      int at = 0;
      for (int s = 1; s < slots; ++s)
        if (free_at[s] < free_at[at]) at = s;
      free_at[at] += dur;
      if (free_at[at] > end) end = free_at[at];
    };
    for (int bb = 0; bb < batch; ++bb) {
      for (int r = 0; r < row_blocks - shared_blocks; ++r) place(chunks + fixed_cost);
      for (int r = 0; r < shared_blocks; ++r)
        for (int q = 0; q < parts; ++q) place((q + 1) * chunks / parts - q * chunks / parts + fixed_cost);
    }
    return end;
  };
  double best_t = makespan(0, 1);
  int limit = chunks / min_chunks;
  if (limit > max_parts) limit = max_parts;
  for (int parts = 2; parts <= limit; ++parts) {
    const int max_shared = row_blocks < slots ? row_blocks : slots;
    for (int sh = 1; sh <= max_shared; ++sh) {
      const double t = makespan(sh, parts) + shared_cost;
      if (t < best_t * 0.97) {
        best_t = t;
        best = {row_blocks - sh, parts};
      }
    }
  }
  memo[memo_next] = {batch, row_blocks, chunks, min_chunks, max_parts, cluster_slots, fixed_cost, shared_cost, best, true};
  memo_next = (memo_next + 1) % kMemo;
  return best;
}

size_t plan_workspace_bytes(const RowBlockPlan& plan, int batch, int row_blocks, int rows_per_block, int N,
                            int cluster_size) {
  const size_t shared = static_cast<size_t>(row_blocks - plan.whole_blocks);
  if (shared == 0 || plan.parts <= 1) return 0;
  return static_cast<size_t>(plan.parts) * batch * shared * rows_per_block * N * sizeof(float) +
         static_cast<size_t>(batch) * shared * cluster_size * sizeof(int);
}

}  // namespace ditto_b200
