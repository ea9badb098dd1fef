// Host-side helpers shared by the launchers: error text of the calling thread, cached TMA tensor-map
// encoding, and a once-per-device guard for function attributes.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>

namespace ditto_b200 {

// Text behind DITTO_ERR_CUDA / DITTO_ERR_DRIVER for ditto_b200_last_cuda_error() (one buffer per thread).
void set_error(const char* what, const char* detail);
const char* last_error_text();
// Records cudaGetErrorString(e) under `what` and returns DITTO_ERR_CUDA.
int cuda_fail(const char* what, cudaError_t e);

// Tiled tensor map over 16-bit elements with 128-byte-swizzled boxes, rank 2 to 4.
//   dims[r]          extent of dimension r in elements, dims[0] innermost (contiguous)
//   strides_bytes[r] byte stride of dimension r + 1 (rank - 1 entries, multiples of 16)
//   box[r]           box extent of dimension r (box[0] * 2 bytes = 128)
// Out-of-range parts of a box read as zero.  A map is a pure function of these arguments, and callers
// with pre-allocated buffers present the same ones call after call, so the last few encodings are kept
// per thread; a repeated launch then makes no driver call at all.  Returns a DITTO_* code.
int make_tensor_map(CUtensorMap* map, bool bf16, const void* base, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box);

// How the row blocks of an MLP-chain call are spread over thread-block clusters: the first `whole_blocks`
// row blocks (of every batch entry) are computed by one cluster each, the others by `parts` clusters each,
// every one taking a range of the hidden dimension; their fp32 partials of Y are combined through scratch
// memory.  parts == 1 (or whole_blocks == row_blocks): no scratch memory is needed.
struct RowBlockPlan {
  int whole_blocks;
  int parts;
};
// The plan with the shortest modelled run time on a device that holds `cluster_slots` clusters at once.
// Clusters are dispatched in item order to whichever place frees up first; an item's duration is modelled as
// its hidden chunks plus `fixed_cost` (start-up and write-out, in chunk units, from timelines of the kernel).
// `shared_cost` is what sharing adds to the run (the partials' round trip through scratch memory, the last
// cluster's combining pass, the counter reset in front of the launch), in the same units.
// A part never gets fewer than `min_chunks` chunks nor are there more than `max_parts` parts.
RowBlockPlan plan_row_blocks(int batch, int row_blocks, int chunks, int min_chunks, int max_parts, int cluster_slots,
                             double fixed_cost, double shared_cost);
// Scratch bytes of a plan: parts slabs of fp32 [batch][shared rows][N] and one counter per (batch, shared
// row block, CTA of the cluster).
size_t plan_workspace_bytes(const RowBlockPlan& plan, int batch, int row_blocks, int rows_per_block, int N,
                            int cluster_size);

// Once-per-device guard: `done` is a static of the calling launcher (one per kernel instantiation), bit d
// set once device d has been configured.  Returns the current device in *dev.
constexpr int kMaxDevices = 64;
inline cudaError_t current_device_checked(int* dev) {
  cudaError_t e = cudaGetDevice(dev);
  if (e != cudaSuccess) return e;
  return (*dev < 0 || *dev >= kMaxDevices) ? cudaErrorInvalidDevice : cudaSuccess;
}
inline bool device_configured(const std::atomic<unsigned long long>& done, int dev) {
  return (done.load(std::memory_order_acquire) >> dev) & 1ull;
}
inline void mark_device_configured(std::atomic<unsigned long long>& done, int dev) {
  done.fetch_or(1ull << dev, std::memory_order_release);
}

}  // namespace ditto_b200
