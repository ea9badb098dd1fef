#include "mlp_sm100.cuh"

#include "../../include/ditto_b200.h"

namespace ditto_b200 {

int launch_mlp_chain(const void*, const void*, const void*, void*, int, int, int, int, int, bool, int, int, int*,
                     cudaStream_t) {
  return DITTO_ERR_UNSUPPORTED;
}

}  // namespace ditto_b200
