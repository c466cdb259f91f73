#include "common.cuh"
namespace based {
int launch_linattn_prefill_tc(const void*, const void*, const void*, void*, void*, void*, int, int, int, int,
                              Strides3, Strides3, Strides3, Strides3, int, float, cudaStream_t) {
  return BASED_ERR_IMPL;
}
}  // namespace based
