// Throughput kernels for the hot S6 shape class (placeholder: not yet enabled).
#include "common.cuh"
#include "dispatch.h"

namespace b200 {
bool selscan_fwd_fast_supported(const b200_selscan_fwd_args &) { return false; }
bool selscan_bwd_fast_supported(const b200_selscan_bwd_args &) { return false; }
int selscan_fwd_fast(const b200_selscan_fwd_args &, cudaStream_t) { return B200_ERR_UNSUPPORTED; }
int selscan_bwd_fast(const b200_selscan_bwd_args &, cudaStream_t) { return B200_ERR_UNSUPPORTED; }
}  // namespace b200
