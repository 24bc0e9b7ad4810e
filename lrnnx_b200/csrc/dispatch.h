// Internal (C++) entry points behind the extern "C" layer in api.cu.
#pragma once
#include <cuda_runtime.h>
#include "../../include/lrnnx_b200.h"

namespace b200 {

constexpr int kSlStage = 32;      // stage_h spacing of the streaming kernels (selscan_sl.cu)
constexpr int kFastStage = 256;   // stage_h spacing of the lane-scan kernels (selscan_fast.cu)

// coverage kernels: every variant (selscan_generic.cu)
int selscan_fwd_generic(const b200_selscan_fwd_args &a, cudaStream_t st);
int selscan_bwd_generic(const b200_selscan_bwd_args &a, cudaStream_t st);

// throughput kernels for the hot S6 shape class (selscan_fast.cu)
bool selscan_fwd_fast_supported(const b200_selscan_fwd_args &a);
bool selscan_bwd_fast_supported(const b200_selscan_bwd_args &a);
int selscan_fwd_fast(const b200_selscan_fwd_args &a, cudaStream_t st);
int selscan_bwd_fast(const b200_selscan_bwd_args &a, cudaStream_t st);

// streaming kernels for the same shape class when there are enough rows (selscan_sl.cu)
bool selscan_fwd_sl_supported(const b200_selscan_fwd_args &a);
bool selscan_bwd_sl_supported(const b200_selscan_bwd_args &a);
int selscan_fwd_sl(const b200_selscan_fwd_args &a, cudaStream_t st);
int selscan_bwd_sl(const b200_selscan_bwd_args &a, cudaStream_t st);

// status word of the tensor-core projection kernel (cgemm_tc.cu)
int cgemm_status_read();

// status word of the decode-step pipeline (ssu.cu): non-zero after an expired bounded wait
int ssu_status_read();

}  // namespace b200
