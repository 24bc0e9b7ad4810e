// extern "C" entry points of liblrnnx_b200.so: argument validation and
// dispatch to the kernels.  See include/lrnnx_b200.h for the contract.
#include "common.cuh"
#include "dispatch.h"
#include <cstring>

namespace b200 {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static int check_selscan(const b200_selscan_fwd_args &a) {
  B200_REQUIRE(a.u && a.delta && a.A && a.B && a.C, B200_ERR_NULL, "selscan: u, delta, A, B, C must be non-null");
  B200_REQUIRE(a.batch > 0 && a.dim > 0 && a.seqlen > 0 && a.dstate > 0, B200_ERR_SHAPE,
               "selscan: batch, dim, seqlen, dstate must be positive");
  // same limit as csrc/selective_scan/selective_scan_cpu.cpp:327
  B200_REQUIRE(a.dstate <= kMaxDState, B200_ERR_SHAPE, "selective_scan only supports state dimension <= 256");
  B200_REQUIRE(a.n_groups >= 1 && a.dim % a.n_groups == 0, B200_ERR_SHAPE,
               "selscan: dim (%d) must be a multiple of n_groups (%d)", a.dim, a.n_groups);
  B200_REQUIRE(a.dtype == B200_F32 || a.dtype == B200_F16 || a.dtype == B200_BF16, B200_ERR_DTYPE,
               "selscan: unknown activation dtype %d", a.dtype);
  B200_REQUIRE(a.method >= B200_DISC_ZOH && a.method <= B200_DISC_S7, B200_ERR_DTYPE,
               "Discretization method not supported");
  // csrc/selective_scan/selective_scan_cpu.cpp:299-305
  B200_REQUIRE(!(a.method == B200_DISC_S7 && a.is_complex), B200_ERR_DTYPE,
               "S7 discretization only supports real (float) weights, not complex");
  B200_REQUIRE(!(a.method == B200_DISC_RGLRU && a.is_complex), B200_ERR_DTYPE,
               "RGLRU discretization only supports real (float) weights, not complex");
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" {

const char *b200_last_error(void) { return g_err; }
int b200_abi_version(void) { return 5; }

// size of an argument block as this library was compiled; lets a binding
// verify its own struct layout before the first call
int b200_sizeof(const char *name) {
  if (!name) return -1;
  if (!strcmp(name, "b200_selscan_fwd_args")) return (int)sizeof(b200_selscan_fwd_args);
  if (!strcmp(name, "b200_selscan_bwd_args")) return (int)sizeof(b200_selscan_bwd_args);
  if (!strcmp(name, "b200_selscan_fixup_args")) return (int)sizeof(b200_selscan_fixup_args);
  if (!strcmp(name, "b200_selscan_adjsum_args")) return (int)sizeof(b200_selscan_adjsum_args);
  if (!strcmp(name, "b200_simpscan_args")) return (int)sizeof(b200_simpscan_args);
  if (!strcmp(name, "b200_ssu_args")) return (int)sizeof(b200_ssu_args);
  if (!strcmp(name, "b200_s4_args")) return (int)sizeof(b200_s4_args);
  if (!strcmp(name, "b200_s5_step_args")) return (int)sizeof(b200_s5_step_args);
  if (!strcmp(name, "b200_conv1d_args")) return (int)sizeof(b200_conv1d_args);
  if (!strcmp(name, "b200_rmsnorm_args")) return (int)sizeof(b200_rmsnorm_args);
  if (!strcmp(name, "b200_cgemm_args")) return (int)sizeof(b200_cgemm_args);
  if (!strcmp(name, "b200_cgemm_planes_args")) return (int)sizeof(b200_cgemm_planes_args);
  if (!strcmp(name, "b200_cgemm_grad_args")) return (int)sizeof(b200_cgemm_grad_args);
  if (!strcmp(name, "b200_xent_args")) return (int)sizeof(b200_xent_args);
  if (!strcmp(name, "b200_skinny_linear_args")) return (int)sizeof(b200_skinny_linear_args);
  return -1;
}

int b200_selscan_fwd(const b200_selscan_fwd_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "selscan_fwd: null argument block");
  if (int e = check_selscan(*args)) return e;
  B200_REQUIRE(args->out && args->x, B200_ERR_NULL, "selscan_fwd: out and x must be non-null");
  B200_REQUIRE(!args->z || args->out_z, B200_ERR_NULL, "selscan_fwd: out_z is required when z is given");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // stage states are written only with the spacing the chosen kernel works in
  b200_selscan_fwd_args a = *args;
  if (selscan_fwd_sl_supported(a)) {
    if (a.stage_len != kSlStage) a.stage_h = nullptr;
    return selscan_fwd_sl(a, st);
  }
  if (selscan_fwd_fast_supported(a)) {
    if (a.stage_len != kFastStage) a.stage_h = nullptr;
    return selscan_fwd_fast(a, st);
  }
  B200_REQUIRE(args->l_segments <= 1, B200_ERR_UNSUPPORTED,
               "selscan_fwd: l_segments > 1 is only available on the throughput-kernel shape class");
  return selscan_fwd_generic(*args, st);
}

int b200_selscan_stage_states(const b200_selscan_fwd_args *args) {
  if (!args || check_selscan(*args) || args->l_segments > 1) return 0;
  b200_selscan_fwd_args a = *args;
  a.stage_h = nullptr;
  if (selscan_fwd_sl_supported(a)) return kSlStage;
  if (selscan_fwd_fast_supported(a)) return kFastStage;
  return 0;
}

int b200_selscan_bwd(const b200_selscan_bwd_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "selscan_bwd: null argument block");
  if (int e = check_selscan(args->f)) return e;
  const b200_selscan_fwd_args &f = args->f;
  B200_REQUIRE(args->dout && args->du && args->ddelta && args->dA && args->dB && args->dC, B200_ERR_NULL,
               "selscan_bwd: dout, du, ddelta, dA, dB, dC must be non-null");
  // csrc/selective_scan/selective_scan_cpu.cpp:573
  B200_REQUIRE(f.x || f.seqlen <= kChunk, B200_ERR_NULL, "selscan_bwd: x is required when seqlen > 2048");
  // csrc/selective_scan/selective_scan_cpu.cpp:550
  B200_REQUIRE(!f.z || (f.out && args->dz), B200_ERR_NULL, "selscan_bwd: out and dz are required when z is given");
  B200_REQUIRE(!f.deltaA || args->ddeltaA, B200_ERR_NULL, "selscan_bwd: ddeltaA is required when deltaA is given");
  B200_REQUIRE(!f.D || args->dD, B200_ERR_NULL, "selscan_bwd: dD is required when D is given");
  B200_REQUIRE(!f.delta_bias || args->ddelta_bias, B200_ERR_NULL,
               "selscan_bwd: ddelta_bias is required when delta_bias is given");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (args->h_in || args->q_in) {      // a slice of a sequence-parallel backward: the coverage kernel takes both
    B200_REQUIRE(!f.is_complex, B200_ERR_UNSUPPORTED, "selscan_bwd: h_in / q_in need a real A");
    return selscan_bwd_generic(*args, st);
  }
  if (selscan_bwd_sl_supported(*args)) return selscan_bwd_sl(*args, st);
  if (selscan_bwd_fast_supported(*args)) {
    b200_selscan_bwd_args a = *args;
    if (a.f.stage_len != kFastStage) a.f.stage_h = nullptr;    // states of another spacing: recompute
    return selscan_bwd_fast(a, st);
  }
  return selscan_bwd_generic(*args, st);
}

}  // extern "C"
