// Entry points not implemented yet.
#include "common.cuh"
extern "C" {
int b200_selscan_fixup(const b200_selscan_fixup_args *, void *) { b200::set_error("not implemented"); return B200_ERR_UNSUPPORTED; }
int b200_simpscan_fwd(const b200_simpscan_args *, void *) { b200::set_error("not implemented"); return B200_ERR_UNSUPPORTED; }
int b200_simpscan_bwd(const b200_simpscan_args *, void *) { b200::set_error("not implemented"); return B200_ERR_UNSUPPORTED; }
int b200_ssu_step(const b200_ssu_args *, void *) { b200::set_error("not implemented"); return B200_ERR_UNSUPPORTED; }
int b200_cauchy_fwd(const b200_s4_args *, void *) { b200::set_error("not implemented"); return B200_ERR_UNSUPPORTED; }
int b200_cauchy_bwd(const b200_s4_args *, void *) { b200::set_error("not implemented"); return B200_ERR_UNSUPPORTED; }
int b200_vand_fwd(const b200_s4_args *, void *) { b200::set_error("not implemented"); return B200_ERR_UNSUPPORTED; }
int b200_vand_bwd(const b200_s4_args *, void *) { b200::set_error("not implemented"); return B200_ERR_UNSUPPORTED; }
}
