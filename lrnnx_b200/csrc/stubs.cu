// Entry points not implemented yet.
#include "common.cuh"
extern "C" {
int b200_selscan_fixup(const b200_selscan_fixup_args *, void *) { b200::set_error("not implemented"); return B200_ERR_UNSUPPORTED; }
}
