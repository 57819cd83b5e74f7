#include "launch.cuh"
namespace sd {
int launch_bwd_preprocess(const splitd_params*, cudaStream_t) { return fail(SPLITD_ERR_UNSUPPORTED, "not built yet"); }
int launch_bwd_dq(const splitd_params*, cudaStream_t) { return fail(SPLITD_ERR_UNSUPPORTED, "not built yet"); }
int launch_bwd_dkdv(const splitd_params*, cudaStream_t) { return fail(SPLITD_ERR_UNSUPPORTED, "not built yet"); }
size_t bwd_rowstat_elems(const splitd_params*) { return 0; }
size_t bwd_workspace_bytes(const splitd_params*) { return 0; }
}
