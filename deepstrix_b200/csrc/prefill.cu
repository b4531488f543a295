// Prefill-size grouped GEMM on tcgen05.  Not built yet: every batch size runs
// the grouped-GEMV kernels.
#include "prefill.cuh"

namespace dsx {

int prefill_workspace_create(PrefillWorkspace* ws, const dsx_moe_config&) {
    ws->ready = false;
    return DSX_OK;
}
void prefill_workspace_free(PrefillWorkspace*) {}
bool prefill_wanted(const PrefillWorkspace& ws, const dsx_moe_config&, int, int64_t T) { return ws.ready && T >= ws.min_tokens; }
int prefill_forward(PrefillWorkspace*, const dsx_moe_config&, const PrefillCall&, cudaStream_t) {
    return set_error(DSX_ERR_UNSUPPORTED, "prefill path not built");
}

}  // namespace dsx
