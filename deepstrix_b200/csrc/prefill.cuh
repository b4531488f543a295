// Prefill-size grouped GEMM on tcgen05 (interface used by api.cu).
#pragma once
#include "dsx_common.cuh"

namespace dsx {

struct PrefillWorkspace {
    bool ready = false;
    int min_tokens = 1 << 30;  // batches of at least this many tokens take the tensor-core path
};

struct PrefillCall {
    const __nv_bfloat16* x;
    int64_t T;
    const int32_t* selected;
    const float* route_w;
    int expert_lo, n_local;
    bool filter_picks, with_shared;
    __nv_bfloat16* out;
    int32_t *hist, *offsets, *perm, *work_items, *n_work_items;
    int32_t work_cap;
    GroupScratch gs;
    float* partial;
    uint32_t* error_word;
    int sm_count;
    int fmt;
    const uint8_t *gu_nib, *gu_sc, *dn_nib, *dn_sc;
    int64_t gu_nib_stride, gu_sc_stride, dn_nib_stride, dn_sc_stride;
    const uint8_t *sh_gu_nib, *sh_gu_sc, *sh_dn_nib, *sh_dn_sc;
};

int prefill_workspace_create(PrefillWorkspace* ws, const dsx_moe_config& cfg);
void prefill_workspace_free(PrefillWorkspace* ws);
bool prefill_wanted(const PrefillWorkspace& ws, const dsx_moe_config& cfg, int fmt, int64_t T);
int prefill_forward(PrefillWorkspace* ws, const dsx_moe_config& cfg, const PrefillCall& call, cudaStream_t stream);

}  // namespace dsx
