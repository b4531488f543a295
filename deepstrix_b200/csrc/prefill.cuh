// Prefill-size grouped GEMM on tcgen05 (interface used by api.cu).
#pragma once
#include <cuda.h>

#include "dsx_common.cuh"

namespace dsx {

struct PrefillSeg {   // a run of <= 256 expert-sorted token rows of one expert
    int32_t expert;   // local slot, or n_local for the shared expert
    int32_t row0;     // first row in the sorted activation / mid buffers
    int32_t n;        // rows
    int32_t pad;
};

struct PrefillWorkspace {
    bool ready = false;
    int min_tokens = 1 << 30;  // batches of at least this many tokens take the tensor-core path
    int64_t cap_rows = 0;      // rows of xperm / mid the tensor maps cover
    int64_t H = 0, F = 0;
    int fmt = DSX_FMT_MXFP4;   // format of the stores the weight maps describe
    __half* xperm = nullptr;   // [cap_rows, H] f16: token rows in expert-sorted order, then all tokens (shared expert); null until a store needs it
    PrefillSeg* segs = nullptr;
    int32_t* n_segs = nullptr;
    int32_t seg_cap = 0;
    int small_max = 0;         // experts with at most this many rows go to the grouped GEMV instead (0: none)
    int32_t* small_items = nullptr;   // their work items (expert << 16 | first member), one per expert
    int32_t* n_small = nullptr;
    CUtensorMap tmap_x[4];     // xperm as [cap_rows, H], boxes of 64 columns x 64 / 128 / 192 / 256 rows, 128-byte swizzle
    CUtensorMap tmap_mid[4];   // mid   as [cap_rows, F]
    // packed-weight planes as 4-D tensors [slot][row tile][column tile][bytes as u32]; index 0 routed, 1 shared
    CUtensorMap tmap_gu_nib[2], tmap_gu_sc[2], tmap_dn_nib[2], tmap_dn_sc[2];
    const void* mapped_gu_nib[2] = {nullptr, nullptr};   // planes the maps above were encoded for
    const void* mapped_dn_nib[2] = {nullptr, nullptr};
    // ---- block-scaled MXFP4 path (prefill_mx.cu)
    bool mx_ready = false;
    uint8_t* xq = nullptr;          // [3 terms][cap_rows][K/2]: the sorted rows (then mid) as packed E2M1 terms
    int64_t mx_term_stride = 0;     // bytes between terms
    uint8_t* sfb = nullptr;         // their block scales: [segment][K/128][term][512]
    int32_t* mx_inv_perm = nullptr; // [max_tokens * n_used]: expert-sorted position of every pick (-1: not placed here)
    PrefillSeg* mx_segs = nullptr;  // segments of at most 192 rows
    int32_t mx_seg_cap = 0;
    int mx_pair_mode = -1;          // the block-scaled GEMMs as CTA pairs: -1 decided per call, 0 never, 1 always
    CUtensorMap tmap_xq2[3], tmap_mq2[3]; // the same for CTA pairs: boxes of 32 / 64 / 96 rows (half a segment per CTA)
    CUtensorMap tmap_xq[3], tmap_mq[3];   // xq as (bytes, row, term) for K = hidden / K = ffn, boxes of 64 / 128 / 192 rows
    CUtensorMap tmap_km_gu[2], tmap_km_dn[2];            // K-major code planes; index 0 routed, 1 shared
    const void* mapped_km_gu[2] = {nullptr, nullptr};
    const void* mapped_km_dn[2] = {nullptr, nullptr};
    int mapped_km_slots[2] = {0, 0};
};

struct PrefillCall {
    const __nv_bfloat16* x;
    int64_t T;
    const int32_t* selected;
    const float* route_w;
    int expert_lo, n_local;
    bool filter_picks, with_shared;
    bool skip_combine;         // stop after the partial rows (the caller reduces them)
    __nv_bfloat16* out;
    __nv_bfloat16* const* out_rows;   // optional: where each row of the result goes instead of out (null entries: nowhere)
    int32_t *hist, *offsets, *perm;
    GroupScratch gs;
    __half* mid;
    float* partial;
    uint32_t* error_word;
    int sm_count;
    int n_used;
    int fmt;
    float clamp;
    const uint8_t *gu_nib, *gu_sc, *dn_nib, *dn_sc;
    int64_t gu_nib_stride, gu_sc_stride, dn_nib_stride, dn_sc_stride;
    const uint8_t *sh_gu_nib, *sh_gu_sc, *sh_dn_nib, *sh_dn_sc;
    // tensor-core planes of an MXFP4 store (null otherwise)
    const uint8_t *km_gu, *km_dn, *sf_gu, *sf_dn;
    int64_t km_gu_stride, km_dn_stride, sf_gu_stride, sf_dn_stride;
    const uint8_t *sh_km_gu, *sh_km_dn, *sh_sf_gu, *sh_sf_dn;
};

// f16_rows: allocate the f16 copy of the sorted rows now (stores that take the f16-operand kernels)
int prefill_workspace_create(PrefillWorkspace* ws, const dsx_moe_config& cfg, int n_used, __half* mid, bool f16_rows);
int prefill_f16_rows_ensure(PrefillWorkspace* ws);   // allocates that copy if it is missing (not during a capture)
void prefill_workspace_free(PrefillWorkspace* ws);
bool prefill_wanted(const PrefillWorkspace& ws, const dsx_moe_config& cfg, int fmt, int64_t T);
int prefill_forward(PrefillWorkspace* ws, const dsx_moe_config& cfg, const PrefillCall& call, cudaStream_t stream);
// shared by the two tensor-core files
int tmap_encode(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const cuuint64_t* dims, const cuuint64_t* strides,
                const cuuint32_t* box, CUtensorMapSwizzle swizzle);
int launch_build_segments(const int32_t* offsets, int n_local, int64_t P, int T_shared, int seg_rows, PrefillSeg* segs, int32_t* n_segs,
                          int cap, int small_max, int32_t* small_items, int32_t* n_small, cudaStream_t stream);
// block-scaled MXFP4 path (prefill_mx.cu); the workspace must have been through prefill_workspace_create
int prefill_mx_workspace_create(PrefillWorkspace* ws, const dsx_moe_config& cfg, int n_used);
void prefill_mx_workspace_free(PrefillWorkspace* ws);
int prefill_mx_forward(PrefillWorkspace* ws, const dsx_moe_config& cfg, const PrefillCall& call, cudaStream_t stream);

}  // namespace dsx
