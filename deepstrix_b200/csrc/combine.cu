// Weighted combine / unpermute: slot-order sum of the per-pick partial rows,
// plus the shared expert's row, written as bf16.
//
// Reference counterparts (paths relative to the deepstrix repository):
//   crates/v4flash-kernels/kernels/q2_k_accumulate_matvec_par.hip:705-766  q2_k_reduce_partials
//       out[b,row] = 0 + p[b,0,row] + ... + p[b,k-1,row] (routing weights already folded into p)
//   crates/v4flash-kernels/src/ffn.rs:118-151  vec_add_inplace: ffn_moe += ffn_shared
// No float atomics: the order of additions is fixed, so the result is reproducible.
#include "dsx_common.cuh"

// One thread per (token, 8 consecutive columns), grid-stride (any grid covers the batch).  Unmangled name: the kernel
// is also shipped as a stand-alone code object (deepstrix_b200/kernels/dsx_combine.cubin) for callers that load kernels
// through dsx_module_load_data / dsx_module_get_function, the way the reference embeds its kernels.
// A thread requests four partial rows at a time (a rolled load-add loop issues one load per round trip), and which
// picks count is decided once per warp: a warp lies inside one token's row whenever hidden is a multiple of 256.
// out_rows (optional, [T] row pointers) replaces out: rows are stored where the table points, null entries skipped.
extern "C" __global__ void __launch_bounds__(256)
dsx_combine_kernel(const float* __restrict__ partial, int64_t T, int n_used, int64_t H, int with_shared,
               const int32_t* __restrict__ selected, int expert_lo, int n_local, __nv_bfloat16* __restrict__ out,
               __nv_bfloat16* const* __restrict__ out_rows) {
    dsx::pdl_launch_dependents();
    dsx::pdl_wait();   // partial rows come from the down kernel
    const int64_t per_row = H >> 3, total = T * per_row;
    const bool warp_in_row = (per_row & 31) == 0;
    for (int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < total; gid += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = gid / per_row, c = gid - t * per_row;
        // where the row goes: out[t], or (out_rows given) wherever the table says -- another GPU's memory included, which is how an
        // expert-parallel owner hands its partial rows back without a copy pass -- and nowhere for a null entry
        __nv_bfloat16* dst = out_rows != nullptr ? out_rows[t] : out + t * H;
        if (dst == nullptr) continue;
        // bit s: pick s of the token counts (expert-parallel form: picks owned elsewhere were never computed)
        uint32_t mask = n_used >= 32 ? 0xFFFFFFFFu : (1u << n_used) - 1u;
        if (selected != nullptr) {
            if (warp_in_row) {   // the warp's 32 threads share the token: lane s looks at pick s
                const int lane = threadIdx.x & 31;
                bool own = false;
                if (lane < n_used) {
                    const int e = selected[t * n_used + lane] - expert_lo;
                    own = e >= 0 && e < n_local;
                }
                mask = __ballot_sync(0xFFFFFFFFu, own);
            } else {
                mask = 0u;
                for (int s = 0; s < n_used; s++) {
                    const int e = selected[t * n_used + s] - expert_lo;
                    if (e >= 0 && e < n_local) mask |= 1u << s;
                }
            }
        }
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] = 0.f;
        const float4* base = reinterpret_cast<const float4*>(partial + t * n_used * H) + 2 * c;
        const int64_t row4 = H >> 2;   // float4 per partial row
        auto add8 = [&](const float4& a, const float4& b) {
            acc[0] = __fadd_rn(acc[0], a.x); acc[1] = __fadd_rn(acc[1], a.y); acc[2] = __fadd_rn(acc[2], a.z); acc[3] = __fadd_rn(acc[3], a.w);
            acc[4] = __fadd_rn(acc[4], b.x); acc[5] = __fadd_rn(acc[5], b.y); acc[6] = __fadd_rn(acc[6], b.z); acc[7] = __fadd_rn(acc[7], b.w);
        };
        // the counted picks in slot order, four rows requested at a time
        for (uint32_t m = mask; m != 0u;) {
            int s[4];
            bool ok[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                ok[j] = m != 0u;
                s[j] = ok[j] ? __ffs(m) - 1 : 0;
                m &= m - 1u;   // (0 stays 0)
            }
            float4 va[4], vb[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float4* p = base + (int64_t)s[j] * row4;
                va[j] = ok[j] ? p[0] : make_float4(0.f, 0.f, 0.f, 0.f);
                vb[j] = ok[j] ? p[1] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (ok[j]) add8(va[j], vb[j]);
        }
        if (with_shared) {
            const float4* p = reinterpret_cast<const float4*>(partial + (T * n_used + t) * H) + 2 * c;
            add8(p[0], p[1]);
        }
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            ow[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *(reinterpret_cast<uint4*>(dst) + c) = o;
    }
}

namespace dsx {

int launch_combine(const float* partial, int64_t T, int n_used, int64_t H, int with_shared, const int32_t* selected,
                   int expert_lo, int n_local, __nv_bfloat16* out, cudaStream_t stream, __nv_bfloat16* const* out_rows) {
    DSX_REQUIRE(H % 8 == 0, "combine: hidden must be a multiple of 8");
    if (T == 0) return DSX_OK;
    const int64_t n = T * (H / 8);
    DSX_CUDA(launch_pdl(dsx_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, partial, T, n_used, H, with_shared,
                        selected, expert_lo, n_local, out, out_rows));
    DSX_LAUNCHED();
    return DSX_OK;
}

}  // namespace dsx
