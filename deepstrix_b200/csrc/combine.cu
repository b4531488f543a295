// Weighted combine / unpermute: slot-order sum of the per-pick partial rows,
// plus the shared expert's row, written as bf16.
//
// Reference counterparts (paths relative to the deepstrix repository):
//   crates/v4flash-kernels/kernels/q2_k_accumulate_matvec_par.hip:705-766  q2_k_reduce_partials
//       out[b,row] = 0 + p[b,0,row] + ... + p[b,k-1,row] (routing weights already folded into p)
//   crates/v4flash-kernels/src/ffn.rs:118-151  vec_add_inplace: ffn_moe += ffn_shared
// No float atomics: the order of additions is fixed, so the result is reproducible.
#include "dsx_common.cuh"

// One thread per (token, 4 consecutive rows).  Unmangled name: the kernel is also shipped as a stand-alone
// code object (deepstrix_b200/kernels/dsx_combine.cubin) for callers that load kernels through
// dsx_module_load_data / dsx_module_get_function, the way the reference embeds its kernels.
extern "C" __global__ void __launch_bounds__(256)
dsx_combine_kernel(const float* __restrict__ partial, int64_t T, int n_used, int64_t H, int with_shared,
               const int32_t* __restrict__ selected, int expert_lo, int n_local, __nv_bfloat16* __restrict__ out) {
    dsx::pdl_launch_dependents();
    dsx::pdl_wait();   // partial rows come from the down kernel
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t per_row = H >> 2;
    if (gid >= T * per_row) return;
    const int64_t t = gid / per_row, c = gid - t * per_row;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < n_used; s++) {
        if (selected != nullptr) {  // expert-parallel form: picks owned elsewhere were never computed
            const int e = selected[t * n_used + s] - expert_lo;
            if (e < 0 || e >= n_local) continue;
        }
        const float4 p = *(reinterpret_cast<const float4*>(partial + (t * n_used + s) * H) + c);
        acc.x = __fadd_rn(acc.x, p.x);
        acc.y = __fadd_rn(acc.y, p.y);
        acc.z = __fadd_rn(acc.z, p.z);
        acc.w = __fadd_rn(acc.w, p.w);
    }
    if (with_shared) {
        const float4 p = *(reinterpret_cast<const float4*>(partial + (T * n_used + t) * H) + c);
        acc.x = __fadd_rn(acc.x, p.x);
        acc.y = __fadd_rn(acc.y, p.y);
        acc.z = __fadd_rn(acc.z, p.z);
        acc.w = __fadd_rn(acc.w, p.w);
    }
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&lo);
    o.y = *reinterpret_cast<const uint32_t*>(&hi);
    *(reinterpret_cast<uint2*>(out + t * H) + c) = o;
}

namespace dsx {

int launch_combine(const float* partial, int64_t T, int n_used, int64_t H, int with_shared, const int32_t* selected,
                   int expert_lo, int n_local, __nv_bfloat16* out, cudaStream_t stream) {
    DSX_REQUIRE(H % 4 == 0, "combine: hidden must be a multiple of 4");
    if (T == 0) return DSX_OK;
    const int64_t n = T * (H / 4);
    DSX_CUDA(launch_pdl(dsx_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, partial, T, n_used, H, with_shared,
                        selected, expert_lo, n_local, out));
    DSX_LAUNCHED();
    return DSX_OK;
}

}  // namespace dsx
