// Stand-alone element-wise operators of the expert path that a caller may launch by itself instead of the
// whole-layer call: Q8_K activation quantise, weighted clamp + SwiGLU, in-place vector add, indexed gather.
// All four stream their operands once (HBM-bound; grids of whole waves of the device's SMs, 16-byte accesses
// where the layout allows them).
#include "dsx_common.cuh"

namespace dsx {
namespace {

constexpr int kQ8kBlock = 256;       // values per Q8_K block
constexpr int kQ8kBytes = 292;       // f32 d | i8 qs[256] | i16 bsums[16]

// One warp per block of 256 values; lane L holds values 8L .. 8L+7.
// Which of several equal |x| supplies the sign of the scale follows the reference kernel's reduction tree
// (stride 128 .. 1, the upper element taken only when strictly larger): among the largest |x| the winner is the
// index whose 8 bits, reversed, form the smallest number.
__global__ void __launch_bounds__(256)
q8_k_quantize_kernel(const float* __restrict__ x, int64_t n_blocks, uint8_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * 8;
    for (int64_t b = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); b < n_blocks; b += warps) {
        const float4* in = reinterpret_cast<const float4*>(x + b * kQ8kBlock) + 2 * lane;
        const float4 lo = __ldg(in), hi = __ldg(in + 1);
        const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        uint8_t* blk = out + b * kQ8kBytes;
        if (amax == 0.0f) {
            for (int i = lane; i < kQ8kBytes / 4; i += 32) reinterpret_cast<uint32_t*>(blk)[i] = 0u;
            continue;
        }
        uint32_t best = 256u;     // smallest reversed index among this lane's values that reach amax
        float signed_max = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t rev = __brev((uint32_t)(8 * lane + j)) >> 24;
            if (fabsf(v[j]) == amax && rev < best) { best = rev; signed_max = v[j]; }
        }
        uint32_t win = best;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) win = min(win, __shfl_xor_sync(0xFFFFFFFFu, win, o));
        const int owner = __ffs(__ballot_sync(0xFFFFFFFFu, best == win)) - 1;
        const float mxv = __shfl_sync(0xFFFFFFFFu, signed_max, owner);
        const float iscale = __fdiv_rn(-127.0f, mxv);
        int sum = 0;
        uint32_t packed[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 8; j++) {
            int q = (int)rintf(__fmul_rn(iscale, v[j]));
            q = max(-128, min(127, q));
            sum += q;
            packed[j >> 2] |= (uint32_t)(q & 0xFF) << (8 * (j & 3));
        }
        uint32_t* qs = reinterpret_cast<uint32_t*>(blk + 4) + 2 * lane;   // blocks are 4-byte aligned (292 = 4 * 73)
        qs[0] = packed[0];
        qs[1] = packed[1];
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);                      // 16 values = two lanes
        if ((lane & 1) == 0) reinterpret_cast<int16_t*>(blk + 260)[lane >> 1] = (int16_t)sum;
        if (lane == 0) *reinterpret_cast<float*>(blk) = __fdiv_rn(1.0f, iscale);
    }
}

// mid[e, r] = silu(min(gate, c)) * clamp(up, -c, c) * expert_w[e]; the exponential is the deterministic one the
// routers use (IEEE add / mul / fma only), so a CPU restatement gives the same bits.
__global__ void __launch_bounds__(256)
swiglu_clamp_weighted_kernel(float* __restrict__ mid, const float* __restrict__ gate, const float* __restrict__ up,
                             const float* __restrict__ expert_w, float clamp, int64_t ff_exp, int64_t n_experts) {
    const int64_t n4 = ff_exp >> 2, total4 = n4 * n_experts;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total4; i += (int64_t)gridDim.x * 256) {
        const float w = __ldg(expert_w + i / n4);
        const float4 g4 = __ldg(reinterpret_cast<const float4*>(gate) + i), u4 = __ldg(reinterpret_cast<const float4*>(up) + i);
        float g[4] = {g4.x, g4.y, g4.z, g4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w}, m[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (clamp > 1.0e-6f) {
                g[j] = fminf(g[j], clamp);
                u[j] = fminf(fmaxf(u[j], -clamp), clamp);
            }
            const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, det_expf(-g[j])));
            m[j] = __fmul_rn(__fmul_rn(__fmul_rn(g[j], sig), u[j]), w);
        }
        reinterpret_cast<float4*>(mid)[i] = make_float4(m[0], m[1], m[2], m[3]);
    }
}

__global__ void __launch_bounds__(256)
vec_add_inplace_kernel(float* __restrict__ out, const float* __restrict__ rhs, int64_t n, bool vec) {
    const int64_t stride = (int64_t)gridDim.x * 256, i0 = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (vec) {
        for (int64_t i = i0; i < (n >> 2); i += stride) {
            float4 a = reinterpret_cast<float4*>(out)[i];
            const float4 b = __ldg(reinterpret_cast<const float4*>(rhs) + i);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            reinterpret_cast<float4*>(out)[i] = a;
        }
        for (int64_t i = (n & ~(int64_t)3) + i0; i < n; i += stride) out[i] += rhs[i];
    } else {
        for (int64_t i = i0; i < n; i += stride) out[i] += rhs[i];
    }
}

__global__ void __launch_bounds__(256)
gather_f32_kernel(float* __restrict__ out, const float* __restrict__ src, const int32_t* __restrict__ idx, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
        const int32_t j = __ldg(idx + i);
        out[i] = j >= 0 ? __ldg(src + j) : -INFINITY;
    }
}

// whole waves of the device's SMs (8 resident blocks of 256 threads each), no more blocks than there is work
int grid_for(int64_t work_items_of_256, unsigned* blocks) {
    int dev = 0, sms = 0;
    DSX_CUDA(cudaGetDevice(&dev));
    DSX_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t cap = (int64_t)sms * 8;
    *blocks = (unsigned)(work_items_of_256 < cap ? (work_items_of_256 < 1 ? 1 : work_items_of_256) : cap);
    return DSX_OK;
}

}  // namespace
}  // namespace dsx

using namespace dsx;

extern "C" {

int dsx_q8_k_quantize(const float* x, int64_t n_blocks, void* out, dsx_stream_t stream) {
    DSX_REQUIRE(n_blocks >= 0, "q8_k_quantize: %lld blocks", (long long)n_blocks);
    if (n_blocks == 0) return DSX_OK;
    DSX_REQUIRE(x && out, "q8_k_quantize: null argument");
    DSX_REQUIRE((((uintptr_t)x & 15) | ((uintptr_t)out & 3)) == 0, "q8_k_quantize: x must be 16-byte and out 4-byte aligned");
    unsigned blocks;
    if (int rc = grid_for((n_blocks + 7) / 8, &blocks)) return rc;
    q8_k_quantize_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, n_blocks, (uint8_t*)out);
    DSX_LAUNCHED();
    return DSX_OK;
}

int dsx_swiglu_clamp_weighted(float* mid, const float* gate, const float* up, const float* expert_w, float clamp, int64_t ff_exp,
                              int64_t n_experts, dsx_stream_t stream) {
    DSX_REQUIRE(ff_exp >= 0 && n_experts >= 0 && ff_exp % 4 == 0, "swiglu_clamp_weighted: %lld experts of %lld rows (a multiple of 4)",
                (long long)n_experts, (long long)ff_exp);
    if (ff_exp == 0 || n_experts == 0) return DSX_OK;
    DSX_REQUIRE(mid && gate && up && expert_w, "swiglu_clamp_weighted: null argument");
    DSX_REQUIRE((((uintptr_t)mid | (uintptr_t)gate | (uintptr_t)up) & 15) == 0, "swiglu_clamp_weighted: rows must be 16-byte aligned");
    unsigned blocks;
    if (int rc = grid_for((ff_exp / 4 * n_experts + 255) / 256, &blocks)) return rc;
    swiglu_clamp_weighted_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(mid, gate, up, expert_w, clamp, ff_exp, n_experts);
    DSX_LAUNCHED();
    return DSX_OK;
}

int dsx_vec_add_inplace(float* out, const float* rhs, int64_t n, dsx_stream_t stream) {
    DSX_REQUIRE(n >= 0, "vec_add_inplace: %lld elements", (long long)n);
    if (n == 0) return DSX_OK;
    DSX_REQUIRE(out && rhs, "vec_add_inplace: null argument");
    const bool vec = (((uintptr_t)out | (uintptr_t)rhs) & 15) == 0;
    unsigned blocks;
    if (int rc = grid_for(((vec ? n / 4 + 3 : n) + 255) / 256, &blocks)) return rc;
    vec_add_inplace_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(out, rhs, n, vec);
    DSX_LAUNCHED();
    return DSX_OK;
}

int dsx_gather_f32(float* out, const float* src, const int32_t* idx, int64_t n, dsx_stream_t stream) {
    DSX_REQUIRE(n >= 0, "gather_f32: %lld elements", (long long)n);
    if (n == 0) return DSX_OK;
    DSX_REQUIRE(out && src && idx, "gather_f32: null argument");
    unsigned blocks;
    if (int rc = grid_for((n + 255) / 256, &blocks)) return rc;
    gather_f32_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(out, src, idx, n);
    DSX_LAUNCHED();
    return DSX_OK;
}

}  // extern "C"
