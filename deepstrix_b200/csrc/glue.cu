// The two steps either side of the MoE path: the RMSNorm that produces the layer's input rows and
// the residual mix that consumes its output.
//
// Reference counterparts (paths relative to the deepstrix repository):
//   crates/v4flash-kernels/kernels/rms_norm.hip:12-84   rms_norm_weighted[_batched]
//       out[i] = x[i] * rsqrt(mean(x^2) + eps) * weight[i]; thread t of 256 sums x[t + 256 j]^2 in
//       double, the 256 partials are cast to f32 and folded by a shared-memory tree (stride 128..1)
//       wrapper RmsNorm::launch_weighted_batched, crates/v4flash-kernels/src/rms_norm.rs:161-205
//   crates/v4flash-kernels/kernels/hc_post.hip:15-68    hc_post[_batched]
//       out_hc[dst, d] = block_out[d] * post[dst] + sum_src comb[dst + src * n_hc] * residual_hc[src, d]
//       wrapper crates/v4flash-kernels/src/head.rs:267-372; call het/forward_layer.rs:3130-3152
//
// Both keep the reference's order of operations.  Where the reference's compiler is free to choose
// (rsqrtf, contraction of a * b + c) this file fixes one choice, the same as the CPU oracle:
// 1 / sqrt with IEEE division and square root, and a fused multiply-add per mixing term.
// Here the norm writes the bf16 rows the MoE layer reads (and, optionally, the f32 rows as the
// reference does), and the mix reads the layer's bf16 output directly: one pass over HBM each.
#include <algorithm>
#include <atomic>

#include "dsx_common.cuh"

namespace dsx {
namespace {

constexpr int kNormThreads = 256;
// Error word of the kernels in this file (bit 1: a row's bulk copy never arrived); read and
// cleared by dsx_glue_check.
__device__ uint32_t g_glue_error = 0;

// kNormRegs: values a thread keeps in registers (rows up to 256 * kNormRegs columns are read once; 0 = re-read
// the row).  Instantiated for a few sizes so that a 4096-column row does not pay the registers of an 8192-column one.
template <int kNormRegs>
__global__ void __launch_bounds__(kNormThreads)
rms_norm_rows_kernel(const float* __restrict__ x, const float* __restrict__ weight, int n, float eps, float* __restrict__ out_f32,
                     __nv_bfloat16* __restrict__ out_bf16) {
    __shared__ float sdata[kNormThreads];
    const int tid = threadIdx.x;
    const float* xb = x + (int64_t)blockIdx.x * n;
    constexpr bool in_regs = kNormRegs > 0;
    float v[kNormRegs > 0 ? kNormRegs : 1];
    double partial = 0.0;
    if constexpr (in_regs) {
#pragma unroll
        for (int j = 0; j < kNormRegs; j++) {
            const int i = tid + kNormThreads * j;
            v[j] = i < n ? xb[i] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < kNormRegs; j++)
            if (tid + kNormThreads * j < n) partial += (double)v[j] * (double)v[j];
    } else {
        for (int i = tid; i < n; i += kNormThreads) {
            const float a = xb[i];
            partial += (double)a * (double)a;
        }
    }
    // the reference's tree: sdata[t] += sdata[t + stride] for stride 128, 64, ..., 1.  Strides 128..32 go
    // through shared memory; 16..1 are the same additions as shuffles inside the first warp.
    sdata[tid] = (float)partial;
    __syncthreads();
    if (tid < 128) sdata[tid] = __fadd_rn(sdata[tid], sdata[tid + 128]);
    __syncthreads();
    if (tid < 64) sdata[tid] = __fadd_rn(sdata[tid], sdata[tid + 64]);
    __syncthreads();
    if (tid < 32) {
        float s = __fadd_rn(sdata[tid], sdata[tid + 32]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s = __fadd_rn(s, __shfl_down_sync(0xFFFFFFFFu, s, off));
        if (tid == 0) sdata[0] = s;
    }
    __syncthreads();
    const float mean_sq = __fdiv_rn(sdata[0], (float)n);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, eps)));
    auto emit = [&](int i, float a) {
        const float r = __fmul_rn(__fmul_rn(a, scale), weight[i]);
        if (out_f32 != nullptr) out_f32[(int64_t)blockIdx.x * n + i] = r;
        if (out_bf16 != nullptr) out_bf16[(int64_t)blockIdx.x * n + i] = __float2bfloat16_rn(r);
    };
    if constexpr (in_regs) {
#pragma unroll
        for (int j = 0; j < kNormRegs; j++) {
            const int i = tid + kNormThreads * j;
            if (i < n) emit(i, v[j]);
        }
    } else {
        for (int i = tid; i < n; i += kNormThreads) emit(i, xb[i]);
    }
}

// The same arithmetic at HBM speed: persistent blocks, every block walks rows b, b + grid, ... with two
// row buffers in shared memory; one thread fetches the next row with a bulk async copy (mbarrier
// complete_tx) while the block reduces and stores the current one.  Every thread still takes ITS
// elements (t + 256 j, the reference's assignment) from shared memory, so sums and results are the
// same bits; results go back through the buffer and leave 16 bytes per lane.  The wait on a row is
// bounded; a block whose wait runs out stops (its remaining rows stay unwritten).
__device__ __forceinline__ uint32_t g_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__global__ void __launch_bounds__(kNormThreads)
rms_norm_rows_vec_kernel(const float* __restrict__ x, const float* __restrict__ weight, int n, int64_t T, float eps,
                         float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16) {
    extern __shared__ __align__(16) float sbuf[];   // [2][n]
    __shared__ float sdata[kNormThreads];
    __shared__ __align__(8) uint64_t s_bar[2];
    const int tid = threadIdx.x;
    const uint32_t row_bytes = (uint32_t)n * 4u;
    auto fetch = [&](int64_t r, int b) {   // thread 0
        const uint32_t bar = g_smem_u32(&s_bar[b]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(row_bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         g_smem_u32(sbuf + (size_t)b * n)),
                     "l"(x + r * n), "r"(row_bytes), "r"(bar)
                     : "memory");
    };
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(g_smem_u32(&s_bar[0])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(g_smem_u32(&s_bar[1])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if ((int64_t)blockIdx.x < T) fetch(blockIdx.x, 0);
    }
    __syncthreads();
    int k = 0;
    for (int64_t r = blockIdx.x; r < T; r += gridDim.x, k++) {
        const int b = k & 1;
        if (tid == 0 && r + gridDim.x < T) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the other buffer was last written by this block's threads
            fetch(r + gridDim.x, b ^ 1);
        }
        {   // bounded wait for this row
            const uint32_t bar = g_smem_u32(&s_bar[b]), parity = (uint32_t)((k >> 1) & 1);
            uint32_t ok = 0;
            for (uint32_t i = 0; i < (1u << 22) && !ok; i++)
                asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                             : "=r"(ok)
                             : "r"(bar), "r"(parity)
                             : "memory");
            if (!ok) {   // the row never arrived: report it and stop (this block's remaining rows stay unwritten)
                if (tid == 0) atomicOr(&g_glue_error, 1u);
                return;
            }
        }
        float* srow = sbuf + (size_t)b * n;
        double partial = 0.0;
        for (int i = tid; i < n; i += kNormThreads) {
            const float a = srow[i];
            partial += (double)a * (double)a;
        }
        sdata[tid] = (float)partial;
        __syncthreads();
        if (tid < 128) sdata[tid] = __fadd_rn(sdata[tid], sdata[tid + 128]);
        __syncthreads();
        if (tid < 64) sdata[tid] = __fadd_rn(sdata[tid], sdata[tid + 64]);
        __syncthreads();
        if (tid < 32) {
            float s = __fadd_rn(sdata[tid], sdata[tid + 32]);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) s = __fadd_rn(s, __shfl_down_sync(0xFFFFFFFFu, s, off));
            if (tid == 0) sdata[0] = s;
        }
        __syncthreads();
        const float mean_sq = __fdiv_rn(sdata[0], (float)n);
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, eps)));
        for (int i = tid; i < n; i += kNormThreads) srow[i] = __fmul_rn(__fmul_rn(srow[i], scale), __ldg(weight + i));   // own elements only
        __syncthreads();
        if (out_f32 != nullptr) {
            float4* o4 = reinterpret_cast<float4*>(out_f32 + r * n);
            for (int i = tid; i < (n >> 2); i += kNormThreads) o4[i] = reinterpret_cast<const float4*>(srow)[i];
        }
        if (out_bf16 != nullptr) {
            uint4* o8 = reinterpret_cast<uint4*>(out_bf16 + r * n);
            for (int i = tid; i < (n >> 3); i += kNormThreads) {
                const float4 a = reinterpret_cast<const float4*>(srow)[2 * i], c = reinterpret_cast<const float4*>(srow)[2 * i + 1];
                const __nv_bfloat162 h0 = __floats2bfloat162_rn(a.x, a.y), h1 = __floats2bfloat162_rn(a.z, a.w);
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(c.x, c.y), h3 = __floats2bfloat162_rn(c.z, c.w);
                uint4 o;
                o.x = *reinterpret_cast<const uint32_t*>(&h0); o.y = *reinterpret_cast<const uint32_t*>(&h1);
                o.z = *reinterpret_cast<const uint32_t*>(&h2); o.w = *reinterpret_cast<const uint32_t*>(&h3);
                o8[i] = o;
            }
        }
        __syncthreads();   // everyone is done with this buffer (and with sdata) before it is fetched into again
    }
}

// One thread per (token, destination stream, column): any number of streams.
template <bool BF16_IN>
__global__ void __launch_bounds__(256)
hc_post_kernel(const void* __restrict__ block_out, const float* __restrict__ residual_hc, const float* __restrict__ post,
               const float* __restrict__ comb, int n_embd, int n_hc, float* __restrict__ out_hc) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= n_embd) return;
    const int dst = blockIdx.y;
    const int64_t b = blockIdx.z;
    float bo;
    if (BF16_IN) bo = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(block_out)[b * n_embd + d]);
    else bo = reinterpret_cast<const float*>(block_out)[b * n_embd + d];
    const float* rh = residual_hc + b * n_hc * n_embd;
    const float* cb = comb + b * n_hc * n_hc;
    float acc = __fmul_rn(bo, post[b * n_hc + dst]);
    for (int src = 0; src < n_hc; src++) acc = __fmaf_rn(cb[dst + src * n_hc], rh[(int64_t)src * n_embd + d], acc);
    out_hc[(b * n_hc + dst) * n_embd + d] = acc;
}

// The reference's four streams: one thread per (token, 4 columns) reads every residual stream once
// (16-byte loads) and writes all four destinations.  Same operations per element as above.
template <bool BF16_IN>
__global__ void __launch_bounds__(256)
hc_post4_kernel(const void* __restrict__ block_out, const float* __restrict__ residual_hc, const float* __restrict__ post,
                const float* __restrict__ comb, int n_embd, int64_t n_tok, float* __restrict__ out_hc) {
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_row = n_embd >> 2;
    if (gid >= n_tok * per_row) return;
    const int64_t b = gid / per_row;
    const int c = (int)(gid - b * per_row);
    float bo[4];
    if (BF16_IN) {
        const uint2 v = *(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(block_out) + b * n_embd) + c);
        bo[0] = __uint_as_float(v.x << 16); bo[1] = __uint_as_float(v.x & 0xFFFF0000u);
        bo[2] = __uint_as_float(v.y << 16); bo[3] = __uint_as_float(v.y & 0xFFFF0000u);
    } else {
        const float4 v = *(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(block_out) + b * n_embd) + c);
        bo[0] = v.x; bo[1] = v.y; bo[2] = v.z; bo[3] = v.w;
    }
    float4 r[4];
#pragma unroll
    for (int src = 0; src < 4; src++) r[src] = *(reinterpret_cast<const float4*>(residual_hc + (b * 4 + src) * n_embd) + c);
    const float* cb = comb + b * 16;
#pragma unroll
    for (int dst = 0; dst < 4; dst++) {
        const float p = post[b * 4 + dst];
        float a[4];
#pragma unroll
        for (int i = 0; i < 4; i++) a[i] = __fmul_rn(bo[i], p);
#pragma unroll
        for (int src = 0; src < 4; src++) {
            const float k = cb[dst + src * 4];
            a[0] = __fmaf_rn(k, r[src].x, a[0]);
            a[1] = __fmaf_rn(k, r[src].y, a[1]);
            a[2] = __fmaf_rn(k, r[src].z, a[2]);
            a[3] = __fmaf_rn(k, r[src].w, a[3]);
        }
        *(reinterpret_cast<float4*>(out_hc + (b * 4 + dst) * n_embd) + c) = make_float4(a[0], a[1], a[2], a[3]);
    }
}

}  // namespace
}  // namespace dsx

using namespace dsx;

extern "C" {

int dsx_rms_norm_rows(const float* x, const float* weight, int64_t T, int64_t n, float eps, float* out_f32, void* out_bf16,
                      dsx_stream_t stream) {
    DSX_REQUIRE(T >= 0 && n >= 1 && n <= (1 << 30), "rms_norm_rows: %lld rows of %lld columns", (long long)T, (long long)n);
    if (T == 0) return DSX_OK;
    DSX_REQUIRE(x && weight && (out_f32 || out_bf16), "rms_norm_rows: null argument");
    DSX_REQUIRE(T <= 0x7FFFFFFF, "rms_norm_rows: too many rows");
    const bool vec = n % 8 == 0 && n * 8 <= 96 * 1024 && (((uintptr_t)x | (uintptr_t)out_f32 | (uintptr_t)out_bf16) & 15) == 0;
    if (vec) {
        // persistent grid: a few blocks per SM.  The opt-in to 96 KB of shared memory is a per-device
        // setting, so it is made (and the SM count read) once for every device this entry point meets.
        constexpr int kMaxDevices = 64;
        static std::atomic<int> sm_counts[kMaxDevices];
        int dev = 0;
        DSX_CUDA(cudaGetDevice(&dev));
        DSX_REQUIRE(dev >= 0 && dev < kMaxDevices, "rms_norm_rows: device index %d out of range", dev);
        int sm_count = sm_counts[dev].load(std::memory_order_acquire);
        if (sm_count == 0) {
            DSX_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
            DSX_CUDA(cudaFuncSetAttribute(rms_norm_rows_vec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
            sm_counts[dev].store(sm_count, std::memory_order_release);
        }
        const size_t smem = (size_t)n * 8;
        const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(6, (200 * 1024) / (smem + 2048)));
        const unsigned blocks = (unsigned)std::min<int64_t>(T, (int64_t)sm_count * per_sm);
        rms_norm_rows_vec_kernel<<<blocks, kNormThreads, smem, (cudaStream_t)stream>>>(x, weight, (int)n, T, eps, out_f32, (__nv_bfloat16*)out_bf16);
        DSX_LAUNCHED();
        return DSX_OK;
    }
    const int per_thread = (int)((n + kNormThreads - 1) / kNormThreads);
#define DSX_NORM_LAUNCH(R) rms_norm_rows_kernel<R><<<(unsigned)T, kNormThreads, 0, (cudaStream_t)stream>>>(x, weight, (int)n, eps, out_f32, (__nv_bfloat16*)out_bf16)
    if (per_thread <= 8) DSX_NORM_LAUNCH(8);
    else if (per_thread <= 16) DSX_NORM_LAUNCH(16);
    else if (per_thread <= 24) DSX_NORM_LAUNCH(24);
    else if (per_thread <= 32) DSX_NORM_LAUNCH(32);
    else DSX_NORM_LAUNCH(0);
#undef DSX_NORM_LAUNCH
    DSX_LAUNCHED();
    return DSX_OK;
}

int dsx_glue_check(dsx_stream_t stream_, uint32_t* error_word) {
    cudaStream_t stream = (cudaStream_t)stream_;
    uint32_t w = 0;
    DSX_CUDA(cudaMemcpyFromSymbolAsync(&w, g_glue_error, 4, 0, cudaMemcpyDeviceToHost, stream));
    DSX_CUDA(cudaStreamSynchronize(stream));
    if (w) {
        const uint32_t zero = 0;
        DSX_CUDA(cudaMemcpyToSymbolAsync(g_glue_error, &zero, 4, 0, cudaMemcpyHostToDevice, stream));
        DSX_CUDA(cudaStreamSynchronize(stream));
    }
    if (error_word) *error_word = w;
    if (w) return set_error(DSX_ERR_DEVICE, "a norm / residual-mix kernel reported error word 0x%x (a bounded wait ran out)", w);
    return DSX_OK;
}

int dsx_hc_post(const void* block_out, int block_out_is_bf16, const float* residual_hc, const float* post, const float* comb, int64_t T,
                int64_t n_embd, int n_hc, float* out_hc, dsx_stream_t stream) {
    DSX_REQUIRE(T >= 0 && n_embd >= 1 && n_hc >= 1 && n_hc <= 65535, "hc_post: %lld tokens, %lld columns, %d streams", (long long)T,
                (long long)n_embd, n_hc);
    if (T == 0) return DSX_OK;
    DSX_REQUIRE(block_out && residual_hc && post && comb && out_hc, "hc_post: null argument");
    const bool vec = n_hc == 4 && n_embd % 4 == 0 && (((uintptr_t)block_out | (uintptr_t)residual_hc | (uintptr_t)out_hc) & 15) == 0;
    if (vec) {
        const int64_t nthr = T * (n_embd / 4);
        const unsigned blocks = (unsigned)((nthr + 255) / 256);
        if (block_out_is_bf16)
            hc_post4_kernel<true><<<blocks, 256, 0, (cudaStream_t)stream>>>(block_out, residual_hc, post, comb, (int)n_embd, T, out_hc);
        else
            hc_post4_kernel<false><<<blocks, 256, 0, (cudaStream_t)stream>>>(block_out, residual_hc, post, comb, (int)n_embd, T, out_hc);
        DSX_LAUNCHED();
        return DSX_OK;
    }
    DSX_REQUIRE(T <= 65535, "hc_post: at most 65535 tokens per call unless n_hc == 4 with 16-byte aligned rows");
    const dim3 grid((unsigned)((n_embd + 255) / 256), (unsigned)n_hc, (unsigned)T);
    if (block_out_is_bf16)
        hc_post_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(block_out, residual_hc, post, comb, (int)n_embd, n_hc, out_hc);
    else
        hc_post_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(block_out, residual_hc, post, comb, (int)n_embd, n_hc, out_hc);
    DSX_LAUNCHED();
    return DSX_OK;
}

}  // extern "C"
