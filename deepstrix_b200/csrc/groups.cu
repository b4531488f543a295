// Token -> expert histogram, offsets, stable permutation and work items.
//
// Reference counterparts (paths relative to the deepstrix repository):
//   crates/v4flash-kernels/kernels/expert_sel_count.hip:17-28     histogram
//   crates/v4flash-kernels/kernels/moe_group_builder.hip:32-51     group inversion (atomic order)
//   crates/v4flash-kernels/kernels/moe_work_items_builder.hip:61-145  prefix sum + work items sorted by expert
//   crates/v4flash-kernels/kernels/b2_fast_chain.hip:46-128        fused single-block builder with the
//                                                                  deterministic (token, slot) member order
// The reference's atomic builder leaves member order unspecified; this one is a
// stable counting sort, so hist, offsets AND perm are reproducible bit for bit:
// warp ballots (match_any) rank equal experts inside a 32-pick step, per-warp
// and per-block prefix sums order the steps.
#include <mutex>

#include "groups.cuh"

namespace dsx {
namespace {

using namespace groupdev;
constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxExperts = 512;

// Single block: T*k <= kGroupChunk.
__global__ void __launch_bounds__(kThreads)
group_build_small_kernel(const int32_t* __restrict__ sel, int64_t P, int E, int lo, int chunk, int shared_T,
                         int32_t* hist, int32_t* offsets, int32_t* perm, int32_t* work_items, int32_t* n_work_items,
                         int32_t work_cap) {
    extern __shared__ int wh[];
    __shared__ int s_warp[kWarps + 1];
    build_small<kThreads>(sel, P, E, lo, chunk, shared_T, hist, offsets, perm, work_items, n_work_items, work_cap, wh, s_warp);
}

__global__ void __launch_bounds__(kThreads)
group_count_kernel(const int32_t* __restrict__ sel, int64_t P, int E, int lo, int32_t* __restrict__ chunk_hist) {
    extern __shared__ int wh[];
    chunk_count<kThreads>(sel, P, (int64_t)blockIdx.x * kGroupChunk, E, lo, wh);
    for (int e = threadIdx.x; e < E; e += kThreads) {
        int h = 0;
        for (int w = 0; w < kWarps; w++) h += wh[w * E + e];
        chunk_hist[(int64_t)blockIdx.x * E + e] = h;
    }
}

__global__ void __launch_bounds__(kThreads)
group_scan_kernel(int n_chunks, int E, int chunk, int shared_T, int32_t* chunk_hist, int32_t* hist, int32_t* offsets,
                  int32_t* work_items, int32_t* n_work_items, int32_t work_cap) {
    __shared__ int s_warp[kWarps + 1];
    const int e = threadIdx.x;
    int run = 0;
    if (e < E)
        for (int c = 0; c < n_chunks; c++) {
            const int v = chunk_hist[(int64_t)c * E + e];
            chunk_hist[(int64_t)c * E + e] = run;  // picks of e in earlier chunks
            run += v;
        }
    write_offsets_and_items<kThreads>(e, E, run, chunk, shared_T, hist, offsets, work_items, n_work_items, work_cap, s_warp);
}

__global__ void __launch_bounds__(kThreads)
group_place_kernel(const int32_t* __restrict__ sel, int64_t P, int E, int lo, const int32_t* __restrict__ chunk_hist,
                   const int32_t* __restrict__ offsets, int32_t* __restrict__ perm) {
    extern __shared__ int wh[];
    const int64_t base = (int64_t)blockIdx.x * kGroupChunk;
    chunk_count<kThreads>(sel, P, base, E, lo, wh);
    for (int e = threadIdx.x; e < E; e += kThreads) {
        int run = offsets[e] + chunk_hist[(int64_t)blockIdx.x * E + e];
        for (int w = 0; w < kWarps; w++) {
            const int v = wh[w * E + e];
            wh[w * E + e] = run;
            run += v;
        }
    }
    __syncthreads();
    chunk_place<kThreads>(sel, P, base, E, lo, wh, perm);
}

// Scratch of the allocation-free entry point: the per-chunk histograms of the
// multi-block counting sort, for at most kStaticMaxChunks chunks of kGroupChunk
// picks (131072 picks, e.g. 16384 tokens x top-8).  128 KiB of device memory on
// every GPU that loads the library, held until the process exits.
constexpr int kStaticMaxChunks = 64;
static __device__ __align__(256) int32_t g_static_chunk_hist[kStaticMaxChunks * kMaxExperts];

}  // namespace

// Device address of g_static_chunk_hist on the CURRENT device.  In host code the
// array's name is only a handle for cudaGetSymbolAddress, never a pointer a
// kernel may receive; the lookup is done once per device and cached.
static int static_scratch(int32_t** out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static int32_t* cache[kMaxDevices] = {};
    int dev = 0;
    DSX_CUDA(cudaGetDevice(&dev));
    DSX_REQUIRE(dev >= 0 && dev < kMaxDevices, "group_build_static: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev] == nullptr) {
        void* p = nullptr;
        DSX_CUDA(cudaGetSymbolAddress(&p, g_static_chunk_hist));
        cache[dev] = static_cast<int32_t*>(p);
    }
    *out = cache[dev];
    return DSX_OK;
}

int launch_group_build_static(const int32_t* selected, int64_t T, int n_used, int n_expert, int chunk, int32_t* hist,
                              int32_t* offsets, int32_t* perm, int32_t* work_items, int32_t* n_work_items, int32_t work_cap,
                              cudaStream_t stream) {
    const int64_t P = T * n_used;
    const int64_t n_chunks = (P + kGroupChunk - 1) / kGroupChunk;
    if (n_expert > kMaxExperts)
        return set_error(DSX_ERR_UNSUPPORTED, "group_build_static: %d experts exceed the built-in scratch (at most %d)", n_expert,
                         kMaxExperts);
    if (n_chunks > kStaticMaxChunks)
        return set_error(DSX_ERR_UNSUPPORTED,
                         "group_build_static: %lld picks exceed the built-in scratch (at most %d picks); use dsx_moe_group_build",
                         (long long)P, kStaticMaxChunks * kGroupChunk);
    GroupScratch gs{};
    if (int rc = static_scratch(&gs.chunk_hist)) return rc;
    gs.capacity_chunks = kStaticMaxChunks;
    return launch_group_build(selected, T, n_used, n_expert, 0, chunk, 0, hist, offsets, perm, work_items, n_work_items, work_cap,
                              gs, stream);
}

int launch_group_build(const int32_t* selected, int64_t T, int n_used, int n_expert, int expert_lo, int chunk,
                       int shared_items_for_T, int32_t* hist, int32_t* offsets, int32_t* perm, int32_t* work_items,
                       int32_t* n_work_items, int32_t work_cap, GroupScratch scratch, cudaStream_t stream) {
    DSX_REQUIRE(n_expert >= 1 && n_expert <= kMaxExperts, "group_build: n_expert %d out of range (1..%d)", n_expert, kMaxExperts);
    DSX_REQUIRE(chunk >= 1, "group_build: chunk must be positive");
    DSX_REQUIRE(work_items == nullptr || T < 65536, "group_build: packed work items need fewer than 65536 tokens");
    const int64_t P = T * n_used;
    const size_t smem = sizeof(int) * (size_t)kWarps * (size_t)n_expert;
    if (P <= kGroupChunk) {
        group_build_small_kernel<<<1, kThreads, smem, stream>>>(selected, P, n_expert, expert_lo, chunk, shared_items_for_T,
                                                                hist, offsets, perm, work_items, n_work_items, work_cap);
        DSX_LAUNCHED();
        return DSX_OK;
    }
    const int64_t n_chunks = (P + kGroupChunk - 1) / kGroupChunk;
    DSX_REQUIRE(scratch.chunk_hist != nullptr && scratch.capacity_chunks >= n_chunks,
                "group_build: scratch holds %lld chunks, %lld needed", (long long)scratch.capacity_chunks, (long long)n_chunks);
    group_count_kernel<<<(unsigned)n_chunks, kThreads, smem, stream>>>(selected, P, n_expert, expert_lo, scratch.chunk_hist);
    DSX_LAUNCHED();
    group_scan_kernel<<<1, kThreads, 0, stream>>>((int)n_chunks, n_expert, chunk, shared_items_for_T, scratch.chunk_hist, hist,
                                                  offsets, work_items, n_work_items, work_cap);
    DSX_LAUNCHED();
    group_place_kernel<<<(unsigned)n_chunks, kThreads, smem, stream>>>(selected, P, n_expert, expert_lo, scratch.chunk_hist,
                                                                      offsets, perm);
    DSX_LAUNCHED();
    return DSX_OK;
}


// Expert-selection statistics bank (crates/v4flash-kernels/kernels/expert_sel_count.hip:17-28,
// src/expert_sel_count.rs:34): counts[layer_off + sel[i]] += 1 for every pick; ids outside
// [0, n_expert) are dropped.  Integer atomics: the totals do not depend on the order.
namespace {
__global__ void expert_sel_count_kernel(unsigned int* __restrict__ counts, const int32_t* __restrict__ selected, unsigned int layer_off,
                                        unsigned int n_expert, int64_t total) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int e = selected[i];
    if (e < 0 || (unsigned int)e >= n_expert) return;
    atomicAdd(&counts[layer_off + (unsigned int)e], 1u);
}
}  // namespace

int launch_expert_sel_count(unsigned int* counts, const int32_t* selected, unsigned int layer_off, unsigned int n_expert, int64_t total,
                            cudaStream_t stream) {
    if (total == 0) return DSX_OK;
    expert_sel_count_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(counts, selected, layer_off, n_expert, total);
    DSX_LAUNCHED();
    return DSX_OK;
}

}  // namespace dsx
