// Device building blocks of the stable counting sort (histogram, offsets, permutation, work
// items), templated on the block size so that both the stand-alone group-build kernels (512
// threads) and the fused decode router (256 threads) use the same code.  See groups.cu.
#pragma once
#include "dsx_common.cuh"

namespace dsx {
namespace groupdev {

// wh[w*E + e] = picks of local expert e inside warp w's slice of the chunk.
template <int NT, int CHUNK = kGroupChunk>
__device__ void chunk_count(const int32_t* __restrict__ sel, int64_t P, int64_t chunk_base, int E, int lo, int* wh) {
    constexpr int kIt = (CHUNK / (NT / 32)) / 32;
    for (int i = threadIdx.x; i < (NT / 32) * E; i += NT) wh[i] = 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int ev[kIt];   // all picks of the thread first: the loads overlap instead of queueing behind the atomics
#pragma unroll
    for (int it = 0; it < kIt; it++) {
        const int64_t idx = chunk_base + warp * (CHUNK / (NT / 32)) + it * 32 + lane;
        ev[it] = idx < P ? sel[idx] - lo : -1;
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < kIt; it++)
        if (ev[it] >= 0 && ev[it] < E) atomicAdd(&wh[warp * E + ev[it]], 1);
    __syncthreads();
}

// Exclusive scan of one value per thread over the block (NT threads).
template <int NT>
__device__ int block_exclusive_scan(int v, int* total, int* s_warp /*[(NT / 32)+1]*/) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int inc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(0xFFFFFFFFu, inc, off);
        if (lane >= off) inc += o;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = lane < (NT / 32) ? s_warp[lane] : 0;
        int winc = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int o = __shfl_up_sync(0xFFFFFFFFu, winc, off);
            if (lane >= off) winc += o;
        }
        if (lane < (NT / 32)) s_warp[lane] = winc - w;
        if (lane == (NT / 32) - 1) s_warp[(NT / 32)] = winc;
    }
    __syncthreads();
    const int res = s_warp[warp] + inc - v;
    *total = s_warp[(NT / 32)];
    __syncthreads();
    return res;
}

// From hist (one expert per thread): offsets, work items (+ shared-expert items).
template <int NT>
__device__ int write_offsets_and_items(int e, int E, int h, int chunk, int shared_T, int32_t* hist, int32_t* offsets,
                                       int32_t* work_items, int32_t* n_work_items, int32_t work_cap, int* s_warp,
                                       int32_t* s_off = nullptr /* [E+1] */, int32_t* s_items = nullptr /* [work_cap] */,
                                       int* s_n_items = nullptr) {
    int total;
    const int off = block_exclusive_scan<NT>(e < E ? h : 0, &total, s_warp);
    if (e < E) {
        hist[e] = h;
        offsets[e] = off;
        if (s_off) s_off[e] = off;
    }
    if (threadIdx.x == 0) {
        offsets[E] = total;
        if (s_off) s_off[E] = total;
    }
    if (work_items != nullptr) {
        const int ni = (e < E) ? (h + chunk - 1) / chunk : 0;
        int n_items;
        const int ibase = block_exclusive_scan<NT>(ni, &n_items, s_warp);
        for (int c = 0; c < ni; c++) {
            const int p = ibase + c;
            if (p < work_cap) {
                const int32_t wi = (int32_t)(((uint32_t)e << 16) | (((uint32_t)(c * chunk)) & 0xFFFFu));
                work_items[p] = wi;
                if (s_items) s_items[p] = wi;
            }
        }
        // the shared expert is appended as pseudo expert id E over all tokens
        const int n_sh = (shared_T + chunk - 1) / chunk;
        for (int c = threadIdx.x; c < n_sh; c += NT) {
            const int p = n_items + c;
            if (p < work_cap) {
                const int32_t wi = (int32_t)(((uint32_t)E << 16) | (((uint32_t)(c * chunk)) & 0xFFFFu));
                work_items[p] = wi;
                if (s_items) s_items[p] = wi;
            }
        }
        if (threadIdx.x == 0) {
            n_work_items[0] = n_items + n_sh;
            if (s_n_items) *s_n_items = min(n_items + n_sh, work_cap);
        }
    }
    return off;   // first sorted position of expert e
}

// Stable placement of this block's chunk.  wh[w*E+e] holds the first free
// position of expert e for warp w; each warp walks its slice in order.
template <int NT, int CHUNK = kGroupChunk>
__device__ void chunk_place(const int32_t* __restrict__ sel, int64_t P, int64_t chunk_base, int E, int lo, int* wh,
                            int32_t* __restrict__ perm, int32_t* s_perm = nullptr /* shared-memory copy of perm */) {
    constexpr int kIt = (CHUNK / (NT / 32)) / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int ev[kIt];
#pragma unroll
    for (int it = 0; it < kIt; it++) {
        const int64_t idx = chunk_base + warp * (CHUNK / (NT / 32)) + it * 32 + lane;
        int e = idx < P ? sel[idx] - lo : -1;
        ev[it] = (e < 0 || e >= E) ? -1 : e;
    }
#pragma unroll
    for (int it = 0; it < kIt; it++) {
        const int64_t idx = chunk_base + warp * (CHUNK / (NT / 32)) + it * 32 + lane;
        const int e = ev[it];
        const int key = e >= 0 ? e : (0x40000000 | lane);
        const uint32_t mask = __match_any_sync(0xFFFFFFFFu, key);
        const int rank = __popc(mask & ((1u << lane) - 1u));
        if (e >= 0) {
            const int pos = wh[warp * E + e] + rank;
            perm[pos] = (int32_t)idx;
            if (s_perm) s_perm[pos] = (int32_t)idx;
        }
        __syncwarp();
        if (e >= 0 && rank == 0) wh[warp * E + e] += __popc(mask);
        __syncwarp();
    }
}

// One expert per thread (needs E <= NT): the whole build for T*k <= CHUNK picks inside one block.
// wh: NT/32 * E ints of shared memory, s_warp: NT/32 + 1 ints.  `sel` may point to shared memory.
template <int NT, int CHUNK = kGroupChunk>
__device__ void build_small(const int32_t* __restrict__ sel, int64_t P, int E, int lo, int chunk, int shared_T, int32_t* hist,
                            int32_t* offsets, int32_t* perm, int32_t* work_items, int32_t* n_work_items, int32_t work_cap,
                            int* wh, int* s_warp) {
    chunk_count<NT, CHUNK>(sel, P, 0, E, lo, wh);
    const int e = threadIdx.x;
    int h = 0;
    if (e < E)
        for (int w = 0; w < NT / 32; w++) h += wh[w * E + e];
    int run = write_offsets_and_items<NT>(e, E, h, chunk, shared_T, hist, offsets, work_items, n_work_items, work_cap, s_warp);
    if (e < E) {
        for (int w = 0; w < NT / 32; w++) {
            const int v = wh[w * E + e];
            wh[w * E + e] = run;
            run += v;
        }
    }
    __syncthreads();
    chunk_place<NT, CHUNK>(sel, P, 0, E, lo, wh, perm);
}

// build_small plus one ItemRec per work item (chunk of 8 tokens), for the decode router.
// sel / s_w: picks and routing weights of all P <= CHUNK picks in shared memory; scratch: shared
// memory for (NT/32)*E + CHUNK + work_cap + E + 2 ints.
template <int NT, int CHUNK>
__device__ void build_small_with_recs(const int32_t* sel, const float* s_w, int T, int n_used, int E, int shared_T, int32_t* hist,
                                      int32_t* offsets, int32_t* perm, int32_t* work_items, int32_t* n_work_items, int32_t work_cap,
                                      ItemRec* recs, int* scratch, int* s_warp) {
    const int P = T * n_used;
    int* wh = scratch;
    int32_t* s_perm = scratch + (NT / 32) * E;
    int32_t* s_items = s_perm + CHUNK;
    int32_t* s_off = s_items + work_cap;
    int* s_n_items = s_off + E + 1;
    chunk_count<NT, CHUNK>(sel, P, 0, E, 0, wh);
    const int e = threadIdx.x;
    int h = 0;
    if (e < E)
        for (int w = 0; w < NT / 32; w++) h += wh[w * E + e];
    int run = write_offsets_and_items<NT>(e, E, h, 8, shared_T, hist, offsets, work_items, n_work_items, work_cap, s_warp, s_off, s_items,
                                          s_n_items);
    if (e < E) {
        for (int w = 0; w < NT / 32; w++) {
            const int v = wh[w * E + e];
            wh[w * E + e] = run;
            run += v;
        }
    }
    __syncthreads();
    chunk_place<NT, CHUNK>(sel, P, 0, E, 0, wh, perm, s_perm);
    __syncthreads();
    const int n_items = *s_n_items;
    for (int idx = threadIdx.x; idx < n_items * 8; idx += NT) {
        const int i = idx >> 3, j = idx & 7;
        const uint32_t wi = (uint32_t)s_items[i];
        const int ex = (int)(wi >> 16), start = (int)(wi & 0xFFFFu);
        int n, tok, mid_row, out_row;
        float w;
        if (ex == E) {   // shared expert: tokens start..start+7, weight 1
            n = min(8, shared_T - start);
            tok = start + j;
            mid_row = out_row = P + start + j;
            w = 1.0f;
        } else {
            const int seg0 = s_off[ex];
            n = min(8, s_off[ex + 1] - seg0 - start);
            const int p = seg0 + start + min(j, n - 1);
            const int ts = s_perm[p];
            tok = ts / n_used;
            mid_row = p;
            out_row = ts;
            w = s_w[ts];
        }
        ItemRec* r = recs + i;
        if (j == 0) { r->expert = ex; r->n_tok = n; }
        r->tok[j] = tok;
        r->mid_row[j] = mid_row;
        r->out_row[j] = out_row;
        r->w[j] = w;
    }
}

// The same result for at most 32 picks (a handful of decode tokens), in four block barriers instead of
// a dozen: every thread counts the picks of, and below, its own expert directly (the picks are in
// shared memory), one block scan numbers the work items, and one warp places the picks (position =
// picks of smaller experts + earlier picks of the same expert, by match_any).  Needs E <= NT.
// scratch: shared memory for 32 + work_cap + E + 2 ints.
template <int NT>
__device__ void build_tiny_with_recs(const int32_t* sel, const float* s_w, int T, int n_used, int E, int shared_T, int32_t* hist,
                                     int32_t* offsets, int32_t* perm, int32_t* work_items, int32_t* n_work_items, int32_t work_cap,
                                     ItemRec* recs, int* scratch, int* s_warp) {
    const int P = T * n_used;   // <= 32
    int32_t* s_perm = scratch;
    int32_t* s_items = s_perm + 32;
    int32_t* s_off = s_items + work_cap;
    int* s_n_items = s_off + E + 1;
    const int e = threadIdx.x;
    int h = 0, below = 0, valid = 0;
    for (int i = 0; i < P; i++) {
        const int v = sel[i];
        h += (v == e) ? 1 : 0;
        below += (v >= 0 && v < e) ? 1 : 0;
        valid += (v >= 0 && v < E) ? 1 : 0;
    }
    if (e < E) {
        hist[e] = h;
        offsets[e] = below;
        s_off[e] = below;
    }
    if (e == 0) {
        offsets[E] = valid;
        s_off[E] = valid;
    }
    const int ni = (e < E) ? (h + 7) >> 3 : 0;
    int n_items;
    const int ibase = block_exclusive_scan<NT>(ni, &n_items, s_warp);   // its barriers also publish s_off
    for (int c = 0; c < ni; c++) {
        const int p = ibase + c;
        if (p < work_cap) {
            const int32_t wi = (int32_t)(((uint32_t)e << 16) | (uint32_t)(c * 8));
            work_items[p] = wi;
            s_items[p] = wi;
        }
    }
    const int n_sh = (shared_T + 7) >> 3;   // the shared expert is appended as pseudo expert id E over all tokens
    for (int c = threadIdx.x; c < n_sh; c += NT) {
        const int p = n_items + c;
        if (p < work_cap) {
            const int32_t wi = (int32_t)(((uint32_t)E << 16) | (uint32_t)(c * 8));
            work_items[p] = wi;
            s_items[p] = wi;
        }
    }
    if (threadIdx.x == 0) {
        n_work_items[0] = n_items + n_sh;
        *s_n_items = min(n_items + n_sh, work_cap);
    }
    if (threadIdx.x < 32) {   // stable placement by one warp
        const int i = threadIdx.x;
        const int v = i < P ? sel[i] : -1;
        const bool ok = v >= 0 && v < E;
        const int key = ok ? v : (0x40000000 | i);
        const uint32_t mask = __match_any_sync(0xFFFFFFFFu, key);
        if (ok) {
            const int pos = s_off[v] + __popc(mask & ((1u << i) - 1u));
            perm[pos] = i;
            s_perm[pos] = i;
        }
    }
    __syncthreads();
    const int total = *s_n_items;
    for (int idx = threadIdx.x; idx < total * 8; idx += NT) {
        const int i = idx >> 3, j = idx & 7;
        const uint32_t wi = (uint32_t)s_items[i];
        const int ex = (int)(wi >> 16), start = (int)(wi & 0xFFFFu);
        int n, tok, mid_row, out_row;
        float w;
        if (ex == E) {   // shared expert: tokens start..start+7, weight 1
            n = min(8, shared_T - start);
            tok = start + j;
            mid_row = out_row = P + start + j;
            w = 1.0f;
        } else {
            const int seg0 = s_off[ex];
            n = min(8, s_off[ex + 1] - seg0 - start);
            const int p = seg0 + start + min(j, n - 1);
            const int ts = s_perm[p];
            tok = ts / n_used;
            mid_row = p;
            out_row = ts;
            w = s_w[ts];
        }
        ItemRec* r = recs + i;
        if (j == 0) { r->expert = ex; r->n_tok = n; }
        r->tok[j] = tok;
        r->mid_row[j] = mid_row;
        r->out_row[j] = out_row;
        r->w[j] = w;
    }
}

}  // namespace groupdev
}  // namespace dsx
