// Expert-weight repack: source layouts of the reference's loaders -> the tile
// layout described in dsx_common.cuh, and its inverse (for bit-parity tests).
//
// Reference counterparts: the CPU repack in crates/v4flash-core/src/hf_v41.rs:1207-1229
// and the GPU twin crates/v4flash-kernels/kernels/mxfp4_repack.hip:35-65 (HF ->
// super-block v2).  Here the destination is this library's own layout, so the
// kernels accept all three MXFP4 layouts the reference moves between (HF,
// ggml 17-byte blocks, super-block v2) and both Q8_0 forms.
#include <algorithm>

#include "dsx_common.cuh"

namespace dsx {
namespace {

__device__ __forceinline__ uint32_t mxfp4_src_code(int layout, const uint8_t* q, int64_t K, int64_t row, int64_t k) {
    if (layout == DSX_SRC_MXFP4_HF) {
        const uint8_t b = q[row * (K >> 1) + (k >> 1)];
        return (k & 1) ? (b >> 4) : (b & 0xF);
    }
    const int j = (int)(k & 31);
    uint8_t b;
    if (layout == DSX_SRC_MXFP4_GGML) {
        b = q[(row * (K >> 5) + (k >> 5)) * 17 + 1 + (j & 15)];
    } else {  // super-block v2: 136 B per 256 columns, nibbles of block b at 16*b
        b = q[row * (K >> 5) * 17 + (k >> 8) * 136 + ((k & 255) >> 5) * 16 + (j & 15)];
    }
    return (j < 16) ? (b & 0xF) : (b >> 4);
}

__device__ __forceinline__ uint8_t mxfp4_src_scale(int layout, const uint8_t* q, const uint8_t* s, int64_t K,
                                                   int64_t row, int64_t blk) {
    if (layout == DSX_SRC_MXFP4_HF) return s[row * (K >> 5) + blk];
    if (layout == DSX_SRC_MXFP4_GGML) return q[(row * (K >> 5) + blk) * 17];
    return q[row * (K >> 5) * 17 + (blk >> 3) * 136 + 128 + (blk & 7)];
}

// One thread per (sub-tile, lane): writes the lane's 16 code bytes and, for
// t == 0, the 4 scale bytes of lane group g.
__global__ void repack_mxfp4_kernel(int layout, const uint8_t* __restrict__ q, const uint8_t* __restrict__ s,
                                    int64_t rows, int64_t K, uint8_t* __restrict__ nib, uint8_t* __restrict__ sc,
                                    int pair_stride, int pair_index, int64_t src_q_stride, int64_t src_s_stride,
                                    int64_t dst_nib_stride, int64_t dst_sc_stride) {
    const int64_t n_kt = K >> 6;
    const int64_t n_sub = (rows >> 4) * n_kt;
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t sub = gid >> 5;
    if (sub >= n_sub) return;
    const int lane = (int)(gid & 31), g = lane >> 2, t = lane & 3;
    const int64_t mat = blockIdx.y;
    q += mat * src_q_stride;
    if (s) s += mat * src_s_stride;
    nib += mat * dst_nib_stride;
    sc += mat * dst_sc_stride;
    const int64_t rt = sub / n_kt, kt = sub - rt * n_kt;
    const int64_t r0 = rt * 16 + g, r1 = r0 + 8;
    uint32_t words[4];
#pragma unroll
    for (int st = 0; st < 4; st++) {
        const int64_t c = kt * 64 + 32 * (st >> 1) + 8 * t + 4 * (st & 1);
        uint32_t w = 0;
        w |= (mxfp4_src_code(layout, q, K, r0, c + 0) | (mxfp4_src_code(layout, q, K, r0, c + 1) << 4)) << 0;
        w |= (mxfp4_src_code(layout, q, K, r1, c + 0) | (mxfp4_src_code(layout, q, K, r1, c + 1) << 4)) << 8;
        w |= (mxfp4_src_code(layout, q, K, r0, c + 2) | (mxfp4_src_code(layout, q, K, r0, c + 3) << 4)) << 16;
        w |= (mxfp4_src_code(layout, q, K, r1, c + 2) | (mxfp4_src_code(layout, q, K, r1, c + 3) << 4)) << 24;
        words[st] = w;
    }
    const int64_t dsub = sub * pair_stride + pair_index;
    *reinterpret_cast<uint4*>(nib + dsub * kSubNibBytes + lane * 16) = make_uint4(words[0], words[1], words[2], words[3]);
    if (t == 0) {
        uint32_t v = 0;
        v |= (uint32_t)mxfp4_src_scale(layout, q, s, K, r0, kt * 2 + 0) << 0;
        v |= (uint32_t)mxfp4_src_scale(layout, q, s, K, r0, kt * 2 + 1) << 8;
        v |= (uint32_t)mxfp4_src_scale(layout, q, s, K, r1, kt * 2 + 0) << 16;
        v |= (uint32_t)mxfp4_src_scale(layout, q, s, K, r1, kt * 2 + 1) << 24;
        *reinterpret_cast<uint32_t*>(sc + dsub * kSubScBytes + g * 4) = v;
    }
}

__device__ __forceinline__ uint8_t q8_src_code(int layout, const uint8_t* q, int64_t K, int64_t row, int64_t k) {
    if (layout == DSX_SRC_Q8_0_SPLIT) return q[row * K + k];
    return q[(row * (K >> 5) + (k >> 5)) * 34 + 2 + (k & 31)];
}
__device__ __forceinline__ uint16_t q8_src_scale(int layout, const uint8_t* q, const uint8_t* s, int64_t K, int64_t row,
                                                 int64_t blk) {
    if (layout == DSX_SRC_Q8_0_SPLIT) return reinterpret_cast<const uint16_t*>(s)[row * (K >> 5) + blk];
    const uint8_t* p = q + (row * (K >> 5) + blk) * 34;
    return (uint16_t)(p[0] | (p[1] << 8));
}

__global__ void repack_q8_0_kernel(int layout, const uint8_t* __restrict__ q, const uint8_t* __restrict__ s,
                                   int64_t rows, int64_t K, uint8_t* __restrict__ nib, uint8_t* __restrict__ sc,
                                   int pair_stride, int pair_index, int64_t src_q_stride, int64_t src_s_stride,
                                   int64_t dst_nib_stride, int64_t dst_sc_stride) {
    const int64_t n_kt = K >> 5;
    const int64_t n_sub = (rows >> 4) * n_kt;
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t sub = gid >> 5;
    if (sub >= n_sub) return;
    const int lane = (int)(gid & 31), g = lane >> 2, t = lane & 3;
    const int64_t mat = blockIdx.y;
    q += mat * src_q_stride;
    if (s) s += mat * src_s_stride;
    nib += mat * dst_nib_stride;
    sc += mat * dst_sc_stride;
    const int64_t rt = sub / n_kt, kt = sub - rt * n_kt;
    const int64_t r0 = rt * 16 + g, r1 = r0 + 8;
    uint32_t words[4];
#pragma unroll
    for (int st = 0; st < 2; st++) {
        const int64_t c = kt * 32 + 8 * t + 4 * st;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int64_t r = h ? r1 : r0;
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) w |= (uint32_t)(q8_src_code(layout, q, K, r, c + j) ^ 0x80u) << (8 * j);
            words[2 * st + h] = w;
        }
    }
    const int64_t dsub = sub * pair_stride + pair_index;
    *reinterpret_cast<uint4*>(nib + dsub * kSubNibBytes + lane * 16) = make_uint4(words[0], words[1], words[2], words[3]);
    if (t == 0) {
        const uint32_t v = (uint32_t)q8_src_scale(layout, q, s, K, r0, kt) | ((uint32_t)q8_src_scale(layout, q, s, K, r1, kt) << 16);
        *reinterpret_cast<uint32_t*>(sc + dsub * kSubScBytes + g * 4) = v;
    }
}

// Inverse: one thread per (row, 32-column block) -> HF bytes (MXFP4) or split int8 + f16 (Q8_0).
__global__ void unpack_kernel(int fmt, const uint8_t* __restrict__ nib, const uint8_t* __restrict__ sc, int64_t rows,
                              int64_t K, int pair_stride, int pair_index, uint8_t* __restrict__ q_out,
                              uint8_t* __restrict__ s_out) {
    const int64_t nb = K >> 5;
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= rows * nb) return;
    const int64_t row = gid / nb, blk = gid - row * nb;
    const int64_t rt = row >> 4;
    const int r = (int)(row & 15), g = r & 7, hi_row = r >> 3;
    if (fmt == DSX_FMT_MXFP4) {
        const int64_t n_kt = K >> 6, kt = blk >> 1;
        const int b = (int)(blk & 1);
        const int64_t dsub = (rt * n_kt + kt) * pair_stride + pair_index;
        const uint8_t* tile = nib + dsub * kSubNibBytes;
        uint8_t codes[32];
        for (int within = 0; within < 32; within++) {
            const int t = within >> 3, rem = within & 7, st = 2 * b + (rem >> 2), j = rem & 3;
            const uint8_t byte = tile[(g * 4 + t) * 16 + st * 4 + (j >> 1) * 2 + hi_row];
            codes[within] = (j & 1) ? (byte >> 4) : (byte & 0xF);
        }
        for (int i = 0; i < 16; i++) q_out[row * (K >> 1) + blk * 16 + i] = (uint8_t)(codes[2 * i] | (codes[2 * i + 1] << 4));
        s_out[row * nb + blk] = sc[dsub * kSubScBytes + g * 4 + hi_row * 2 + b];
    } else {
        const int64_t n_kt = K >> 5, kt = blk;
        const int64_t dsub = (rt * n_kt + kt) * pair_stride + pair_index;
        const uint8_t* tile = nib + dsub * kSubNibBytes;
        for (int within = 0; within < 32; within++) {
            const int t = within >> 3, rem = within & 7, st = rem >> 2, j = rem & 3;
            q_out[row * K + blk * 32 + within] = tile[(g * 4 + t) * 16 + (2 * st + hi_row) * 4 + j] ^ 0x80u;
        }
        reinterpret_cast<uint16_t*>(s_out)[row * nb + blk] =
            *reinterpret_cast<const uint16_t*>(sc + dsub * kSubScBytes + g * 4 + hi_row * 2);
    }
}

// The tensor-core planes of an MXFP4 matrix (prefill_mx.cu): codes K-major, i.e. the HF byte layout
// [row][K/2] with element 2i in the low nibble, and the E8M0 block scales cut into the 512-byte chunks
// the block-scaled MMA takes its scale factors from: chunk = 128 rows x 4 blocks (128 columns), byte
// (row % 32) * 16 + (row / 32 % 4) * 4 + (block % 4).  Chunks are ordered [group][K / 128][4]: for gate and up a
// group is 256 rows of both matrices, its chunks (gate rows 0-127, up rows 0-127, gate rows 128-255, up rows
// 128-255); for down a group is 512 rows, its chunks the four 128-row quarters.  The two chunks one pipeline stage
// of one tile of the GEMM needs (gate + up of 128 rows; two 128-row quarters) are one contiguous half of a group.
// One thread per (row, 32-column block).
__global__ void kmajor_mxfp4_kernel(int layout, const uint8_t* __restrict__ q, const uint8_t* __restrict__ s, int64_t rows, int64_t K,
                                    int pair_index, int64_t src_q_stride, int64_t src_s_stride, uint8_t* __restrict__ km,
                                    int64_t km_stride, uint8_t* __restrict__ sf, int64_t sf_stride) {
    const int64_t nb = K >> 5;
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= rows * nb) return;
    const int64_t row = gid / nb, blk = gid - row * nb;
    const int64_t mat = blockIdx.y;
    q += mat * src_q_stride;
    if (s) s += mat * src_s_stride;
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t v = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) v |= mxfp4_src_code(layout, q, K, row, blk * 32 + i * 8 + j) << (4 * j);
        w[i] = v;
    }
    uint8_t* kdst = km + mat * km_stride + (pair_index > 0 ? rows * (K >> 1) : 0) + row * (K >> 1) + blk * 16;
    *reinterpret_cast<uint4*>(kdst) = make_uint4(w[0], w[1], w[2], w[3]);
    const int64_t n_kc = K >> 7;
    const int64_t chunk = pair_index >= 0 ? ((row >> 8) * n_kc + (blk >> 2)) * 4 + ((row >> 7) & 1) * 2 + pair_index
                                          : ((row >> 9) * n_kc + (blk >> 2)) * 4 + ((row >> 7) & 3);
    sf[mat * sf_stride + chunk * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (blk & 3)] = mxfp4_src_scale(layout, q, s, K, row, blk);
}

// Largest byte of a scale plane (E8M0 exponents), folded into *out with atomicMax.
__global__ void max_byte_kernel(const uint8_t* __restrict__ p, int64_t n_words, uint32_t* out) {
    uint32_t m = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t w = reinterpret_cast<const uint32_t*>(p)[i];
        m = max(m, max(max(w & 0xFFu, (w >> 8) & 0xFFu), max((w >> 16) & 0xFFu, w >> 24)));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
    if ((threadIdx.x & 31) == 0 && m) atomicMax(out, m);
}

}  // namespace

int launch_max_byte(const uint8_t* p, int64_t bytes, uint32_t* out, cudaStream_t stream) {
    const int64_t n_words = bytes / 4;
    if (n_words == 0) return DSX_OK;
    max_byte_kernel<<<(unsigned)std::min<int64_t>(1024, (n_words + 255) / 256), 256, 0, stream>>>(p, n_words, out);
    DSX_LAUNCHED();
    return DSX_OK;
}

int launch_kmajor_mxfp4(int src_layout, const uint8_t* q, const uint8_t* s, int64_t rows, int64_t K, int pair_index, int n_mats,
                        int64_t src_q_stride, int64_t src_s_stride, uint8_t* km, int64_t km_stride, uint8_t* sf, int64_t sf_stride,
                        cudaStream_t stream) {
    DSX_REQUIRE(rows % 256 == 0 && K % 128 == 0 && (pair_index >= 0 || rows % 512 == 0), "kmajor: rows %lld / K %lld not tileable",
                (long long)rows, (long long)K);
    DSX_REQUIRE(src_layout >= DSX_SRC_MXFP4_HF && src_layout <= DSX_SRC_MXFP4_SB2, "kmajor: layout %d is not MXFP4", src_layout);
    const int64_t n_threads = rows * (K >> 5);
    dim3 grid((unsigned)((n_threads + 255) / 256), (unsigned)n_mats);
    kmajor_mxfp4_kernel<<<grid, 256, 0, stream>>>(src_layout, q, s, rows, K, pair_index, src_q_stride, src_s_stride, km, km_stride, sf,
                                                  sf_stride);
    DSX_LAUNCHED();
    return DSX_OK;
}

int launch_repack(int fmt, int src_layout, const uint8_t* q, const uint8_t* s, int64_t rows, int64_t K, uint8_t* nib,
                  uint8_t* sc, int pair_stride, int pair_index, int n_mats, int64_t src_q_stride, int64_t src_s_stride,
                  int64_t dst_nib_stride, int64_t dst_sc_stride, cudaStream_t stream) {
    const int tk = tile_k(fmt);
    DSX_REQUIRE(rows % 16 == 0 && K % tk == 0 && K % 256 == 0, "repack: rows %lld / K %lld not tileable", (long long)rows,
                (long long)K);
    const int64_t n_threads = (rows / 16) * (K / tk) * 32;
    dim3 grid((unsigned)((n_threads + 255) / 256), (unsigned)n_mats);
    if (fmt == DSX_FMT_MXFP4) {
        DSX_REQUIRE(src_layout >= DSX_SRC_MXFP4_HF && src_layout <= DSX_SRC_MXFP4_SB2, "repack: layout %d is not MXFP4", src_layout);
        DSX_REQUIRE(src_layout != DSX_SRC_MXFP4_HF || s != nullptr, "repack: HF layout needs a scale array");
        repack_mxfp4_kernel<<<grid, 256, 0, stream>>>(src_layout, q, s, rows, K, nib, sc, pair_stride, pair_index,
                                                      src_q_stride, src_s_stride, dst_nib_stride, dst_sc_stride);
    } else {
        DSX_REQUIRE(src_layout == DSX_SRC_Q8_0_BLOCKS || src_layout == DSX_SRC_Q8_0_SPLIT, "repack: layout %d is not Q8_0", src_layout);
        DSX_REQUIRE(src_layout != DSX_SRC_Q8_0_SPLIT || s != nullptr, "repack: split layout needs a scale array");
        repack_q8_0_kernel<<<grid, 256, 0, stream>>>(src_layout, q, s, rows, K, nib, sc, pair_stride, pair_index,
                                                     src_q_stride, src_s_stride, dst_nib_stride, dst_sc_stride);
    }
    DSX_LAUNCHED();
    return DSX_OK;
}

int launch_unpack(int fmt, const uint8_t* nib, const uint8_t* sc, int64_t rows, int64_t K, int pair_stride,
                  int pair_index, uint8_t* q_out, uint8_t* s_out, cudaStream_t stream) {
    const int64_t n = rows * (K / 32);
    unpack_kernel<<<(unsigned)((n + 127) / 128), 128, 0, stream>>>(fmt, nib, sc, rows, K, pair_stride, pair_index, q_out, s_out);
    DSX_LAUNCHED();
    return DSX_OK;
}

}  // namespace dsx
