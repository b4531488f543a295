/*
 * dsx_oracle.c -- CPU restatement of deepstrix's routed-MoE hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, imports or
 * calls this file: it is the checker the GPU kernels are compared against, and
 * the CPU baseline that the benchmark times beside them.
 *
 * Every function cites the reference file:line (paths relative to the
 * deepstrix repository) whose arithmetic it restates.  The reference itself is
 * Rust + HIP and cannot be compiled without cargo/hipcc, so this is a port,
 * pinned against the reference's own known-answer vectors:
 *   - external/ds4-dump/quants_selftest_expected.inc:93-137 (MXFP4 dequant bits)
 *   - crates/v4flash-core/src/hf_v41.rs:1321-1382 (E4M3 / E8M0 / Q8_0 / nibble tests)
 *   - crates/v4flash-kernels/src/het/dispatch.rs:746-748 (work-item bound literals)
 *   - scripts/v41_oracle/kernel.py (dequant_fp4 / act_quant / fp4_act_quant / fp4_gemm outputs)
 * Parts with no counterpart in the reference (group-limited routing, Q8_0
 * routed experts, bf16 activations) are "parity unpinned": defined here under
 * the reference's conventions.  So are the router's alternatives / score range /
 * cache prior and the two steps either side of the layer (RMSNorm, residual mix): the
 * reference has kernels for them but no known-answer vector, so they are
 * restated from the kernel text alone.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see Makefile).
 * -ffp-contract=off matters: the router arithmetic must round exactly like the
 * explicit __fmaf_rn/__fmul_rn sequence of the CUDA kernels.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define DSXO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ scalars */

static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

/* crates/v4flash-kernels/src/mxfp4_tables.rs:8 -- E2M1 values doubled. */
static const int8_t KVALUES_MXFP4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

/* crates/v4flash-kernels/src/mxfp4_tables.rs:37-45 -- 2^(e-128), denormal for e<2. */
DSXO_API float dsxo_e8m0_half(uint8_t e) {
    uint32_t bits = (e < 2) ? (0x00200000u << e) : (((uint32_t)e - 1u) << 23);
    return bits_f32(bits);
}

/* crates/v4flash-core/src/hf_v41.rs:97-105 -- torch float8_e8m0fnu: 2^(e-127). */
DSXO_API float dsxo_e8m0(uint8_t e) {
    if (e == 0xFF) return NAN;
    if (e == 0) return bits_f32(1u << 22);
    return bits_f32((uint32_t)e << 23);
}

/* crates/v4flash-core/src/hf_v41.rs:107-118 -- torch float8_e4m3fn. */
DSXO_API float dsxo_e4m3(uint8_t b) {
    if ((b & 0x7F) == 0x7F) return NAN;
    float sign = (b & 0x80) ? -1.0f : 1.0f;
    int e = (b >> 3) & 0xF;
    float m = (float)(b & 7);
    float v = (e == 0) ? m * ldexpf(1.0f, -9) : (1.0f + m / 8.0f) * ldexpf(1.0f, e - 7);
    return sign * v;
}

static float f16_to_f32(uint16_t h) {
    uint32_t s = (uint32_t)(h & 0x8000) << 16;
    uint32_t e = (h >> 10) & 0x1F, m = h & 0x3FF;
    if (e == 0) {
        if (m == 0) return bits_f32(s);
        float v = ldexpf((float)m, -24);
        return (s ? -v : v);
    }
    if (e == 31) return bits_f32(s | 0x7F800000u | (m << 13));
    return bits_f32(s | ((e + 112) << 23) | (m << 13));
}

static uint16_t f32_to_f16(float f) { /* round to nearest even */
    uint32_t x = f32_bits(f);
    uint32_t s = (x >> 16) & 0x8000;
    int32_t e = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    uint32_t m = x & 0x7FFFFF;
    if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(s | 0x7C00 | (m ? 0x200 : 0));
    if (e >= 31) return (uint16_t)(s | 0x7C00);
    if (e <= 0) {
        if (e < -10) return (uint16_t)s;
        m |= 0x800000;
        int shift = 14 - e;
        uint32_t r = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (r & 1))) r++;
        return (uint16_t)(s | r);
    }
    uint32_t r = ((uint32_t)e << 10) | (m >> 13);
    uint32_t rem = m & 0x1FFF;
    if (rem > 0x1000 || (rem == 0x1000 && (r & 1))) r++;
    return (uint16_t)(s | r);
}

DSXO_API float dsxo_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
DSXO_API uint16_t dsxo_f32_to_f16(float f) { return f32_to_f16(f); }

static inline float bf16_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }
static inline uint16_t f32_to_bf16(float f) { /* RNE; NaN kept quiet */
    uint32_t x = f32_bits(f);
    if ((x & 0x7FFFFFFF) > 0x7F800000) return (uint16_t)((x >> 16) | 0x40);
    return (uint16_t)((x + 0x7FFF + ((x >> 16) & 1)) >> 16);
}
DSXO_API void dsxo_f32_to_bf16(const float* x, uint16_t* y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = f32_to_bf16(x[i]);
}
DSXO_API void dsxo_bf16_to_f32(const uint16_t* x, float* y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = bf16_to_f32(x[i]);
}

/* ------------------------------------------------- MXFP4 layouts and dequant */

/* ggml 17-byte block `e | qs[16]`: element j = low nibble of qs[j], element
 * j+16 = high nibble (crates/v4flash-kernels/kernels/mxfp4_matvec.hip:5-9);
 * value = kvalue * e8m0_half(e).  Checked bit-for-bit against
 * external/ds4-dump/quants_selftest_expected.inc:93-137. */
DSXO_API void dsxo_mxfp4_dequant_ggml(const uint8_t* blocks, int64_t n_blocks, float* out) {
    for (int64_t b = 0; b < n_blocks; b++) {
        const uint8_t* blk = blocks + b * 17;
        float d = dsxo_e8m0_half(blk[0]);
        for (int j = 0; j < 16; j++) {
            out[b * 32 + j] = (float)KVALUES_MXFP4[blk[1 + j] & 0xF] * d;
            out[b * 32 + 16 + j] = (float)KVALUES_MXFP4[blk[1 + j] >> 4] * d;
        }
    }
}

/* Super-block v2 (136 B per 256 elements): eight 16-byte ggml-order nibble
 * blocks at k*16, eight scales at 128+k (crates/v4flash-kernels/src/mxfp4_tables.rs:10-35). */
DSXO_API void dsxo_mxfp4_dequant_sb2(const uint8_t* sb, int64_t n_super, float* out) {
    for (int64_t s = 0; s < n_super; s++) {
        const uint8_t* w = sb + s * 136;
        for (int b = 0; b < 8; b++) {
            float d = dsxo_e8m0_half(w[128 + b]);
            const uint8_t* qs = w + b * 16;
            for (int j = 0; j < 16; j++) {
                out[s * 256 + b * 32 + j] = (float)KVALUES_MXFP4[qs[j] & 0xF] * d;
                out[s * 256 + b * 32 + 16 + j] = (float)KVALUES_MXFP4[qs[j] >> 4] * d;
            }
        }
    }
}

/* HF layout: packed [rows, K/2] with element 2i in the low nibble of byte i,
 * scales [rows, K/32] E8M0; value = E2M1 * 2^(e-127)
 * (scripts/v41_oracle/kernel.py:18-21,63-70; docs/v41/ARCH_SPEC.md:176-177).
 * Computed as kvalue * 2^(e-128), which is the same real number. */
DSXO_API void dsxo_mxfp4_dequant_hf(const uint8_t* packed, const uint8_t* scales,
                                    int64_t rows, int64_t K, float* out) {
    const int64_t half = K / 2, nb = K / 32;
    for (int64_t r = 0; r < rows; r++)
        for (int64_t i = 0; i < half; i++) {
            float d = dsxo_e8m0_half(scales[r * nb + i / 16]);
            uint8_t q = packed[r * half + i];
            out[r * K + 2 * i] = (float)KVALUES_MXFP4[q & 0xF] * d;
            out[r * K + 2 * i + 1] = (float)KVALUES_MXFP4[q >> 4] * d;
        }
}

/* HF -> super-block v2, crates/v4flash-core/src/hf_v41.rs:1207-1229 (and the
 * GPU twin kernels/mxfp4_repack.hip:35-65). dst is rows * (K/32) * 17 bytes. */
DSXO_API void dsxo_mxfp4_repack_hf_to_sb2(const uint8_t* packed, const uint8_t* scales,
                                          int64_t rows, int64_t K, uint8_t* dst) {
    const int64_t half = K / 2, nb = K / 32;
    for (int64_t r = 0; r < rows; r++) {
        const uint8_t* prow = packed + r * half;
        const uint8_t* srow = scales + r * nb;
        uint8_t* drow = dst + r * nb * 17;
        for (int64_t sb = 0; sb < nb / 8; sb++) {
            uint8_t* sup = drow + sb * 136;
            for (int k = 0; k < 8; k++) {
                int64_t j = sb * 8 + k;
                sup[128 + k] = srow[j];
                const uint8_t* pb = prow + j * 16;
                for (int i = 0; i < 8; i++) {
                    uint8_t lo = pb[i], hi = pb[8 + i];
                    sup[k * 16 + 2 * i] = (uint8_t)((lo & 0x0F) | (hi << 4));
                    sup[k * 16 + 1 + 2 * i] = (uint8_t)((lo >> 4) | (hi & 0xF0));
                }
            }
        }
    }
}

/* ggml 17-byte blocks -> HF layout (inverse nibble shuffle), for loaders that
 * receive GGUF bytes. */
DSXO_API void dsxo_mxfp4_repack_ggml_to_hf(const uint8_t* blocks, int64_t rows, int64_t K,
                                           uint8_t* packed, uint8_t* scales) {
    const int64_t nb = K / 32;
    for (int64_t r = 0; r < rows; r++)
        for (int64_t b = 0; b < nb; b++) {
            const uint8_t* blk = blocks + (r * nb + b) * 17;
            scales[r * nb + b] = blk[0];
            uint8_t el[32];
            for (int j = 0; j < 16; j++) { el[j] = blk[1 + j] & 0xF; el[16 + j] = blk[1 + j] >> 4; }
            for (int i = 0; i < 16; i++)
                packed[r * (K / 2) + b * 16 + i] = (uint8_t)(el[2 * i] | (el[2 * i + 1] << 4));
        }
}

DSXO_API void dsxo_mxfp4_repack_sb2_to_hf(const uint8_t* sb, int64_t rows, int64_t K,
                                          uint8_t* packed, uint8_t* scales) {
    const int64_t nb = K / 32;
    for (int64_t r = 0; r < rows; r++)
        for (int64_t s = 0; s < nb / 8; s++) {
            const uint8_t* sup = sb + r * nb * 17 + s * 136;
            for (int k = 0; k < 8; k++) {
                int64_t b = s * 8 + k;
                scales[r * nb + b] = sup[128 + k];
                uint8_t el[32];
                for (int j = 0; j < 16; j++) { el[j] = sup[k * 16 + j] & 0xF; el[16 + j] = sup[k * 16 + j] >> 4; }
                for (int i = 0; i < 16; i++)
                    packed[r * (K / 2) + b * 16 + i] = (uint8_t)(el[2 * i] | (el[2 * i + 1] << 4));
            }
        }
}

/* ------------------------------------------------------------------- Q8_0 */

/* Weight quantiser, crates/v4flash-core/src/hf_v41.rs:127-137: d = amax/127,
 * q = round-half-away(x/d), stored f16(d) | i8[32]. */
DSXO_API void dsxo_q8_0_quantize_block(const float* x, uint8_t* out34) {
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) { float a = fabsf(x[i]); if (a > amax) amax = a; }
    float d = amax / 127.0f;
    float id = (d == 0.0f) ? 0.0f : 1.0f / d;
    uint16_t h = f32_to_f16(d);
    out34[0] = (uint8_t)(h & 0xFF);
    out34[1] = (uint8_t)(h >> 8);
    for (int i = 0; i < 32; i++) out34[2 + i] = (uint8_t)(int8_t)roundf(x[i] * id);
}

/* 34-byte blocks `f16 d | i8[32]` -> f32 (crates/v4flash-kernels/kernels/q8_0_matvec.hip:5-16). */
DSXO_API void dsxo_q8_0_dequant(const uint8_t* blocks, int64_t n_blocks, float* out) {
    for (int64_t b = 0; b < n_blocks; b++) {
        const uint8_t* blk = blocks + b * 34;
        float d = f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int i = 0; i < 32; i++) out[b * 32 + i] = d * (float)(int8_t)blk[2 + i];
    }
}

/* Activation quantiser of the Q8_0 GEMV, kernels/q8_0_matvec.hip:150-176. */
DSXO_API void dsxo_q8_0_quantize_act(const float* x, int64_t n_blocks, int8_t* xq, float* xscale) {
    for (int64_t b = 0; b < n_blocks; b++) {
        const float* xb = x + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(xb[i]));
        float d = amax / 127.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        xscale[b] = d;
        for (int i = 0; i < 32; i++) {
            long q = lrintf(xb[i] * id);
            if (q > 127) q = 127;
            if (q < -128) q = -128;
            xq[b * 32 + i] = (int8_t)q;
        }
    }
}

/* ------------------------------------------------------------------- Q8_K */

/* kernels/q8_k_quantize.hip:35-89 (host mirror tests/mxfp4_pair_oracle.rs:44-74).
 * Block = f32 d | i8[256] | i16 bsums[16] = 292 bytes. */
DSXO_API void dsxo_q8_k_quantize(const float* x, int64_t n_blocks, uint8_t* out) {
    for (int64_t b = 0; b < n_blocks; b++) {
        const float* xb = x + b * 256;
        uint8_t* blk = out + b * 292;
        /* the kernel's pairwise tree (stride 128..1, upper half taken only when
         * strictly larger) decides which of several equal |x| supplies the sign */
        float s_amax[256], s_max[256];
        for (int i = 0; i < 256; i++) { s_amax[i] = fabsf(xb[i]); s_max[i] = xb[i]; }
        for (int stride = 128; stride > 0; stride >>= 1)
            for (int i = 0; i < stride; i++)
                if (s_amax[i + stride] > s_amax[i]) { s_amax[i] = s_amax[i + stride]; s_max[i] = s_max[i + stride]; }
        float amax = s_amax[0], mxv = s_max[0];
        int8_t* qs = (int8_t*)(blk + 4);
        int16_t* bs = (int16_t*)(blk + 260);
        if (amax == 0.0f) { memset(blk, 0, 292); continue; }
        float iscale = -127.0f / mxv;
        for (int g = 0; g < 16; g++) {
            int sum = 0;
            for (int i = 0; i < 16; i++) {
                int q = (int)rintf(iscale * xb[g * 16 + i]);
                if (q > 127) q = 127;
                if (q < -128) q = -128;
                qs[g * 16 + i] = (int8_t)q;
                sum += q;
            }
            bs[g] = (int16_t)sum;
        }
        float d = 1.0f / iscale;
        memcpy(blk, &d, 4);
    }
}

/* crates/v4flash-kernels/src/mxfp4_tables.rs:49-74 -- super-block v2 weights
 * against Q8_K activations: exact int32 sum per 32-block, f32 scale. */
DSXO_API float dsxo_dot_mxfp4_q8k(int64_t n_super, const uint8_t* w_bytes, const uint8_t* y_bytes) {
    float sumf = 0.0f;
    for (int64_t s = 0; s < n_super; s++) {
        const uint8_t* w = w_bytes + s * 136;
        const uint8_t* y = y_bytes + s * 292;
        float yd; memcpy(&yd, y, 4);
        const int8_t* q8 = (const int8_t*)(y + 4);
        float acc = 0.0f;
        for (int b = 0; b < 8; b++) {
            float scale = dsxo_e8m0_half(w[128 + b]);
            const uint8_t* qs = w + b * 16;
            int32_t sumi = 0;
            for (int j = 0; j < 16; j++) {
                sumi += (int32_t)KVALUES_MXFP4[qs[j] & 0xF] * q8[b * 32 + j];
                sumi += (int32_t)KVALUES_MXFP4[qs[j] >> 4] * q8[b * 32 + 16 + j];
            }
            acc += scale * (float)sumi;
        }
        sumf += yd * acc;
    }
    return sumf;
}

/* ----------------------------------------------------------------- router */

/* Deterministic exp / log built from IEEE +,*,fma only, so the CUDA kernel
 * (same sequence with __fmaf_rn etc.) and this file round identically.  The
 * reference calls libm expf/log1pf (kernels/router_topk.hip:32-36,
 * kernels/laguna_ops.hip:59); these agree with libm to a few ulp. */
static float det_expf(float x) {
    x = fminf(fmaxf(x, -87.0f), 88.0f);
    float n = floorf(fmaf(x, 1.44269504088896341f, 0.5f));
    float r = fmaf(n, -0.693359375f, x);
    r = fmaf(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float r2 = r * r;
    float y = fmaf(p, r2, r);
    y = y + 1.0f;
    return y * bits_f32((uint32_t)((int32_t)n + 127) << 23);
}

static float det_logf(float u) { /* u > 0, normal */
    uint32_t b = f32_bits(u);
    int32_t e = (int32_t)(b >> 23) - 126;
    float m = bits_f32((b & 0x007FFFFFu) | 0x3F000000u); /* [0.5,1) */
    if (m < 0.707106781186547524f) { e -= 1; m = (m + m) - 1.0f; } else { m = m - 1.0f; }
    float z = m * m;
    float y = 7.0376836292e-2f;
    y = fmaf(y, m, -1.1514610310e-1f);
    y = fmaf(y, m, 1.1676998740e-1f);
    y = fmaf(y, m, -1.2420140846e-1f);
    y = fmaf(y, m, 1.4249322787e-1f);
    y = fmaf(y, m, -1.6668057665e-1f);
    y = fmaf(y, m, 2.0000714765e-1f);
    y = fmaf(y, m, -2.4999993993e-1f);
    y = fmaf(y, m, 3.3333331174e-1f);
    y = y * m;
    y = y * z;
    float fe = (float)e;
    y = fmaf(fe, -2.12194440e-4f, y);
    y = fmaf(z, -0.5f, y);
    float r = m + y;
    r = fmaf(fe, 0.693359375f, r);
    return r;
}

static float det_log1pf(float y) { /* y >= 0 */
    float u = 1.0f + y;
    if (u == 1.0f) return y;
    float d = u - 1.0f;
    return det_logf(u) * (y / d);
}

DSXO_API float dsxo_det_expf(float x) { return det_expf(x); }

/* kernels/swiglu_clamp_weighted.hip:16-37: mid[e, r] = silu(min(g, c)) * clamp(u, -c, c) * w[e], left to right in
 * f32.  use_det != 0 evaluates the exponential with det_expf (IEEE add / mul / fma only, what the CUDA operator
 * does: bit-exact against it); 0 uses libm's expf as the reference source reads (the two differ by rounding only). */
DSXO_API void dsxo_swiglu_clamp_weighted(float* mid, const float* gate, const float* up, const float* expert_w, float clamp,
                                         int64_t ff_exp, int64_t n_experts, int use_det) {
    for (int64_t e = 0; e < n_experts; e++)
        for (int64_t r = 0; r < ff_exp; r++) {
            float g = gate[e * ff_exp + r], u = up[e * ff_exp + r];
            if (clamp > 1.0e-6f) {
                if (g > clamp) g = clamp;
                if (u > clamp) u = clamp;
                if (u < -clamp) u = -clamp;
            }
            const float ex = use_det ? det_expf(-g) : expf(-g);
            const float sig = 1.0f / (1.0f + ex);
            float m = g * sig;
            m = m * u;
            m = m * expert_w[e];
            mid[e * ff_exp + r] = m;
        }
}
DSXO_API float dsxo_det_log1pf(float x) { return det_log1pf(x); }

/* kernels/router_topk.hip:32-36 */
static float softplus_stable(float x) {
    if (x > 20.0f) return x;
    if (x < -20.0f) return det_expf(x);
    return det_log1pf(det_expf(x));
}

enum { DSXO_SCORE_SQRT_SOFTPLUS = 0, DSXO_SCORE_SIGMOID = 1 };

DSXO_API float dsxo_router_prob(float logit, int score_fn) {
    if (score_fn == DSXO_SCORE_SIGMOID) return 1.0f / (1.0f + det_expf(-logit)); /* laguna_ops.hip:59 */
    return sqrtf(softplus_stable(logit));                                         /* router_topk.hip:71 */
}

/* Router selection for T rows.
 *   p = f(logit); s = p + bias (kernels/router_topk.hip:71-75)
 *   top-k: k argmax passes, strictly greater wins, equal -> lower index, winner
 *          masked (kernels/router_topk_par.hip:33-64; serial form router_topk.hip:86-101)
 *   w_j = p[sel_j] / max(sum_j p[sel_j], eps) * scale, sum in slot order
 *          (router_topk.hip:103-125).
 * Group limit (NOT in the reference; DeepSeek-V3 convention, parity unpinned):
 *   experts split into n_group contiguous groups; group score = sum of the two
 *   largest s in the group; the topk_group best groups (ties -> lower group)
 *   stay, all other experts are masked to -inf before the top-k.
 *   n_group <= 1 gives the reference algorithm unchanged. */
/* Top-k with the reference's extras (kernels/router_topk_par.hip:18-21,75-81,140-160,164-171,
 * 231-236): n_alt further argmax passes after the first n_used ("alternatives", ranks
 * n_used+1 .. n_used+n_alt; the picks and weights do not depend on n_alt), their weights
 * prob(alt) / (sum of the n_used picks' probs) * scale, and the token's selection-score range
 * max - min over all experts (taken before the group limit masks anything).  alts, alt_w and
 * range_out may be NULL. */
DSXO_API void dsxo_router_topk_ex(const float* logits, const float* bias, int64_t T, int n_expert,
                                  int n_used, int n_group, int topk_group, int score_fn,
                                  float scale, float eps, int32_t* selected, float* weights,
                                  int n_alt, int32_t* alts, float* alt_w, float* range_out) {
    if (!alts) n_alt = 0;
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; t++) {
        float* p = (float*)malloc(sizeof(float) * (size_t)n_expert * 2);
        float* s = p + n_expert;
        const float* lg = logits + t * n_expert;
        float mx = -INFINITY, mn = INFINITY;
        for (int e = 0; e < n_expert; e++) {
            p[e] = dsxo_router_prob(lg[e], score_fn);
            s[e] = bias ? (p[e] + bias[e]) : p[e];
            mx = fmaxf(mx, s[e]);
            mn = fminf(mn, s[e]);
        }
        if (range_out) range_out[t] = mx - mn;
        if (n_group > 1) {
            int per = n_expert / n_group;
            float gs[64];
            int keep[64];
            for (int g = 0; g < n_group; g++) {
                float m1 = -INFINITY, m2 = -INFINITY;
                for (int i = 0; i < per; i++) {
                    float v = s[g * per + i];
                    if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
                }
                gs[g] = m1 + m2;
                keep[g] = 0;
            }
            for (int g = 0; g < n_group; g++) {
                int rank = 0;
                for (int h = 0; h < n_group; h++)
                    if (gs[h] > gs[g] || (gs[h] == gs[g] && h < g)) rank++;
                keep[g] = rank < topk_group;
            }
            for (int e = 0; e < n_expert; e++)
                if (!keep[e / per]) s[e] = -INFINITY;
        }
        int32_t all[64];
        for (int j = 0; j < n_used + n_alt; j++) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < n_expert; e++) {
                int taken = 0;
                for (int q = 0; q < j; q++) if (all[q] == e) taken = 1;
                if (taken) continue;
                if (best < 0 || s[e] > bv) { best = e; bv = s[e]; }
            }
            all[j] = best;
        }
        int32_t* sel = selected + t * n_used;
        for (int j = 0; j < n_used; j++) sel[j] = all[j];
        float sum = 0.0f;
        for (int j = 0; j < n_used; j++) sum += p[sel[j]];
        if (sum < eps) sum = eps;
        for (int j = 0; j < n_used; j++) weights[t * n_used + j] = p[sel[j]] / sum * scale;
        for (int j = 0; j < n_alt; j++) {
            alts[t * n_alt + j] = all[n_used + j];
            if (alt_w) alt_w[t * n_alt + j] = p[all[n_used + j]] / sum * scale;
        }
        free(p);
    }
}

DSXO_API void dsxo_router_topk(const float* logits, const float* bias, int64_t T, int n_expert,
                               int n_used, int n_group, int topk_group, int score_fn,
                               float scale, float eps, int32_t* selected, float* weights) {
    dsxo_router_topk_ex(logits, bias, T, n_expert, n_used, n_group, topk_group, score_fn, scale, eps, selected, weights, 0, NULL, NULL, NULL);
}

/* Top-k with the cache prior (kernels/router_topk_par.hip:82-99,173-210).  No group limit. */
DSXO_API void dsxo_router_topk_prior(const float* logits, const float* bias, int64_t T, int n_expert, int n_used, int score_fn,
                                     float scale, float eps, int32_t* selected, float* weights, int n_alt, int32_t* alts,
                                     float* alt_w, const float* prior, int n_protect, int prior_dry, int32_t* orig_sel) {
    if (!alts) n_alt = 0;
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; t++) {
        float* p = (float*)malloc(sizeof(float) * (size_t)n_expert * 3);
        float* s = p + n_expert;
        float* boost = s + n_expert;
        const float* lg = logits + t * n_expert;
        for (int e = 0; e < n_expert; e++) {
            p[e] = dsxo_router_prob(lg[e], score_fn);
            s[e] = bias ? (p[e] + bias[e]) : p[e];
            boost[e] = s[e] + prior[e];
        }
        int32_t orig[64], sel[64];
        for (int j = 0; j < n_used; j++) {          /* the original top-n_used on the plain scores */
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < n_expert; e++) {
                int taken = 0;
                for (int q = 0; q < j; q++) if (orig[q] == e) taken = 1;
                if (taken) continue;
                if (best < 0 || s[e] > bv) { best = e; bv = s[e]; }
            }
            orig[j] = best;
        }
        for (int j = 0; j < n_protect; j++) sel[j] = orig[j];
        for (int j = n_protect; j < n_used + n_alt; j++) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < n_expert; e++) {
                int taken = 0;
                for (int q = 0; q < j; q++) if (sel[q] == e) taken = 1;
                if (taken) continue;
                if (best < 0 || boost[e] > bv) { best = e; bv = boost[e]; }
            }
            sel[j] = best;
        }
        if (prior_dry)
            for (int j = 0; j < n_used; j++) { int32_t tmp = sel[j]; sel[j] = orig[j]; orig[j] = tmp; }
        float sum = 0.0f;
        for (int j = 0; j < n_used; j++) sum += p[sel[j]];
        if (sum < eps) sum = eps;
        for (int j = 0; j < n_used; j++) {
            selected[t * n_used + j] = sel[j];
            weights[t * n_used + j] = p[sel[j]] / sum * scale;
            if (orig_sel) orig_sel[t * n_used + j] = orig[j];
        }
        for (int j = 0; j < n_alt; j++) {
            alts[t * n_alt + j] = sel[n_used + j];
            if (alt_w) alt_w[t * n_alt + j] = p[sel[n_used + j]] / sum * scale;
        }
        free(p);
    }
}

/* RMSNorm of rows (kernels/rms_norm.hip:48-84): partial j (of 256) = sum over m of x[j + 256 m]^2 in
 * double, cast to f32; the 256 partials fold by a stride-128..1 tree; scale = 1 / sqrt(mean + eps);
 * out = (x * scale) * weight.  The reference's rsqrtf is an approximation of the same value. */
DSXO_API void dsxo_rms_norm_rows(const float* x, const float* weight, int64_t T, int64_t n, float eps, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; t++) {
        const float* xb = x + t * n;
        float sd[256];
        for (int j = 0; j < 256; j++) {
            double partial = 0.0;
            for (int64_t i = j; i < n; i += 256) partial += (double)xb[i] * (double)xb[i];
            sd[j] = (float)partial;
        }
        for (int stride = 128; stride > 0; stride >>= 1)
            for (int j = 0; j < stride; j++) sd[j] = sd[j] + sd[j + stride];
        const float mean_sq = sd[0] / (float)n;
        const float scale = 1.0f / sqrtf(mean_sq + eps);
        for (int64_t i = 0; i < n; i++) out[t * n + i] = (xb[i] * scale) * weight[i];
    }
}

/* Residual mix (kernels/hc_post.hip:36-68): acc = block_out * post[dst]; acc = fma(comb[dst + src*n_hc],
 * residual[src], acc) for src ascending. */
DSXO_API void dsxo_hc_post(const float* block_out, const float* residual_hc, const float* post, const float* comb,
                           int64_t T, int64_t n_embd, int n_hc, float* out_hc) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; t++)
        for (int dst = 0; dst < n_hc; dst++)
            for (int64_t d = 0; d < n_embd; d++) {
                float acc = block_out[t * n_embd + d] * post[t * n_hc + dst];
                for (int src = 0; src < n_hc; src++)
                    acc = fmaf(comb[t * n_hc * n_hc + dst + src * n_hc], residual_hc[(t * n_hc + src) * n_embd + d], acc);
                out_hc[(t * n_hc + dst) * n_embd + d] = acc;
            }
}

/* Router logits: x[T,H] (f32) . W[E,H]^T, f32 inputs, accumulated in double
 * (kernels/f16_matvec.hip:26-45 accumulates f32 per lane then a wave
 * reduction; any f32 association is within 1e-6 of this). */
DSXO_API void dsxo_router_logits(const float* x, const float* W, int64_t T, int n_expert,
                                 int64_t H, float* logits) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t t = 0; t < T; t++)
        for (int e = 0; e < n_expert; e++) {
            double acc = 0.0;
            for (int64_t k = 0; k < H; k++) acc += (double)W[(int64_t)e * H + k] * (double)x[t * H + k];
            logits[t * n_expert + e] = (float)acc;
        }
}

/* ----------------------------------------------- histogram / permute / items */

/* hist[e] = picks of e (kernels/expert_sel_count.hip:17-28,
 * kernels/moe_group_builder.hip:45-47; ids <0 or >= n_expert skipped);
 * offsets = exclusive prefix sum over ascending e
 * (kernels/moe_work_items_builder.hip:102-118); member order inside a group =
 * ascending t*k+s (kernels/b2_fast_chain.hip:94-105); perm[offset[e]+pos] = t*k+s.
 * offsets has n_expert+1 entries.  Returns the number of placed picks. */
DSXO_API int64_t dsxo_group_build(const int32_t* selected, int64_t T, int n_used, int n_expert,
                                  int32_t* hist, int32_t* offsets, int32_t* perm) {
    memset(hist, 0, sizeof(int32_t) * (size_t)n_expert);
    for (int64_t i = 0; i < T * n_used; i++) {
        int32_t e = selected[i];
        if (e >= 0 && e < n_expert) hist[e]++;
    }
    offsets[0] = 0;
    for (int e = 0; e < n_expert; e++) offsets[e + 1] = offsets[e] + hist[e];
    int32_t* cur = (int32_t*)malloc(sizeof(int32_t) * (size_t)n_expert);
    memcpy(cur, offsets, sizeof(int32_t) * (size_t)n_expert);
    for (int64_t i = 0; i < T * n_used; i++) {
        int32_t e = selected[i];
        if (e >= 0 && e < n_expert) perm[cur[e]++] = (int32_t)i;
    }
    free(cur);
    return offsets[n_expert];
}

/* Work items sorted by expert, `(e<<16) | member_start`, ceil(count/chunk) per
 * expert (kernels/moe_work_items_builder.hip:61-145 split variant; packing
 * src/moe_group_builder.rs:18-31).  Returns the item count. */
DSXO_API int32_t dsxo_work_items(const int32_t* hist, int n_expert, int chunk, int32_t* items, int32_t cap) {
    int32_t n = 0;
    for (int e = 0; e < n_expert; e++)
        for (int32_t st = 0; st < hist[e]; st += chunk) {
            if (n < cap) items[n] = (int32_t)(((uint32_t)e << 16) | ((uint32_t)st & 0xFFFFu));
            n++;
        }
    return n;
}

/* crates/v4flash-kernels/src/het/dispatch.rs:444-454 */
DSXO_API uint32_t dsxo_wi_upper_bound(uint64_t members, uint32_t groups, uint32_t chunk, uint64_t cap) {
    uint64_t m = members;
    uint64_t g = m < groups ? m : groups;
    uint32_t c = chunk ? chunk : 1;
    uint64_t b = g + (m + c - 1) / c;
    if (b > m) b = m;
    if (b > cap) b = cap;
    return (uint32_t)b;
}

/* ------------------------------------------------- activation quantisers */

/* f32 -> nearest float8_e4m3fn value (round to nearest even, |x| <= 448 on entry), as a float.
 * scripts/v41_oracle/kernel.py:81-82 (_fake_fp8 = torch's f32 -> float8_e4m3fn cast). */
static float round_e4m3(float x) {
    float a = fabsf(x);
    if (a == 0.0f) return x;
    int e;
    frexpf(a, &e);                 /* a = m * 2^e, m in [0.5, 1) */
    int ex = e - 1;                /* a in [2^ex, 2^(ex+1)) */
    if (ex < -6) ex = -6;          /* subnormals share the smallest normal's spacing 2^-9 */
    const float step = ldexpf(1.0f, ex - 3);
    float q = nearbyintf(a / step) * step;   /* default rounding mode: nearest even */
    if (q > 448.0f) q = 448.0f;
    return copysignf(q, x);
}

/* act_quant with block 32 and ue8m0 scales (scripts/v41_oracle/kernel.py:85-106): per 32 values
 * s = 2^ceil(log2(max(amax, 1e-4) / 448)), y = e4m3(clamp(x / s, +-448)); out = y * s. */
DSXO_API void dsxo_act_quant_e4m3(const float* x, int64_t n, float* out) {
    for (int64_t b = 0; b < n / 32; b++) {
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[b * 32 + i]));
        if (amax < 1e-4f) amax = 1e-4f;
        const float s = exp2f(ceilf(log2f(amax / 448.0f)));
        for (int i = 0; i < 32; i++) {
            float v = x[b * 32 + i] / s;
            if (v > 448.0f) v = 448.0f;
            if (v < -448.0f) v = -448.0f;
            out[b * 32 + i] = round_e4m3(v) * s;
        }
    }
}

/* Nearest E2M1 magnitude code (0..7 -> 0, .5, 1, 1.5, 2, 3, 4, 6), ties to the even mantissa, saturating:
 * scripts/v41_oracle/kernel.py:109-126 (_fake_fp4). */
static int e2m1_code(float a) {
    static const float grid[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    if (a >= 6.0f) return 7;
    int lo = 0;
    while (lo < 7 && grid[lo + 1] <= a) lo++;
    const float dl = a - grid[lo], du = grid[lo + 1] - a;
    if (dl < du) return lo;
    if (du < dl) return lo + 1;
    return (lo & 1) ? lo + 1 : lo;   /* even codes have an even mantissa */
}

/* The MXFP4 expansion of an activation row used by the block-scaled tensor-core kernel: term t is the
 * reference's FP4 fake-quant (fp4_act_quant with E8M0 scales and block 32, scripts/v41_oracle/kernel.py:129-147:
 * s = 2^ceil(log2(amax / 6)), codes = nearest E2M1 of x / s) of what terms 0..t-1 left over.  The scale is found
 * from the bits of amax (amax = m * 2^E: s = 2^(E-2), doubled when m > 1.5), which is that formula without a
 * logarithm, with the E8M0 byte kept inside 1..253.  Every step is exact in f32.
 * codes: n_terms x n/2 bytes (element 2i in the low nibble), scales: n_terms x n/32 E8M0 bytes, sum: the
 * n values the terms add up to (any output may be NULL). */
DSXO_API void dsxo_act_terms_mxfp4(const float* x, int64_t n, int n_terms, uint8_t* codes, uint8_t* scales, float* sum) {
    float* res = (float*)malloc(sizeof(float) * (size_t)n);
    memcpy(res, x, sizeof(float) * (size_t)n);
    if (sum) memset(sum, 0, sizeof(float) * (size_t)n);
    for (int t = 0; t < n_terms; t++)
        for (int64_t b = 0; b < n / 32; b++) {
            float amax = 0.0f;
            for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(res[b * 32 + i]));
            const uint32_t bits = f32_bits(amax);
            int e = (int)(bits >> 23) - 2 + ((bits & 0x7FFFFFu) > 0x400000u ? 1 : 0);
            if (e < 1) e = 1;
            if (e > 253) e = 253;
            const float s = bits_f32((uint32_t)e << 23), inv = bits_f32((uint32_t)(254 - e) << 23);
            if (scales) scales[(int64_t)t * (n / 32) + b] = (uint8_t)e;
            for (int i = 0; i < 32; i++) {
                const int64_t j = b * 32 + i;
                const float v = res[j] * inv;
                const int c = e2m1_code(fabsf(v)) | (v < 0.0f || (v == 0.0f && signbit(v)) ? 8 : 0);
                const float d = (float)KVALUES_MXFP4[c] * 0.5f * s;
                if (codes) {
                    uint8_t* p = codes + (int64_t)t * (n / 2) + j / 2;
                    *p = (j & 1) ? (uint8_t)((*p & 0x0F) | (c << 4)) : (uint8_t)((*p & 0xF0) | c);
                }
                if (sum) sum[j] += d;
                res[j] -= d;
            }
        }
    free(res);
}

/* What a row of activations becomes before a product, by act_mode:
 *   0      unchanged (the dequantised-f32 reference, the tolerance target)
 *   1      one E4M3 term (act_quant above: the model's own FP8 activation numerics, docs/v41/ARCH_SPEC.md:131-133)
 *   2      two E4M3 terms (the second quantises what the first left over)
 *   10 + k k MXFP4 terms (dsxo_act_terms_mxfp4) */
static void apply_act_mode(int act_mode, float* row, int64_t n) {
    if (act_mode == 0) return;
    float* tmp = (float*)malloc(sizeof(float) * (size_t)n);
    if (act_mode == 1 || act_mode == 2) {
        dsxo_act_quant_e4m3(row, n, tmp);
        if (act_mode == 2) {
            float* res = (float*)malloc(sizeof(float) * (size_t)n);
            float* t2 = (float*)malloc(sizeof(float) * (size_t)n);
            for (int64_t i = 0; i < n; i++) res[i] = row[i] - tmp[i];
            dsxo_act_quant_e4m3(res, n, t2);
            for (int64_t i = 0; i < n; i++) tmp[i] += t2[i];
            free(res); free(t2);
        }
    } else {
        dsxo_act_terms_mxfp4(row, n, act_mode - 10, NULL, NULL, tmp);
    }
    memcpy(row, tmp, sizeof(float) * (size_t)n);
    free(tmp);
}

/* ------------------------------------------------------------ expert FFN */

enum { DSXO_FMT_MXFP4 = 0, DSXO_FMT_Q8_0 = 1 };

/* A weight matrix [rows, K] in its canonical host layout:
 *   MXFP4: HF layout -- q = packed [rows, K/2], s = E8M0 [rows, K/32]
 *   Q8_0 : q = int8 [rows, K], s = f16 bits [rows, K/32] (the split form of
 *          crates/v4flash-kernels/src/weights.rs:215-240)                   */
static void dequant_row(int fmt, const uint8_t* q, const uint8_t* s, int64_t K, int64_t r, float* out) {
    const int64_t nb = K / 32;
    if (fmt == DSXO_FMT_MXFP4) {
        const uint8_t* qr = q + r * (K / 2);
        for (int64_t b = 0; b < nb; b++) {
            float d = dsxo_e8m0_half(s[r * nb + b]);
            for (int i = 0; i < 16; i++) {
                uint8_t v = qr[b * 16 + i];
                out[b * 32 + 2 * i] = (float)KVALUES_MXFP4[v & 0xF] * d;
                out[b * 32 + 2 * i + 1] = (float)KVALUES_MXFP4[v >> 4] * d;
            }
        }
    } else {
        const int8_t* qr = (const int8_t*)q + r * K;
        const uint16_t* sr = (const uint16_t*)s + r * nb;
        for (int64_t b = 0; b < nb; b++) {
            float d = f16_to_f32(sr[b]);
            for (int i = 0; i < 32; i++) out[b * 32 + i] = d * (float)qr[b * 32 + i];
        }
    }
}

DSXO_API void dsxo_dequant_matrix(int fmt, const uint8_t* q, const uint8_t* s, int64_t rows, int64_t K, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) dequant_row(fmt, q, s, K, r, out + r * K);
}

static inline int64_t qbytes(int fmt, int64_t rows, int64_t K) { return fmt == DSXO_FMT_MXFP4 ? rows * K / 2 : rows * K; }
static inline int64_t sbytes(int fmt, int64_t rows, int64_t K) { return fmt == DSXO_FMT_MXFP4 ? rows * K / 32 : rows * K / 32 * 2; }

/* One expert FFN applied to n activation rows (dequantised-weight arithmetic):
 *   g = Wg x, u = Wu x; clamp (kernels/swiglu_clamp_weighted.hip:28-33: g<=c,
 *   |u|<=c, only when c>1e-6); mid = g*sigmoid(g)*u*w (:34-35; the routing
 *   weight multiplies mid, docs/v41/ARCH_SPEC.md:128); out = Wd mid
 *   (kernels/mxfp4_matvec.hip:141-154).
 * Dots accumulate in double over dequantised f32 weights.  mid_round: 0 = keep
 * f32, 1 = round mid to f16, 2 = round mid to bf16 (what the GPU paths store
 * between the two products). */
static void expert_ffn(int fmt, const uint8_t* gq, const uint8_t* gs, const uint8_t* uq, const uint8_t* us,
                       const uint8_t* dq, const uint8_t* ds, int64_t H, int64_t F, float clamp,
                       int n, const float* const* xs, const float* ws, float* const* outs, int mid_round, int act_mode) {
    float* mid = (float*)malloc(sizeof(float) * (size_t)(F * n));
#pragma omp parallel
    {
        float* row = (float*)malloc(sizeof(float) * (size_t)(H > F ? H : F) * 2);
        float* row2 = row + (H > F ? H : F);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < F; r++) {
            dequant_row(fmt, gq, gs, H, r, row);
            dequant_row(fmt, uq, us, H, r, row2);
            /* four tokens at a time: eight independent sums in flight, each still added in k order */
            double ag4[4], au4[4];
            for (int i = 0; i < n; i++) {
                if ((i & 3) == 0) {
                    const int m4 = n - i < 4 ? n - i : 4;
                    const float* x0 = xs[i];
                    const float* x1 = xs[i + (m4 > 1 ? 1 : 0)];
                    const float* x2 = xs[i + (m4 > 2 ? 2 : 0)];
                    const float* x3 = xs[i + (m4 > 3 ? 3 : 0)];
                    double g0 = 0.0, g1 = 0.0, g2 = 0.0, g3 = 0.0, u0 = 0.0, u1 = 0.0, u2 = 0.0, u3 = 0.0;
                    for (int64_t k = 0; k < H; k++) {
                        const double a = (double)row[k], b = (double)row2[k];
                        g0 += a * x0[k]; u0 += b * x0[k];
                        g1 += a * x1[k]; u1 += b * x1[k];
                        g2 += a * x2[k]; u2 += b * x2[k];
                        g3 += a * x3[k]; u3 += b * x3[k];
                    }
                    ag4[0] = g0; ag4[1] = g1; ag4[2] = g2; ag4[3] = g3;
                    au4[0] = u0; au4[1] = u1; au4[2] = u2; au4[3] = u3;
                }
                float g = (float)ag4[i & 3], u = (float)au4[i & 3];
                if (clamp > 1.0e-6f) {
                    if (g > clamp) g = clamp;
                    if (u > clamp) u = clamp;
                    if (u < -clamp) u = -clamp;
                }
                float sig = 1.0f / (1.0f + expf(-g));
                float m = g * sig * u * ws[i];
                if (mid_round == 1) m = f16_to_f32(f32_to_f16(m));
                else if (mid_round == 2) m = bf16_to_f32(f32_to_bf16(m));
                mid[(int64_t)i * F + r] = m;
            }
        }
        if (act_mode != 0) {   /* the rows of mid as the second product's kernel sees them */
#pragma omp for schedule(static)
            for (int i = 0; i < n; i++) apply_act_mode(act_mode, mid + (int64_t)i * F, F);
        }
#pragma omp for schedule(static)
        for (int64_t r = 0; r < H; r++) {
            dequant_row(fmt, dq, ds, F, r, row);
            for (int i = 0; i < n; i += 4) {
                const int m4 = n - i < 4 ? n - i : 4;
                const float* m0 = mid + (int64_t)i * F;
                const float* m1 = mid + (int64_t)(i + (m4 > 1 ? 1 : 0)) * F;
                const float* m2 = mid + (int64_t)(i + (m4 > 2 ? 2 : 0)) * F;
                const float* m3 = mid + (int64_t)(i + (m4 > 3 ? 3 : 0)) * F;
                double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
                for (int64_t k = 0; k < F; k++) {
                    const double w = (double)row[k];
                    a0 += w * m0[k]; a1 += w * m1[k]; a2 += w * m2[k]; a3 += w * m3[k];
                }
                outs[i][r] = (float)a0;
                if (m4 > 1) outs[i + 1][r] = (float)a1;
                if (m4 > 2) outs[i + 2][r] = (float)a2;
                if (m4 > 3) outs[i + 3][r] = (float)a3;
            }
        }
        free(row);
    }
    free(mid);
}

/* Whole MoE layer, dequantised-f32 reference (the tolerance target):
 *   partial[t,s,:] = expert(sel[t,s])(x[t]) with weight w[t,s]
 *   out[t,:] = 0 + partial[t,0] + ... + partial[t,k-1]   (slot order,
 *              kernels/q2_k_accumulate_matvec_par.hip:724-729)
 *   out[t,:] += shared(x[t])                             (src/ffn.rs:118-151 vec_add)
 * Expert e of a routed matrix lives at e * bytes_per_expert in each plane.
 * shared_* may be NULL (no shared expert).  partials_out (optional) receives
 * the [T*k+T, H] rows (routed in (t,s) order, then shared). */
DSXO_API void dsxo_moe_layer_act(
        int fmt, int64_t T, int64_t H, int64_t F, int n_expert, int n_used,
        const float* x_in, const int32_t* selected, const float* weights,
        const uint8_t* gate_q, const uint8_t* gate_s, const uint8_t* up_q, const uint8_t* up_s,
        const uint8_t* down_q, const uint8_t* down_s,
        int shared_fmt, int64_t Fs,
        const uint8_t* sg_q, const uint8_t* sg_s, const uint8_t* su_q, const uint8_t* su_s,
        const uint8_t* sd_q, const uint8_t* sd_s,
        float clamp, int mid_round, int act_mode, float* out, float* partials_out) {
    const int64_t P = T * n_used;
    /* act_mode != 0: both products see their activation rows (x, then mid) through apply_act_mode */
    float* xq = NULL;
    const float* x = x_in;
    if (act_mode != 0) {
        xq = (float*)malloc(sizeof(float) * (size_t)(T * H));
        memcpy(xq, x_in, sizeof(float) * (size_t)(T * H));
#pragma omp parallel for schedule(static)
        for (int64_t t = 0; t < T; t++) apply_act_mode(act_mode, xq + t * H, H);
        x = xq;
    }
    float* partial = partials_out ? partials_out : (float*)malloc(sizeof(float) * (size_t)((P + T) * H));
    memset(partial, 0, sizeof(float) * (size_t)((P + T) * H));
    int32_t* hist = (int32_t*)malloc(sizeof(int32_t) * (size_t)n_expert);
    int32_t* offs = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n_expert + 1));
    int32_t* perm = (int32_t*)malloc(sizeof(int32_t) * (size_t)(P > 0 ? P : 1));
    dsxo_group_build(selected, T, n_used, n_expert, hist, offs, perm);
    const int64_t gq_b = qbytes(fmt, F, H), gs_b = sbytes(fmt, F, H);
    const int64_t dq_b = qbytes(fmt, H, F), ds_b = sbytes(fmt, H, F);
    for (int e = 0; e < n_expert; e++) {
        int n = hist[e];
        if (!n) continue;
        const float** xs = (const float**)malloc(sizeof(float*) * (size_t)n);
        float** outs = (float**)malloc(sizeof(float*) * (size_t)n);
        float* ws = (float*)malloc(sizeof(float) * (size_t)n);
        for (int i = 0; i < n; i++) {
            int32_t ts = perm[offs[e] + i];
            xs[i] = x + (int64_t)(ts / n_used) * H;
            outs[i] = partial + (int64_t)ts * H;
            ws[i] = weights[ts];
        }
        expert_ffn(fmt, gate_q + e * gq_b, gate_s + e * gs_b, up_q + e * gq_b, up_s + e * gs_b,
                   down_q + e * dq_b, down_s + e * ds_b, H, F, clamp, n, xs, ws, outs, mid_round, act_mode);
        free(xs); free(outs); free(ws);
    }
    if (sg_q) {
        const float** xs = (const float**)malloc(sizeof(float*) * (size_t)T);
        float** outs = (float**)malloc(sizeof(float*) * (size_t)T);
        float* ws = (float*)malloc(sizeof(float) * (size_t)T);
        for (int64_t t = 0; t < T; t++) { xs[t] = x + t * H; outs[t] = partial + (P + t) * H; ws[t] = 1.0f; }
        expert_ffn(shared_fmt, sg_q, sg_s, su_q, su_s, sd_q, sd_s, H, Fs, clamp, (int)T, xs, ws, outs, mid_round, act_mode);
        free(xs); free(outs); free(ws);
    }
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; t++)
        for (int64_t r = 0; r < H; r++) {
            float acc = 0.0f;
            for (int s = 0; s < n_used; s++) acc += partial[(t * n_used + s) * H + r];
            if (sg_q) acc += partial[(P + t) * H + r];
            out[t * H + r] = acc;
        }
    free(hist); free(offs); free(perm);
    free(xq);
    if (!partials_out) free(partial);
}

DSXO_API void dsxo_moe_layer_f32(
        int fmt, int64_t T, int64_t H, int64_t F, int n_expert, int n_used,
        const float* x, const int32_t* selected, const float* weights,
        const uint8_t* gate_q, const uint8_t* gate_s, const uint8_t* up_q, const uint8_t* up_s,
        const uint8_t* down_q, const uint8_t* down_s,
        int shared_fmt, int64_t Fs,
        const uint8_t* sg_q, const uint8_t* sg_s, const uint8_t* su_q, const uint8_t* su_s,
        const uint8_t* sd_q, const uint8_t* sd_s,
        float clamp, int mid_round, float* out, float* partials_out) {
    dsxo_moe_layer_act(fmt, T, H, F, n_expert, n_used, x, selected, weights, gate_q, gate_s, up_q, up_s, down_q, down_s, shared_fmt, Fs,
                       sg_q, sg_s, su_q, su_s, sd_q, sd_s, clamp, mid_round, 0, out, partials_out);
}

/* Reference-numerics variant of one routed pick for MXFP4 (the int8 path the
 * HIP kernels run): x -> Q8_K, g/u = MXFP4.Q8_K dots
 * (kernels/mxfp4_pair_matvec.hip:118-149), clamp+SwiGLU+weight, mid -> Q8_K
 * (het/forward_prefill.rs:11884-11892), down dot.  Weights arrive in HF layout
 * and are repacked to super-block v2 row by row.  out has H floats. */
DSXO_API void dsxo_expert_ref_int_mxfp4(const uint8_t* gq, const uint8_t* gs, const uint8_t* uq, const uint8_t* us,
                                        const uint8_t* dq, const uint8_t* ds, int64_t H, int64_t F,
                                        float clamp, const float* x, float w, float* out) {
    uint8_t* xq = (uint8_t*)malloc((size_t)(H / 256 * 292));
    dsxo_q8_k_quantize(x, H / 256, xq);
    float* mid = (float*)malloc(sizeof(float) * (size_t)F);
#pragma omp parallel
    {
        uint8_t* rowg = (uint8_t*)malloc((size_t)((H > F ? H : F) / 32 * 17) * 2);
        uint8_t* rowu = rowg + (H > F ? H : F) / 32 * 17;
#pragma omp for schedule(static)
        for (int64_t r = 0; r < F; r++) {
            dsxo_mxfp4_repack_hf_to_sb2(gq + r * H / 2, gs + r * H / 32, 1, H, rowg);
            dsxo_mxfp4_repack_hf_to_sb2(uq + r * H / 2, us + r * H / 32, 1, H, rowu);
            float g = dsxo_dot_mxfp4_q8k(H / 256, rowg, xq);
            float u = dsxo_dot_mxfp4_q8k(H / 256, rowu, xq);
            if (clamp > 1.0e-6f) {
                if (g > clamp) g = clamp;
                if (u > clamp) u = clamp;
                if (u < -clamp) u = -clamp;
            }
            float sig = 1.0f / (1.0f + expf(-g));
            mid[r] = g * sig * u * w;
        }
        free(rowg);
    }
    uint8_t* mq = (uint8_t*)malloc((size_t)(F / 256 * 292));
    dsxo_q8_k_quantize(mid, F / 256, mq);
#pragma omp parallel
    {
        uint8_t* rowd = (uint8_t*)malloc((size_t)(F / 32 * 17));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < H; r++) {
            dsxo_mxfp4_repack_hf_to_sb2(dq + r * F / 2, ds + r * F / 32, 1, F, rowd);
            out[r] = dsxo_dot_mxfp4_q8k(F / 256, rowd, mq);
        }
        free(rowd);
    }
    free(xq); free(mid); free(mq);
}

DSXO_API int dsxo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
