/* moe_oracle.c -- CPU restatement of the reference's quantized MoE feed-forward path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: the test-suite,
 * the smoke check and the benchmark's CPU-baseline leg are its only users.  Nothing in the
 * shipped library links, loads or calls it.
 *
 * Every function names the reference code it restates (paths are relative to the reference
 * project root).  Integer results (routing indices, Q8_1 bytes, per-block integer dots, the
 * dispatch permutation) are meant to be compared bit for bit; fp32 results within the stated
 * tolerance, because float summation order and the host's expf differ from the GPU's.
 *
 * Pinning: the known-answer values held by the reference's own tests are checked against this
 * file in tests/test_oracle_golden.py (top-k cases of src/moe_forward.rs:321-404 and
 * src/raw_forward.rs:1856-1904, Q8_1 cases of ffi/src/lib.rs:965-1044, Q8_0 block of
 * src/gguf_loader.rs:1765-1790, SwiGLU values of src/expert.rs:356-411, dot/sigmoid-gate
 * cases of src/scratch_pool.rs:412-491), and on a GPU box the reference's own kernels
 * (chimere-server/kernels/chimere_kernels.cu compiled for sm_100a into oracle/_ref/) are run
 * on the same inputs.  The K-quant decoders and dots (Q4_K, Q5_K, Q6_K) are checked in tests/test_kquants.py against
 * an independent decoder (the gguf Python package's dequantize) and with the reference's own Q5_K tests
 * (ffi/src/lib.rs:1150-1270).  Not pinned by anything in the reference (no implementation there):
 * Q4_0 x Q8_1 integer dots, the dispatch permutation, the sigmoid/top-6 router variant and
 * the squared-ReLU expert -- for those this file is the definition ("parity unpinned").
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../include/chimere_b200_moe.h"

static const uint32_t iq3s_grid[512] = {
#include "iq3s_grid.inc"
};

#define Q8_1_BYTES 36
#define Q4_0_BYTES 18
#define Q8_0_BYTES 34
#define IQ3S_BYTES 110
#define Q4_K_BYTES 144
#define Q5_K_BYTES 176
#define Q6_K_BYTES 210

/* ------------------------------------------------------------------ f16 <-> f32 (IEEE) --- */

/* Round-to-nearest-even f32 -> f16, what __float2half does in ggml_quantize_q8_1
 * (chimere-server/kernels/chimere_kernels.cu:1522). */
uint16_t orc_f32_to_f16(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | (ax > 0x7F800000u ? 0x7E00u : 0x7C00u));
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);           /* rounds to inf */
    if (ax < 0x33000001u) return (uint16_t)sign;                         /* rounds to zero (< 2^-25) */
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }                  /* subnormal result */
    else { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7FFFFFu; }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q));                                /* carry into exponent is correct */
}

float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, x;
    if (e == 0) {
        if (m == 0) x = sign;
        else { float r = (float)m * (1.0f / 16777216.0f); memcpy(&x, &r, 4); x |= sign; }
    } else if (e == 31) x = sign | 0x7F800000u | (m << 13);
    else x = sign | ((e + 112u) << 23) | (m << 13);
    float f; memcpy(&f, &x, 4); return f;
}

/* Truncating f32 -> f16 with subnormals flushed, as the reference's own helper does
 * (chimere_kernels.cu:49-60); used only by the own-dialect Q8_1 quantizer below. */
static uint16_t f32_to_f16_trunc(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    uint32_t sign = (u >> 31) & 1u;
    int e = (int)((u >> 23) & 0xFFu) - 127;
    uint32_t m = u & 0x7FFFFFu;
    if (e >= 16) return (uint16_t)((sign << 15) | 0x7C00u);
    if (e < -14) return (uint16_t)(sign << 15);
    return (uint16_t)((sign << 15) | ((uint32_t)(e + 15) << 10) | (m >> 13));
}

/* --------------------------------------------------------------------- router pieces ---- */

/* One dot product in the reference's summation order: 256 partial sums, partial p taking
 * elements p, p+256, ... with one fused multiply-add each (nvcc contracts acc += a*b), then a
 * binary tree over the 256 partials with strides 128..1.
 * f32_gemv_kernel, chimere_kernels.cu:706-741; dot_product_kernel, src/scratch_pool.rs:243-261. */
float orc_dot_strided256(const float* a, const float* x, int n) {
    float part[256];
    for (int p = 0; p < 256; p++) {
        float acc = 0.0f;
        for (int j = p; j < n; j += 256) acc = fmaf(a[j], x[j], acc);
        part[p] = acc;
    }
    for (int s = 128; s > 0; s >>= 1)
        for (int p = 0; p < s; p++) part[p] += part[p + s];
    return part[0];
}

/* Router logits for one token: logits[e] = W[e] . x (+ bias[e]).  moe_ffn.rs:1099-1110. */
void orc_router_logits(const float* W, const float* bias, const float* x, int E, int H, float* logits) {
    for (int e = 0; e < E; e++) {
        float v = orc_dot_strided256(W + (size_t)e * H, x, H);
        logits[e] = bias ? v + bias[e] : v;
    }
}

/* k largest of score[0..E) by repeated strict-greater scan from index 0, so the lowest index
 * wins a tie; selected entries are overwritten with -1.  chimere_kernels.cu:1201-1216. */
static float select_topk(float* score, int E, int k, int32_t* idx, float* w) {
    float wsum = 0.0f;
    for (int j = 0; j < k; j++) {
        int best = 0; float bv = -1.0f;
        for (int i = 0; i < E; i++) if (score[i] > bv) { bv = score[i]; best = i; }
        idx[j] = best; w[j] = bv; wsum += bv; score[best] = -1.0f;
    }
    return wsum;
}

/* Softmax over E logits, top-k on the probabilities, weights renormalised by multiplying with
 * 1/sum.  topk_softmax, chimere_kernels.cu:1150-1223 (block of 256 threads, E <= 256): the
 * exponentials are summed by a tree with strides 128..1 where element i+stride is added into
 * element i only when i+stride < E.  probs_out (optional) receives the E probabilities. */
void orc_topk_softmax(const float* logits, int E, int k, int32_t* idx, float* w, float* probs_out) {
    float p[256], ev[256];
    float mx = logits[0];
    for (int i = 1; i < E; i++) mx = fmaxf(mx, logits[i]);
    for (int i = 0; i < E; i++) { ev[i] = expf(logits[i] - mx); p[i] = ev[i]; }
    for (int s = 128; s > 0; s >>= 1)
        for (int i = 0; i < s; i++) if (i + s < E) p[i] += p[i + s];
    float sum = p[0];
    for (int i = 0; i < E; i++) p[i] = (sum > 0.0f) ? ev[i] / sum : 1.0f / (float)E;
    if (probs_out) memcpy(probs_out, p, sizeof(float) * (size_t)E);
    float wsum = select_topk(p, E, k, idx, w);
    if (wsum > 0.0f) { float inv = 1.0f / wsum; for (int j = 0; j < k; j++) w[j] *= inv; }
}

/* Sigmoid scores, top-k, selected scores normalised to sum 1 and multiplied by `scale`.
 * Not implemented in the reference's own sources (it runs inside libllama,
 * src/generic_model.rs:1-15); this follows the benchmark configuration's wording and uses
 * the same selection loop and the same "multiply by 1/sum" as the softmax router. */
void orc_topk_sigmoid(const float* logits, int E, int k, float scale, int32_t* idx, float* w, float* probs_out) {
    float p[256];
    for (int i = 0; i < E; i++) p[i] = 1.0f / (1.0f + expf(-logits[i]));
    if (probs_out) memcpy(probs_out, p, sizeof(float) * (size_t)E);
    float wsum = select_topk(p, E, k, idx, w);
    if (wsum > 0.0f) { float inv = 1.0f / wsum; for (int j = 0; j < k; j++) w[j] = w[j] * inv * scale; }
}

/* ----------------------------------------------------------------- Q8_1 quantization ---- */

/* ggml-compatible Q8_1 of n floats (n multiple of 32): per block d = amax/127 (fp32),
 * q = (int8)roundf(x/d), stored d = f16_rn(d), s = f16_rn(sum of the raw floats), the sum taken
 * as an xor-butterfly over the 32 lanes (offsets 16,8,4,2,1).
 * ggml_quantize_q8_1, chimere_kernels.cu:1495-1523; reductions :1327-1342. */
void orc_quantize_q8_1(const float* x, uint8_t* out, int n) {
    for (int b = 0; b < n / 32; b++) {
        const float* xb = x + (size_t)b * 32;
        uint8_t* ob = out + (size_t)b * Q8_1_BYTES;
        float amax = 0.0f, s[32];
        for (int i = 0; i < 32; i++) { amax = fmaxf(amax, fabsf(xb[i])); s[i] = xb[i]; }
        for (int off = 16; off > 0; off >>= 1) {
            float t[32];
            for (int i = 0; i < 32; i++) t[i] = s[i] + s[i ^ off];
            memcpy(s, t, sizeof s);
        }
        float d = amax / 127.0f;
        for (int i = 0; i < 32; i++)
            ((int8_t*)ob)[4 + i] = (amax == 0.0f) ? (int8_t)0 : (int8_t)roundf(xb[i] / d);
        uint16_t dh = orc_f32_to_f16(d), sh = orc_f32_to_f16(s[0]);
        memcpy(ob, &dh, 2); memcpy(ob + 2, &sh, 2);
    }
}

/* The reference's own dialect: d = amax/127, q = (int)(x*(1/d) +- 0.5) clamped to +-127,
 * d stored truncated to f16, s = f16_trunc(d * sum q).  quantize_q8_1_block,
 * chimere_kernels.cu:754-777.  Kept to show where the two dialects agree. */
void orc_quantize_q8_1_own(const float* x, uint8_t* out, int n) {
    for (int b = 0; b < n / 32; b++) {
        const float* xb = x + (size_t)b * 32;
        uint8_t* ob = out + (size_t)b * Q8_1_BYTES;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) { float ax = xb[i] < 0.0f ? -xb[i] : xb[i]; if (ax > amax) amax = ax; }
        float scale = amax / 127.0f;
        float inv = (scale > 0.0f) ? (1.0f / scale) : 0.0f;
        int sum = 0;
        for (int i = 0; i < 32; i++) {
            float fq = xb[i] * inv;
            int q = (int)(fq + (fq >= 0.0f ? 0.5f : -0.5f));
            if (q > 127) q = 127;
            if (q < -127) q = -127;
            ((int8_t*)ob)[4 + i] = (int8_t)q; sum += q;
        }
        uint16_t dh = f32_to_f16_trunc(scale), sh = f32_to_f16_trunc(scale * (float)sum);
        memcpy(ob, &dh, 2); memcpy(ob + 2, &sh, 2);
    }
}

/* ------------------------------------------------------------- per-block integer dots --- */

/* IQ3_S sub-block `sg` (32 weights) of a 110-byte super-block against one Q8_1 block:
 * sumi = (sum of +-grid * q8) * (1 + 2*scale_nibble).  Layout: d f16 @0, qs[64] @2, qh[8] @66,
 * signs[32] @74, scales[4] @106.  Grid index = qs byte | (bit of qh) << 8; sign bit i of the
 * sub-block's 32 sign bits negates weight i.  dot_iq3s_q8_subgroup, chimere_kernels.cu:788-862;
 * decode order as dequantize_iq3_s, src/gguf_loader.rs:1022-1170. */
static inline int32_t iq3s_sub_sumi(const uint8_t* blk, const int8_t* q8, int sg) {
    const uint8_t* qs = blk + 2 + sg * 8;
    uint32_t qh = blk[66 + sg];
    const uint8_t* sgn = blk + 74 + sg * 4;
    int32_t sumi = 0;
    for (int g = 0; g < 8; g++) {
        uint32_t gi = qs[g] | (((qh >> g) & 1u) << 8);
        uint32_t gv = iq3s_grid[gi];
        uint32_t sb = sgn[g >> 1] >> ((g & 1) * 4);
        for (int i = 0; i < 4; i++) {
            int32_t m = (int32_t)((gv >> (8 * i)) & 0xFFu);
            if ((sb >> i) & 1u) m = -m;
            sumi += m * (int32_t)q8[g * 4 + i];
        }
    }
    uint8_t scb = blk[106 + sg / 2];
    int nib = (sg & 1) ? (scb >> 4) : (scb & 0x0F);
    return sumi * (1 + 2 * nib);
}

/* Q4_0 block (f16 d, 16 bytes; low nibbles = elements 0..15, high = 16..31, value nibble-8;
 * dequantize_q4_0, src/gguf_loader.rs:752-772) against one Q8_1 block: sum (nib-8)*q8.
 * The reference has no own Q4_0 x Q8_1 kernel; this is its dequantisation rule applied to
 * integers. */
static inline int32_t q4_0_sumi(const uint8_t* blk, const int8_t* q8) {
    int32_t sumi = 0;
    for (int j = 0; j < 16; j++) {
        int lo = (blk[2 + j] & 0x0F) - 8, hi = (blk[2 + j] >> 4) - 8;
        sumi += lo * (int32_t)q8[j] + hi * (int32_t)q8[j + 16];
    }
    return sumi;
}

/* Q8_0 block (f16 d, 32 int8; dequantize_q8_0, src/gguf_loader.rs:793-837) against one Q8_1
 * block.  dot_q8_0_q8_1, src/kernels/gemv_q8_0.rs:230-255. */
static inline int32_t q8_0_sumi(const uint8_t* blk, const int8_t* q8) {
    int32_t sumi = 0;
    const int8_t* qw = (const int8_t*)(blk + 2);
    for (int j = 0; j < 32; j++) sumi += (int32_t)qw[j] * (int32_t)q8[j];
    return sumi;
}

int64_t orc_row_bytes(int type, int ncols) {
    switch (type) {
        case CHIMERE_TYPE_Q4_0: return (int64_t)(ncols / 32) * Q4_0_BYTES;
        case CHIMERE_TYPE_Q8_0: return (int64_t)(ncols / 32) * Q8_0_BYTES;
        case CHIMERE_TYPE_IQ3_S: return (int64_t)(ncols / 256) * IQ3S_BYTES;
        case CHIMERE_TYPE_Q4_K: return (int64_t)(ncols / 256) * Q4_K_BYTES;
        case CHIMERE_TYPE_Q5_K: return (int64_t)(ncols / 256) * Q5_K_BYTES;
        case CHIMERE_TYPE_Q6_K: return (int64_t)(ncols / 256) * Q6_K_BYTES;
        default: return -1;
    }
}

/* Block b (32 columns) of one weight row: integer dot and the row's f16 scale for it. */
static inline int32_t row_block_sumi(int type, const uint8_t* row, int b, const int8_t* q8, float* dw) {
    uint16_t dh;
    switch (type) {
        case CHIMERE_TYPE_Q4_0: { const uint8_t* blk = row + (size_t)b * Q4_0_BYTES; memcpy(&dh, blk, 2); *dw = orc_f16_to_f32(dh); return q4_0_sumi(blk, q8); }
        case CHIMERE_TYPE_Q8_0: { const uint8_t* blk = row + (size_t)b * Q8_0_BYTES; memcpy(&dh, blk, 2); *dw = orc_f16_to_f32(dh); return q8_0_sumi(blk, q8); }
        default: { const uint8_t* blk = row + (size_t)(b / 8) * IQ3S_BYTES; memcpy(&dh, blk, 2); *dw = orc_f16_to_f32(dh); return iq3s_sub_sumi(blk, q8, b % 8); }
    }
}

/* sumi[nrows][ncols/32]: the exact integer block dots of `nrows` rows against one Q8_1 row. */
void orc_block_sumi(int type, const void* W, const void* xq8, int32_t* sumi, int ncols, int nrows) {
    int nb = ncols / 32; int64_t rb = orc_row_bytes(type, ncols);
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < nrows; r++) {
        const uint8_t* row = (const uint8_t*)W + (size_t)r * rb;
        for (int b = 0; b < nb; b++) {
            float dw;
            sumi[(size_t)r * nb + b] = row_block_sumi(type, row, b, (const int8_t*)xq8 + (size_t)b * Q8_1_BYTES + 4, &dw);
        }
    }
}

/* One GEMV row: sum over blocks of d_w * d_x * (float)sumi, d_w and d_x the f16-stored scales.
 * gemv_iq3s_q8 / dot_iq3s_q8_subgroup, chimere_kernels.cu:860-861,874-925;
 * gemv_q8_0_q8, src/kernels/gemv_q8_0.rs:253-254.  Blocks are added in ascending order
 * (the reference's order is a property of its launch shape; fp32 results are compared with a
 * tolerance). */
static float kquant_row_dot(int type, const uint8_t* row, const uint8_t* xq8, int ncols);
static int is_kquant(int type);
static inline float row_dot(int type, const uint8_t* row, const uint8_t* xq8, int nb) {
    if (is_kquant(type)) return kquant_row_dot(type, row, xq8, nb * 32);   /* a K-quant shared expert (moe_ffn.rs:1597-1650) */
    float acc = 0.0f;
    for (int b = 0; b < nb; b++) {
        const uint8_t* xb = xq8 + (size_t)b * Q8_1_BYTES;
        uint16_t dxh; memcpy(&dxh, xb, 2);
        float dw; int32_t s = row_block_sumi(type, row, b, (const int8_t*)xb + 4, &dw);
        acc = fmaf(dw * orc_f16_to_f32(dxh), (float)s, acc);   /* nvcc contracts sum += d*d*(float)sumi */
    }
    return acc;
}

/* ---- K-quant super-blocks of 256 weights (the shared expert of the production files is Q5_K; wrappers
 * ffi/ggml_cuda_gemv.cu:118-172).  Layouts as the reference reads them:
 *   Q5_K 176 B: f16 d, f16 dmin, scales[12] (eight 6-bit scales and eight 6-bit mins), qh[32], qs[128]
 *               -- ffi/src/lib.rs:51-54,396-443, src/gguf_loader.rs (dequantize_q5_k)
 *   Q4_K 144 B: the same without qh -- src/gguf_loader.rs:1274-1345
 *   Q6_K 210 B: ql[128], qh[64], int8 scales[16] (one per 16 weights), f16 d -- src/gguf_loader.rs:855-927
 * Sub-block j (32 weights) of a Q4_K/Q5_K super-block: nibbles of qs[32*(j/2) .. +32), low for even j, high for
 * odd j; Q5_K adds 16 where bit j of qh[l] is set.  weight = d*sc_j*q - dmin*m_j. */
static inline void scale_min_k4(int j, const uint8_t* sc, int* s, int* m) {   /* ffi/src/lib.rs:368-383 */
    if (j < 4) { *s = sc[j] & 63; *m = sc[j + 4] & 63; }
    else { *s = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); *m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
}
/* the 32 unsigned quants of sub-block j */
static inline void q45k_sub_quants(int type, const uint8_t* blk, int j, int32_t* q) {
    const uint8_t* qh = blk + 16;
    const uint8_t* qs = blk + (type == CHIMERE_TYPE_Q5_K ? 48 : 16) + 32 * (j / 2);
    for (int l = 0; l < 32; l++) {
        int v = (j & 1) ? (qs[l] >> 4) : (qs[l] & 0x0F);
        if (type == CHIMERE_TYPE_Q5_K && ((qh[l] >> j) & 1)) v += 16;
        q[l] = v;
    }
}
/* the 32 signed quants of sub-block j (0..7) of a Q6_K super-block and its two scales (first / second 16 weights) */
static inline void q6k_sub_quants(const uint8_t* blk, int j, int32_t* q, int* sc_a, int* sc_b) {
    const int grp = j / 4, s = j % 4;
    const uint8_t* ql = blk + 64 * grp + 32 * (s & 1);
    const uint8_t* qh = blk + 128 + 32 * grp;
    const int8_t* sc = (const int8_t*)(blk + 192) + 8 * grp + 2 * s;
    for (int l = 0; l < 32; l++) {
        const int nib = (s >> 1) ? (ql[l] >> 4) : (ql[l] & 0x0F);
        q[l] = (nib | (((qh[l] >> (2 * s)) & 3) << 4)) - 32;
    }
    *sc_a = sc[0]; *sc_b = sc[1];
}
static int is_kquant(int type) { return type == CHIMERE_TYPE_Q4_K || type == CHIMERE_TYPE_Q5_K || type == CHIMERE_TYPE_Q6_K; }

/* One row of a K-quant matrix against one Q8_1 row (f16 d, f16 s = d * sum of quants): the formula of
 * vec_dot_q5_k_q8_1, ffi/src/lib.rs:385-499 -- per sub-block d*d8*sc*dot, minus dmin*m*s8 -- in f32, sub-blocks ascending. */
static float kquant_row_dot(int type, const uint8_t* row, const uint8_t* xq8, int ncols) {
    float acc = 0.0f;
    const int bytes = type == CHIMERE_TYPE_Q4_K ? Q4_K_BYTES : type == CHIMERE_TYPE_Q5_K ? Q5_K_BYTES : Q6_K_BYTES;
    for (int sb = 0; sb < ncols / 256; sb++) {
        const uint8_t* blk = row + (size_t)sb * bytes;
        uint16_t h;
        float d, dmin = 0.0f;
        if (type == CHIMERE_TYPE_Q6_K) { memcpy(&h, blk + 208, 2); d = orc_f16_to_f32(h); }
        else { memcpy(&h, blk, 2); d = orc_f16_to_f32(h); memcpy(&h, blk + 2, 2); dmin = orc_f16_to_f32(h); }
        for (int j = 0; j < 8; j++) {
            const uint8_t* xb = xq8 + (size_t)(sb * 8 + j) * Q8_1_BYTES;
            const int8_t* q8 = (const int8_t*)xb + 4;
            memcpy(&h, xb, 2); const float d8 = orc_f16_to_f32(h);
            memcpy(&h, xb + 2, 2); const float s8 = orc_f16_to_f32(h);
            int32_t q[32];
            if (type == CHIMERE_TYPE_Q6_K) {
                int sa, sb2; q6k_sub_quants(blk, j, q, &sa, &sb2);
                int32_t da = 0, db = 0;
                for (int l = 0; l < 16; l++) { da += q[l] * (int32_t)q8[l]; db += q[16 + l] * (int32_t)q8[16 + l]; }
                acc = fmaf(d * d8, (float)(sa * da + sb2 * db), acc);
            } else {
                int sc, mn; scale_min_k4(j, blk + 4, &sc, &mn);
                q45k_sub_quants(type, blk, j, q);
                int32_t dot = 0;
                for (int l = 0; l < 32; l++) dot += q[l] * (int32_t)q8[l];
                acc = fmaf(d * d8, (float)(sc * dot), acc);
                acc = fmaf(-(dmin * (float)mn), s8, acc);
            }
        }
    }
    return acc;
}

/* y[nrows] = W . x_q8 for one Q8_1 input row (chimere_mmvq_* semantics, ffi/ggml_cuda_gemv.cu:105-172). */
void orc_gemv(int type, const void* W, const void* xq8, float* y, int ncols, int nrows) {
    int nb = ncols / 32; int64_t rb = orc_row_bytes(type, ncols);
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < nrows; r++)
        y[r] = row_dot(type, (const uint8_t*)W + (size_t)r * rb, (const uint8_t*)xq8, nb);
}

/* Dequantise n elements (n multiple of the block size) -- gguf_loader.rs:752-772 (Q4_0),
 * :793-837 (Q8_0), :1022-1170 (IQ3_S) / dequant_iq3s chimere_kernels.cu:203-290. */
void orc_dequant(int type, const void* W, float* out, int64_t n) {
    const uint8_t* p = (const uint8_t*)W;
    if (is_kquant(type)) {   /* gguf_loader.rs:855-927 (Q6_K), :1274-1345 (Q4_K); ffi/src/lib.rs:576-640 (Q5_K) */
        const int bytes = type == CHIMERE_TYPE_Q4_K ? Q4_K_BYTES : type == CHIMERE_TYPE_Q5_K ? Q5_K_BYTES : Q6_K_BYTES;
        for (int64_t b = 0; b < n / 256; b++) {
            const uint8_t* blk = p + b * bytes;
            uint16_t h;
            for (int j = 0; j < 8; j++) {
                int32_t q[32];
                if (type == CHIMERE_TYPE_Q6_K) {
                    memcpy(&h, blk + 208, 2); const float d = orc_f16_to_f32(h);
                    int sa, sb; q6k_sub_quants(blk, j, q, &sa, &sb);
                    for (int l = 0; l < 32; l++) out[b * 256 + j * 32 + l] = d * (float)(l < 16 ? sa : sb) * (float)q[l];
                } else {
                    memcpy(&h, blk, 2); const float d = orc_f16_to_f32(h);
                    memcpy(&h, blk + 2, 2); const float dmin = orc_f16_to_f32(h);
                    int sc, mn; scale_min_k4(j, blk + 4, &sc, &mn);
                    q45k_sub_quants(type, blk, j, q);
                    for (int l = 0; l < 32; l++) out[b * 256 + j * 32 + l] = d * (float)sc * (float)q[l] - dmin * (float)mn;
                }
            }
        }
        return;
    }
    if (type == CHIMERE_TYPE_Q4_0) {
        for (int64_t b = 0; b < n / 32; b++) {
            const uint8_t* blk = p + b * Q4_0_BYTES; uint16_t dh; memcpy(&dh, blk, 2); float d = orc_f16_to_f32(dh);
            for (int j = 0; j < 16; j++) {
                out[b * 32 + j] = (float)((blk[2 + j] & 0x0F) - 8) * d;
                out[b * 32 + j + 16] = (float)((blk[2 + j] >> 4) - 8) * d;
            }
        }
    } else if (type == CHIMERE_TYPE_Q8_0) {
        for (int64_t b = 0; b < n / 32; b++) {
            const uint8_t* blk = p + b * Q8_0_BYTES; uint16_t dh; memcpy(&dh, blk, 2); float d = orc_f16_to_f32(dh);
            for (int j = 0; j < 32; j++) out[b * 32 + j] = (float)((const int8_t*)blk)[2 + j] * d;
        }
    } else {
        for (int64_t b = 0; b < n / 256; b++) {
            const uint8_t* blk = p + b * IQ3S_BYTES; uint16_t dh; memcpy(&dh, blk, 2); float d = orc_f16_to_f32(dh);
            for (int sg = 0; sg < 8; sg++) {
                uint8_t scb = blk[106 + sg / 2];
                float db = d * (float)(1 + 2 * ((sg & 1) ? (scb >> 4) : (scb & 0x0F)));
                uint32_t qh = blk[66 + sg];
                for (int g = 0; g < 8; g++) {
                    uint32_t gv = iq3s_grid[blk[2 + sg * 8 + g] | (((qh >> g) & 1u) << 8)];
                    uint32_t sb = blk[74 + sg * 4 + (g >> 1)] >> ((g & 1) * 4);
                    for (int i = 0; i < 4; i++) {
                        float m = (float)((gv >> (8 * i)) & 0xFFu);
                        out[b * 256 + sg * 32 + g * 4 + i] = db * (((sb >> i) & 1u) ? -m : m);
                    }
                }
            }
        }
    }
}

/* --------------------------------------------------------------- elementwise pieces ----- */

/* silu(g) * u with silu(g) = g / (1 + expf(-g)).  silu_mul_batched_kernel,
 * chimere_kernels.cu:1533-1547; src/kernels/fused_ops.rs:34-45. */
float orc_swiglu(float g, float u) { return g / (1.0f + expf(-g)) * u; }
/* relu(u)^2 (gateless; docs/journey-2026-04-24.md:182-186 pins relu(up)^2, not relu(up)^2*up). */
float orc_relu2(float u) { float r = u > 0.0f ? u : 0.0f; return r * r; }

/* out[i] = sh[i] * sigmoid(logit) + routed[i].  sigmoid_gate_add_kernel, src/scratch_pool.rs:266-277. */
void orc_sigmoid_gate_add(const float* sh, float logit, const float* routed, float* out, int n) {
    float scale = 1.0f / (1.0f + expf(-logit));
    for (int i = 0; i < n; i++) out[i] = fmaf(sh[i], scale, routed[i]);   /* contracted by nvcc */
}

/* out[h] = sum_k w[k] * y[k][h], k ascending.  weighted_combine_kernel, chimere_kernels.cu:1551-1565. */
void orc_weighted_combine(const float* y, const float* w, float* out, int H, int k) {
    for (int h = 0; h < H; h++) {
        float s = 0.0f;
        for (int j = 0; j < k; j++) s = fmaf(w[j], y[(size_t)j * H + h], s);   /* contracted by nvcc */
        out[h] = s;
    }
}

/* y = x / sqrt(mean(x^2) + eps), unit weight (the benchmark's layer stack). */
void orc_rmsnorm(const float* x, float* y, int T, int H, float eps) {
    #pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        double ss = 0.0;
        for (int h = 0; h < H; h++) ss += (double)x[(size_t)t * H + h] * x[(size_t)t * H + h];
        float inv = 1.0f / sqrtf((float)(ss / H) + eps);
        for (int h = 0; h < H; h++) y[(size_t)t * H + h] = x[(size_t)t * H + h] * inv;
    }
}

/* residual += hidden; normed = residual / sqrt(mean(residual^2) + eps) * weight, for T rows of length n.
 * fused_add_residual_rmsnorm, src/kernels/fused_ops.rs:91-140 (one block of 256 threads per row): thread i sums the
 * squares of elements i, i+256, ... (nvcc contracts sum += v*v), the 256 sums meet in a tree with strides 128..1, and
 * every element is (residual * inv_rms) * weight with inv_rms = 1 / sqrtf(sum / n + eps). */
void orc_add_residual_rmsnorm(const float* hidden, float* residual, const float* weight, float* normed, int T, int n, float eps) {
    for (int t = 0; t < T; t++) {
        const float* h = hidden + (size_t)t * n; float* r = residual + (size_t)t * n; float* o = normed + (size_t)t * n;
        float part[256];
        for (int p = 0; p < 256; p++) {
            float acc = 0.0f;
            for (int i = p; i < n; i += 256) { float v = h[i] + r[i]; r[i] = v; acc = fmaf(v, v, acc); }
            part[p] = acc;
        }
        for (int s = 128; s > 0; s >>= 1)
            for (int p = 0; p < s; p++) part[p] += part[p + s];
        float rms = sqrtf(part[0] / (float)n + eps);
        float inv = 1.0f / rms;
        for (int i = 0; i < n; i++) o[i] = r[i] * inv * weight[i];
    }
}

/* ------------------------------------------------------------------- dispatch order ----- */

/* Stable counting sort of the pairs p = t*k + j by expert id: offsets[E+1], perm[T*k].
 * The reference never permutes tokens (its prefill loops over tokens,
 * src/qwen35_model/compute_graph.rs:1787-1808); this is the canonical grouped order. */
void orc_permute(const int32_t* idx, int T, int k, int E, int32_t* perm, int32_t* offsets) {
    memset(offsets, 0, sizeof(int32_t) * (size_t)(E + 1));
    for (int p = 0; p < T * k; p++) offsets[idx[p] + 1]++;
    for (int e = 0; e < E; e++) offsets[e + 1] += offsets[e];
    int32_t* cur = (int32_t*)malloc(sizeof(int32_t) * (size_t)E);
    memcpy(cur, offsets, sizeof(int32_t) * (size_t)E);
    for (int p = 0; p < T * k; p++) perm[cur[idx[p]]++] = p;
    free(cur);
}

/* ------------------------------------------------------------------- whole layer -------- */

/* y[T][H] = MoE(x[T][H]) with host pointers in `w`.  Follows forward_moe_cudarc_with_cache
 * (moe_ffn.rs:1094-1766) step by step -- router GEMV, top-k, Q8_1 of x (:1099-1204); gate and up
 * GEMVs and the activation per selected expert (:1206-1305); Q8_1 of the intermediates
 * (:1307-1323); down GEMVs (:1325-1373); weighted combine in slot order (:1375-1384); the shared
 * expert (:1597-1730) and the sigmoid gate add (:1736-1766) -- with the loops over tokens,
 * slots and rows spread over the host threads (tokens are processed in chunks of 64).
 * Optional taps (any may be NULL):
 *   topk_idx[T][k], topk_w[T][k], logits[T][E], x_q8[T][H/32*36],
 *   inter_q8[T][k+1][Fmax/32*36] (slot k = shared expert), sh_logit[T]. */
/* forced_idx (optional, [T][k]): take these expert ids instead of the oracle's own top-k and give them the weights
 * the router would: the probabilities of those experts, renormalised (and scaled) exactly as after a selection.
 * The GPU tests use it where the host's expf and the GPU's differ in the last place and flip a near-tie: the rest
 * of the layer is then still checked on the GPU's routing. */
int orc_moe_forward_ex(const chimere_moe_layer* w, const float* x, float* y, int T, const int32_t* forced_idx,
                       int32_t* topk_idx, float* topk_w, float* logits_out, uint8_t* x_q8_out,
                       uint8_t* inter_q8_out, float* sh_logit_out) {
    const int H = w->H, E = w->E, F = w->F, Fs = w->F_s, k = w->top_k;
    if (E > 256 || k > 16 || H % 32 || F % 32 || Fs % 32) return -1;
    const int dual = w->act == CHIMERE_ACT_SWIGLU;
    const int Fmax = F > Fs ? F : Fs;
    const int S = k + (Fs > 0 ? 1 : 0);                    /* slots per token, the last one shared */
    const size_t xq_row = (size_t)(H / 32) * Q8_1_BYTES, iq_row = (size_t)(Fmax / 32) * Q8_1_BYTES;
    enum { CHUNK = 64 };
    int32_t* idx = (int32_t*)malloc(sizeof(int32_t) * CHUNK * 16);
    float* wt = (float*)malloc(sizeof(float) * CHUNK * 16);
    float* shl = (float*)calloc(CHUNK, sizeof(float));
    uint8_t* xq = (uint8_t*)malloc(xq_row * CHUNK);
    float* inter = (float*)malloc(sizeof(float) * (size_t)CHUNK * S * Fmax);
    uint8_t* iq = (uint8_t*)malloc(iq_row * (size_t)CHUNK * S);
    float* eout = (float*)malloc(sizeof(float) * (size_t)CHUNK * S * H);
    for (int t0 = 0; t0 < T; t0 += CHUNK) {
        const int nt = (T - t0 < CHUNK) ? T - t0 : CHUNK;
        /* router, top-k, Q8_1 of the input rows */
        #pragma omp parallel for schedule(dynamic, 1)
        for (int i = 0; i < nt; i++) {
            const int t = t0 + i;
            const float* xt = x + (size_t)t * H;
            float logits[256];
            orc_router_logits(w->router_w, w->router_bias, xt, E, H, logits);
            float probs[256];
            if (w->route_mode == CHIMERE_ROUTE_SOFTMAX_RENORM) {
                orc_topk_softmax(logits, E, k, idx + i * 16, wt + i * 16, probs);
                if (w->route_scale != 1.0f) for (int j = 0; j < k; j++) wt[i * 16 + j] *= w->route_scale;
            } else orc_topk_sigmoid(logits, E, k, w->route_scale, idx + i * 16, wt + i * 16, probs);
            if (forced_idx) {
                float wsum = 0.0f;
                for (int j = 0; j < k; j++) {
                    idx[i * 16 + j] = forced_idx[(size_t)t * k + j];
                    wt[i * 16 + j] = probs[idx[i * 16 + j]];
                    wsum += wt[i * 16 + j];
                }
                if (wsum > 0.0f) { const float inv = 1.0f / wsum; for (int j = 0; j < k; j++) wt[i * 16 + j] *= inv; }
                if (w->route_mode != CHIMERE_ROUTE_SOFTMAX_RENORM || w->route_scale != 1.0f)
                    for (int j = 0; j < k; j++) wt[i * 16 + j] *= w->route_scale;
            }
            orc_quantize_q8_1(xt, xq + (size_t)i * xq_row, H);
            if (Fs > 0 && w->shexp_gate_w) shl[i] = orc_dot_strided256(xt, w->shexp_gate_w, H);
            if (topk_idx) memcpy(topk_idx + (size_t)t * k, idx + i * 16, sizeof(int32_t) * (size_t)k);
            if (topk_w) memcpy(topk_w + (size_t)t * k, wt + i * 16, sizeof(float) * (size_t)k);
            if (logits_out) memcpy(logits_out + (size_t)t * E, logits, sizeof(float) * (size_t)E);
            if (x_q8_out) memcpy(x_q8_out + (size_t)t * xq_row, xq + (size_t)i * xq_row, xq_row);
            if (sh_logit_out && Fs > 0 && w->shexp_gate_w) sh_logit_out[t] = shl[i];
        }
        /* gate / up rows and the activation, one (token, slot, row) at a time */
        #pragma omp parallel for collapse(2) schedule(dynamic, 16)
        for (int p = 0; p < nt * S; p++) {
            for (int r = 0; r < Fmax; r++) {
                const int i = p / S, j = p % S, sh = (j == k);
                const int Fe = sh ? Fs : F;
                if (r >= Fe) continue;
                const int tu = sh ? w->type_sh_up : w->type_up, tg = sh ? w->type_sh_gate : w->type_gate;
                const uint8_t* Wu = sh ? (const uint8_t*)w->sh_up : (const uint8_t*)w->up_exps + (size_t)idx[i * 16 + j] * w->stride_up;
                const uint8_t* xr = xq + (size_t)i * xq_row;
                float u = row_dot(tu, Wu + (size_t)r * orc_row_bytes(tu, H), xr, H / 32), v;
                if (dual) {
                    const uint8_t* Wg = sh ? (const uint8_t*)w->sh_gate : (const uint8_t*)w->gate_exps + (size_t)idx[i * 16 + j] * w->stride_gate;
                    v = orc_swiglu(row_dot(tg, Wg + (size_t)r * orc_row_bytes(tg, H), xr, H / 32), u);
                } else v = orc_relu2(u);
                inter[(size_t)p * Fmax + r] = v;
            }
        }
        /* Q8_1 of the intermediates */
        #pragma omp parallel for schedule(static)
        for (int p = 0; p < nt * S; p++) {
            const int i = p / S, j = p % S;
            const int Fe = (j == k) ? Fs : F;
            memset(iq + (size_t)p * iq_row, 0, iq_row);
            orc_quantize_q8_1(inter + (size_t)p * Fmax, iq + (size_t)p * iq_row, Fe);
            if (inter_q8_out) memcpy(inter_q8_out + ((size_t)(t0 + i) * (k + 1) + j) * iq_row, iq + (size_t)p * iq_row, iq_row);
        }
        /* down rows */
        #pragma omp parallel for collapse(2) schedule(dynamic, 16)
        for (int p = 0; p < nt * S; p++) {
            for (int h = 0; h < H; h++) {
                const int i = p / S, j = p % S, sh = (j == k);
                const int Fe = sh ? Fs : F;
                const int td = sh ? w->type_sh_down : w->type_down;
                const uint8_t* Wd = sh ? (const uint8_t*)w->sh_down : (const uint8_t*)w->down_exps + (size_t)idx[i * 16 + j] * w->stride_down;
                eout[(size_t)p * H + h] = row_dot(td, Wd + (size_t)h * orc_row_bytes(td, Fe), iq + (size_t)p * iq_row, Fe / 32);
            }
        }
        /* combine in slot order, then the shared expert */
        #pragma omp parallel for schedule(static)
        for (int i = 0; i < nt; i++) {
            float* yt = y + (size_t)(t0 + i) * H;
            orc_weighted_combine(eout + (size_t)i * S * H, wt + i * 16, yt, H, k);
            if (Fs > 0) {
                const float* sh = eout + ((size_t)i * S + k) * H;
                if (w->shexp_gate_w) orc_sigmoid_gate_add(sh, shl[i], yt, yt, H);
                else for (int h = 0; h < H; h++) yt[h] = sh[h] + yt[h];
            }
        }
    }
    free(idx); free(wt); free(shl); free(xq); free(inter); free(iq); free(eout);
    return 0;
}

int orc_moe_forward(const chimere_moe_layer* w, const float* x, float* y, int T,
                    int32_t* topk_idx, float* topk_w, float* logits_out, uint8_t* x_q8_out,
                    uint8_t* inter_q8_out, float* sh_logit_out) {
    return orc_moe_forward_ex(w, x, y, T, NULL, topk_idx, topk_w, logits_out, x_q8_out, inter_q8_out, sh_logit_out);
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
