// Plain GEMV on K-quant super-blocks (Q4_K, Q5_K, Q6_K) against one Q8_1 row: the entries chimere_mmvq_q4k / _q5k / _q6k
// that the reference binds to its dependency's mul_mat_vec_*_K_q8_1 kernels (ffi/ggml_cuda_gemv.cu:118-172).  The
// production files keep the shared expert in Q5_K (moe_ffn.rs:1597-1650); the routed experts never use these types.
//
// A warp owns one output row (and up to eight input rows).  Lane l takes the 32-weight sub-blocks l, l+32, ... of the row:
// it reads the sub-block's quants as eight 32-bit words once, the Q8_1 block of every input row beside it, and adds
//     d * d8 * sc_j * dot - dmin * m_j * s8        (Q4_K, Q5_K: six-bit scale sc_j and min m_j, s8 = d8 * sum of the quants)
//     d * d8 * (sc_a * dot_a + sc_b * dot_b)       (Q6_K: one int8 scale per 16 weights)
// in ascending sub-block order; the lanes' sums meet in a butterfly.  HBM-bound: a row is read once, coalesced by
// super-block (consecutive lanes read consecutive 32-weight pieces), the Q8_1 row stays in L1/L2.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"

namespace chimere {

namespace {

constexpr int kRowsPerCta = 8;   // warps per CTA

__device__ __forceinline__ uint32_t ld32(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }

// six-bit scale and min of sub-block j from the twelve packed bytes (ffi/src/lib.rs:368-383)
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* sc, int& s, int& m) {
    if (j < 4) { s = sc[j] & 63; m = sc[j + 4] & 63; }
    else { s = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
}

template <int TYPE> struct KBlock;
template <> struct KBlock<CHIMERE_TYPE_Q4_K> { static constexpr int kBytes = 144, kQs = 16; };
template <> struct KBlock<CHIMERE_TYPE_Q5_K> { static constexpr int kBytes = 176, kQs = 48; };
template <> struct KBlock<CHIMERE_TYPE_Q6_K> { static constexpr int kBytes = 210, kQs = 0; };

// A decoded 32-weight sub-block: eight words of four quants each and what scales them.
struct SubBlock {
    int w[8];
    float d, dmin;   // super-block scales (dmin unused for Q6_K)
    int sc, mn;      // Q4_K / Q5_K: six-bit scale and min; Q6_K: the int8 scales of the first and the second 16 weights
};

template <int TYPE>
__device__ __forceinline__ void decode_sub(const uint8_t* blk, int j, SubBlock& s) {
    if (TYPE == CHIMERE_TYPE_Q6_K) {
        // 210-byte blocks are only 2-byte aligned
        const int grp = j >> 2, q = j & 3;
        const uint8_t* ql = blk + 64 * grp + 32 * (q & 1);
        const uint8_t* qh = blk + 128 + 32 * grp;
        const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192) + 8 * grp + 2 * q;
        s.d = h2f(ld_u16(blk + 208)); s.dmin = 0.0f;
        s.sc = sc[0]; s.mn = sc[1];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const uint32_t lo = ld_u32_a2(ql + 4 * g), hi = ld_u32_a2(qh + 4 * g);
            const uint32_t nib = (q >> 1) ? (lo >> 4) & 0x0F0F0F0Fu : lo & 0x0F0F0F0Fu;
            const uint32_t v = nib | (((hi >> (2 * q)) & 0x03030303u) << 4);      // 0..63 per byte
            s.w[g] = (int)__vsub4(v, 0x20202020u);                                // -32..31 per byte
        }
    } else {
        s.d = h2f(ld_u16(blk)); s.dmin = h2f(ld_u16(blk + 2));
        scale_min_k4(j, blk + 4, s.sc, s.mn);
        const uint8_t* qs = blk + KBlock<TYPE>::kQs + 32 * (j >> 1);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const uint32_t lo = ld32(qs + 4 * g);
            uint32_t v = (j & 1) ? (lo >> 4) & 0x0F0F0F0Fu : lo & 0x0F0F0F0Fu;
            if (TYPE == CHIMERE_TYPE_Q5_K) v |= ((ld32(blk + 16 + 4 * g) >> j) & 0x01010101u) << 4;
            s.w[g] = (int)v;
        }
    }
}

// ... against one Q8_1 block `xb` (36 bytes: f16 d, f16 s, 32 int8).
template <int TYPE>
__device__ __forceinline__ float dot_sub(const SubBlock& s, const uint8_t* xb) {
    const __half2 ds = *reinterpret_cast<const __half2*>(xb);
    const float d8 = __low2float(ds), s8 = __high2float(ds);
    if (TYPE == CHIMERE_TYPE_Q6_K) {
        int da = 0, db = 0;
#pragma unroll
        for (int g = 0; g < 4; ++g) { da = __dp4a(s.w[g], (int)ld32(xb + 4 + 4 * g), da); db = __dp4a(s.w[4 + g], (int)ld32(xb + 20 + 4 * g), db); }
        return s.d * d8 * (float)(s.sc * da + s.mn * db);
    } else {
        int dot = 0;
#pragma unroll
        for (int g = 0; g < 8; ++g) dot = __dp4a(s.w[g], (int)ld32(xb + 4 + 4 * g), dot);
        return fmaf(-(s.dmin * (float)s.mn), s8, s.d * d8 * (float)(s.sc * dot));
    }
}

// grid = (row groups, groups of tpc <= kTokensPerCta input rows, matrices).  A sub-block is decoded once and used for every input
// row of the CTA's group.  mode 0: y = v; 1: y += v; 2: y += sigmoid(logit[t]) * v (the sigmoid-gated shared expert added
// to the routed sum, scratch_pool.rs:266-277).  blockIdx.z = 1 takes the second matrix / output (gate beside up).
constexpr int kTokensPerCta = 8;
template <int TYPE>
__global__ void __launch_bounds__(32 * kRowsPerCta) kquant_mmvq_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ w2,
                                                                      const uint8_t* __restrict__ xq8, int64_t x_stride, float* __restrict__ y,
                                                                      float* __restrict__ y2, int64_t y_stride, int n_inputs, int tpc, int ncols,
                                                                      int nrows, int mode, const float* __restrict__ logit) {
    const int lane = threadIdx.x & 31, row = blockIdx.x * kRowsPerCta + (threadIdx.x >> 5);
    const int t0 = blockIdx.y * tpc, nt = min(tpc, n_inputs - t0);   // tpc <= kTokensPerCta input rows per CTA
    griddep_wait();   // (a no-op unless launched programmatically behind the kernel that writes the inputs)
    if (threadIdx.x == 0) griddep_launch();
    if (row >= nrows) return;
    if (blockIdx.z) { w = w2; y = y2; }
    const int nsub = ncols >> 5;
    const uint8_t* rowp = w + (size_t)row * (size_t)(ncols >> 8) * KBlock<TYPE>::kBytes;
    const uint8_t* xr = xq8 + (size_t)t0 * x_stride;
    float acc[kTokensPerCta];
#pragma unroll
    for (int i = 0; i < kTokensPerCta; ++i) acc[i] = 0.0f;
    for (int sb = lane; sb < nsub; sb += 32) {
        SubBlock s;
        decode_sub<TYPE>(rowp + (size_t)(sb >> 3) * KBlock<TYPE>::kBytes, sb & 7, s);
#pragma unroll
        for (int i = 0; i < kTokensPerCta; ++i)
            if (i < nt) acc[i] += dot_sub<TYPE>(s, xr + (size_t)i * x_stride + (size_t)sb * kQ81Bytes);
    }
#pragma unroll
    for (int i = 0; i < kTokensPerCta; ++i) {
        if (i < nt) {
            float v = acc[i];
#pragma unroll
            for (int sft = 16; sft > 0; sft >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sft);
            if (lane == 0) {
                float* out = y + (size_t)(t0 + i) * y_stride + row;
                if (mode == 0) *out = v;
                else if (mode == 1) *out = v + *out;
                else *out = fmaf(v, sigmoid_ref(logit[t0 + i]), *out);
            }
        }
    }
}

// One warp per (row t, block b of 32): v = silu(g) * u (or relu(u)^2 without a gate row) -> one Q8_1 block, as the gate/up
// kernels write their intermediates (d = amax / 127 in f16, s = the sum of the 32 values).
__global__ void __launch_bounds__(256) act_q8_1_kernel(const float* __restrict__ g, const float* __restrict__ u, int64_t in_stride,
                                                       uint8_t* __restrict__ out, int64_t out_stride, int T, int F) {
    const int lane = threadIdx.x & 31, nb = F >> 5;
    const int64_t wid = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    griddep_wait();
    if (threadIdx.x == 0) griddep_launch();
    if (wid >= (int64_t)T * nb) return;
    const int t = (int)(wid / nb), b = (int)(wid - (int64_t)t * nb);
    const float uu = u[(size_t)t * in_stride + b * 32 + lane];
    float v;
    if (g) v = silu_mul_ref(g[(size_t)t * in_stride + b * 32 + lane], uu);
    else { const float r = fmaxf(uu, 0.0f); v = r * r; }
    float amax = fabsf(v), sum = v;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
        sum += __shfl_xor_sync(0xffffffffu, sum, s);
    }
    const float d = amax / 127.0f;
    uint8_t* blk = out + (size_t)t * out_stride + (size_t)b * kQ81Bytes;
    reinterpret_cast<int8_t*>(blk)[4 + lane] = (amax == 0.0f) ? (int8_t)0 : (int8_t)roundf(v / d);
    if (lane == 0) *reinterpret_cast<__half2*>(blk) = __halves2half2(__float2half(d), __float2half(sum));
}

}  // namespace

// w2 / y2 (optional): a second matrix of the same type and shape against the same inputs, in the same launch.
// chained: launch programmatically behind the previous kernel of the stream.
cudaError_t launch_mmvq_kquant_batched(int wtype, const void* w, const void* w2, const void* xq8, int64_t x_stride, float* y, float* y2,
                                       int64_t y_stride, int n_inputs, int ncols, int nrows, int mode, const float* logit, bool chained,
                                       cudaStream_t stream) {
    if (nrows <= 0 || n_inputs <= 0) return cudaSuccess;
    if (ncols <= 0 || (ncols & 255) || ((uintptr_t)xq8 & 3) || (x_stride & 3) || n_inputs > 65535 || (mode == 2 && !logit)) return cudaErrorInvalidValue;
    const uintptr_t wbits = (uintptr_t)w | (uintptr_t)w2;
    // input rows per CTA: as many as still leave a grid of two CTAs per SM (a small batch wants the CTAs, a large one the reuse)
    const int row_groups = (nrows + kRowsPerCta - 1) / kRowsPerCta;
    int tpc = kTokensPerCta;
    while (tpc > 1 && (int64_t)row_groups * ((n_inputs + tpc - 1) / tpc) * (w2 ? 2 : 1) < 2 * sm_count()) tpc >>= 1;
    const dim3 grid(row_groups, (n_inputs + tpc - 1) / tpc, w2 ? 2 : 1);
    const uint8_t* wp = (const uint8_t*)w;
    const uint8_t* wp2 = (const uint8_t*)w2;
    const uint8_t* xp = (const uint8_t*)xq8;
    auto go = [&](auto kernel) {
        if (chained) return launch_pdl(kernel, grid, 32 * kRowsPerCta, 0, stream, wp, wp2, xp, x_stride, y, y2, y_stride, n_inputs, tpc, ncols, nrows, mode, logit);
        kernel<<<grid, 32 * kRowsPerCta, 0, stream>>>(wp, wp2, xp, x_stride, y, y2, y_stride, n_inputs, tpc, ncols, nrows, mode, logit);
        return cudaGetLastError();
    };
    switch (wtype) {
        case CHIMERE_TYPE_Q4_K: return (wbits & 3) ? cudaErrorInvalidValue : go(kquant_mmvq_kernel<CHIMERE_TYPE_Q4_K>);
        case CHIMERE_TYPE_Q5_K: return (wbits & 3) ? cudaErrorInvalidValue : go(kquant_mmvq_kernel<CHIMERE_TYPE_Q5_K>);
        case CHIMERE_TYPE_Q6_K: return (wbits & 1) ? cudaErrorInvalidValue : go(kquant_mmvq_kernel<CHIMERE_TYPE_Q6_K>);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_mmvq_kquant(int wtype, const void* w, const void* xq8, float* y, int ncols, int nrows, cudaStream_t stream) {
    return launch_mmvq_kquant_batched(wtype, w, nullptr, xq8, 0, y, nullptr, 0, 1, ncols, nrows, 0, nullptr, false, stream);
}

cudaError_t launch_act_q8_1(const float* g, const float* u, int64_t in_stride, void* out, int64_t out_stride, int T, int F, cudaStream_t stream) {
    if (T <= 0 || F <= 0) return cudaSuccess;
    if (F & 31) return cudaErrorInvalidValue;
    const int64_t warps = (int64_t)T * (F >> 5);
    return launch_pdl(act_q8_1_kernel, dim3((unsigned)((warps + 7) / 8)), 256, 0, stream, g, u, in_stride, (uint8_t*)out, out_stride, T, F);
}

}  // namespace chimere
