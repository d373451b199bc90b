// gemv_tiled.cu -- the decode-path GEMV kernels on tiled32 weights (see tiled.cuh).
//
// One warp = 32 consecutive rows of one expert matrix, lane = row: a warp-wide 128-bit load is one
// contiguous 512-byte read of the tiled layout and hands every lane whole 32-weight units of its own
// row, which are decoded in registers and multiplied (dp4a) with the tokens' Q8_1 activations.  The
// activations of the work entry's tokens are staged once per CTA in shared memory as an int8 plane and
// an f32 scale plane and read as warp-wide broadcasts.  The eight warps of a CTA are WR row tiles x WK
// slices of K; slices meet in shared memory and are added in a fixed order.
//
// Two kernels share this core.  bulk_kernel (the one that normally runs) brings every warp's contiguous piece of the
// tiled layout into shared memory with one cp.async.bulk per matrix and reads the units back from there;
// tile_kernel loads them straight into registers (ld.global.nc, 128 bits per lane) and is the fallback for shapes
// whose row tile does not fit shared memory.  Measurements on B200 showed this path to be bound by the latency of
// the chain every work item starts with (work entry -> weights and activations -> dot products -> reduction) and by
// the tails of the CTA waves, not by bandwidth; a persistent variant with per-warp rings was slower than letting the
// hardware start fresh CTAs, so the kernels stay one work item per CTA with several CTAs resident per SM.
//
//   STAGE_GATE_UP : act(gate . x, up . x) -> Q8_1 blocks of the intermediates
//                   (replaces moe_ffn.rs:1206-1323 and :1597-1700 of the reference)
//   STAGE_DOWN    : down . inter -> per-pair rows; the CTA that completes a token's row tile adds the
//                   rows up in slot order with the routing weights and the sigmoid-gated shared
//                   expert (replaces moe_ffn.rs:1325-1384 and :1700-1766)
#include "common.cuh"
#include "kernels.h"
#include "tiled.cuh"

namespace chimere {

constexpr int kWarpsT = 8;
constexpr int kThreadsT = 32 * kWarpsT;
constexpr int kStageGateUp = 0, kStageDown = 1;

struct TileSmem { uint32_t aq, ad, red, total, q_row, d_row; };
__host__ __device__ inline TileSmem tile_smem(int ncols_max, int wr, int wk, bool dual) {
    TileSmem s;
    s.q_row = (uint32_t)ncols_max;
    s.d_row = ((uint32_t)(ncols_max / 32) * 8 + 15u) & ~15u;
    uint32_t o = 0;
    s.aq = o; o += kMaxGroupTokens * s.q_row;
    s.ad = o; o += kMaxGroupTokens * s.d_row;
    s.red = o; o += (uint32_t)(dual ? 2 : 1) * wk * kMaxGroupTokens * 32 * wr * 4;
    s.total = o;
    return s;
}

// Activations of `mp` tokens into shared memory: the int8 plane (row pitch qrow bytes) and, per unit, the pair
// { f32 scale, correction word } (row pitch drow bytes; see tiled.cuh for the correction).  row_of(i) names the
// global row of token i.  A thread copies 16 quants; the two halves of a unit sit in neighbouring lanes, which
// exchange their sums.  Every thread of the CTA must call this (warp-wide shuffles).
template <int TYPE, typename RowOf>
__device__ __forceinline__ void stage_tokens(const GemvParams& p, uint8_t* aq, uint8_t* ad, int qrow, int drow, int mp, int ncols, int tid,
                                             int nthreads, RowOf row_of) {
    const int vq = ncols >> 4, total = mp * vq;
    for (int v0 = 0; v0 < total; v0 += nthreads) {
        const int v = v0 + tid;
        const bool ok = v < total;
        int i = 0, c = 0;
        uint4 x = make_uint4(0u, 0u, 0u, 0u);
        float d = 0.0f;
        if (ok) {
            i = v / vq; c = v - i * vq;
            const int irow = row_of(i);
            x = __ldcg(reinterpret_cast<const uint4*>(p.in_soa_q + (size_t)irow * p.in_soa_q_stride) + c);
            if (!(c & 1)) d = __ldcg(p.in_soa_d + (size_t)irow * p.in_soa_d_stride + (c >> 1));
            *reinterpret_cast<uint4*>(aq + i * qrow + c * 16) = x;
        }
        const int s = sum16(x);
        const int so = __shfl_xor_sync(0xffffffffu, s, 1);
        if (ok && !(c & 1))
            *reinterpret_cast<uint2*>(ad + i * drow + (c >> 1) * 8) = make_uint2(__float_as_uint(d), (uint32_t)Tiled<TYPE>::correction(s, so));
    }
}

// One pass over groups g0, g0+gstep, ... < ngroups of the tile at `tile` (global memory) for M tokens whose int8
// rows start at shared address aq (row pitch qrow) and whose f32 scales start at shared address ad (row pitch
// drow bytes): acc[i] += (scale_w * scale_x) * integer block dot.
// The units of one group against M tokens.  FULL: all kGroupUnits units are there (no per-unit test).
// Types with one weight scale per group (Tiled<TYPE>::kGroupScale) multiply by it once per group.
template <int TYPE, int M, bool FULL>
__device__ __forceinline__ void group_units(const typename Tiled<TYPE>::Regs& r, int g, int nu, uint32_t aq, int qrow, uint32_t ad,
                                            int drow, int mrem, float (&acc)[M]) {
    using TT = Tiled<TYPE>;
    float part[M];
#pragma unroll
    for (int i = 0; i < M; ++i) part[i] = 0.0f;
#pragma unroll
    for (int u = 0; u < kGroupUnits; ++u) {
        if (FULL || u < nu) {
            int w[8];
            TT::decode(r, u, w);
            const uint32_t qb = aq + (g * kGroupUnits + u) * 32, db = ad + (g * kGroupUnits + u) * 8;
#pragma unroll
            for (int i = 0; i < M; ++i) {
                if (M == 1 || i < mrem) {
                    const uint4 q0 = lds128(qb + i * qrow), q1 = lds128(qb + i * qrow + 16);
                    const uint2 dc = lds64(db + i * drow);   // the token's scale and correction word for this unit
                    const float dx = __uint_as_float(dc.x);
                    const float t = (float)unit_dot<TYPE>(w, q0, q1, (int)dc.y, r, u);
                    if (TT::kGroupScale) part[i] = fmaf(t, dx, part[i]);
                    else acc[i] = fmaf(TT::dscale(r, u) * dx, t, acc[i]);
                }
            }
        }
    }
    if (TT::kGroupScale) {
        const float dw = TT::dscale(r, 0);
#pragma unroll
        for (int i = 0; i < M; ++i)
            if (M == 1 || i < mrem) acc[i] = fmaf(dw, part[i], acc[i]);
    }
}

// The same for one token against the same group of two matrices (up and gate rows of one tile): the token's quants,
// scale and correction word are fetched once per unit and serve both, and the two dot chains are independent.
template <int TYPE, bool FULL>
__device__ __forceinline__ void group_units_pair(const typename Tiled<TYPE>::Regs& ra, const typename Tiled<TYPE>::Regs& rb, int g, int nu,
                                                 uint32_t aq, uint32_t ad, float& acc_a, float& acc_b) {
    using TT = Tiled<TYPE>;
    float part_a = 0.0f, part_b = 0.0f;
#pragma unroll
    for (int u = 0; u < kGroupUnits; ++u) {
        if (FULL || u < nu) {
            const uint32_t qb = aq + (g * kGroupUnits + u) * 32, db = ad + (g * kGroupUnits + u) * 8;
            const uint4 q0 = lds128(qb), q1 = lds128(qb + 16);
            const uint2 dc = lds64(db);
            const float dx = __uint_as_float(dc.x);
            int wa[8], wb[8];
            TT::decode(ra, u, wa);
            TT::decode(rb, u, wb);
            const float ta = (float)unit_dot<TYPE>(wa, q0, q1, (int)dc.y, ra, u);
            const float tb = (float)unit_dot<TYPE>(wb, q0, q1, (int)dc.y, rb, u);
            if (TT::kGroupScale) { part_a = fmaf(ta, dx, part_a); part_b = fmaf(tb, dx, part_b); }
            else { acc_a = fmaf(TT::dscale(ra, u) * dx, ta, acc_a); acc_b = fmaf(TT::dscale(rb, u) * dx, tb, acc_b); }
        }
    }
    if (TT::kGroupScale) {
        acc_a = fmaf(TT::dscale(ra, 0), part_a, acc_a);
        acc_b = fmaf(TT::dscale(rb, 0), part_b, acc_b);
    }
}

// One pass over groups g0, g0+gstep, ... < ngroups of the tile at `tile` (global memory) for M tokens whose int8
// rows start at shared address aq (row pitch qrow) and whose f32 scales start at shared address ad (row pitch
// drow bytes): acc[i] += (scale_w * scale_x) * integer block dot.
template <int TYPE, int M>
__device__ __forceinline__ void dot_pass(const uint8_t* tile, int g0, int ngroups, int gstep, int lane, int nb, uint32_t aq,
                                         int qrow, uint32_t ad, int drow, int mrem, float (&acc)[M]) {
    using TT = Tiled<TYPE>;
    for (int g = g0; g < ngroups; g += gstep) {
        const int nu = min(kGroupUnits, nb - g * kGroupUnits);
        typename TT::Regs r;
        TT::load(tile, g, lane, nu, r);
        if (nu == kGroupUnits) group_units<TYPE, M, true>(r, g, nu, aq, qrow, ad, drow, mrem, acc);
        else group_units<TYPE, M, false>(r, g, nu, aq, qrow, ad, drow, mrem, acc);
    }
}

__device__ __forceinline__ float sum_slices(const float* red, int mat, int wk, int i, int width, int col) {
    float v = 0.0f;
    for (int k = 0; k < wk; ++k) v += red[((mat * wk + k) * kMaxGroupTokens + i) * width + col];
    return v;
}

// grid = (row items, max entries); an instance handles the entries whose weight type is TYPE.
template <int TYPE, int STAGE, bool DUAL>
__global__ void __launch_bounds__(kThreadsT, 4) tile_kernel(const GemvParams p, int wk, int wr) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_row[kMaxGroupTokens];   // pair row of each token (output row of gate/up, input row of down)
    __shared__ int s_tok[kMaxGroupTokens];
    __shared__ int s_done[kMaxGroupTokens];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nthreads = (int)blockDim.x, nwarps = nthreads >> 5;
    griddep_wait();
    if (threadIdx.x == 0) griddep_launch();
    // one look-up names everything the CTA needs: the entry (expert, token count, pair rows)
    const int4* entv = reinterpret_cast<const int4*>(p.group_list + kListHeader + kListEntry * blockIdx.y);
    const int n_entries = __ldcg(p.group_list);
    const int4 e0 = __ldcg(entv), e1 = __ldcg(entv + 1), e2 = __ldcg(entv + 2);
    if ((int)blockIdx.y >= n_entries) return;
    const int expert = e0.x, m = e0.z;
    const bool shared = expert < 0;
    if ((shared ? p.type_shared : p.type_routed) != TYPE) return;
    const int nrows = shared ? p.nrows_shared : p.nrows_routed;
    const int ncols = shared ? p.ncols_shared : p.ncols_routed, nb = ncols >> 5;
    const int width = 32 * wr, tile0 = blockIdx.x * wr, tiles_total = nrows / 32;
    if (tile0 >= tiles_total) return;
    const TileSmem ts = tile_smem(max(p.ncols_routed, p.ncols_shared), wr, wk, DUAL);
    float* red = reinterpret_cast<float*>(smem + ts.red);
    const uint32_t aq = smem_u32(smem + ts.aq), ad = smem_u32(smem + ts.ad);
    const int qrow = (int)ts.q_row, drow = (int)ts.d_row;

    // the warp's weights do not depend on the activations: start their first loads before staging
    const int wr_id = warp / wk, wk_id = warp - wr_id * wk;
    const bool tile_valid = tile0 + wr_id < tiles_total;
    const int64_t tb = Tiled<TYPE>::tile_bytes(ncols);
    const uint8_t* wa = (STAGE == kStageGateUp ? (shared ? p.sh_b : p.w_b + (size_t)expert * p.stride_b)
                                               : (shared ? p.sh_a : p.w_a + (size_t)expert * p.stride_a)) + (size_t)(tile0 + wr_id) * tb;
    const uint8_t* wb = DUAL ? (shared ? p.sh_a : p.w_a + (size_t)expert * p.stride_a) + (size_t)(tile0 + wr_id) * tb : nullptr;
    const int ngroups = (nb + kGroupUnits - 1) / kGroupUnits;
    if (tile_valid) {
        // ask for the warp's units now: they arrive in L2 while the activations are staged
        for (int g = wk_id; g < ngroups; g += wk) {
            const int nu = min(kGroupUnits, nb - g * kGroupUnits);
            Tiled<TYPE>::prefetch(wa, g, lane, nu);
            if (DUAL) Tiled<TYPE>::prefetch(wb, g, lane, nu);
        }
    }
    if (tid < kMaxGroupTokens) {
        const int rows[kMaxGroupTokens] = {e1.x, e1.y, e1.z, e1.w, e2.x, e2.y, e2.z, e2.w};
        int prow = 0;
#pragma unroll
        for (int j = 0; j < kMaxGroupTokens; ++j) if (j == tid) prow = rows[j];
        s_row[tid] = prow;
        s_tok[tid] = shared ? prow - p.T * p.top_k : prow / p.top_k;
    }
    __syncthreads();
    // activations of the entry's tokens
    stage_tokens<TYPE>(p, smem + ts.aq, smem + ts.ad, qrow, drow, m, ncols, tid, nthreads,
                       [&](int i) { return (STAGE == kStageGateUp) ? s_tok[i] : s_row[i]; });
    __syncthreads();

#pragma unroll
    for (int mat = 0; mat < (DUAL ? 2 : 1); ++mat) {
        // one set of accumulators: the partial sums of a matrix go to shared memory before the next starts
        float acc[kMaxGroupTokens];
#pragma unroll
        for (int i = 0; i < kMaxGroupTokens; ++i) acc[i] = 0.0f;
        const uint8_t* tile = mat == 0 ? wa : wb;
        if (tile_valid) {
            if (m == 1) {
                float a1[1] = {0.0f};
                dot_pass<TYPE, 1>(tile, wk_id, ngroups, wk, lane, nb, aq, qrow, ad, drow, 1, a1);
                acc[0] = a1[0];
            } else if (m == 2) {
                float a2[2] = {0.0f, 0.0f};
                dot_pass<TYPE, 2>(tile, wk_id, ngroups, wk, lane, nb, aq, qrow, ad, drow, 2, a2);
                acc[0] = a2[0]; acc[1] = a2[1];
            } else {
                // at most four tokens per pass; tokens 4..7 stream the tile again (it is in L2 by then)
                float a4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                dot_pass<TYPE, 4>(tile, wk_id, ngroups, wk, lane, nb, aq, qrow, ad, drow, m, a4);
                acc[0] = a4[0]; acc[1] = a4[1]; acc[2] = a4[2]; acc[3] = a4[3];
                if (m > 4) {
                    float b4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    dot_pass<TYPE, 4>(tile, wk_id, ngroups, wk, lane, nb, aq + 4 * qrow, qrow, ad + 4 * drow, drow, m - 4, b4);
                    acc[4] = b4[0]; acc[5] = b4[1]; acc[6] = b4[2]; acc[7] = b4[3];
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kMaxGroupTokens; ++i)
            if (i < m) red[((mat * wk + wk_id) * kMaxGroupTokens + i) * width + wr_id * 32 + lane] = acc[i];
    }
    __syncthreads();

    if (STAGE == kStageGateUp) {
        // (token, row tile): sum the K slices, activation, Q8_1 of the 32 results (lane = element)
        for (int pr = warp; pr < m * wr; pr += nwarps) {
            const int i = pr / wr, wq = pr - i * wr;
            if (tile0 + wq >= tiles_total) continue;
            const float u = sum_slices(red, 0, wk, i, width, wq * 32 + lane);
            float v;
            if (DUAL) v = silu_mul_ref(sum_slices(red, 1, wk, i, width, wq * 32 + lane), u);
            else { const float r = fmaxf(u, 0.0f); v = r * r; }
            float amax = fabsf(v), sum = v;
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) {
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
                sum += __shfl_xor_sync(0xffffffffu, sum, s);
            }
            const float d = amax / 127.0f;
            const int8_t q = (amax == 0.0f) ? (int8_t)0 : (int8_t)roundf(v / d);
            const int orow = s_row[i];
            uint8_t* out = p.inter_q8 + (size_t)orow * p.inter_stride + (size_t)(tile0 + wq) * kQ81Bytes;
            reinterpret_cast<int8_t*>(out)[4 + lane] = q;
            const __half dh = __float2half(d);
            if (lane == 0) *reinterpret_cast<__half2*>(out) = __halves2half2(dh, __float2half(sum));
            // the same block as planes, the form the down stage reads
            p.out_soa_q[(size_t)orow * p.out_soa_q_stride + (size_t)(tile0 + wq) * 32 + lane] = q;
            if (lane == 0) p.out_soa_d[(size_t)orow * p.out_soa_d_stride + (tile0 + wq)] = __half2float(dh);
        }
        return;
    }

    const int H = p.H, r0 = tile0 * 32, rows_here = min(width, H - r0);
    for (int e = tid; e < m * width; e += nthreads) {
        const int i = e / width, c = e - i * width;
        if (c < rows_here) p.pair_out[(size_t)s_row[i] * H + r0 + c] = sum_slices(red, 0, wk, i, width, c);
    }
    if (p.no_combine) return;
    // Whoever completes a token's contributions for this row tile adds them up.  The CTA barrier orders the rows
    // written above before thread 0's counter increment, which releases them and acquires the other arrivals'
    // (both cumulative); the next barrier orders the reads below behind it.
    __syncthreads();
    if (tid == 0) {
        const int expected = p.top_k + (p.nrows_shared > 0 ? 1 : 0);
        // one token: release and acquire in the increment itself; several: one fence on either side of their increments
        if (m > 1) __threadfence();
        for (int i = 0; i < m; ++i) {
            int* ctr = p.combine_ctr + (size_t)s_tok[i] * p.n_row_tiles + blockIdx.x;
            const int c = m > 1 ? atomicAdd(ctr, 1) : atom_add_acq_rel_gpu(ctr, 1);
            s_done[i] = (c == expected - 1);
            if (c == expected - 1) *ctr = 0;
        }
        if (m > 1) __threadfence();
    }
    __syncthreads();
    const int k = p.top_k;
    for (int i = 0; i < m; ++i) {
        if (!s_done[i]) continue;
        const int t = s_tok[i];
        for (int r = tid; r < rows_here; r += nthreads) {
            const int h = r0 + r;
            float sum = 0.0f;   // weighted_combine_kernel (chimere_kernels.cu:1551-1565): slots ascending
            for (int j = 0; j < k; ++j)
                sum = fmaf(p.topk_w[(size_t)t * k + j], __ldcg(p.pair_out + ((size_t)t * k + j) * H + h), sum);
            if (p.nrows_shared > 0) {  // sigmoid_gate_add_kernel (scratch_pool.rs:266-277)
                const float sh = __ldcg(p.pair_out + ((size_t)p.T * k + t) * H + h);
                if (p.sh_gate_logit) sum = fmaf(sh, sigmoid_ref(__ldcg(p.sh_gate_logit + t)), sum);
                else sum = sh + sum;
            }
            p.y[(size_t)t * H + h] = sum;
        }
    }
}

// ------------------------------------------------------------------------------------------
// The same work with the weights brought in by bulk asynchronous copies.
//
// A CTA's weights are one contiguous piece of the tiled layout per (matrix, row tile, K slice), so every warp
// asks for its own pieces with one cp.async.bulk each as soon as the work entry is known and waits for them on
// its own mbarrier: no address arithmetic, no register staging and no L2 prefetch in the inner loop, and the
// copies run while the CTA stages the activations.  Units are then read from shared memory with the same
// 128-bit-per-lane pattern (conflict-free).  A CTA holds all its weights at once; several CTAs per SM keep
// enough bytes in flight.  Tokens are taken `mt` at a time so that the planes stay small.
struct BulkSmem { uint32_t w_slot, aq, ad, red, total, q_row, d_row; };
__host__ __device__ inline BulkSmem bulk_smem(uint32_t tile_bytes_max, int ncols_max, int wr, int wk, int nmat, int mt, bool need_red) {
    BulkSmem s;
    s.w_slot = (tile_bytes_max + 127u) & ~127u;
    s.q_row = (uint32_t)ncols_max;
    s.d_row = ((uint32_t)(ncols_max / 32) * 8 + 15u) & ~15u;
    uint32_t o = (uint32_t)nmat * wr * s.w_slot;
    s.aq = o; o += (uint32_t)mt * s.q_row;
    s.ad = o; o += (uint32_t)mt * s.d_row;
    s.red = o; o += need_red ? (uint32_t)nmat * wk * mt * 32 * wr * 4 : 0u;
    s.total = o;
    return s;
}

template <int TYPE, int M>
__device__ __forceinline__ void dot_pass_s(uint32_t tile, int g0, int g1, int lane, int nb, uint32_t aq, int qrow, uint32_t ad, int drow,
                                           int mrem, float (&acc)[M]) {
    using TT = Tiled<TYPE>;
    for (int g = g0; g < g1; ++g) {
        const int nu = min(kGroupUnits, nb - g * kGroupUnits);
        typename TT::Regs r;
        TT::loads(tile, g, lane, nu, r);
        if (nu == kGroupUnits) group_units<TYPE, M, true>(r, g, nu, aq, qrow, ad, drow, mrem, acc);
        else group_units<TYPE, M, false>(r, g, nu, aq, qrow, ad, drow, mrem, acc);
    }
}

template <int TYPE>
__device__ __forceinline__ void dot_pass_pair_s(uint32_t tile_a, uint32_t tile_b, int g0, int g1, int lane, int nb, uint32_t aq, uint32_t ad,
                                                float& acc_a, float& acc_b) {
    using TT = Tiled<TYPE>;
    for (int g = g0; g < g1; ++g) {
        const int nu = min(kGroupUnits, nb - g * kGroupUnits);
        typename TT::Regs ra, rb;
        TT::loads(tile_a, g, lane, nu, ra);
        TT::loads(tile_b, g, lane, nu, rb);
        if (nu == kGroupUnits) group_units_pair<TYPE, true>(ra, rb, g, nu, aq, ad, acc_a, acc_b);
        else group_units_pair<TYPE, false>(ra, rb, g, nu, aq, ad, acc_a, acc_b);
    }
}

// grid = (row items, max entries), block = 32 * wr * wk threads (wk = 1 << wk_shift, wr = 1 << wr_shift).
template <int TYPE, int STAGE, bool DUAL, int MT>
__global__ void __launch_bounds__(kThreadsT, 3) bulk_kernel(const GemvParams p, int wk_shift, int wr_shift, uint32_t tile_bytes_max) {
    constexpr int mt = MT;   // tokens per pass
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_row[kMaxGroupTokens];
    __shared__ int s_tok[kMaxGroupTokens];
    __shared__ int s_done[kMaxGroupTokens];
    __shared__ __align__(8) uint64_t s_bar[kWarpsT];
    using TT = Tiled<TYPE>;
    constexpr int kMat = DUAL ? 2 : 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wk = 1 << wk_shift, wr = 1 << wr_shift, nwarps = wk * wr, nthreads = 32 * nwarps;
    // Gate/up follows the kernel that writes the work list: wait for it, then let the down stage's CTAs come in
    // behind this grid.  The down stage is launched after a gate/up grid whose CTAs all passed that wait, so the
    // list is complete when its CTAs start: they look up their entry and ask for their weights first, and wait
    // for the gate/up results only then.
    if (STAGE == kStageGateUp) { griddep_wait(); if (threadIdx.x == 0) griddep_launch(); }
    const int4* entv = reinterpret_cast<const int4*>(p.group_list + kListHeader + kListEntry * blockIdx.y);
    const int n_entries = __ldcg(p.group_list);
    const int4 e0 = __ldcg(entv), e1 = __ldcg(entv + 1), e2 = __ldcg(entv + 2);
    const int expert = e0.x, m = e0.z;
    const bool shared = expert < 0;
    const int nrows = shared ? p.nrows_shared : p.nrows_routed;
    const int ncols = shared ? p.ncols_shared : p.ncols_routed, nb = ncols >> 5;
    const int width = 32 * wr, tile0 = blockIdx.x << wr_shift, tiles_total = nrows >> 5;
    if ((int)blockIdx.y >= n_entries || (shared ? p.type_shared : p.type_routed) != TYPE || tile0 >= tiles_total) {
        // Nothing to do for this CTA.  A down-stage CTA still waits for the grid before it: this grid must not count as
        // complete while the gate/up grid is running, because whatever follows in the stream (a second down instance for
        // the other weight type, the caller's next kernel) depends on this grid only.
        if (STAGE == kStageDown) griddep_wait();
        return;
    }
    // down stage: let the next kernel of the stream (the next layer's router, if it was launched programmatically)
    // bring its CTAs in; it waits for this grid before it touches the workspace
    if (STAGE == kStageDown && tid == 0) griddep_launch();
    const bool need_red = STAGE == kStageGateUp || wk > 1;
    const BulkSmem bs = bulk_smem(tile_bytes_max, max(p.ncols_routed, p.ncols_shared), wr, wk, kMat, mt, need_red);
    float* red = reinterpret_cast<float*>(smem + bs.red);
    const uint32_t aq = smem_u32(smem + bs.aq), ad = smem_u32(smem + bs.ad);
    const int qrow = (int)bs.q_row, drow = (int)bs.d_row;

    // ---- this warp's pieces: K slice [u0, u1) of row tile tile0 + wr_id, of one or two matrices ----
    const int wr_id = warp >> wk_shift, wk_id = warp & (wk - 1);
    const bool tile_valid = tile0 + wr_id < tiles_total;
    const int upw = ((((nb + wk - 1) >> wk_shift) + TT::kChunkUnits - 1) / TT::kChunkUnits) * TT::kChunkUnits;
    const int u0 = min(nb, wk_id * upw), u1 = min(nb, u0 + upw);
    const uint32_t off = TT::unit_offset(u0), bytes = tile_valid ? TT::unit_offset(u1) - off : 0u;
    const int64_t tb = TT::tile_bytes(ncols);
    const uint32_t ws0 = smem_u32(smem) + (uint32_t)wr_id * bs.w_slot, ws1 = ws0 + (uint32_t)wr * bs.w_slot;
    if (bytes > 0 && lane == 0) {
        const uint8_t* wa = (STAGE == kStageGateUp ? (shared ? p.sh_b : p.w_b + (size_t)expert * p.stride_b)
                                                   : (shared ? p.sh_a : p.w_a + (size_t)expert * p.stride_a)) + (size_t)(tile0 + wr_id) * tb;
        mbar_init(&s_bar[warp], 1);
        mbar_fence_init();
        mbar_expect_tx(&s_bar[warp], bytes * kMat);
        bulk_g2s(smem + (size_t)wr_id * bs.w_slot + off, wa + off, bytes, &s_bar[warp]);
        if (DUAL) {
            const uint8_t* wb = (shared ? p.sh_a : p.w_a + (size_t)expert * p.stride_a) + (size_t)(tile0 + wr_id) * tb;
            bulk_g2s(smem + (size_t)(wr + wr_id) * bs.w_slot + off, wb + off, bytes, &s_bar[warp]);
        }
    }
    if (tid < kMaxGroupTokens) {
        const int rows[kMaxGroupTokens] = {e1.x, e1.y, e1.z, e1.w, e2.x, e2.y, e2.z, e2.w};
        int prow = 0;
#pragma unroll
        for (int j = 0; j < kMaxGroupTokens; ++j) if (j == tid) prow = rows[j];
        s_row[tid] = prow;
        s_tok[tid] = shared ? prow - p.T * p.top_k : prow / p.top_k;
    }
    if (STAGE == kStageDown) griddep_wait();
    __syncthreads();   // also orders lane 0's barrier set-up before the other lanes' wait

    const int g0 = u0 / kGroupUnits, g1 = (u1 + kGroupUnits - 1) / kGroupUnits;
    const int H = p.H, r0 = tile0 * 32, rows_here = min(width, H - r0);
    bool arrived = false;
    for (int i0 = 0; i0 < m; i0 += mt) {
        const int mp = min(mt, m - i0);
        if (i0 > 0) __syncthreads();   // the planes and partial sums of the previous tokens are no longer read
        // activations of tokens i0 .. i0+mp
        stage_tokens<TYPE>(p, smem + bs.aq, smem + bs.ad, qrow, drow, mp, ncols, tid, nthreads,
                           [&](int i) { return (STAGE == kStageGateUp) ? s_tok[i0 + i] : s_row[i0 + i]; });
        __syncthreads();
        if (!arrived) {
            if (bytes > 0 && !mbar_wait(&s_bar[warp], 0)) {
                if (lane == 0 && p.status) atomicOr(p.status, kStatusWaitTimeout);
                mbar_wait(&s_bar[warp], 0);   // give the copies in flight a second, equally bounded, chance before going on
            }
            arrived = true;
        }
        if (DUAL && need_red && (MT == 1 || mp == 1)) {
            // one token, gate and up rows of the tile together: the token's values are fetched once for both
            float au = 0.0f, ag = 0.0f;
            if (bytes > 0) dot_pass_pair_s<TYPE>(ws0, ws1, g0, g1, lane, nb, aq, ad, au, ag);
            red[(wk_id * mt) * width + wr_id * 32 + lane] = au;
            red[((wk + wk_id) * mt) * width + wr_id * 32 + lane] = ag;
        } else
#pragma unroll
        for (int mat = 0; mat < kMat; ++mat) {
            float acc[MT];
#pragma unroll
            for (int i = 0; i < MT; ++i) acc[i] = 0.0f;
            const uint32_t tile = mat == 0 ? ws0 : ws1;
            if (bytes > 0) {
                if (MT == 1 || mp == 1) {
                    float a1[1] = {0.0f};
                    dot_pass_s<TYPE, 1>(tile, g0, g1, lane, nb, aq, qrow, ad, drow, 1, a1);
                    acc[0] = a1[0];
                } else if (MT == 2 || mp == 2) {
                    float a2[2] = {0.0f, 0.0f};
                    dot_pass_s<TYPE, 2>(tile, g0, g1, lane, nb, aq, qrow, ad, drow, 2, a2);
                    acc[0] = a2[0]; acc[MT > 1 ? 1 : 0] = a2[1];
                } else {
                    // four tokens at a time; tokens 4..7 read the weights from shared memory again
#pragma unroll
                    for (int h = 0; h < MT / 4; ++h) {
                        if (4 * h < mp) {
                            float a4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                            dot_pass_s<TYPE, 4>(tile, g0, g1, lane, nb, aq + 4 * h * qrow, qrow, ad + 4 * h * drow, drow, mp - 4 * h, a4);
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[(4 * h + i) < MT ? 4 * h + i : 0] = a4[i];
                        }
                    }
                }
            }
            if (need_red) {
#pragma unroll
                for (int i = 0; i < MT; ++i)
                    if (i < mp) red[((mat * wk + wk_id) * mt + i) * width + wr_id * 32 + lane] = acc[i];
            } else if (tile_valid) {
                // a warp owns its rows' whole sums: straight to the per-pair rows
#pragma unroll
                for (int i = 0; i < MT; ++i)
                    if (i < mp) p.pair_out[(size_t)s_row[i0 + i] * H + r0 + wr_id * 32 + lane] = acc[i];
            }
        }
        if (!need_red) continue;
        __syncthreads();
        if (STAGE == kStageGateUp) {
            // (token, row tile): sum the K slices, activation, Q8_1 of the 32 results (lane = element)
            for (int pr = warp; pr < (mp << wr_shift); pr += nwarps) {
                const int i = pr >> wr_shift, wq = pr & (wr - 1);
                if (tile0 + wq >= tiles_total) continue;
                float u = 0.0f, g = 0.0f;
                for (int k = 0; k < wk; ++k) {
                    u += red[(k * mt + i) * width + wq * 32 + lane];
                    if (DUAL) g += red[((wk + k) * mt + i) * width + wq * 32 + lane];
                }
                float v;
                if (DUAL) v = silu_mul_ref(g, u);
                else { const float r = fmaxf(u, 0.0f); v = r * r; }
                float amax = fabsf(v), sum = v;
#pragma unroll
                for (int s = 16; s > 0; s >>= 1) {
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
                    sum += __shfl_xor_sync(0xffffffffu, sum, s);
                }
                const float d = amax / 127.0f;
                const int8_t q = (amax == 0.0f) ? (int8_t)0 : (int8_t)roundf(v / d);
                const int orow = s_row[i0 + i];
                uint8_t* out = p.inter_q8 + (size_t)orow * p.inter_stride + (size_t)(tile0 + wq) * kQ81Bytes;
                reinterpret_cast<int8_t*>(out)[4 + lane] = q;
                const __half dh = __float2half(d);
                if (lane == 0) *reinterpret_cast<__half2*>(out) = __halves2half2(dh, __float2half(sum));
                p.out_soa_q[(size_t)orow * p.out_soa_q_stride + (size_t)(tile0 + wq) * 32 + lane] = q;
                if (lane == 0) p.out_soa_d[(size_t)orow * p.out_soa_d_stride + (tile0 + wq)] = __half2float(dh);
            }
        } else {
            for (int e = tid; e < mp * width; e += nthreads) {
                const int i = e / width, c = e - i * width;
                if (c < rows_here) {
                    float v = 0.0f;
                    for (int k = 0; k < wk; ++k) v += red[(k * mt + i) * width + c];
                    p.pair_out[(size_t)s_row[i0 + i] * H + r0 + c] = v;
                }
            }
        }
    }
    if (STAGE == kStageGateUp || p.no_combine) return;
    // Whoever completes a token's contributions for this row item adds them up (see tile_kernel).
    __syncthreads();
    if (tid == 0) {
        const int expected = p.top_k + (p.nrows_shared > 0 ? 1 : 0);
        // one token: release and acquire in the increment itself; several: one fence on either side of their increments
        if (m > 1) __threadfence();
        for (int i = 0; i < m; ++i) {
            int* ctr = p.combine_ctr + (size_t)s_tok[i] * p.n_row_tiles + blockIdx.x;
            const int c = m > 1 ? atomicAdd(ctr, 1) : atom_add_acq_rel_gpu(ctr, 1);
            s_done[i] = (c == expected - 1);
            if (c == expected - 1) *ctr = 0;
        }
        if (m > 1) __threadfence();
    }
    __syncthreads();
    const int k = p.top_k;
    for (int i = 0; i < m; ++i) {
        if (!s_done[i]) continue;
        const int t = s_tok[i];
        for (int r = tid; r < rows_here; r += nthreads) {
            const int h = r0 + r;
            float sum = 0.0f;   // weighted_combine_kernel (chimere_kernels.cu:1551-1565): slots ascending
            for (int j = 0; j < k; ++j)
                sum = fmaf(p.topk_w[(size_t)t * k + j], __ldcg(p.pair_out + ((size_t)t * k + j) * H + h), sum);
            if (p.nrows_shared > 0) {  // sigmoid_gate_add_kernel (scratch_pool.rs:266-277)
                const float sh = __ldcg(p.pair_out + ((size_t)p.T * k + t) * H + h);
                if (p.sh_gate_logit) sum = fmaf(sh, sigmoid_ref(__ldcg(p.sh_gate_logit + t)), sum);
                else sum = sh + sum;
            }
            p.y[(size_t)t * H + h] = sum;
        }
    }
}

// ------------------------------------------------------------------ launchers --------------
struct Geom { int wk, wr; };
static int ngroups_of(int ncols) { return (ncols / 32 + kGroupUnits - 1) / kGroupUnits; }
static int64_t tile_bytes_of(int type, int ncols) { return tiled_matrix_bytes(type, 32, ncols); }
static int log2i(int v) { int s = 0; while ((1 << s) < v) ++s; return s; }

// Gate/up: one row tile per CTA, its K range cut over the eight warps.
static Geom geom_for(int ngroups_min) {
    int wk = kWarpsT;
    while (wk > 1 && wk > ngroups_min) wk >>= 1;
    return Geom{wk, kWarpsT / wk};
}
TiledGeomHost tiled_gate_up_geom(int type_routed, int type_shared, int H, bool has_shared) {
    (void)type_routed; (void)type_shared; (void)has_shared;
    const Geom t = geom_for(ngroups_of(H));
    return TiledGeomHost{t.wk, t.wr};
}
// Down stage: rows are short (F columns), so a warp keeps a whole row tile to itself when that leaves it at most
// four groups; the CTA takes as many row tiles as keep its weights near 40 KB.  The same split for every batch
// size: a token's sums are added in the same order whatever its batch.
TiledGeomHost tiled_down_geom(int type_routed, int F, int type_shared, int F_s, int T) {
    (void)T;
    int g = ngroups_of(F);
    int64_t tb = tile_bytes_of(type_routed, F);
    if (F_s > 0) { g = min(g, ngroups_of(F_s)); tb = max(tb, tile_bytes_of(type_shared, F_s)); }
    int wk = 1;
    while (wk < kWarpsT && g / wk > 4) wk <<= 1;
    int wr = kWarpsT / wk;
    while (wr > 1 && (int64_t)wr * tb > 40 * 1024) wr >>= 1;
    return TiledGeomHost{wk, wr};
}

template <int TYPE, int STAGE, bool DUAL>
static cudaError_t launch_tile_t(const GemvParams& p, int max_entries, int wk, int wr, cudaStream_t stream) {
    const TileSmem ts = tile_smem(max(p.ncols_routed, p.ncols_shared), wr, wk, DUAL);
    if (ts.total > 200 * 1024) return cudaErrorInvalidValue;
    static bool attr_done[64] = {};
    cudaError_t e = max_smem_once(tile_kernel<TYPE, STAGE, DUAL>, 200 * 1024, attr_done);
    if (e != cudaSuccess) return e;
    const int rows = max(p.nrows_routed, p.nrows_shared);
    const int items = (rows / 32 + wr - 1) / wr;
    return launch_pdl(tile_kernel<TYPE, STAGE, DUAL>, dim3(items, max_entries), 32 * wk * wr, ts.total, stream, p, wk, wr);
}

// How the bulk-copy kernel fits an SM: CTAs per SM and tokens per pass.  ok = false: the weights of one CTA do not
// fit, or something is not 16-byte aligned; the caller then takes the kernel that loads through registers.
struct BulkPlan { bool ok; int mt; uint32_t tile_bytes_max, smem; };
static BulkPlan plan_bulk(const GemvParams& p, int stage, bool dual, int wk, int wr) {
    BulkPlan b{false, 0, 0, 0};
    const bool gu = stage == kStageGateUp;
    int64_t tb = tile_bytes_of(p.type_routed, p.ncols_routed);
    if (p.nrows_shared > 0) tb = max(tb, tile_bytes_of(p.type_shared, p.ncols_shared));
    const uintptr_t ptrs = (uintptr_t)p.w_a | (uintptr_t)p.w_b | (uintptr_t)p.sh_a | (uintptr_t)p.sh_b | (uintptr_t)p.in_soa_q |
                           (uintptr_t)p.stride_a | (uintptr_t)p.stride_b | (uintptr_t)p.in_soa_q_stride;
    if (ptrs & 15) return b;
    const int nmat = dual ? 2 : 1;
    const bool need_red = gu || wk > 1;
    const int ncols_max = max(p.ncols_routed, p.ncols_shared);
    const int threads = 32 * wk * wr;
    const int sm_bytes = 228 * 1024, per_cta = 1024 + 192;   // an SM's shared memory; per CTA the system's reserve and the kernel's static variables
    const int max_ctas = min(8, 1536 / threads);
    // decode-size batches: as many CTAs per SM as fit one token per pass, then as many tokens as still fit;
    // larger batches: at least four tokens per pass if that fits at all
    const int mt_floor = (p.T > 16 && !p.few_tokens) ? 4 : 1;
    for (int floor_mt = mt_floor; floor_mt >= 1 && !b.ok; floor_mt = (floor_mt == 1 ? 0 : 1)) {
        int ctas = 0;
        for (int c = max_ctas; c >= 1; --c)
            if ((int64_t)bulk_smem((uint32_t)tb, ncols_max, wr, wk, nmat, floor_mt, need_red).total <= sm_bytes / c - per_cta) { ctas = c; break; }
        if (!ctas) continue;
        for (int mt = kMaxGroupTokens; mt >= floor_mt; mt >>= 1)
            if ((int64_t)bulk_smem((uint32_t)tb, ncols_max, wr, wk, nmat, mt, need_red).total <= sm_bytes / ctas - per_cta) {
                b.ok = true; b.mt = mt; b.tile_bytes_max = (uint32_t)tb;
                b.smem = bulk_smem((uint32_t)tb, ncols_max, wr, wk, nmat, mt, need_red).total;
                break;
            }
    }
    return b;
}

template <int TYPE, int STAGE, bool DUAL, int MT>
static cudaError_t launch_bulk_m(const GemvParams& p, int max_entries, int wk, int wr, const BulkPlan& b, cudaStream_t stream) {
    static bool attr_done[64] = {};
    cudaError_t e = max_smem_once(bulk_kernel<TYPE, STAGE, DUAL, MT>, 226 * 1024, attr_done);
    if (e != cudaSuccess) return e;
    const int rows = max(p.nrows_routed, p.nrows_shared);
    const int items = (rows / 32 + wr - 1) / wr;
    return launch_pdl(bulk_kernel<TYPE, STAGE, DUAL, MT>, dim3(items, max_entries), 32 * wk * wr, b.smem, stream, p, log2i(wk), log2i(wr),
                      b.tile_bytes_max);
}
template <int TYPE, int STAGE, bool DUAL>
static cudaError_t launch_bulk_t(const GemvParams& p, int max_entries, int wk, int wr, const BulkPlan& b, cudaStream_t stream) {
    switch (b.mt) {
        case 1: return launch_bulk_m<TYPE, STAGE, DUAL, 1>(p, max_entries, wk, wr, b, stream);
        case 2: return launch_bulk_m<TYPE, STAGE, DUAL, 2>(p, max_entries, wk, wr, b, stream);
        case 4: return launch_bulk_m<TYPE, STAGE, DUAL, 4>(p, max_entries, wk, wr, b, stream);
        default: return launch_bulk_m<TYPE, STAGE, DUAL, 8>(p, max_entries, wk, wr, b, stream);
    }
}

template <int STAGE>
static cudaError_t dispatch_tile(int type, const GemvParams& p, int max_entries, int wk, int wr, cudaStream_t stream) {
    const bool dual = STAGE == kStageGateUp && p.act == CHIMERE_ACT_SWIGLU;
    const BulkPlan b = plan_bulk(p, STAGE, dual, wk, wr);
#define CHIMERE_LAUNCH(T_, D_) \
    (b.ok ? launch_bulk_t<T_, STAGE, D_>(p, max_entries, wk, wr, b, stream) : launch_tile_t<T_, STAGE, D_>(p, max_entries, wk, wr, stream))
    switch (type) {
        case CHIMERE_TYPE_Q4_0: return dual ? CHIMERE_LAUNCH(CHIMERE_TYPE_Q4_0, true) : CHIMERE_LAUNCH(CHIMERE_TYPE_Q4_0, false);
        case CHIMERE_TYPE_Q8_0: return dual ? CHIMERE_LAUNCH(CHIMERE_TYPE_Q8_0, true) : CHIMERE_LAUNCH(CHIMERE_TYPE_Q8_0, false);
        case CHIMERE_TYPE_IQ3_S: return dual ? CHIMERE_LAUNCH(CHIMERE_TYPE_IQ3_S, true) : CHIMERE_LAUNCH(CHIMERE_TYPE_IQ3_S, false);
        default: return cudaErrorInvalidValue;
    }
#undef CHIMERE_LAUNCH
}

cudaError_t launch_gate_up_tiled(const GemvParams& p, int max_entries, cudaStream_t stream) {
    const TiledGeomHost g = tiled_gate_up_geom(p.type_routed, p.type_shared, p.H, p.nrows_shared > 0);
    cudaError_t e = dispatch_tile<kStageGateUp>(p.type_routed, p, max_entries, g.wk, g.wr, stream);
    if (e == cudaSuccess && p.nrows_shared > 0 && p.type_shared != p.type_routed)
        e = dispatch_tile<kStageGateUp>(p.type_shared, p, max_entries, g.wk, g.wr, stream);
    return e;
}

// p.n_row_tiles must be ceil(H / (32 * wr)) with the geometry of tiled_down_geom
cudaError_t launch_down_tiled(const GemvParams& p, int max_entries, cudaStream_t stream) {
    const TiledGeomHost g = tiled_down_geom(p.type_routed, p.ncols_routed, p.type_shared, p.nrows_shared > 0 ? p.ncols_shared : 0, p.T);
    cudaError_t e = dispatch_tile<kStageDown>(p.type_routed, p, max_entries, g.wk, g.wr, stream);
    if (e == cudaSuccess && p.nrows_shared > 0 && p.type_shared != p.type_routed)
        e = dispatch_tile<kStageDown>(p.type_shared, p, max_entries, g.wk, g.wr, stream);
    return e;
}

}  // namespace chimere
