// gemv_tiled.cu -- the decode-path GEMV kernels on tiled32 weights (see tiled.cuh).
//
// One warp = 32 consecutive rows of one expert matrix, lane = row.  A warp streams its part of
// the K range with contiguous 512-byte reads (128 bits per lane) straight into registers, decodes
// in registers and multiplies with the tokens' Q8_1 activations, which sit in shared memory as an
// int8 plane + f32 scale plane and are read as warp-wide broadcasts.  The eight warps of a CTA
// are WR row tiles x WK slices of K; slices are added up through shared memory in a fixed order.
//
//   gate_up_tiled_kernel : act(gate . x, up . x) -> Q8_1 blocks of the intermediates
//                          (replaces moe_ffn.rs:1206-1323 and :1597-1700 of the reference)
//   down_tiled_kernel    : down . inter -> per-pair rows, then the weighted combine in slot order
//                          plus the sigmoid-gated shared expert by whichever CTA completes a
//                          token's row tile (replaces moe_ffn.rs:1325-1384 and :1700-1766)
#include "common.cuh"
#include "kernels.h"
#include "tiled.cuh"

namespace chimere {

constexpr int kThreadsT = 256;

// acc[i] += sum over the units of one group of (scale_w * scale_x) * integer block dot, for up to M tokens
template <int TYPE, int M>
__device__ __forceinline__ void group_dot(const typename Tiled<TYPE>::Regs& r, int nu, int unit0, const int8_t* aq,
                                          const float* ad, int ncols, int nb, int m, float (&acc)[M]) {
    using TT = Tiled<TYPE>;
#pragma unroll
    for (int u = 0; u < TT::kGroupUnits; ++u) {
        if (u < nu) {
            int w[8];
            TT::decode(r, u, w);
            const float dw = TT::dscale(r, u);
            const int b = unit0 + u;
#pragma unroll
            for (int i = 0; i < M; ++i) {
                if (i < m) {
                    const int4* q = reinterpret_cast<const int4*>(aq + (size_t)i * ncols + b * 32);
                    const int4 q0 = q[0], q1 = q[1];
                    int s = __dp4a(w[0], q0.x, 0);
                    s = __dp4a(w[1], q0.y, s); s = __dp4a(w[2], q0.z, s); s = __dp4a(w[3], q0.w, s);
                    s = __dp4a(w[4], q1.x, s); s = __dp4a(w[5], q1.y, s); s = __dp4a(w[6], q1.z, s); s = __dp4a(w[7], q1.w, s);
                    acc[i] = fmaf(dw * ad[i * nb + b], (float)TT::finish(s, r, u), acc[i]);
                }
            }
        }
    }
}

// Q8_1 rows (36-byte blocks) -> int8 plane aq[i][ncols] and f32 scale plane ad[i][nb]
__device__ __forceinline__ void stage_q8_rows(const uint8_t* const* rows, int m, int nb, int ncols, int8_t* aq, float* ad, int tid) {
    for (int i = 0; i < m; ++i) {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(rows[i]);
        uint32_t* dq = reinterpret_cast<uint32_t*>(aq + (size_t)i * ncols);
        for (int wd = tid; wd < nb * 9; wd += kThreadsT) {
            const int b = wd / 9, r = wd - b * 9;
            const uint32_t v = __ldcg(src + wd);
            if (r == 0) ad[i * nb + b] = h2f(v & 0xFFFFu);
            else dq[b * 8 + (r - 1)] = v;
        }
    }
}

struct TiledGeom { int wk, wr; };
__host__ __device__ inline TiledGeom tiled_geom(int ngroups_min) {
    int wk = 8;
    while (wk > 1 && wk > ngroups_min) wk >>= 1;
    return TiledGeom{wk, 8 / wk};
}

struct TiledSmem { uint32_t aq, ad, red, total; };
__host__ __device__ inline TiledSmem tiled_smem(int ncols, int wr, int wk, bool dual) {
    TiledSmem s;
    uint32_t o = 0;
    s.aq = o; o += (uint32_t)kMaxGroupTokens * ncols;
    s.ad = o; o += (uint32_t)kMaxGroupTokens * (ncols / 32) * 4;
    o = (o + 15u) & ~15u;
    s.red = o; o += (uint32_t)(dual ? 2 : 1) * wk * kMaxGroupTokens * 32 * wr * 4;
    s.total = o;
    return s;
}

// The shared front part of both kernels: every warp accumulates its (row tile, K slice) for the
// entry's tokens and leaves the partial sums in red[(mat * wk + k) * 8 + i][wr * 32 + lane].
template <int TYPE, bool DUAL, int M>
__device__ __forceinline__ void tile_partials(const uint8_t* tile_a, const uint8_t* tile_b, bool valid, int wk_id, int wk, int wr_id,
                                              int wr, int lane, int ncols, int m, const int8_t* aq, const float* ad, float* red) {
    using TT = Tiled<TYPE>;
    const int nb = ncols >> 5;
    const int ngroups = (nb + TT::kGroupUnits - 1) / TT::kGroupUnits;
    float aa[M], ab[M];
#pragma unroll
    for (int i = 0; i < M; ++i) { aa[i] = 0.0f; ab[i] = 0.0f; }
    if (valid) {
        for (int grp = wk_id; grp < ngroups; grp += wk) {
            const int nu = min(TT::kGroupUnits, nb - grp * TT::kGroupUnits);
            typename TT::Regs ra, rb;
            TT::load(tile_a, grp, lane, nu, ra);
            if (DUAL) TT::load(tile_b, grp, lane, nu, rb);
            group_dot<TYPE, M>(ra, nu, grp * TT::kGroupUnits, aq, ad, ncols, nb, m, aa);
            if (DUAL) group_dot<TYPE, M>(rb, nu, grp * TT::kGroupUnits, aq, ad, ncols, nb, m, ab);
        }
    }
    const int col = wr_id * 32 + lane, width = 32 * wr;
#pragma unroll
    for (int i = 0; i < M; ++i) {
        if (i < m) {
            red[((0 * wk + wk_id) * kMaxGroupTokens + i) * width + col] = aa[i];
            if (DUAL) red[((1 * wk + wk_id) * kMaxGroupTokens + i) * width + col] = ab[i];
        }
    }
}

template <int TYPE, bool DUAL>
__device__ __forceinline__ void tile_partials_m(const uint8_t* tile_a, const uint8_t* tile_b, bool valid, int wk_id, int wk, int wr_id,
                                                int wr, int lane, int ncols, int m, const int8_t* aq, const float* ad, float* red) {
    if (m == 1) tile_partials<TYPE, DUAL, 1>(tile_a, tile_b, valid, wk_id, wk, wr_id, wr, lane, ncols, m, aq, ad, red);
    else if (m == 2) tile_partials<TYPE, DUAL, 2>(tile_a, tile_b, valid, wk_id, wk, wr_id, wr, lane, ncols, m, aq, ad, red);
    else if (m <= 4) tile_partials<TYPE, DUAL, 4>(tile_a, tile_b, valid, wk_id, wk, wr_id, wr, lane, ncols, m, aq, ad, red);
    else tile_partials<TYPE, DUAL, 8>(tile_a, tile_b, valid, wk_id, wk, wr_id, wr, lane, ncols, m, aq, ad, red);
}

__device__ __forceinline__ float sum_slices(const float* red, int mat, int wk, int i, int width, int col) {
    float v = 0.0f;
    for (int k = 0; k < wk; ++k) v += red[((mat * wk + k) * kMaxGroupTokens + i) * width + col];
    return v;
}

// grid = (ceil(max rows / (32*wr)), max entries); an instance handles the entries of its weight type
template <int TYPE, bool DUAL>
__global__ void __launch_bounds__(kThreadsT) gate_up_tiled_kernel(const GemvParams p, int wk, int wr) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ const uint8_t* s_rows[kMaxGroupTokens];
    __shared__ int s_out_row[kMaxGroupTokens];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if ((int)blockIdx.y >= __ldcg(p.group_list)) return;
    const int* ent = p.group_list + kListHeader + 4 * blockIdx.y;
    const int expert = __ldcg(ent), start = __ldcg(ent + 1), m = __ldcg(ent + 2);
    const bool shared = expert < 0;
    if ((shared ? p.type_shared : p.type_routed) != TYPE) return;
    const int nrows = shared ? p.nrows_shared : p.nrows_routed;
    if ((int)blockIdx.x * 32 * wr >= nrows) return;
    const int ncols = p.H, nb = ncols >> 5;
    const TiledSmem sp = tiled_smem(ncols, wr, wk, DUAL);
    int8_t* aq = reinterpret_cast<int8_t*>(smem + sp.aq);
    float* ad = reinterpret_cast<float*>(smem + sp.ad);
    float* red = reinterpret_cast<float*>(smem + sp.red);

    if (tid < m) {
        int t, orow;
        if (shared) { t = start + tid; orow = p.T * p.top_k + t; }
        else { const int q = __ldcg(p.perm + start + tid); t = q / p.top_k; orow = q; }
        s_rows[tid] = p.in_q8 + (size_t)t * p.in_stride;
        s_out_row[tid] = orow;
    }
    __syncthreads();
    stage_q8_rows(s_rows, m, nb, ncols, aq, ad, tid);
    __syncthreads();

    const int wr_id = warp / wk, wk_id = warp - wr_id * wk;
    const int tile = blockIdx.x * wr + wr_id;
    const bool valid = tile * 32 < nrows;
    const int64_t tb = Tiled<TYPE>::tile_bytes(ncols);
    const uint8_t* up = (shared ? p.sh_b : p.w_b + (size_t)expert * p.stride_b) + (size_t)tile * tb;
    const uint8_t* gate = DUAL ? (shared ? p.sh_a : p.w_a + (size_t)expert * p.stride_a) + (size_t)tile * tb : nullptr;
    tile_partials_m<TYPE, DUAL>(up, gate, valid, wk_id, wk, wr_id, wr, lane, ncols, m, aq, ad, red);
    __syncthreads();

    // (token, row tile) pairs: sum the K slices, activation, Q8_1 of the 32 results (lane = element)
    const int width = 32 * wr;
    for (int pr = warp; pr < m * wr; pr += 8) {
        const int i = pr / wr, wq = pr - i * wr;
        const int t32 = blockIdx.x * wr + wq;
        if (t32 * 32 >= nrows) continue;
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
        uint8_t* out = p.inter_q8 + (size_t)s_out_row[i] * p.inter_stride + (size_t)t32 * kQ81Bytes;
        reinterpret_cast<int8_t*>(out)[4 + lane] = q;
        if (lane == 0) *reinterpret_cast<__half2*>(out) = __halves2half2(__float2half(d), __float2half(sum));
    }
}

template <int TYPE>
__global__ void __launch_bounds__(kThreadsT) down_tiled_kernel(const GemvParams p, int wk, int wr) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ const uint8_t* s_rows[kMaxGroupTokens];
    __shared__ int s_out_row[kMaxGroupTokens];
    __shared__ int s_tok[kMaxGroupTokens];
    __shared__ int s_done[kMaxGroupTokens];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if ((int)blockIdx.y >= __ldcg(p.group_list)) return;
    const int* ent = p.group_list + kListHeader + 4 * blockIdx.y;
    const int expert = __ldcg(ent), start = __ldcg(ent + 1), m = __ldcg(ent + 2);
    const bool shared = expert < 0;
    if ((shared ? p.type_shared : p.type_routed) != TYPE) return;
    const int H = p.H;
    const int ncols = shared ? p.ncols_shared : p.ncols_routed, nb = ncols >> 5;
    const int width = 32 * wr;
    const int r0 = blockIdx.x * width;
    if (r0 >= H) return;
    const TiledSmem sp = tiled_smem(max(p.ncols_routed, p.ncols_shared), wr, wk, false);
    int8_t* aq = reinterpret_cast<int8_t*>(smem + sp.aq);
    float* ad = reinterpret_cast<float*>(smem + sp.ad);
    float* red = reinterpret_cast<float*>(smem + sp.red);

    if (tid < m) {
        int t, irow;
        if (shared) { t = start + tid; irow = p.T * p.top_k + t; }
        else { irow = __ldcg(p.perm + start + tid); t = irow / p.top_k; }
        s_rows[tid] = p.in_q8 + (size_t)irow * p.in_stride;
        s_out_row[tid] = irow;
        s_tok[tid] = t;
    }
    __syncthreads();
    stage_q8_rows(s_rows, m, nb, ncols, aq, ad, tid);
    __syncthreads();

    const int wr_id = warp / wk, wk_id = warp - wr_id * wk;
    const int tile = blockIdx.x * wr + wr_id;
    const bool valid = tile * 32 < H;
    const uint8_t* wt = (shared ? p.sh_a : p.w_a + (size_t)expert * p.stride_a) + (size_t)tile * Tiled<TYPE>::tile_bytes(ncols);
    tile_partials_m<TYPE, false>(wt, nullptr, valid, wk_id, wk, wr_id, wr, lane, ncols, m, aq, ad, red);
    __syncthreads();

    const int rows_here = min(width, H - r0);
    for (int e = tid; e < m * width; e += kThreadsT) {
        const int i = e / width, c = e - i * width;
        if (c < rows_here) p.pair_out[(size_t)s_out_row[i] * H + r0 + c] = sum_slices(red, 0, wk, i, width, c);
    }

    // ---- combine: whoever completes a token's contributions for this row tile adds them up ----
    __threadfence();
    __syncthreads();
    const int expected = p.top_k + (p.nrows_shared > 0 ? 1 : 0);
    if (tid < m) {
        int* ctr = p.combine_ctr + (size_t)s_tok[tid] * p.n_row_tiles + blockIdx.x;
        const int c = atomicAdd(ctr, 1);
        s_done[tid] = (c == expected - 1);
        if (c == expected - 1) *ctr = 0;
    }
    __syncthreads();
    __threadfence();
    const int k = p.top_k;
    for (int i = 0; i < m; ++i) {
        if (!s_done[i]) continue;
        const int t = s_tok[i];
        for (int r = tid; r < rows_here; r += kThreadsT) {
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
static int ngroups_of(int type, int ncols) {
    const int nb = ncols / 32;
    const int gu = (type == CHIMERE_TYPE_Q8_0) ? 4 : 8;
    return (nb + gu - 1) / gu;
}

TiledGeomHost tiled_gate_up_geom(int type_routed, int type_shared, int H, bool has_shared) {
    int g = ngroups_of(type_routed, H);
    if (has_shared) g = min(g, ngroups_of(type_shared, H));
    const TiledGeom t = tiled_geom(g);
    return TiledGeomHost{t.wk, t.wr};
}
TiledGeomHost tiled_down_geom(int type_routed, int F, int type_shared, int F_s) {
    int g = ngroups_of(type_routed, F);
    if (F_s > 0) g = min(g, ngroups_of(type_shared, F_s));
    const TiledGeom t = tiled_geom(g);
    return TiledGeomHost{t.wk, t.wr};
}

template <int TYPE, bool DUAL>
static cudaError_t launch_gate_up_tiled_t(const GemvParams& p, int max_entries, int wk, int wr, cudaStream_t stream) {
    const size_t smem = tiled_smem(p.H, wr, wk, DUAL).total;
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(gate_up_tiled_kernel<TYPE, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    const int tiles = (max(p.nrows_routed, p.nrows_shared) + 32 * wr - 1) / (32 * wr);
    gate_up_tiled_kernel<TYPE, DUAL><<<dim3(tiles, max_entries), kThreadsT, smem, stream>>>(p, wk, wr);
    return cudaGetLastError();
}

static cudaError_t dispatch_gate_up_tiled(int type, const GemvParams& p, int max_entries, int wk, int wr, cudaStream_t stream) {
    const bool dual = p.act == CHIMERE_ACT_SWIGLU;
    switch (type) {
        case CHIMERE_TYPE_Q4_0: return dual ? launch_gate_up_tiled_t<CHIMERE_TYPE_Q4_0, true>(p, max_entries, wk, wr, stream)
                                            : launch_gate_up_tiled_t<CHIMERE_TYPE_Q4_0, false>(p, max_entries, wk, wr, stream);
        case CHIMERE_TYPE_Q8_0: return dual ? launch_gate_up_tiled_t<CHIMERE_TYPE_Q8_0, true>(p, max_entries, wk, wr, stream)
                                            : launch_gate_up_tiled_t<CHIMERE_TYPE_Q8_0, false>(p, max_entries, wk, wr, stream);
        case CHIMERE_TYPE_IQ3_S: return dual ? launch_gate_up_tiled_t<CHIMERE_TYPE_IQ3_S, true>(p, max_entries, wk, wr, stream)
                                             : launch_gate_up_tiled_t<CHIMERE_TYPE_IQ3_S, false>(p, max_entries, wk, wr, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gate_up_tiled(const GemvParams& p, int max_entries, cudaStream_t stream) {
    const TiledGeomHost g = tiled_gate_up_geom(p.type_routed, p.type_shared, p.H, p.nrows_shared > 0);
    cudaError_t e = dispatch_gate_up_tiled(p.type_routed, p, max_entries, g.wk, g.wr, stream);
    if (e == cudaSuccess && p.nrows_shared > 0 && p.type_shared != p.type_routed)
        e = dispatch_gate_up_tiled(p.type_shared, p, max_entries, g.wk, g.wr, stream);
    return e;
}

template <int TYPE>
static cudaError_t launch_down_tiled_t(const GemvParams& p, int max_entries, int wk, int wr, cudaStream_t stream) {
    const size_t smem = tiled_smem(max(p.ncols_routed, p.ncols_shared), wr, wk, false).total;
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(down_tiled_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    down_tiled_kernel<TYPE><<<dim3(p.n_row_tiles, max_entries), kThreadsT, smem, stream>>>(p, wk, wr);
    return cudaGetLastError();
}

static cudaError_t dispatch_down_tiled(int type, const GemvParams& p, int max_entries, int wk, int wr, cudaStream_t stream) {
    switch (type) {
        case CHIMERE_TYPE_Q4_0: return launch_down_tiled_t<CHIMERE_TYPE_Q4_0>(p, max_entries, wk, wr, stream);
        case CHIMERE_TYPE_Q8_0: return launch_down_tiled_t<CHIMERE_TYPE_Q8_0>(p, max_entries, wk, wr, stream);
        case CHIMERE_TYPE_IQ3_S: return launch_down_tiled_t<CHIMERE_TYPE_IQ3_S>(p, max_entries, wk, wr, stream);
        default: return cudaErrorInvalidValue;
    }
}

// p.n_row_tiles must be ceil(H / (32 * wr)) with the geometry of tiled_down_geom
cudaError_t launch_down_tiled(const GemvParams& p, int max_entries, cudaStream_t stream) {
    const TiledGeomHost g = tiled_down_geom(p.type_routed, p.ncols_routed, p.type_shared, p.nrows_shared > 0 ? p.ncols_shared : 0);
    cudaError_t e = dispatch_down_tiled(p.type_routed, p, max_entries, g.wk, g.wr, stream);
    if (e == cudaSuccess && p.nrows_shared > 0 && p.type_shared != p.type_routed)
        e = dispatch_down_tiled(p.type_shared, p, max_entries, g.wk, g.wr, stream);
    return e;
}

}  // namespace chimere
