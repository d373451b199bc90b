// router.cu -- routing front end of the MoE layer, one launch for T tokens:
//   router logits (+ shared-expert gate logit), softmax / sigmoid top-k, Q8_1 of the input rows,
//   dispatch permutation and the work list of the grouped GEMV kernels.
//
// Arithmetic order is the reference's, so that logits, probabilities, indices and weights are
// bit-identical to its kernels on the same GPU:
//   f32_gemv_kernel      chimere-server/kernels/chimere_kernels.cu:706-741
//   dot_product_kernel   chimere-server/src/scratch_pool.rs:243-261
//   topk_softmax         chimere-server/kernels/chimere_kernels.cu:1150-1223
//   ggml_quantize_q8_1   chimere-server/kernels/chimere_kernels.cu:1495-1523
#include "common.cuh"
#include "kernels.h"

namespace chimere {

// Sum of 256 partials held in shared memory in the order of a binary tree with strides
// 128, 64, ..., 1 (element i+stride added into element i), done by one warp.
__device__ __forceinline__ float tree256(const float* r, int lane) {
    float a0 = r[lane] + r[lane + 128];
    float a1 = r[lane + 32] + r[lane + 160];
    float a2 = r[lane + 64] + r[lane + 192];
    float a3 = r[lane + 96] + r[lane + 224];
    float b0 = a0 + a2;
    float b1 = a1 + a3;
    float v = b0 + b1;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_down_sync(0xffffffffu, v, s);
    return v;  // valid in lane 0
}

// Q8_1 of one 32-float block by one warp; lane = element.
__device__ __forceinline__ void quantize_block_q8_1(float xi, uint8_t* out, int lane, int8_t* plane_q, float* plane_d) {
    float amax = fabsf(xi), sum = xi;
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        sum += __shfl_xor_sync(0xffffffffu, sum, m);
    }
    const float d = amax / 127.0f;
    const int8_t q = (amax == 0.0f) ? (int8_t)0 : (int8_t)roundf(xi / d);
    reinterpret_cast<int8_t*>(out)[4 + lane] = q;
    const __half dh = __float2half(d);
    if (lane == 0) *reinterpret_cast<__half2*>(out) = __halves2half2(dh, __float2half(sum));
    // the same block as planes (what the tiled GEMV kernels stream)
    plane_q[lane] = q;
    if (lane == 0) *plane_d = __half2float(dh);
}

// One token's scores -> top-k, by one warp.  Lane l owns experts l, l+32, ...
__device__ void topk_warp(const RouteParams& p, const float* logit_row, int t, int lane, float* tree_scratch, int* ids_out) {
    const int E = p.E, k = p.top_k;
    float v[8], pr[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        v[i] = (e < E) ? __ldcg(logit_row + e) : -1.0e30f;
    }
    if (p.route_mode == CHIMERE_ROUTE_SOFTMAX_RENORM) {
        float mx = v[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) mx = fmaxf(mx, v[i]);
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
        float ev[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane + 32 * i;
            ev[i] = (e < E) ? expf(v[i] - mx) : 0.0f;
            tree_scratch[e] = ev[i];
        }
        __syncwarp();
        float sum = tree256(tree_scratch, lane);
        sum = __shfl_sync(0xffffffffu, sum, 0);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) pr[i] = (sum > 0.0f) ? (ev[i] / sum) : (1.0f / (float)E);
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) pr[i] = 1.0f / (1.0f + expf(-v[i]));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (lane + 32 * i >= E) pr[i] = -2.0f;  // never selected

    // Selection on integer keys: probabilities are >= 0, so their bit patterns order like the values; key 0 = not
    // available (beyond E, or already taken).  One warp-wide max and one warp-wide min per slot (redux.sync) instead
    // of a shuffle butterfly: the largest value wins, equal values go to the lowest index, like a strict-greater
    // scan from index 0.
    uint32_t key[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) key[i] = (lane + 32 * i < E) ? __float_as_uint(pr[i]) + 1u : 0u;
    float wsum = 0.0f;
    float wsel = 0.0f;  // lane j keeps the weight of slot j
    int isel = 0;
    for (int j = 0; j < k; ++j) {
        uint32_t lm = key[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) lm = max(lm, key[i]);
        const uint32_t m = __reduce_max_sync(0xffffffffu, lm);
        uint32_t cand = 0xffffffffu;   // lowest index in this lane that holds the maximum
#pragma unroll
        for (int i = 7; i >= 0; --i)
            if (key[i] == m) cand = (uint32_t)(lane + 32 * i);
        const int bi = (int)__reduce_min_sync(0xffffffffu, cand);
        const float bv = __uint_as_float(m - 1u);
        wsum += bv;
        if (lane == j) { wsel = bv; isel = bi; }
        if ((bi & 31) == lane) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i == (bi >> 5)) key[i] = 0u;
        }
    }
    if (lane < k) {
        float w = wsel;
        if (wsum > 0.0f) {
            const float inv = 1.0f / wsum;
            w = w * inv;
        }
        if (p.route_mode != CHIMERE_ROUTE_SOFTMAX_RENORM || p.route_scale != 1.0f) w = w * p.route_scale;
        p.topk_idx[(size_t)t * k + lane] = isel;
        p.topk_w[(size_t)t * k + lane] = w;
        if (ids_out) ids_out[lane] = isel;
    }
}

// Stable counting sort of the T*k pairs by expert, plus the GEMV work list.  One CTA of 256.
// s_ids: the T*k expert ids in shared memory if the caller has them there (else they are read from p.topk_idx).
// Each warp takes one contiguous eighth of the pairs: it counts its pairs per expert, the counts are turned into
// every warp's first position within every expert, and the warp places its pairs in order; so the only CTA
// barriers are between those steps, however many pairs there are.  The work entries are then filled by all
// threads (entry -> expert by bisection of the entry offsets).
constexpr int kDispatchSmemInts = 256 + 256 + 2048 + 32 + 288 + 1024;
// The dispatch step is written for 256 threads; in a larger CTA only the first 256 threads call it, so its meeting
// point is a named barrier of those threads (in a CTA of 256 it is the same as a CTA-wide barrier).
__device__ __forceinline__ void dispatch_sync() { asm volatile("bar.sync 2, 256;" ::: "memory"); }
// ids_room: ints of shared memory behind the kDispatchSmemInts of scratch; if the ids fit there they are fetched
// once, all loads in flight together, instead of one dependent load per step of the two passes.
// The same result for at most 32 pairs whose ids are in shared memory (a decode batch of up to four tokens): every thread counts directly --
// pair q its position (ids below its own, equal ids before it), thread e the offset of expert e -- and the work entries
// come from the sorted ids by two ballots.  Two barriers instead of six and no scratch to clear: a third of the time.
constexpr int kSmallDispatchPairs = 32;   // (at 64 pairs the direct counting is no faster than the general form)
__device__ void build_dispatch_small(const RouteParams& p, int* smem_i, const int* s_ids) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int E = p.E, P = p.T * p.top_k;
    int* s_sid = smem_i;          // [64] expert ids in sorted order (room for two warps of positions)
    int* s_perm = smem_i + 64;    // [64] the permutation
    int* s_lead = smem_i + 128;   // [2] distinct experts among sorted positions 0..31 / 32..63
    const int my_e = tid < P ? s_ids[tid] : -1;
    const bool valid = my_e >= 0 && my_e < E;
    int below_tid = 0, below_mine = 0, before_me = 0, total = 0;
    for (int q = 0; q < P; ++q) {
        const int e = s_ids[q];                      // (the same address in every thread: a broadcast)
        const bool v = e >= 0 && e < E;
        total += v;
        below_tid += v && e < tid;
        below_mine += v && e < my_e;
        before_me += q < tid && e == my_e;
    }
    if (tid < E) p.offsets[tid] = below_tid;
    if (tid == 0) p.offsets[E] = total;
    if (valid) {
        const int pos = below_mine + before_me;
        p.perm[pos] = tid;
        s_perm[pos] = tid;
        s_sid[pos] = my_e;
    }
    // shared-expert entries first (all tokens, identity order), as in the general form
    const int sgt = shared_group_tokens(p.T);
    const int nsh = p.has_shared ? (p.T + sgt - 1) / sgt : 0;
    const int nsh_listed = p.list_mode == 2 ? 0 : nsh;
    for (int i = tid; i < nsh_listed; i += 256) {
        int* ent = p.group_list + kListHeader + kListEntry * i;
        const int t0 = i * sgt, mm = min(sgt, p.T - t0);
        ent[0] = -1; ent[1] = t0; ent[2] = mm; ent[3] = 0;
        for (int j = 0; j < kMaxGroupTokens; ++j) ent[4 + j] = j < mm ? p.T * p.top_k + t0 + j : 0;
    }
    dispatch_sync();
    // sorted position tid starts a new expert?  (warps 0 and 1 hold the 64 positions)
    unsigned lead = 0u;
    if (warp < 2) {
        const bool first = tid < total && (tid == 0 || s_sid[tid] != s_sid[tid - 1]);
        lead = __ballot_sync(0xffffffffu, first);
        if (lane == 0) s_lead[warp] = __popc(lead);
    }
    dispatch_sync();
    const int total_routed = p.list_mode != 0 ? 0 : s_lead[0] + s_lead[1];
    if (tid == 0) {
        p.group_list[0] = total_routed + nsh_listed;
        p.group_list[1] = total_routed;
        p.group_list[2] = nsh_listed;
        p.group_list[3] = 0;
    }
    if (warp < 2 && total_routed > 0 && ((lead >> lane) & 1u)) {
        const int idx = __popc(lead & ((1u << lane) - 1u)) + (warp == 1 ? s_lead[0] : 0);
        const int e = s_sid[tid];
        int mm = 1;
        while (mm < kMaxGroupTokens && tid + mm < total && s_sid[tid + mm] == e) ++mm;   // (an expert has at most T <= 8 pairs here)
        int* ent = p.group_list + kListHeader + kListEntry * (nsh + idx);
        ent[0] = e; ent[1] = tid; ent[2] = mm; ent[3] = 0;
        for (int j = 0; j < kMaxGroupTokens; ++j) ent[4 + j] = j < mm ? s_perm[tid + j] : 0;
    }
}

__device__ void build_dispatch(const RouteParams& p, int* smem_i, const int* s_ids, int ids_room) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int E = p.E, P = p.T * p.top_k;
    if (s_ids && P <= kSmallDispatchPairs && p.T <= kMaxGroupTokens) { build_dispatch_small(p, smem_i, s_ids); return; }
    if (!s_ids && P <= ids_room) {
        int* stage = smem_i + kDispatchSmemInts;
        const int istr0 = p.idx_stride > 1 ? p.idx_stride : 1;
        for (int q = tid; q < P; q += 256) stage[q] = __ldcg(p.topk_idx + (size_t)q * istr0);
        s_ids = stage;   // visible after the barrier below
    }
    int* hist = smem_i;               // [256] pairs per expert
    int* cursor = smem_i + 256;       // [256] first position of each expert
    int* warp_cnt = smem_i + 512;     // [8][256] per warp: pairs of each expert, then the warp's next position within it
    int* scan = smem_i + 2560;        // [32]
    int* ent_base = smem_i + 2592;    // [257] first routed entry of each expert, [256] = their number
    int* s_perm = smem_i + 2880;      // [1024] copy of the permutation when it is that short
    const bool perm_in_smem = P <= 1024;
    for (int i = tid; i < 2048; i += 256) warp_cnt[i] = 0;
    dispatch_sync();
    // ids outside [0, E) mark pairs that are not there (padding of a fixed-size exchange): they get no work
    const int istr = p.idx_stride > 1 ? p.idx_stride : 1;
    const int chunk = (((P + 7) >> 3) + 31) & ~31;
    const int q0 = min(P, warp * chunk), q1 = min(P, q0 + chunk);
    for (int base = q0; base < q1; base += 32) {
        const int q = base + lane;
        int e = q < q1 ? (s_ids ? s_ids[q] : __ldcg(p.topk_idx + (size_t)q * istr)) : -1;
        const bool valid = e >= 0 && e < E;
        if (!valid) e = 0x40000000 + lane;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (valid && (same & ((1u << lane) - 1u)) == 0u) warp_cnt[warp * 256 + e] += __popc(same);
        __syncwarp();
    }
    dispatch_sync();
    // thread = expert: its pair count, and where each warp's pairs start within it
    int cnt = 0;
    if (tid < E) {
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const int t = warp_cnt[w * 256 + tid];
            warp_cnt[w * 256 + tid] = cnt;
            cnt += t;
        }
    }
    hist[tid] = cnt;
    // exclusive scans over the experts: pair offsets and work-entry offsets
    const int nent = (cnt + kMaxGroupTokens - 1) / kMaxGroupTokens;
    int incl_c = cnt, incl_n = nent;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, incl_c, s), b = __shfl_up_sync(0xffffffffu, incl_n, s);
        if (lane >= s) { incl_c += a; incl_n += b; }
    }
    if (lane == 31) { scan[warp] = incl_c; scan[8 + warp] = incl_n; }
    dispatch_sync();
    int base_c = 0, base_n = 0;
    for (int w = 0; w < warp; ++w) { base_c += scan[w]; base_n += scan[8 + w]; }
    const int off = base_c + incl_c - cnt;      // exclusive
    const int ent0 = base_n + incl_n - nent;
    cursor[tid] = off;
    ent_base[tid] = ent0;
    if (tid < E) p.offsets[tid] = off;
    if (tid == 255) {
        p.offsets[E] = base_c + incl_c;  // tid 255 holds the inclusive total (cnt = 0 beyond E)
        ent_base[256] = base_n + incl_n;
    }
    int total_routed = 0;
    for (int w = 0; w < 8; ++w) total_routed += scan[8 + w];
    // shared-expert entries first (all tokens, identity order), then the routed ones
    const int sgt = shared_group_tokens(p.T);
    const int nsh = p.has_shared ? (p.T + sgt - 1) / sgt : 0;
    if (p.list_mode != 0) total_routed = 0;
    for (int i = tid; i < (p.list_mode == 2 ? 0 : nsh); i += 256) {
        int* ent = p.group_list + kListHeader + kListEntry * i;
        const int t0 = i * sgt, mm = min(sgt, p.T - t0);
        ent[0] = -1; ent[1] = t0; ent[2] = mm; ent[3] = 0;
        for (int j = 0; j < kMaxGroupTokens; ++j) ent[4 + j] = j < mm ? p.T * p.top_k + t0 + j : 0;
    }
    if (tid == 0) {
        const int nsh_listed = p.list_mode == 2 ? 0 : nsh;
        p.group_list[0] = total_routed + nsh_listed;
        p.group_list[1] = total_routed;
        p.group_list[2] = nsh_listed;
        p.group_list[3] = 0;
    }
    dispatch_sync();   // cursor and the warps' first positions are in place
    // stable placement: each warp walks its pairs in order
    for (int base = q0; base < q1; base += 32) {
        const int q = base + lane;
        int e = q < q1 ? (s_ids ? s_ids[q] : __ldcg(p.topk_idx + (size_t)q * istr)) : -1;
        const bool valid = e >= 0 && e < E;
        if (!valid) e = 0x40000000 + lane;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(same & ((1u << lane) - 1u));
        if (valid) {
            const int pos = cursor[e] + warp_cnt[warp * 256 + e] + rank;
            p.perm[pos] = q;
            if (perm_in_smem) s_perm[pos] = q;
        }
        __syncwarp();
        if (valid && rank == 0) warp_cnt[warp * 256 + e] += __popc(same);
        __syncwarp();
    }
    dispatch_sync();
    // the routed entries with their pair rows (perm was written by this CTA: visible after the barrier above)
    for (int idx = tid; idx < total_routed; idx += 256) {
        int lo = 0, hi = 256;   // ent_base[lo] <= idx < ent_base[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (ent_base[mid] <= idx) lo = mid; else hi = mid;
        }
        const int e = lo, i = idx - ent_base[e], c = hist[e], o = cursor[e];
        const int mm = min(kMaxGroupTokens, c - i * kMaxGroupTokens);
        int* ent = p.group_list + kListHeader + kListEntry * (nsh + idx);
        ent[0] = e;
        ent[1] = o + i * kMaxGroupTokens;
        ent[2] = mm;
        ent[3] = 0;
        for (int j = 0; j < kMaxGroupTokens; ++j)
            ent[4 + j] = j < mm ? (perm_in_smem ? s_perm[o + i * kMaxGroupTokens + j] : p.perm[o + i * kMaxGroupTokens + j]) : 0;
    }
}

// grid = (row tiles, token tiles), 256 threads.  Thread p owns partial sum p of every output of
// the tile: elements p, p+256, ... in ascending order, one fused multiply-add each.
template <int TT, int TE>
__global__ void __launch_bounds__(256) route_kernel(const RouteParams p) {
    extern __shared__ __align__(16) float smem_f[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H = p.H, E = p.E;
    const int nrows = E + (p.shexp_gate_w ? 1 : 0);
    const int t0 = blockIdx.y * TT, r0 = blockIdx.x * TE;
    const int n_rtiles = gridDim.x;

    // ---- partial dot products; the router rows come from DRAM, so their loads go out first and the Q8_1 of
    //      this token tile's input rows (blocks dealt round-robin to the row tiles) runs while they are in flight ----
    float acc[TT][TE];
#pragma unroll
    for (int a = 0; a < TT; ++a)
#pragma unroll
        for (int b = 0; b < TE; ++b) acc[a][b] = 0.0f;
    const float* wrow[TE];
#pragma unroll
    for (int b = 0; b < TE; ++b) {
        const int r = r0 + b;
        wrow[b] = (r < E) ? p.router_w + (size_t)r * H : ((r == E && r < nrows) ? p.shexp_gate_w : nullptr);
    }
    constexpr int kStep = (TE <= 2) ? 8 : 2;   // elements per thread whose loads are in flight together
    for (int j0 = 0; j0 < H; j0 += kStep * 256) {
        float wv[kStep][TE];
#pragma unroll
        for (int i = 0; i < kStep; ++i) {
            const int j = j0 + i * 256 + tid;
#pragma unroll
            for (int b = 0; b < TE; ++b) wv[i][b] = (j < H && wrow[b]) ? __ldg(wrow[b] + j) : 0.0f;
        }
        if (j0 == 0) {
            // The router rows are constants of the layer: their loads were issued above, possibly while the previous
            // kernel of the stream was still running (programmatic launch).  Everything that kernel may have written
            // (the input rows) or may still be reading (the workspace) is touched only after this wait.
            griddep_wait();
            if (tid == 0) griddep_launch();   // the grouped GEMV that follows may bring its CTAs in; it waits for this grid itself
            const int nbH = H >> 5;
            const int nt = min(TT, p.T - t0);
            for (int q = blockIdx.x * 8 + warp; q < nt * nbH; q += n_rtiles * 8) {
                const int tt = q / nbH, b = q - tt * nbH;
                const float xi = p.x[(size_t)(t0 + tt) * H + b * 32 + lane];
                quantize_block_q8_1(xi, p.x_q8 + ((size_t)(t0 + tt) * nbH + b) * kQ81Bytes, lane,
                                    p.x_soa_q + (size_t)(t0 + tt) * H + b * 32, p.x_soa_d + (size_t)(t0 + tt) * p.x_soa_d_stride + b);
            }
        }
        float xv[kStep][TT];
#pragma unroll
        for (int i = 0; i < kStep; ++i) {
            const int j = j0 + i * 256 + tid;
#pragma unroll
            for (int a = 0; a < TT; ++a) xv[i][a] = (j < H && t0 + a < p.T) ? p.x[(size_t)(t0 + a) * H + j] : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < kStep; ++i) {   // ascending j, one fused multiply-add each
            if (j0 + i * 256 + tid < H) {
#pragma unroll
                for (int a = 0; a < TT; ++a)
#pragma unroll
                    for (int b = 0; b < TE; ++b) acc[a][b] = fmaf(wv[i][b], xv[i][a], acc[a][b]);
            }
        }
    }
    float* red = smem_f;  // [TT*TE][256]
#pragma unroll
    for (int a = 0; a < TT; ++a)
#pragma unroll
        for (int b = 0; b < TE; ++b) red[(a * TE + b) * 256 + tid] = acc[a][b];
    __syncthreads();
    for (int o = warp; o < TT * TE; o += 8) {
        const float v = tree256(red + o * 256, lane);
        const int a = o / TE, b = o - a * TE;
        const int t = t0 + a, r = r0 + b;
        if (lane == 0 && t < p.T && r < nrows) {
            if (r < E) p.router_logits[(size_t)t * E + r] = p.router_bias ? v + p.router_bias[r] : v;
            else p.sh_gate_logit[t] = v;
        }
    }

    // ---- last CTA of the token tile: scores and top-k ----
    __shared__ int s_flag;
    __shared__ int s_ids[TT * kMaxTopK];
    __syncthreads();   // every thread's writes are ordered before thread 0's counter increment, which releases them
    if (tid == 0) s_flag = (atom_add_acq_rel_gpu(&p.counters[kCtrRouteTile + blockIdx.y], 1) == n_rtiles - 1);   // ... and acquires the other CTAs'
    __syncthreads();
    if (!s_flag) return;
    if (tid == 0) p.counters[kCtrRouteTile + blockIdx.y] = 0;
    for (int a = warp; a < TT; a += 8) {
        const int t = t0 + a;
        if (t < p.T) topk_warp(p, p.router_logits + (size_t)t * E, t, lane, red + warp * 256, s_ids + a * p.top_k);
    }

    // ---- last token tile overall: dispatch permutation and work list ----
    if (gridDim.y == 1) {
        // the only token tile: its ids are all in shared memory
        __syncthreads();
        build_dispatch(p, reinterpret_cast<int*>(smem_f), s_ids, 0);
        return;
    }
    __syncthreads();   // every thread's writes are ordered before thread 0's counter increment, which releases them
    if (tid == 0) s_flag = (atom_add_acq_rel_gpu(&p.counters[kCtrRouteAll], 1) == (int)gridDim.y - 1);   // ... and acquires the other CTAs'
    __syncthreads();
    if (!s_flag) return;
    if (tid == 0) p.counters[kCtrRouteAll] = 0;
    build_dispatch(p, reinterpret_cast<int*>(smem_f), nullptr, (int)(TT * TE * 256) - kDispatchSmemInts);
}

// Larger batches.  The order of the additions is fixed (256 partial sums per output, tree of strides 128 .. 1), so
// a thread can only ever own one partial of an output, and the operands of an output tile have to pass through the
// SM once per tile: the kernel is bound by how many outputs a CTA can hold per router row it fetches.
// CTA = kBigGroups token groups of 256 threads.  Thread (g, p) keeps elements p, p+256, ... of eight token rows in
// registers and owns partial p of every output of its group; the router rows come four at a time through a ring of bulk
// copies shared by the CTA's groups.  The 32 x 256 partial sums a group makes per step are left in shared memory and summed
// by the group's eight warps, four outputs each, in the reference's order.  One group per CTA and two CTAs per SM measured
// faster than two groups in one CTA (747 against 834 us at T = 8192, the same at T = 2048): the phases of a step
// (multiply-adds, partial sums to shared memory, tree) use different units, and two independent CTAs overlap them where
// two groups that share their barriers cannot.  A CTA whose row group starts at row 0
// also writes the Q8_1 form of its tokens, from the values it holds anyway.
// grid = (row groups, token tiles of kBigGroups * 8); NC = ceil(H / 256) <= 8 columns per thread; H a multiple of 32.
constexpr int kBigGroups = 1;   // token groups (of 256 threads and kBigTT tokens) per CTA
constexpr int kBigTT = 8, kBigTE = 4, kBigThreads = 256 * kBigGroups, kBigRing = kBigGroups == 1 ? 2 : 4;
constexpr int kBigCtasPerSm = kBigGroups == 1 ? 2 : 1;
constexpr int kBigRedFloats = kBigGroups * kBigTT * kBigTE * 256;        // [group][token][row][256] partial sums of one step
static size_t big_route_smem(int H) { return (size_t)(kBigRedFloats + kBigRing * kBigTE * H) * sizeof(float); }
// The same tree for two outputs whose partials are interleaved (partial i of the pair at r[2 * i], r[2 * i + 1]): one
// 64-bit load serves both, two-wide adds keep each lane's order.  Valid in lane 0.
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) { uint64_t d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ void tree256_pair(const float* r, int lane, float& v0, float& v1) {
    const uint64_t* q = reinterpret_cast<const uint64_t*>(r);
    const uint64_t a0 = add2(q[lane], q[lane + 128]);
    const uint64_t a1 = add2(q[lane + 32], q[lane + 160]);
    const uint64_t a2 = add2(q[lane + 64], q[lane + 192]);
    const uint64_t a3 = add2(q[lane + 96], q[lane + 224]);
    const uint64_t b0 = add2(a0, a2);
    const uint64_t b1 = add2(a1, a3);
    unpack2(add2(b0, b1), v0, v1);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        v0 += __shfl_down_sync(0xffffffffu, v0, s);
        v1 += __shfl_down_sync(0xffffffffu, v1, s);
    }
}

// EXACT: H == NC * 256 (the common case, H = 2048): no bounds tests and constant offsets in the inner loop.
// The partial sums of two neighbouring tokens travel together (two-wide fused multiply-adds, each lane rounded like the
// scalar instruction), so the sums of a step sit in shared memory as [group][token pair][row][partial][2].
template <int NC, bool EXACT>
__global__ void __launch_bounds__(kBigThreads, kBigCtasPerSm) route_big_kernel(const RouteParams p, int rows_per_group, int split_dispatch) {
    extern __shared__ __align__(16) float smem_f[];   // [kBigRedFloats] partial sums, then [kBigRing][kBigTE][H] router rows
    __shared__ __align__(8) uint64_t s_full[kBigRing];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = tid >> 8, pt = tid & 255;
    const int H = EXACT ? NC * 256 : p.H, E = p.E;
    const int nrows = E + (p.shexp_gate_w ? 1 : 0);
    const int t0 = blockIdx.y * (kBigGroups * kBigTT) + g * kBigTT;
    const int r_begin = blockIdx.x * rows_per_group, r_end = min(nrows, r_begin + rows_per_group);
    const int nsteps = (r_end - r_begin + kBigTE - 1) / kBigTE;
    if (tid == 0) griddep_launch();
    float* ring = smem_f + kBigRedFloats;
    auto wrow = [&](int r) -> const float* { return r < E ? p.router_w + (size_t)r * H : p.shexp_gate_w; };
    // thread 0: the rows of step k into ring slot k % kBigRing (rows past r_end are not copied; what the slot holds in
    // their place is multiplied and never stored)
    auto ask = [&](int k) {
        const int r = r_begin + kBigTE * k, slot = k % kBigRing;
        const uint32_t bytes = (uint32_t)H * 4u;
        const int n = min(kBigTE, r_end - r);
        mbar_expect_tx(&s_full[slot], bytes * n);
        for (int b = 0; b < n; ++b) bulk_g2s(ring + ((size_t)slot * kBigTE + b) * H, wrow(r + b), bytes, &s_full[slot]);
    };
    if (tid == 0) {
        for (int i = 0; i < kBigRing; ++i) mbar_init(&s_full[i], 1);
        mbar_fence_init();
        for (int k = 0; k < kBigRing && k < nsteps; ++k) ask(k);
    }
    // what is added to a row's sums before they are stored (a load from global memory at that point would put a trip
    // to L2 behind every output of every step)
    __shared__ float s_bias[kMaxExperts + 1];
    for (int e = tid; e <= kMaxExperts; e += kBigThreads) s_bias[e] = (p.router_bias && e < E) ? p.router_bias[e] : 0.0f;
    uint64_t xv2[kBigTT / 2][NC];   // elements pt + 256 i of tokens (2 a2, 2 a2 + 1)
    {
        const int nbH = H >> 5;
#pragma unroll
        for (int a2 = 0; a2 < kBigTT / 2; ++a2)
#pragma unroll
            for (int i = 0; i < NC; ++i) {
                const int j = i * 256 + pt, ta = t0 + 2 * a2;
                const bool in = EXACT || j < H;
                const float x0 = (in && ta < p.T) ? p.x[(size_t)ta * H + j] : 0.0f;
                const float x1 = (in && ta + 1 < p.T) ? p.x[(size_t)(ta + 1) * H + j] : 0.0f;
                xv2[a2][i] = pack2f(x0, x1);
                if (blockIdx.x == 0) {
                    // Q8_1 of this group's tokens: a warp's 32 threads hold one 32-element block per (token, i)
                    const int b = i * 8 + (pt >> 5);
                    if (b < nbH && ta < p.T)   // (uniform over the warp)
                        quantize_block_q8_1(x0, p.x_q8 + ((size_t)ta * nbH + b) * kQ81Bytes, lane, p.x_soa_q + (size_t)ta * H + b * 32,
                                            p.x_soa_d + (size_t)ta * p.x_soa_d_stride + b);
                    if (b < nbH && ta + 1 < p.T)
                        quantize_block_q8_1(x1, p.x_q8 + ((size_t)(ta + 1) * nbH + b) * kQ81Bytes, lane, p.x_soa_q + (size_t)(ta + 1) * H + b * 32,
                                            p.x_soa_d + (size_t)(ta + 1) * p.x_soa_d_stride + b);
                }
            }
    }
    __syncthreads();   // barriers initialised
    float* red = smem_f + g * (kBigTT * kBigTE * 256) + 2 * pt;   // this thread's pair slot of every (token pair, row)
    for (int k = 0; k < nsteps; ++k) {
        const int r = r_begin + kBigTE * k, slot = k % kBigRing;
        if (!mbar_wait(&s_full[slot], (uint32_t)((k / kBigRing) & 1))) {
            if (p.status && tid == 0) atomicOr(p.status, kStatusWaitTimeout);   // a wait ran out: leave a mark, go on
            mbar_wait(&s_full[slot], (uint32_t)((k / kBigRing) & 1));
        }
        const float* w0 = ring + (size_t)slot * kBigTE * H + pt;
        uint64_t acc2[kBigTT / 2][kBigTE];
#pragma unroll
        for (int a2 = 0; a2 < kBigTT / 2; ++a2)
#pragma unroll
            for (int b = 0; b < kBigTE; ++b) acc2[a2][b] = 0ull;
#pragma unroll
        for (int i = 0; i < NC; ++i) {   // ascending j, one fused multiply-add per output each
            if (EXACT || i * 256 + pt < H) {
#pragma unroll
                for (int b = 0; b < kBigTE; ++b) {
                    const float w = w0[b * H + i * 256];
                    const uint64_t w2 = pack2f(w, w);
#pragma unroll
                    for (int a2 = 0; a2 < kBigTT / 2; ++a2) acc2[a2][b] = fma2(w2, xv2[a2][i], acc2[a2][b]);
                }
            }
        }
        if (k > 0) __syncthreads();   // the sums of the previous step have been read
#pragma unroll
        for (int a2 = 0; a2 < kBigTT / 2; ++a2)
#pragma unroll
            for (int b = 0; b < kBigTE; ++b) *reinterpret_cast<uint64_t*>(red + (a2 * kBigTE + b) * 512) = acc2[a2][b];
        __syncthreads();   // partial sums complete; every thread is done with this ring slot
        if (tid == 0 && k + kBigRing < nsteps) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            ask(k + kBigRing);
        }
        // sixteen warps, two (token pair, row) sums each: warp = (group, token pair, row half)
        {
            const int og = warp >> 3, a2 = (warp >> 1) & 3, bh = warp & 1;
            const float* rb = smem_f + og * (kBigTT * kBigTE * 256) + a2 * (kBigTE * 512);
            const int t = blockIdx.y * (kBigGroups * kBigTT) + og * kBigTT + 2 * a2;
#pragma unroll
            for (int bb = 0; bb < kBigTE / 2; ++bb) {
                const int b = bh * (kBigTE / 2) + bb, rr = r + b;
                float v0, v1;
                tree256_pair(rb + b * 512, lane, v0, v1);
                if (lane == 0 && rr < r_end) {
                    const float bias = s_bias[rr];
                    if (rr < E) {
                        if (t < p.T) p.router_logits[(size_t)t * E + rr] = p.router_bias ? v0 + bias : v0;
                        if (t + 1 < p.T) p.router_logits[(size_t)(t + 1) * E + rr] = p.router_bias ? v1 + bias : v1;
                    } else {
                        if (t < p.T) p.sh_gate_logit[t] = v0;
                        if (t + 1 < p.T) p.sh_gate_logit[t + 1] = v1;
                    }
                }
            }
        }
    }

    // ---- last CTA of the token tile: scores and top-k, one warp per token ----
    __shared__ int s_flag;
    __syncthreads();   // every thread's writes are ordered before thread 0's counter increment, which releases them
    if (tid == 0) s_flag = (atom_add_acq_rel_gpu(&p.counters[kCtrRouteTile + blockIdx.y], 1) == (int)gridDim.x - 1);   // ... and acquires the other CTAs'
    __syncthreads();
    if (!s_flag) return;
    if (tid == 0) p.counters[kCtrRouteTile + blockIdx.y] = 0;
    {
        const int t = blockIdx.y * (kBigGroups * kBigTT) + warp;
        if (t < p.T) topk_warp(p, p.router_logits + (size_t)t * E, t, lane, smem_f + warp * 256, nullptr);
    }
    if (split_dispatch) return;   // three small launches follow and do the dispatch over the whole GPU
    // ---- last token tile overall: dispatch permutation and work list (the first 256 threads) ----
    __syncthreads();   // every thread's writes are ordered before thread 0's counter increment, which releases them
    if (tid == 0) s_flag = (atom_add_acq_rel_gpu(&p.counters[kCtrRouteAll], 1) == (int)gridDim.y - 1);   // ... and acquires the other CTAs'
    __syncthreads();
    if (!s_flag || tid >= 256) return;
    if (tid == 0) p.counters[kCtrRouteAll] = 0;
    build_dispatch(p, reinterpret_cast<int*>(smem_f), nullptr, kBigRedFloats - kDispatchSmemInts);
}

// ---- dispatch of a large batch in three small launches --------------------------------------
// One CTA sorting tens of thousands of pairs is a serial tail of hundreds of microseconds, so large batches split
// the same stable counting sort over the GPU: chunks of 128 consecutive pairs are counted per expert (hist),
// one CTA turns the counts into every chunk's first position within every expert and into the experts' offsets
// (scan), and the chunks place their own pairs (place); whoever finishes last writes the GEMV work list.
// Scratch: hist[chunks][256] + 260 ints behind it, zero before and after (it shares memory with the combine
// counters of the down stage, which need zeros).
constexpr int kDispatchChunk = 128;
__host__ __device__ inline int dispatch_chunks(int P) { return (P + kDispatchChunk - 1) / kDispatchChunk; }
__host__ __device__ inline size_t dispatch_scratch_ints(int P) { return (size_t)dispatch_chunks(P) * 256 + 260; }

__global__ void __launch_bounds__(kDispatchChunk) dispatch_hist_kernel(const RouteParams p, int32_t* hist) {
    __shared__ int s_ids[kDispatchChunk];
    const int tid = threadIdx.x, P = p.T * p.top_k, q = blockIdx.x * kDispatchChunk + tid;
    const int istr = p.idx_stride > 1 ? p.idx_stride : 1;
    int e = q < P ? __ldcg(p.topk_idx + (size_t)q * istr) : -1;
    s_ids[tid] = (e >= 0 && e < p.E) ? e : -1;
    __syncthreads();
    for (int x = tid; x < 256; x += kDispatchChunk) {
        int c = 0;
#pragma unroll 8
        for (int i = 0; i < kDispatchChunk; ++i) c += (s_ids[i] == x);
        hist[(size_t)blockIdx.x * 256 + x] = c;
    }
}

// One CTA of 256: thread = expert.  hist[chunk][e] becomes the number of pairs of expert e in earlier chunks.
__global__ void __launch_bounds__(256) dispatch_scan_kernel(const RouteParams p, int32_t* hist, int nchunks) {
    __shared__ int scan[16];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int run = 0;
    int32_t* col = hist + tid;
    int c = 0;
    for (; c + 8 <= nchunks; c += 8) {   // eight independent loads in flight
        int v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = col[(size_t)(c + i) * 256];
#pragma unroll
        for (int i = 0; i < 8; ++i) { col[(size_t)(c + i) * 256] = run; run += v[i]; }
    }
    for (; c < nchunks; ++c) { const int v = col[(size_t)c * 256]; col[(size_t)c * 256] = run; run += v; }
    const int cnt = tid < p.E ? run : 0;
    const int nent = (cnt + kMaxGroupTokens - 1) / kMaxGroupTokens;
    int incl_c = cnt, incl_n = nent;
#pragma unroll
    for (int sft = 1; sft < 32; sft <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, incl_c, sft), b = __shfl_up_sync(0xffffffffu, incl_n, sft);
        if (lane >= sft) { incl_c += a; incl_n += b; }
    }
    if (lane == 31) { scan[warp] = incl_c; scan[8 + warp] = incl_n; }
    __syncthreads();
    int base_c = 0, base_n = 0;
    for (int w = 0; w < warp; ++w) { base_c += scan[w]; base_n += scan[8 + w]; }
    int32_t* ent_base = hist + (size_t)nchunks * 256;   // [257] first routed entry of each expert, then their number
    if (tid < p.E) p.offsets[tid] = base_c + incl_c - cnt;
    ent_base[tid] = base_n + incl_n - nent;
    if (tid == 255) { p.offsets[p.E] = base_c + incl_c; ent_base[256] = base_n + incl_n; }
}

__global__ void __launch_bounds__(kDispatchChunk) dispatch_place_kernel(const RouteParams p, int32_t* hist, int nchunks) {
    __shared__ int s_ids[kDispatchChunk];
    __shared__ int s_last;
    const int tid = threadIdx.x, P = p.T * p.top_k, q = blockIdx.x * kDispatchChunk + tid;
    const int istr = p.idx_stride > 1 ? p.idx_stride : 1;
    int e = q < P ? __ldcg(p.topk_idx + (size_t)q * istr) : -1;
    if (e < 0 || e >= p.E) e = -1;
    s_ids[tid] = e;
    __syncthreads();
    if (e >= 0) {
        int rank = 0;
        for (int i = 0; i < tid; ++i) rank += (s_ids[i] == e);
        p.perm[__ldcg(p.offsets + e) + __ldcg(hist + (size_t)blockIdx.x * 256 + e) + rank] = q;
    }
    __syncthreads();
    for (int x = tid; x < 256; x += kDispatchChunk) hist[(size_t)blockIdx.x * 256 + x] = 0;   // back to zero for whoever shares this memory
    // ---- the chunk that finishes last writes the work list ----
    int32_t* ent_base = hist + (size_t)nchunks * 256;
    int32_t* done = ent_base + 258;
    __syncthreads();   // every thread's writes are ordered before thread 0's counter increment, which releases them
    if (tid == 0) s_last = (atom_add_acq_rel_gpu(done, 1) == nchunks - 1);   // ... and acquires the other CTAs'
    __syncthreads();
    if (!s_last) return;
    __shared__ int s_ent[257], s_off[257];
    for (int x = tid; x < 257; x += kDispatchChunk) { s_ent[x] = __ldcg(ent_base + x); s_off[x] = x <= p.E ? __ldcg(p.offsets + x) : 0; }
    __syncthreads();
    const int sgt = shared_group_tokens(p.T);
    const int nsh = (p.has_shared && p.list_mode != 2) ? (p.T + sgt - 1) / sgt : 0;
    const int total_routed = p.list_mode == 0 ? s_ent[256] : 0;
    for (int i = tid; i < nsh; i += kDispatchChunk) {
        int* ent = p.group_list + kListHeader + kListEntry * i;
        const int t0 = i * sgt, mm = min(sgt, p.T - t0);
        ent[0] = -1; ent[1] = t0; ent[2] = mm; ent[3] = 0;
        for (int j = 0; j < kMaxGroupTokens; ++j) ent[4 + j] = j < mm ? p.T * p.top_k + t0 + j : 0;
    }
    for (int idx = tid; idx < total_routed; idx += kDispatchChunk) {
        int lo = 0, hi = 256;   // ent_base[lo] <= idx < ent_base[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_ent[mid] <= idx) lo = mid; else hi = mid;
        }
        const int ex = lo, i = idx - s_ent[ex], o = s_off[ex], cnt = s_off[ex + 1] - o;
        const int mm = min(kMaxGroupTokens, cnt - i * kMaxGroupTokens);
        int* ent = p.group_list + kListHeader + kListEntry * (nsh + idx);
        ent[0] = ex; ent[1] = o + i * kMaxGroupTokens; ent[2] = mm; ent[3] = 0;
        for (int j = 0; j < kMaxGroupTokens; ++j) ent[4 + j] = j < mm ? __ldcg(p.perm + o + i * kMaxGroupTokens + j) : 0;
    }
    __syncthreads();
    if (tid == 0) {
        p.group_list[0] = total_routed + nsh; p.group_list[1] = total_routed; p.group_list[2] = nsh; p.group_list[3] = 0;
        *done = 0;
    }
    for (int x = tid; x < 258; x += kDispatchChunk) ent_base[x] = 0;
}

static cudaError_t launch_dispatch_split(const RouteParams& p, cudaStream_t stream) {
    const int nchunks = dispatch_chunks(p.T * p.top_k);
    dispatch_hist_kernel<<<nchunks, kDispatchChunk, 0, stream>>>(p, p.dispatch_scratch);
    dispatch_scan_kernel<<<1, 256, 0, stream>>>(p, p.dispatch_scratch, nchunks);
    dispatch_place_kernel<<<nchunks, kDispatchChunk, 0, stream>>>(p, p.dispatch_scratch, nchunks);
    return cudaGetLastError();
}
// Batches from this many pairs on take the three-launch dispatch (below, the single CTA at the router's end is faster).
constexpr int kSplitDispatchPairs = 4096;
static bool use_split_dispatch(const RouteParams& p) { return p.dispatch_scratch != nullptr && p.T * p.top_k >= kSplitDispatchPairs; }

// ---- counters of the expert-parallel exchange by peer stores (see the kernels further down) ----
__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) { int v; asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void red_release_sys_add(int32_t* p, int v) { asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
// true when *flag reached `expect` within the bound
__device__ __forceinline__ bool wait_flag(const int32_t* flag, int expect) {
    for (int it = 0; it < (1 << 22); ++it) {
        if (ld_acquire_sys(flag) >= expect) return true;
        __nanosleep(40);
    }
    return false;
}

// The dispatch step alone, for callers that bring their own expert ids in p.topk_idx.  An expert-parallel owner rank
// whose rows arrive by peer stores first waits (bounded) for the source ranks' counters and takes them down.
constexpr int kPermuteIdsRoom = 8192;
__global__ void __launch_bounds__(256) permute_kernel(const RouteParams p) {
    extern __shared__ __align__(16) float smem_f[];
    if (p.wait_flags) {
        if ((int)threadIdx.x < p.wait_n) {
            if (!wait_flag(p.wait_flags + threadIdx.x, p.wait_expect) && p.status) atomicOr(p.status, kStatusWaitTimeout);
            p.wait_flags[threadIdx.x] = 0;
        }
        __syncthreads();
    }
    build_dispatch(p, reinterpret_cast<int*>(smem_f), nullptr, kPermuteIdsRoom);
}

// Final step of an expert-parallel layer on the tokens' home rank: routing-weighted sum of the k expert
// rows of every token in slot order (weighted_combine_kernel, chimere_kernels.cu:1551-1565) plus the
// sigmoid-gated shared expert (sigmoid_gate_add_kernel, scratch_pool.rs:266-277).
__global__ void ep_finish_kernel(const float* rows, const int32_t* slot, const float* topk_w, const float* shared_rows,
                                 const float* sh_logit, float* y, int T, int H, int k) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)T * H) return;
    const int t = (int)(idx / H), h = (int)(idx - (int64_t)t * H);
    float sum = 0.0f;
    for (int j = 0; j < k; ++j) {
        const size_t r = slot ? (size_t)slot[t * k + j] : (size_t)t * k + j;   // where pair (t, j) came back
        sum = fmaf(topk_w[(size_t)t * k + j], rows[r * H + h], sum);
    }
    if (shared_rows) {
        const float sh = shared_rows[(size_t)t * H + h];
        if (sh_logit) sum = fmaf(sh, sigmoid_ref(sh_logit[t]), sum);
        else sum = sh + sum;
    }
    y[idx] = sum;
}

// Fixed-size dispatch of an expert-parallel layer.  Slot s = (destination rank d, position i) of the send
// buffer holds the i-th pair (in pair order) whose expert lives on rank d, or id -1 if there are fewer.
// One CTA per slot finds its pair by scanning the T*k ids, copies the pair's Q8_1 planes and local expert
// id, and notes the slot for the way back.  Row: [H int8][d_stride f32][int32 id], row_bytes a multiple of 16.
__global__ void __launch_bounds__(128) ep_pack_kernel(const int32_t* topk_idx, const int8_t* x_q, const float* x_d, int d_stride,
                                                      uint8_t* send, int32_t* slot, int T, int k, int H, int experts_per_rank, int cap,
                                                      int row_bytes) {
    __shared__ int s_pair;
    const int s = blockIdx.x, d = s / cap, i = s - d * cap, P = T * k;
    if (threadIdx.x < 32) {
        // warp 0: the i-th pair with destination d, pairs in ascending order
        int found = -1, seen = 0;
        for (int base = 0; base < P && found < 0; base += 32) {
            const int q = base + threadIdx.x;
            const bool hit = q < P && (__ldcg(topk_idx + q) / experts_per_rank) == d;
            const unsigned m = __ballot_sync(0xffffffffu, hit);
            const int c = __popc(m);
            if (seen + c > i) {
                unsigned mm = m;
                for (int r = 0; r < i - seen; ++r) mm &= mm - 1;   // drop the first i - seen hits
                found = base + __ffs(mm) - 1;
            }
            seen += c;
        }
        if (threadIdx.x == 0) s_pair = found;
    }
    __syncthreads();
    const int pair = s_pair;
    uint8_t* row = send + (size_t)s * row_bytes;
    int32_t* idp = reinterpret_cast<int32_t*>(row + H + 4 * d_stride);
    if (pair < 0) {
        if (threadIdx.x == 0) *idp = -1;
        return;
    }
    const int t = pair / k;
    const uint4* sq = reinterpret_cast<const uint4*>(x_q + (size_t)t * H);
    for (int v = threadIdx.x; v < H / 16; v += blockDim.x) reinterpret_cast<uint4*>(row)[v] = sq[v];
    const float* sd = x_d + (size_t)t * d_stride;
    for (int v = threadIdx.x; v < d_stride; v += blockDim.x) reinterpret_cast<float*>(row + H)[v] = sd[v];
    if (threadIdx.x == 0) {
        *idp = __ldcg(topk_idx + pair) - d * experts_per_rank;
        slot[pair] = s;
    }
}

// ---- expert-parallel exchange by peer stores (decode-size batches) -----------------------------
// Instead of handing the packed rows to a collective, the home rank writes every pair's row straight into its owner's
// receive buffer (peer memory over NVLink, plain stores, no multicast), and the owner writes every (home rank, token)
// partial sum straight into the home rank's buffer.  One counter per (buffer, source rank) says how many of the source's
// CTAs have finished writing their part of this call: every CTA adds one with a system-scope release behind its stores,
// the reader waits (acquire) for the full count and takes the counter down again.  A rank cannot be a call ahead of a peer
// on the same buffers (it needs that peer's answer first), so one counter suffices.
// Every wait is bounded; a wait that runs out raises the status bit and the kernel goes on.
// Row: [H int8][d_stride f32][int32 local expert id | -1][int32 token][f32 routing weight], row_bytes a multiple of 16.
// One CTA per slot s = (destination rank d, position i): the i-th pair (in pair order) whose expert lives on rank d goes
// to row rank * cap + i of rank d's receive buffer; slots without a pair get id -1.
__global__ void __launch_bounds__(128) ep_pack_p2p_kernel(const int32_t* topk_idx, const float* topk_w, const int8_t* x_q, const float* x_d,
                                                          int d_stride, uint8_t* const* peer_recv, int32_t* const* peer_flags,
                                                          int rank, int T, int k, int H, int experts_per_rank, int cap, int row_bytes) {
    __shared__ int s_pair;
    const int s = blockIdx.x, d = s / cap, i = s - d * cap, P = T * k;
    if (threadIdx.x < 32) {
        int found = -1, seen = 0;
        for (int base = 0; base < P && found < 0; base += 32) {
            const int q = base + threadIdx.x;
            const bool hit = q < P && (__ldcg(topk_idx + q) / experts_per_rank) == d;
            const unsigned m = __ballot_sync(0xffffffffu, hit);
            const int c = __popc(m);
            if (seen + c > i) {
                unsigned mm = m;
                for (int r = 0; r < i - seen; ++r) mm &= mm - 1;   // drop the first i - seen hits
                found = base + __ffs(mm) - 1;
            }
            seen += c;
        }
        if (threadIdx.x == 0) s_pair = found;
    }
    __syncthreads();
    const int pair = s_pair;
    uint8_t* row = peer_recv[d] + ((size_t)rank * cap + i) * row_bytes;
    int32_t* tail = reinterpret_cast<int32_t*>(row + H + 4 * d_stride);
    if (pair < 0) {
        if (threadIdx.x == 0) tail[0] = -1;
    } else {
        const int t = pair / k;
        const uint4* sq = reinterpret_cast<const uint4*>(x_q + (size_t)t * H);
        for (int v = threadIdx.x; v < H / 16; v += blockDim.x) reinterpret_cast<uint4*>(row)[v] = sq[v];
        const float* sd = x_d + (size_t)t * d_stride;
        for (int v = threadIdx.x; v < d_stride; v += blockDim.x) reinterpret_cast<float*>(row + H)[v] = sd[v];
        if (threadIdx.x == 0) {
            tail[0] = __ldcg(topk_idx + pair) - d * experts_per_rank;
            tail[1] = t;
            reinterpret_cast<float*>(tail)[2] = __ldcg(topk_w + pair);
        }
    }
    // this CTA's stores, then one more on the destination's counter for this rank (the CTA barrier orders every thread's
    // stores before thread 0's release; releases are cumulative): the reader waits for `cap` of them
    __syncthreads();
    if (threadIdx.x == 0) red_release_sys_add(peer_flags[d] + rank, 1);
}

// Owner side, before its kernels read the received rows: wait for every source rank's counter and take it down.
__global__ void ep_wait_flags_kernel(int32_t* flags, int n, int expect, int32_t* status) {
    const int i = threadIdx.x;
    if (i < n) {
        if (!wait_flag(flags + i, expect) && status) atomicOr(status, kStatusWaitTimeout);
        flags[i] = 0;
    }
}

// Owner side, after the down products: for every (source rank s, token t) the routing-weighted sum of the expert rows of
// that token's pairs on this rank, in slot order, written into rank s's buffer at [this rank][t][H]; then this rank's flag
// there.  grid = (world * T, ceil(H / 256)), 256 threads.
__global__ void __launch_bounds__(256) ep_return_p2p_kernel(const float* pair_rows, const uint8_t* recv, int row_bytes, int tail_off,
                                                            float* const* peer_back, int32_t* const* peer_flags, int rank, int T, int cap,
                                                            int H) {
    __shared__ float s_w[64];
    __shared__ int s_slot[64];
    __shared__ int s_n;
    const int s = blockIdx.x / T, t = blockIdx.x - s * T;
    // the slots of source s that carry a pair of token t (at most top_k <= 8 of them), kept in slot order
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int n = 0;
        for (int base = 0; base < cap; base += 32) {
            const int i = base + lane;
            bool hit = false;
            float wgt = 0.0f;
            if (i < cap) {
                const int32_t* tail = reinterpret_cast<const int32_t*>(recv + ((size_t)s * cap + i) * row_bytes + tail_off);
                hit = __ldcg(tail) >= 0 && __ldcg(tail + 1) == t;
                wgt = __ldcg(reinterpret_cast<const float*>(tail) + 2);
            }
            const unsigned m = __ballot_sync(0xffffffffu, hit);
            const int pos = n + __popc(m & ((1u << lane) - 1u));
            if (hit && pos < 64) { s_slot[pos] = s * cap + i; s_w[pos] = wgt; }
            n += __popc(m);
        }
        if (lane == 0) s_n = min(n, 64);
    }
    __syncthreads();
    const int n = s_n;
    const int h = blockIdx.y * 256 + threadIdx.x;
    if (h < H) {
        float sum = 0.0f;
        for (int j = 0; j < n; ++j) sum = fmaf(s_w[j], __ldcg(pair_rows + (size_t)s_slot[j] * H + h), sum);
        peer_back[s][((size_t)rank * T + t) * H + h] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) red_release_sys_add(peer_flags[s] + rank, 1);   // the home rank waits for T * gridDim.y of these
}

// Home side: y[t] = sum over owner ranks (ascending) of their partial sums + the sigmoid-gated shared expert.  Every CTA
// waits for the owners' flags; the CTA that finishes last takes them down.  ctr: one int of local scratch.
__global__ void __launch_bounds__(256) ep_finish_p2p_kernel(const float* back, int32_t* flags, int world, int expect, const float* shared_rows,
                                                            const float* sh_logit, float* y, int T, int H, int32_t* ctr, int32_t* status) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < world && !wait_flag(flags + threadIdx.x, expect)) s_ok = 0;
    __syncthreads();
    if (!s_ok && threadIdx.x == 0 && status) atomicOr(status, kStatusWaitTimeout);
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < (int64_t)T * H) {
        const int t = (int)(idx / H), h = (int)(idx - (int64_t)t * H);
        float sum = 0.0f;
        for (int o = 0; o < world; ++o) sum += __ldcg(back + ((size_t)o * T + t) * H + h);
        if (shared_rows) {
            const float sh = shared_rows[(size_t)t * H + h];
            if (sh_logit) sum = fmaf(sh, sigmoid_ref(sh_logit[t]), sum);
            else sum = sh + sum;
        }
        y[idx] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ctr, 1) == (int)gridDim.x - 1) {
            *ctr = 0;
            for (int o = 0; o < world; ++o) flags[o] = 0;
        }
    }
}

cudaError_t launch_ep_pack_p2p(const int32_t* topk_idx, const float* topk_w, const int8_t* x_q, const float* x_d, int d_stride,
                               uint8_t* const* peer_recv, int32_t* const* peer_flags, int rank, int T, int k, int H,
                               int experts_per_rank, int world, int cap, int row_bytes, cudaStream_t stream) {
    ep_pack_p2p_kernel<<<world * cap, 128, 0, stream>>>(topk_idx, topk_w, x_q, x_d, d_stride, peer_recv, peer_flags, rank, T, k, H,
                                                        experts_per_rank, cap, row_bytes);
    return cudaGetLastError();
}
cudaError_t launch_ep_wait_flags(int32_t* flags, int n, int expect, int32_t* status, cudaStream_t stream) {
    ep_wait_flags_kernel<<<1, 32, 0, stream>>>(flags, n, expect, status);
    return cudaGetLastError();
}
cudaError_t launch_ep_return_p2p(const float* pair_rows, const uint8_t* recv, int row_bytes, int tail_off, float* const* peer_back,
                                 int32_t* const* peer_flags, int rank, int world, int T, int cap, int H, cudaStream_t stream) {
    ep_return_p2p_kernel<<<dim3(world * T, (H + 255) / 256), 256, 0, stream>>>(pair_rows, recv, row_bytes, tail_off, peer_back, peer_flags, rank,
                                                                              T, cap, H);
    return cudaGetLastError();
}
// the home rank's counters reach T * ceil(H / 256) per owner rank
cudaError_t launch_ep_finish_p2p(const float* back, int32_t* flags, int world, const float* shared_rows, const float* sh_logit, float* y,
                                 int T, int H, int32_t* ctr, int32_t* status, cudaStream_t stream) {
    const int64_t n = (int64_t)T * H;
    if (n <= 0) return cudaSuccess;
    ep_finish_p2p_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(back, flags, world, T * ((H + 255) / 256), shared_rows, sh_logit, y, T, H,
                                                                         ctr, status);
    return cudaGetLastError();
}

static size_t route_smem(int TT, int TE) {
    size_t a = (size_t)TT * TE * 256 * sizeof(float);
    size_t b = kDispatchSmemInts * sizeof(int);
    return a > b ? a : b;
}

cudaError_t launch_permute(const RouteParams& p, cudaStream_t stream) {
    if (use_split_dispatch(p) && !p.wait_flags) return launch_dispatch_split(p, stream);
    permute_kernel<<<1, 256, (kDispatchSmemInts + kPermuteIdsRoom) * sizeof(int), stream>>>(p);
    return cudaGetLastError();
}

// The routing decision of a layer call in the form the drafter tooling stores it: one byte per (token, slot), slots
// in descending-score order (the "ffn_moe_topk-{L}" tensor, I32 [n_expert_used, n_tokens], narrowed to uint8
// [n_tokens][8]; chimere-dflash/extract/target_daemon.cpp:18-23).  `load` (optional) collects how many pairs each expert
// received: the per-expert load metric.
__global__ void routing_trace_kernel(const int32_t* topk_idx, uint8_t* trace, int32_t* load, int n, int E) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = topk_idx[i];
    trace[i] = (uint8_t)e;
    if (load && e >= 0 && e < E) atomicAdd(load + e, 1);
}

cudaError_t launch_routing_trace(const int32_t* topk_idx, uint8_t* trace, int32_t* load, int T, int k, int E, cudaStream_t stream) {
    const int n = T * k;
    if (n <= 0) return cudaSuccess;
    routing_trace_kernel<<<(n + 255) / 256, 256, 0, stream>>>(topk_idx, trace, load, n, E);
    return cudaGetLastError();
}

cudaError_t launch_ep_finish(const float* rows, const int32_t* slot, const float* topk_w, const float* shared_rows, const float* sh_logit,
                             float* y, int T, int H, int k, cudaStream_t stream) {
    const int64_t n = (int64_t)T * H;
    if (n <= 0) return cudaSuccess;
    ep_finish_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(rows, slot, topk_w, shared_rows, sh_logit, y, T, H, k);
    return cudaGetLastError();
}

// Exact-size dispatch (prefill-size batches): the routing kernel's dispatch has already sorted the pairs by expert, and the
// experts of an owner rank are contiguous, so perm[] lists the pairs grouped by destination.  One CTA per sorted position j
// copies pair perm[j]'s row in the same row format as above and notes slot[pair] = j for the way back.
__global__ void __launch_bounds__(128) ep_pack_sorted_kernel(const int32_t* perm, const int32_t* topk_idx, const int8_t* x_q, const float* x_d,
                                                             int d_stride, uint8_t* send, int32_t* slot, int k, int H, int experts_per_rank,
                                                             int row_bytes) {
    const int j = blockIdx.x, pair = __ldcg(perm + j), t = pair / k;
    const int e = __ldcg(topk_idx + pair);
    uint8_t* row = send + (size_t)j * row_bytes;
    const uint4* sq = reinterpret_cast<const uint4*>(x_q + (size_t)t * H);
    for (int v = threadIdx.x; v < H / 16; v += blockDim.x) reinterpret_cast<uint4*>(row)[v] = sq[v];
    const float* sd = x_d + (size_t)t * d_stride;
    for (int v = threadIdx.x; v < d_stride; v += blockDim.x) reinterpret_cast<float*>(row + H)[v] = sd[v];
    if (threadIdx.x == 0) {
        *reinterpret_cast<int32_t*>(row + H + 4 * d_stride) = e % experts_per_rank;
        slot[pair] = j;
    }
}
cudaError_t launch_ep_pack_sorted(const int32_t* perm, const int32_t* topk_idx, const int8_t* x_q, const float* x_d, int d_stride, uint8_t* send,
                                  int32_t* slot, int T, int k, int H, int experts_per_rank, int row_bytes, cudaStream_t stream) {
    if (T * k <= 0) return cudaSuccess;
    ep_pack_sorted_kernel<<<T * k, 128, 0, stream>>>(perm, topk_idx, x_q, x_d, d_stride, send, slot, k, H, experts_per_rank, row_bytes);
    return cudaGetLastError();
}

cudaError_t launch_ep_pack(const int32_t* topk_idx, const int8_t* x_q, const float* x_d, int d_stride, uint8_t* send, int32_t* slot,
                           int T, int k, int H, int experts_per_rank, int world, int cap, int row_bytes, cudaStream_t stream) {
    ep_pack_kernel<<<world * cap, 128, 0, stream>>>(topk_idx, x_q, x_d, d_stride, send, slot, T, k, H, experts_per_rank, cap, row_bytes);
    return cudaGetLastError();
}

cudaError_t launch_route(const RouteParams& p, cudaStream_t stream) {
    const int nrows = p.E + (p.shexp_gate_w ? 1 : 0);
    if (p.T <= 32) {
        constexpr int TT = 8, TE = 2;
        dim3 grid((nrows + TE - 1) / TE, (p.T + TT - 1) / TT);
        return launch_pdl(route_kernel<TT, TE>, grid, 256, route_smem(TT, TE), stream, p);
    } else if (p.H <= 2048 && p.H % 32 == 0) {
        // token tiles of kBigGroups * 8; the router rows are cut into row groups (multiples of four rows) only while there are too few
        // token tiles to fill the GPU, because every row group fetches its tokens again
        const int token_tiles = (p.T + kBigGroups * kBigTT - 1) / (kBigGroups * kBigTT);
        int groups = sm_count() * kBigCtasPerSm / token_tiles;   // (rounded down: a second wave of a few CTAs would double the time)
        const int max_groups = (nrows + kBigTE - 1) / kBigTE;
        groups = groups < 1 ? 1 : (groups > max_groups ? max_groups : groups);
        const int rows_per_group = kBigTE * (((nrows + groups - 1) / groups + kBigTE - 1) / kBigTE);
        const dim3 grid((nrows + rows_per_group - 1) / rows_per_group, token_tiles);
        const size_t smem = big_route_smem(p.H);
        static bool attr_done[64] = {};
        static bool attr_done_x[64] = {};
        const bool split = use_split_dispatch(p);
        if (p.H == 2048) {
            cudaError_t e = max_smem_once(route_big_kernel<8, true>, (int)big_route_smem(2048), attr_done_x);
            if (e != cudaSuccess) return e;
            route_big_kernel<8, true><<<grid, kBigThreads, smem, stream>>>(p, rows_per_group, split ? 1 : 0);
        } else {
            cudaError_t e = max_smem_once(route_big_kernel<8, false>, (int)big_route_smem(2048), attr_done);
            if (e != cudaSuccess) return e;
            route_big_kernel<8, false><<<grid, kBigThreads, smem, stream>>>(p, rows_per_group, split ? 1 : 0);
        }
        if (split) return launch_dispatch_split(p, stream);
    } else {
        constexpr int TT = 8, TE = 8;
        static bool attr_done[64] = {};
        cudaError_t e = max_smem_once(route_kernel<TT, TE>, (int)route_smem(TT, TE), attr_done);
        if (e != cudaSuccess) return e;
        dim3 grid((nrows + TE - 1) / TE, (p.T + TT - 1) / TT);
        route_kernel<TT, TE><<<grid, 256, route_smem(TT, TE), stream>>>(p);
    }
    return cudaGetLastError();
}

}  // namespace chimere

// ------------------------------------------------------------------------------------------
// Routing without any allocation by anyone: chimere_b200_moe_route_noalloc.
//
// Some hosts of this library cannot hand it scratch memory.  A serving process that gave all device
// memory to its own pool at start-up (the reference's server sizes every buffer once, at model
// load), or a caller already inside a region where cudaMalloc is not permitted, has the token rows
// and somewhere to put the routing result, but no spare arena and no way to get one.  For them the
// routing step's scratch lives in the library image itself: one fixed array per GPU, reserved when
// the library is loaded on that GPU and held until the process ends.
//
// In host code the array's name is only a handle, not a device address, so the address is looked
// up once per device with cudaGetSymbolAddress (with that device current) and cached.  The first
// call on a device does this look-up; make that first call outside any stream capture.
// Every call on a device shares the one array: calls that overlap on the GPU (two streams, two
// threads) race.  Nothing here calls cudaMalloc, cudaFree or a library routine that allocates.
namespace chimere {

constexpr int kNoAllocMaxT = 64;        // tokens per call
constexpr int kNoAllocMaxH = 4096;      // hidden size
constexpr size_t kNoAllocCounters = 0;                                                        // 1 KiB of integer scratch
constexpr size_t kNoAllocLogits = 1024;                                                       // [T][256] f32
constexpr size_t kNoAllocShLogit = kNoAllocLogits + (size_t)kNoAllocMaxT * kMaxExperts * 4;   // [T] f32
constexpr size_t kNoAllocXq8 = kNoAllocShLogit + 256;                                         // [T][H/32][36]
constexpr size_t kNoAllocXq = kNoAllocXq8 + (size_t)kNoAllocMaxT * (kNoAllocMaxH / 32) * kQ81Bytes;
constexpr size_t kNoAllocXd = kNoAllocXq + (size_t)kNoAllocMaxT * kNoAllocMaxH;               // [T][H/32] f32
constexpr size_t kNoAllocPerm = kNoAllocXd + (size_t)kNoAllocMaxT * (kNoAllocMaxH / 32) * 4;  // [T*8] i32
constexpr size_t kNoAllocOffsets = kNoAllocPerm + (size_t)kNoAllocMaxT * kMaxTopK * 4;        // [257] i32
constexpr size_t kNoAllocList = kNoAllocOffsets + 1280;                                       // work list
constexpr size_t kNoAllocBytes = kNoAllocList + (size_t)(kListHeader + kListEntry * (kMaxExperts + kNoAllocMaxT * kMaxTopK + kNoAllocMaxT)) * 4 + 256;

static __device__ __align__(256) unsigned char g_route_scratch[kNoAllocBytes];   // ~680 KiB per GPU

}  // namespace chimere

extern "C" int chimere_b200_moe_route_noalloc(const chimere_moe_layer* w, const float* d_x, int T, int32_t* d_topk_idx,
                                              float* d_topk_w, cudaStream_t stream) {
    using namespace chimere;
    if (!w || !d_x || !d_topk_idx || !d_topk_w || !w->router_w) return -1;
    if (w->H <= 0 || w->H % 32 || w->E <= 0 || w->top_k <= 0 || w->top_k > w->E || T <= 0) return -2;
    if (w->route_mode != CHIMERE_ROUTE_SOFTMAX_RENORM && w->route_mode != CHIMERE_ROUTE_SIGMOID_NORM_SCALE) return -2;
    // larger than the built-in scratch was sized for: use chimere_b200_moe_route with a workspace instead
    if (T > kNoAllocMaxT || w->H > kNoAllocMaxH || w->E > kMaxExperts || w->top_k > kMaxTopK) return -7;

    // once per device, with that device current: the array's device address
    static unsigned char* s_base[64] = {nullptr};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return -100 - (int)e;
    if (dev < 0 || dev >= 64) return -2;
    if (!s_base[dev]) {
        // the look-up is not a stream operation and must not happen while `stream` is being captured
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone) return -8;
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_route_scratch);
        if (e != cudaSuccess || !ptr) return -100 - (int)e;
        s_base[dev] = ptr;
    }
    unsigned char* base = s_base[dev];

    // the integer scratch must start at zero; everything else is fully rewritten by the kernel
    e = cudaMemsetAsync(base + kNoAllocCounters, 0, 1024, stream);
    if (e != cudaSuccess) return -100 - (int)e;

    RouteParams p{};
    p.T = T; p.H = w->H; p.E = w->E; p.top_k = w->top_k; p.route_mode = w->route_mode;
    p.has_shared = w->F_s > 0;
    p.route_scale = w->route_scale;
    p.x = d_x; p.router_w = w->router_w; p.router_bias = w->router_bias;
    p.shexp_gate_w = (w->F_s > 0) ? w->shexp_gate_w : nullptr;
    p.counters = (int32_t*)(base + kNoAllocCounters);
    p.router_logits = (float*)(base + kNoAllocLogits);
    p.sh_gate_logit = (float*)(base + kNoAllocShLogit);
    p.x_q8 = base + kNoAllocXq8;
    p.x_soa_q = (int8_t*)(base + kNoAllocXq);
    p.x_soa_d = (float*)(base + kNoAllocXd);
    p.x_soa_d_stride = (w->H / 32 + 3) & ~3;
    p.perm = (int32_t*)(base + kNoAllocPerm);
    p.offsets = (int32_t*)(base + kNoAllocOffsets);
    p.group_list = (int32_t*)(base + kNoAllocList);
    p.topk_idx = d_topk_idx;   // results go straight to the caller's buffers
    p.topk_w = d_topk_w;
    e = launch_route(p, stream);
    return e == cudaSuccess ? 0 : -100 - (int)e;
}
