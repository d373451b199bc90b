// gemv_tiled.cu -- the decode-path GEMV kernels on tiled32 weights (see tiled.cuh).
//
// Persistent CTAs, one per SM: a producer warp walks the CTA's share of the work items and keeps
// a ring of shared-memory stages filled with cp.async.bulk copies (weights come as contiguous
// slabs of the tiled layout, activations as whole Q8_1 rows); eight consumer warps drain it.
// The producer runs ahead across items, so the dependent look-ups that name an item's bytes
// (work list -> permutation -> token row) are off the consumers' critical path and the memory
// system always has a few tens of KB per SM in flight.
//
// Consumer side: one warp = 32 consecutive rows of one expert matrix, lane = row; a lane reads its
// own 16 bytes of every 32-weight unit from the stage (conflict-free 128-bit shared loads), decodes
// in registers and multiplies with the tokens' Q8_1 blocks, read from shared memory as warp-wide
// broadcasts.  The eight warps are WR row tiles x WK slices of K; slices meet in shared memory
// and are added in a fixed order.
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

constexpr int kConsumerWarps = 16;
constexpr int kStreamThreads = 32 * (kConsumerWarps + 1);  // + one producer warp
constexpr int kSlabMax = 36 * 1024 + 1024;                  // bytes of one weight stage
constexpr int kStageGateUp = 0, kStageDown = 1;

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// How an item's weights are cut into slabs (identical on the host, in the producer and in the consumers).
struct SlabPlan {
    int tile_bytes, chunk_bytes, groups_per_chunk, ngroups;
    int whole_tiles;       // 1: a slab is `per` whole tiles; 0: a slab is `per` chunks of the single tile (wr == 1)
    int per, slabs_per_mat;
};
__host__ __device__ inline SlabPlan slab_plan(int tile_bytes, int chunk_bytes, int groups_per_chunk, int nb, int wr) {
    SlabPlan s;
    s.tile_bytes = tile_bytes; s.chunk_bytes = chunk_bytes; s.groups_per_chunk = groups_per_chunk;
    s.ngroups = (nb + kGroupUnits - 1) / kGroupUnits;
    if (tile_bytes <= kSlabMax) {
        s.whole_tiles = 1;
        s.per = kSlabMax / tile_bytes; if (s.per > wr) s.per = wr;
        s.slabs_per_mat = (wr + s.per - 1) / s.per;
    } else {
        s.whole_tiles = 0;
        s.per = kSlabMax / chunk_bytes;
        const int nchunks = (tile_bytes + chunk_bytes - 1) / chunk_bytes;
        s.slabs_per_mat = (nchunks + s.per - 1) / s.per;
    }
    return s;
}

struct StreamSmem { uint32_t bars, meta, red, act, ring, total; int nst; uint32_t act_q_row, act_d_row, act_buf; };
// bars: full[nst] empty[nst] afull[2] aempty[2]; meta: 2 x 64 ints; red; act: 2 buffers of 8 x (int8 row + f32 scale row)
__host__ __device__ inline StreamSmem stream_smem(int ncols_max, int wr, int wk, bool dual) {
    StreamSmem s;
    uint32_t o = 0;
    s.bars = o; o += 256;
    s.meta = o; o += 2 * 64 * 4;
    s.red = o; o += (uint32_t)(dual ? 2 : 1) * wk * kMaxGroupTokens * 32 * wr * 4;
    o = (o + 127u) & ~127u;
    s.act_q_row = (uint32_t)ncols_max;
    s.act_d_row = ((uint32_t)(ncols_max / 32) * 4 + 15u) & ~15u;
    s.act_buf = kMaxGroupTokens * (s.act_q_row + s.act_d_row);
    s.act = o; o += 2u * s.act_buf;
    o = (o + 127u) & ~127u;
    s.ring = o;
    int nst = (int)((220u * 1024u - o) / kSlabMax);
    if (nst > 6) nst = 6;
    s.nst = nst;
    s.total = o + (uint32_t)(nst > 0 ? nst : 0) * kSlabMax;
    return s;
}

// acc[i] += sum over the units of one group of (scale_w * scale_x) * integer block dot, for up to M tokens.
// Activations in shared memory: int8 plane aq[i][qrow], f32 scale plane ad[i][drow / 4].
template <int TYPE, int M>
__device__ __forceinline__ void group_dot(const uint8_t* tile, int grp, int lane, int nu, const uint8_t* aq, int qrow,
                                          const float* ad, int drow_f, int m, float (&acc)[kMaxGroupTokens]) {
    using TT = Tiled<TYPE>;
    typename TT::Regs r;
    TT::load(tile, grp, lane, nu, r);
#pragma unroll
    for (int u = 0; u < kGroupUnits; ++u) {
        if (u < nu) {
            int w[8];
            TT::decode(r, u, w);
            const float dw = TT::dscale(r, u);
            const int b = grp * kGroupUnits + u;
#pragma unroll
            for (int i = 0; i < M; ++i) {
                if (M == 1 || i < m) {
                    const int4* q = reinterpret_cast<const int4*>(aq + (size_t)i * qrow + b * 32);
                    const int4 q0 = q[0], q1 = q[1];
                    int s0 = __dp4a(w[0], q0.x, 0), s1 = __dp4a(w[4], q1.x, 0);   // two independent chains
                    s0 = __dp4a(w[1], q0.y, s0); s1 = __dp4a(w[5], q1.y, s1);
                    s0 = __dp4a(w[2], q0.z, s0); s1 = __dp4a(w[6], q1.z, s1);
                    s0 = __dp4a(w[3], q0.w, s0); s1 = __dp4a(w[7], q1.w, s1);
                    acc[i] = fmaf(dw * ad[i * drow_f + b], (float)TT::finish(s0 + s1, r, u, 0), acc[i]);
                }
            }
        }
    }
}

struct StreamGeom { int wk, wr; };

template <int TYPE, int M>
__device__ __forceinline__ void consume_slab(const uint8_t* stage, const SlabPlan& sp, int si, int wr_id, int wk_id, int wk,
                                             int wr, int lane, int nb, bool row_tile_valid, const uint8_t* aq, int qrow,
                                             const float* ad, int drow_f, int m, float (&acc)[kMaxGroupTokens]) {
    if (!row_tile_valid) return;
    const uint8_t* tile;
    int g0, g1;
    if (sp.whole_tiles) {
        const int t0 = si * sp.per;
        if (wr_id < t0 || wr_id >= t0 + sp.per || wr_id >= wr) return;
        tile = stage + (size_t)(wr_id - t0) * sp.tile_bytes;
        g0 = 0; g1 = sp.ngroups;
    } else {
        if (wr_id != 0) return;
        g0 = si * sp.per * sp.groups_per_chunk; g1 = min(sp.ngroups, g0 + sp.per * sp.groups_per_chunk);
        tile = stage - (size_t)(si * sp.per) * sp.chunk_bytes;
    }
    for (int g = g0 + wk_id; g < g1; g += wk) {
        const int nu = min(kGroupUnits, nb - g * kGroupUnits);
        group_dot<TYPE, M>(tile, g, lane, nu, aq, qrow, ad, drow_f, m, acc);
    }
}

__device__ __forceinline__ float sum_slices(const float* red, int mat, int wk, int i, int width, int col) {
    float v = 0.0f;
    for (int k = 0; k < wk; ++k) v += red[((mat * wk + k) * kMaxGroupTokens + i) * width + col];
    return v;
}

// meta words per item (written by the producer, read by the consumers)
constexpr int kMetaM = 0, kMetaTile0 = 1, kMetaNTilesTotal = 2, kMetaShared = 3, kMetaOutRow = 8, kMetaTok = 16, kMetaValid = 4;

template <int TYPE, int STAGE, bool DUAL>
__global__ void __launch_bounds__(kStreamThreads, 1) stream_kernel(const GemvParams p, int wk, int wr) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // ---- static description of an item ----
    const int ncols_r = p.ncols_routed, ncols_s = p.ncols_shared;
    const int nrows_r = p.nrows_routed, nrows_s = p.nrows_shared;
    const bool do_r = p.type_routed == TYPE, do_s = nrows_s > 0 && p.type_shared == TYPE;
    const int tiles_r = (nrows_r / 32 + wr - 1) / wr, tiles_s = nrows_s > 0 ? (nrows_s / 32 + wr - 1) / wr : 0;  // items per entry
    const StreamSmem ss = stream_smem(max(ncols_r, ncols_s), wr, wk, DUAL);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + ss.bars);
    uint64_t* empty = full + ss.nst;
    uint64_t* afull = empty + ss.nst;
    uint64_t* aempty = afull + 2;
    int* meta = reinterpret_cast<int*>(smem + ss.meta);
    float* red = reinterpret_cast<float*>(smem + ss.red);
    uint8_t* actbuf = smem + ss.act;
    uint8_t* ring = smem + ss.ring;
    const int nst = ss.nst;

    if (tid == 0) {
        for (int i = 0; i < nst; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, kConsumerWarps); }
        for (int i = 0; i < 2; ++i) { mbar_init(afull + i, 1); mbar_init(aempty + i, kConsumerWarps); }
        mbar_fence_init();
    }
    __syncthreads();

    const int n_routed = __ldcg(p.group_list + 1), n_shared = __ldcg(p.group_list + 2);
    const int items_r = do_r ? n_routed * tiles_r : 0, items_s = do_s ? n_shared * tiles_s : 0;
    const int total = items_r + items_s;
    const int n_mats = DUAL ? 2 : 1;
    // Items are handed out through a device-wide queue, the heavy ones (shared expert: every token) first.
    int* queue = p.queue + (STAGE == kStageGateUp ? 0 : 2);   // [0] next item, [1] CTAs finished

    if (warp == kConsumerWarps) {
        // ================================ producer ================================
        if (lane != 0) return;
        int slab_seq = 0;
        for (int n = 0;; ++n) {
            const int it = atomicAdd(queue, 1);
            const int ab = n & 1, aphase = (n >> 1) & 1;
            if (it >= total) {
                // end marker for the consumers, then the last CTA to get here re-arms the queue
                if (!mbar_wait(aempty + ab, aphase ^ 1)) { atomicOr(p.status, kStatusWaitTimeout); return; }
                meta[ab * 64 + kMetaM] = -1;
                mbar_arrive(afull + ab);
                if (atomicAdd(queue + 1, 1) == (int)gridDim.x - 1) { queue[1] = 0; __threadfence(); queue[0] = 0; }
                return;
            }
            const bool shared = it < items_s;
            const int rel = shared ? it : it - items_s;
            const int tiles_e = shared ? tiles_s : tiles_r;
            const int eidx = (shared ? n_routed : 0) + rel / tiles_e, item_tile = rel % tiles_e;
            const int* ent = p.group_list + kListHeader + 4 * eidx;
            const int expert = __ldcg(ent), start = __ldcg(ent + 1), m = __ldcg(ent + 2);
            const int ncols = shared ? ncols_s : ncols_r, nrows = shared ? nrows_s : nrows_r;
            const int tb = (int)Tiled<TYPE>::tile_bytes(ncols);
            const SlabPlan sp = slab_plan(tb, Tiled<TYPE>::kChunkBytes, Tiled<TYPE>::kGroupsPerChunk, ncols / 32, wr);
            const int tiles_total = nrows / 32, tile0 = item_tile * wr;
            const int ntiles_here = min(wr, tiles_total - tile0);
            // activations + meta of this item
            if (!mbar_wait(aempty + ab, aphase ^ 1)) { atomicOr(p.status, kStatusWaitTimeout); return; }
            int* mt = meta + ab * 64;
            mt[kMetaM] = m; mt[kMetaTile0] = tile0; mt[kMetaNTilesTotal] = tiles_total; mt[kMetaShared] = shared ? 1 : 0;
            mt[kMetaValid] = ntiles_here;
            const uint32_t qbytes = (uint32_t)ncols, dbytes = ((uint32_t)(ncols / 32) * 4u + 15u) & ~15u;
            int irow[kMaxGroupTokens];
            for (int i = 0; i < m; ++i) {
                int t, prow;
                if (shared) { t = start + i; prow = p.T * p.top_k + t; }
                else { prow = __ldcg(p.perm + start + i); t = prow / p.top_k; }
                mt[kMetaOutRow + i] = prow; mt[kMetaTok + i] = t;
                irow[i] = (STAGE == kStageGateUp) ? t : prow;
            }
            mbar_expect_tx(afull + ab, (uint32_t)m * (qbytes + dbytes));   // releases the meta words written above
            uint8_t* abuf = actbuf + (size_t)ab * ss.act_buf;
            for (int i = 0; i < m; ++i) {
                bulk_g2s(abuf + (size_t)i * ss.act_q_row, p.in_soa_q + (size_t)irow[i] * p.in_soa_q_stride, qbytes, afull + ab);
                bulk_g2s(abuf + kMaxGroupTokens * ss.act_q_row + (size_t)i * ss.act_d_row,
                         p.in_soa_d + (size_t)irow[i] * p.in_soa_d_stride, dbytes, afull + ab);
            }
            // weight slabs: matrix A (up / down) first, then B (gate)
            for (int mat = 0; mat < n_mats; ++mat) {
                const uint8_t* wbase = (mat == 0) ? (shared ? (STAGE == kStageGateUp ? p.sh_b : p.sh_a)
                                                            : (STAGE == kStageGateUp ? p.w_b + (size_t)expert * p.stride_b
                                                                                     : p.w_a + (size_t)expert * p.stride_a))
                                                  : (shared ? p.sh_a : p.w_a + (size_t)expert * p.stride_a);
                const uint8_t* item_base = wbase + (size_t)tile0 * tb;
                for (int si = 0; si < sp.slabs_per_mat; ++si) {
                    size_t off; uint32_t bytes;
                    if (sp.whole_tiles) {
                        const int t0 = si * sp.per, nt = min(sp.per, ntiles_here - t0);
                        off = (size_t)t0 * tb; bytes = nt > 0 ? (uint32_t)nt * tb : 0u;
                    } else {
                        off = (size_t)(si * sp.per) * sp.chunk_bytes;
                        bytes = (uint32_t)min((int64_t)sp.per * sp.chunk_bytes, (int64_t)tb - (int64_t)off);
                    }
                    const int st = slab_seq % nst, ph = (slab_seq / nst) & 1;
                    if (!mbar_wait(empty + st, ph ^ 1)) { atomicOr(p.status, kStatusWaitTimeout); return; }
                    if (bytes > 0) {
                        mbar_expect_tx(full + st, bytes);
                        bulk_g2s(ring + (size_t)st * kSlabMax, item_base + off, bytes, full + st);
                    } else {
                        mbar_arrive(full + st);
                    }
                    ++slab_seq;
                }
            }
        }
    }

    // ================================ consumers ================================
    const int wr_id = warp / wk, wk_id = warp - wr_id * wk;
    const int width = 32 * wr;
    int slab_seq = 0;
    for (int n = 0;; ++n) {
        const int ab = n & 1, aphase = (n >> 1) & 1;
        if (!mbar_wait(afull + ab, aphase)) { atomicOr(p.status, kStatusWaitTimeout); return; }
        const int* mt = meta + ab * 64;
        const int m = mt[kMetaM], tile0 = mt[kMetaTile0], tiles_total = mt[kMetaNTilesTotal];
        if (m < 0) return;
        const bool shared = mt[kMetaShared] != 0;
        const int ncols = shared ? ncols_s : ncols_r, nb = ncols >> 5;
        const SlabPlan sp = slab_plan((int)Tiled<TYPE>::tile_bytes(ncols), Tiled<TYPE>::kChunkBytes, Tiled<TYPE>::kGroupsPerChunk, nb, wr);
        const uint8_t* aq = actbuf + (size_t)ab * ss.act_buf;
        const float* ad = reinterpret_cast<const float*>(aq + kMaxGroupTokens * ss.act_q_row);
        const int qrow = (int)ss.act_q_row, drow_f = (int)(ss.act_d_row / 4);
        const bool tile_valid = tile0 + wr_id < tiles_total;
        float aa[kMaxGroupTokens], ab_[kMaxGroupTokens];
#pragma unroll
        for (int i = 0; i < kMaxGroupTokens; ++i) { aa[i] = 0.0f; ab_[i] = 0.0f; }
        for (int mat = 0; mat < n_mats; ++mat) {
            for (int si = 0; si < sp.slabs_per_mat; ++si) {
                const int st = slab_seq % nst, ph = (slab_seq / nst) & 1;
                if (!mbar_wait(full + st, ph)) { atomicOr(p.status, kStatusWaitTimeout); return; }
                const uint8_t* stage = ring + (size_t)st * kSlabMax;
#define CHIMERE_CONSUME(MM, ACC) consume_slab<TYPE, MM>(stage, sp, si, wr_id, wk_id, wk, wr, lane, nb, tile_valid, aq, qrow, ad, drow_f, m, ACC)
                if (mat == 0) {
                    if (m == 1) CHIMERE_CONSUME(1, aa); else if (m == 2) CHIMERE_CONSUME(2, aa); else CHIMERE_CONSUME(kMaxGroupTokens, aa);
                } else {
                    if (m == 1) CHIMERE_CONSUME(1, ab_); else if (m == 2) CHIMERE_CONSUME(2, ab_); else CHIMERE_CONSUME(kMaxGroupTokens, ab_);
                }
#undef CHIMERE_CONSUME
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + st);
                ++slab_seq;
            }
        }
        // partial sums of this warp's K slice
#pragma unroll
        for (int i = 0; i < kMaxGroupTokens; ++i) {
            if (i < m) {
                red[((0 * wk + wk_id) * kMaxGroupTokens + i) * width + wr_id * 32 + lane] = aa[i];
                if (DUAL) red[((1 * wk + wk_id) * kMaxGroupTokens + i) * width + wr_id * 32 + lane] = ab_[i];
            }
        }
        consumer_sync();

        if (STAGE == kStageGateUp) {
            // (token, row tile): sum the K slices, activation, Q8_1 of the 32 results (lane = element)
            for (int pr = warp; pr < m * wr; pr += kConsumerWarps) {
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
                uint8_t* out = p.inter_q8 + (size_t)mt[kMetaOutRow + i] * p.inter_stride + (size_t)(tile0 + wq) * kQ81Bytes;
                reinterpret_cast<int8_t*>(out)[4 + lane] = q;
                const __half dh = __float2half(d);
                if (lane == 0) *reinterpret_cast<__half2*>(out) = __halves2half2(dh, __float2half(sum));
                // the same block as planes, the form the down stage streams
                p.out_soa_q[(size_t)mt[kMetaOutRow + i] * p.out_soa_q_stride + (size_t)(tile0 + wq) * 32 + lane] = q;
                if (lane == 0) p.out_soa_d[(size_t)mt[kMetaOutRow + i] * p.out_soa_d_stride + (tile0 + wq)] = __half2float(dh);
            }
        } else {
            const int H = p.H, r0 = tile0 * 32, rows_here = min(width, H - r0);
            const int ctid = tid;  // 0..511 among consumers
            for (int e = ctid; e < m * width; e += 32 * kConsumerWarps) {
                const int i = e / width, c = e - i * width;
                if (c < rows_here) p.pair_out[(size_t)mt[kMetaOutRow + i] * H + r0 + c] = sum_slices(red, 0, wk, i, width, c);
            }
            // whoever completes a token's contributions for this row tile adds them up
            __threadfence();
            consumer_sync();
            int* done = reinterpret_cast<int*>(red);   // red is free now: reuse 8 words as flags
            const int expected = p.top_k + (p.nrows_shared > 0 ? 1 : 0);
            const int row_tile = tile0 / wr;
            consumer_sync();
            if (ctid < m) {
                int* ctr = p.combine_ctr + (size_t)mt[kMetaTok + ctid] * p.n_row_tiles + row_tile;
                const int c = atomicAdd(ctr, 1);
                done[ctid] = (c == expected - 1);
                if (c == expected - 1) *ctr = 0;
            }
            consumer_sync();
            __threadfence();
            const int k = p.top_k;
            for (int i = 0; i < m; ++i) {
                if (!done[i]) continue;
                const int t = mt[kMetaTok + i];
                for (int r = ctid; r < rows_here; r += 32 * kConsumerWarps) {
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
        consumer_sync();   // red, meta and the activation buffer are free again
        if (lane == 0) mbar_arrive(aempty + ab);
    }
}

// ------------------------------------------------------------------ launchers --------------
static int ngroups_of(int type, int ncols) {
    (void)type;
    return (ncols / 32 + kGroupUnits - 1) / kGroupUnits;
}
static StreamGeom geom_for(int ngroups_min) {
    int wk = kConsumerWarps;
    while (wk > 1 && wk > ngroups_min) wk >>= 1;
    return StreamGeom{wk, kConsumerWarps / wk};
}
static int64_t host_tile_bytes(int type, int ncols) { return tiled_matrix_bytes(type, 32, ncols); }

TiledGeomHost tiled_gate_up_geom(int type_routed, int type_shared, int H, bool has_shared) {
    int g = ngroups_of(type_routed, H);
    if (has_shared) g = min(g, ngroups_of(type_shared, H));
    StreamGeom t = geom_for(g);
    // a tile too large for one ring stage is cut along K, which needs one row tile per CTA
    if (host_tile_bytes(type_routed, H) > kSlabMax || (has_shared && host_tile_bytes(type_shared, H) > kSlabMax)) t = StreamGeom{kConsumerWarps, 1};
    return TiledGeomHost{t.wk, t.wr};
}
TiledGeomHost tiled_down_geom(int type_routed, int F, int type_shared, int F_s) {
    int g = ngroups_of(type_routed, F);
    if (F_s > 0) g = min(g, ngroups_of(type_shared, F_s));
    StreamGeom t = geom_for(g);
    if (host_tile_bytes(type_routed, F) > kSlabMax || (F_s > 0 && host_tile_bytes(type_shared, F_s) > kSlabMax)) t = StreamGeom{kConsumerWarps, 1};
    return TiledGeomHost{t.wk, t.wr};
}

static int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

template <int TYPE, int STAGE, bool DUAL>
static cudaError_t launch_stream_t(const GemvParams& p, int wk, int wr, cudaStream_t stream) {
    const StreamSmem ss = stream_smem(max(p.ncols_routed, p.ncols_shared), wr, wk, DUAL);
    if (ss.nst < 2) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(stream_kernel<TYPE, STAGE, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
    if (e != cudaSuccess) return e;
    stream_kernel<TYPE, STAGE, DUAL><<<sm_count(), kStreamThreads, ss.total, stream>>>(p, wk, wr);
    return cudaGetLastError();
}

template <int STAGE>
static cudaError_t dispatch_stream(int type, const GemvParams& p, int wk, int wr, cudaStream_t stream) {
    const bool dual = STAGE == kStageGateUp && p.act == CHIMERE_ACT_SWIGLU;
    switch (type) {
        case CHIMERE_TYPE_Q4_0: return dual ? launch_stream_t<CHIMERE_TYPE_Q4_0, STAGE, true>(p, wk, wr, stream)
                                            : launch_stream_t<CHIMERE_TYPE_Q4_0, STAGE, false>(p, wk, wr, stream);
        case CHIMERE_TYPE_Q8_0: return dual ? launch_stream_t<CHIMERE_TYPE_Q8_0, STAGE, true>(p, wk, wr, stream)
                                            : launch_stream_t<CHIMERE_TYPE_Q8_0, STAGE, false>(p, wk, wr, stream);
        case CHIMERE_TYPE_IQ3_S: return dual ? launch_stream_t<CHIMERE_TYPE_IQ3_S, STAGE, true>(p, wk, wr, stream)
                                             : launch_stream_t<CHIMERE_TYPE_IQ3_S, STAGE, false>(p, wk, wr, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gate_up_tiled(const GemvParams& p, int max_entries, cudaStream_t stream) {
    (void)max_entries;
    const TiledGeomHost g = tiled_gate_up_geom(p.type_routed, p.type_shared, p.H, p.nrows_shared > 0);
    cudaError_t e = dispatch_stream<kStageGateUp>(p.type_routed, p, g.wk, g.wr, stream);
    if (e == cudaSuccess && p.nrows_shared > 0 && p.type_shared != p.type_routed)
        e = dispatch_stream<kStageGateUp>(p.type_shared, p, g.wk, g.wr, stream);
    return e;
}

// p.n_row_tiles must be ceil(H / (32 * wr)) with the geometry of tiled_down_geom
cudaError_t launch_down_tiled(const GemvParams& p, int max_entries, cudaStream_t stream) {
    (void)max_entries;
    const TiledGeomHost g = tiled_down_geom(p.type_routed, p.ncols_routed, p.type_shared, p.nrows_shared > 0 ? p.ncols_shared : 0);
    cudaError_t e = dispatch_stream<kStageDown>(p.type_routed, p, g.wk, g.wr, stream);
    if (e == cudaSuccess && p.nrows_shared > 0 && p.type_shared != p.type_routed)
        e = dispatch_stream<kStageDown>(p.type_shared, p, g.wk, g.wr, stream);
    return e;
}

}  // namespace chimere
