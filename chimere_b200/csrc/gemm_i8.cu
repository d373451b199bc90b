// gemm_i8.cu -- block-scaled int8 GEMM on the 5th-generation tensor cores (tcgen05, sm_100a), the
// prefill-size counterpart of the GEMV kernels.
//
// Math per output element:   D[row][tok] = sum over 32-wide blocks b of
//                            sa[row][b] * sb[tok][b] * (sum_i A[row][32b+i] * B[tok][32b+i])
// i.e. exactly the per-block integer dot of the ggml Q8_0 x Q8_1 / Q4_0 x Q8_1 / IQ3_S x Q8_1 kernels
// (chimere-server/src/kernels/gemv_q8_0.rs:230-255, chimere-server/kernels/chimere_kernels.cu:788-862),
// kept as an exact int32 per block and scaled in fp32 -- the integer results are bit-identical to the
// GEMV path; only the order of the fp32 additions differs.
//
// Operands come in the "mma128" layout made for the MMA: per (128-row tile, block b) 4096 bytes of int8
// in the canonical K-major no-swizzle core-matrix order [k half (2)][row group (16)][row (8)][16 bytes]
// followed by 128 f32 scales.  A plain bulk copy of a (tile, block range) lands MMA-ready in shared
// memory: shared-memory descriptor with leading (K) byte offset 2048 and stride (row group) byte offset 128.
//
// CTA = 18 warps: warp 0 feeds a shared-memory ring with cp.async.bulk; warp 1 owns TMEM (512 columns =
// four 128x128 int32 accumulators) and issues one tcgen05.mma kind::i8 (M 128, N 128, K 32) per block,
// never accumulating across blocks; warps 2..17 read each block's accumulator back (tcgen05.ld; four warps per
// TMEM lane quarter, 32 token columns each), convert, scale and add into fp32 registers (thread = output row)
// with two-wide fp32 instructions, then write the tile.  The read-back is what bounds the kernel: 128 x 128
// values per block against 64 tensor-pipe cycles of MMA.
// All waits are bounded; a wait that runs out raises a status bit and the CTA still frees its TMEM.
#include "common.cuh"
#include "kernels.h"

namespace chimere {

constexpr int kG_TileBytes = 4096 + 512;     // one (128 x 32) int8 block + 128 f32 scales
constexpr int kG_BlocksPerStage = 4;
constexpr int kG_Stages = 4;
constexpr int kG_StageBytes = 2 * kG_BlocksPerStage * kG_TileBytes;   // A blocks then B blocks
constexpr int kG_EpiWarps = 16;                // four per TMEM lane quarter: each takes 32 of the 128 token columns
constexpr int kG_EpiCols = 128 / (kG_EpiWarps / 4);
constexpr int kG_Threads = 32 * (2 + kG_EpiWarps);
constexpr int kG_TmemCols = 512;

__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t saddr) {
    // start address (>>4) | leading byte offset 2048 (>>4) << 16 | stride byte offset 128 (>>4) << 32 | version 1 << 46
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(2048u >> 4) << 16) | ((uint64_t)(128u >> 4) << 32) | (1ull << 46);
}
// D format S32 (2 << 4), A and B signed int8 (1 << 7, 1 << 10), both K-major, N = 128 (>> 3 at bit 17), M = 128 (>> 4 at bit 24)
constexpr uint32_t kG_InstrDesc = (2u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kG_InstrDesc), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}

__device__ __forceinline__ void tc_ld32_nowait(uint32_t taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// int32 -> f32 without the conversion unit: |v| <= 32 * 127 * 128 < 2^22, so v + 0x4B400000 read as a float is
// 12582912 + v exactly, and one fp32 subtraction gives v.  (Integer add and float add run at full rate.)
__device__ __forceinline__ float i2f_exact(int v) { return __int_as_float(v + 0x4B400000) - 12582912.0f; }
// two fp32 lanes in one 64-bit register (sm_100 has two-wide fp32 add / mul / fma)
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi)); return r; }
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) { uint64_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) { uint64_t d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) { uint64_t d; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

struct GemmShared {
    uint64_t full[kG_Stages];        // stage bytes have landed
    uint64_t empty[kG_Stages];       // stage read by the MMAs and by the epilogue (scales)
    uint64_t tfull[2];               // the two accumulators of a block pair are complete
    uint64_t tempty[2];              // ... have been read back
    uint32_t tmem_base;
    int failed;
};

// What a CTA works on: its operands (mma128 tiles), the number of K blocks and of valid token columns.
struct GemmWork {
    const uint8_t* a_src; const uint8_t* b_src;
    int nblocks, n_valid;
    int aux0, aux1, aux2, aux3;   // policy specific
};

// Persistent: CTA c works on output tiles c, c + gridDim.x, ... (128 rows x up to 128 tokens each).
// Policy::work() names tile idx: kWorkOk, kWorkSkip (no such tile, go on) or kWorkEnd (nothing at or after idx).
// Policy::store() consumes the fp32 accumulators, thread = row.  The three roles walk the same sequence of tiles
// on their own; the ring stages and the TMEM buffers are counted across tiles, so the copies and the MMAs of the
// next tile run while the read-back warps finish and store the current one.
constexpr int kWorkOk = 0, kWorkSkip = 1, kWorkEnd = 2;

template <class Policy, class Params>
__global__ void __launch_bounds__(kG_Threads, 1) gemm_i8_kernel(const Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ GemmShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int stride = (int)gridDim.x;

    if (tid == 0) {
        for (int i = 0; i < kG_Stages; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 1 + kG_EpiWarps); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sh.tfull[i], 1); mbar_init(&sh.tempty[i], kG_EpiWarps); }
        sh.failed = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"(kG_TmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            uint32_t sg = 0;   // stages issued so far, over all tiles
            bool ok = true;
            for (int idx = blockIdx.x; ok; idx += stride) {
                GemmWork item;
                const int ws = Policy::work(p, idx, item);
                if (ws == kWorkEnd) break;
                if (ws == kWorkSkip) continue;
                const int nstages = (item.nblocks + kG_BlocksPerStage - 1) / kG_BlocksPerStage;
                for (int s = 0; s < nstages; ++s, ++sg) {
                    const int st = sg % kG_Stages, ph = (sg / kG_Stages) & 1;
                    if (!mbar_wait(&sh.empty[st], ph ^ 1)) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; ok = false; break; }
                    const int b0 = s * kG_BlocksPerStage, nb = min(kG_BlocksPerStage, item.nblocks - b0);
                    uint8_t* dst = smem + (size_t)st * kG_StageBytes;
                    const uint32_t bytes = (uint32_t)nb * kG_TileBytes;
                    mbar_expect_tx(&sh.full[st], 2 * bytes);
                    bulk_g2s(dst, item.a_src + (size_t)b0 * kG_TileBytes, bytes, &sh.full[st]);
                    bulk_g2s(dst + kG_BlocksPerStage * kG_TileBytes, item.b_src + (size_t)b0 * kG_TileBytes, bytes, &sh.full[st]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            uint32_t sg = 0, bg = 0;   // stages / block pairs so far, over all tiles
            bool ok = true;
            for (int idx = blockIdx.x; ok; idx += stride) {
                GemmWork item;
                const int ws = Policy::work(p, idx, item);
                if (ws == kWorkEnd) break;
                if (ws == kWorkSkip) continue;
                const int nstages = (item.nblocks + kG_BlocksPerStage - 1) / kG_BlocksPerStage;
                for (int s = 0; s < nstages && ok; ++s, ++sg) {
                    const int st = sg % kG_Stages, ph = (sg / kG_Stages) & 1;
                    if (!mbar_wait(&sh.full[st], ph)) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; ok = false; break; }
                    tc_fence_after();
                    const int nb = min(kG_BlocksPerStage, item.nblocks - s * kG_BlocksPerStage);
                    const uint32_t sa = smem_u32(smem + (size_t)st * kG_StageBytes);
                    const uint32_t sb = sa + kG_BlocksPerStage * kG_TileBytes;
                    // two blocks per hand-over: accumulator pair bg & 1 = TMEM buffers 2 * (bg & 1) and + 1
                    for (int j = 0; j < nb; j += 2, ++bg) {
                        const int pr = bg & 1, tph = (bg >> 1) & 1;
                        if (!mbar_wait(&sh.tempty[pr], tph ^ 1)) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; ok = false; break; }
                        tc_fence_after();
                        tc_mma_i8(tmem + (2 * pr) * 128, smem_desc_kmajor(sa + j * kG_TileBytes), smem_desc_kmajor(sb + j * kG_TileBytes));
                        if (j + 1 < nb)
                            tc_mma_i8(tmem + (2 * pr + 1) * 128, smem_desc_kmajor(sa + (j + 1) * kG_TileBytes), smem_desc_kmajor(sb + (j + 1) * kG_TileBytes));
                        tc_commit(&sh.tfull[pr]);        // both accumulators ready when these MMAs have finished
                    }
                    tc_commit(&sh.empty[st]);            // ... and the stage's int8 data is no longer needed
                }
            }
        }
    } else {
        // ------------------------------ read-back: thread = output row, 32 token columns ------------------------------
        const int q = warp & 3;                      // TMEM lane quarter this warp may read
        const int part = (warp - 2) >> 2;            // which 32 columns
        const int row = q * 32 + lane;
        const uint64_t neg_magic2 = pack2(__float_as_uint(-12582912.0f), __float_as_uint(-12582912.0f));
        uint32_t sg = 0, bg = 0;   // stages / block pairs so far
        bool ok = true;
        for (int idx = blockIdx.x;; idx += stride) {
            GemmWork item;
            const int ws = Policy::work(p, idx, item);
            if (ws == kWorkEnd) break;
            if (ws == kWorkSkip) continue;
            const int nblocks = item.nblocks;
            const int ncols_here = min(kG_EpiCols, max(0, item.n_valid - part * kG_EpiCols));
            uint64_t acc2[kG_EpiCols / 2];
#pragma unroll
            for (int i = 0; i < kG_EpiCols / 2; ++i) acc2[i] = 0ull;
            // blocks come in pairs (never across a ring stage): one wait and one arrival per pair
            for (int blk = 0; blk < nblocks && ok; ++bg) {
                const int s = blk / kG_BlocksPerStage, j0 = blk - s * kG_BlocksPerStage;
                const int st = (sg + s) % kG_Stages;
                const int nb_stage = min(kG_BlocksPerStage, nblocks - s * kG_BlocksPerStage);
                const int npair = min(2, nb_stage - j0);
                const int pr = bg & 1, tph = (bg >> 1) & 1;
                if (!mbar_wait(&sh.tfull[pr], tph)) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; ok = false; break; }
                tc_fence_after();
                if (ncols_here > 0) {
                    const uint8_t* stage = smem + (size_t)st * kG_StageBytes;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (h < npair) {
                            const int j = j0 + h;
                            const uint32_t sab = *reinterpret_cast<const uint32_t*>(stage + j * kG_TileBytes + 4096 + row * 4);
                            const uint64_t sa2 = pack2(sab, sab);
                            const uint4* sbv = reinterpret_cast<const uint4*>(stage + (kG_BlocksPerStage + j) * kG_TileBytes + 4096) + part * (kG_EpiCols / 4);
                            int v[32];
                            tc_ld32(tmem + ((uint32_t)(q * 32) << 16) + (2 * pr + h) * 128 + part * kG_EpiCols, v);
                            // value + 0x4B400000 read as a float is 12582912 + value (see i2f_exact); the rest runs two columns at a time
#pragma unroll
                            for (int g = 0; g < kG_EpiCols / 4; ++g) {
                                const uint4 sb4 = sbv[g];
                                const uint64_t f01 = add2(pack2((uint32_t)(v[4 * g + 0] + 0x4B400000), (uint32_t)(v[4 * g + 1] + 0x4B400000)), neg_magic2);
                                const uint64_t f23 = add2(pack2((uint32_t)(v[4 * g + 2] + 0x4B400000), (uint32_t)(v[4 * g + 3] + 0x4B400000)), neg_magic2);
                                acc2[2 * g + 0] = fma2(f01, mul2(pack2(sb4.x, sb4.y), sa2), acc2[2 * g + 0]);
                                acc2[2 * g + 1] = fma2(f23, mul2(pack2(sb4.z, sb4.w), sa2), acc2[2 * g + 1]);
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                blk += npair;
                if (lane == 0) {
                    mbar_arrive_cta(&sh.tempty[pr]);
                    if (j0 + npair == nb_stage) mbar_arrive_cta(&sh.empty[st]);   // scales of the stage read
                }
            }
            sg += (uint32_t)((nblocks + kG_BlocksPerStage - 1) / kG_BlocksPerStage);
            float acc[kG_EpiCols];
#pragma unroll
            for (int i = 0; i < kG_EpiCols / 2; ++i) unpack2(acc2[i], acc[2 * i], acc[2 * i + 1]);
            Policy::store(p, item, row, q, part, lane, acc, smem + (size_t)kG_Stages * kG_StageBytes, ok);
            if (!ok) break;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kG_TmemCols) : "memory");
    }
}

__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * kG_EpiWarps) : "memory"); }

// plain fp32 tile store: out[(row0 + r) * ldo + col0 + c] = D[r][c]  (the primitive)
struct PlainPolicy {
    __device__ static __forceinline__ int work(const GemmParams& p, int idx, GemmWork& w) {
        if (idx >= p.n_items) return kWorkEnd;
        const GemmItem it = p.items[idx];
        w.a_src = p.a_base + it.a_offset; w.b_src = p.b_base + it.b_offset;
        w.nblocks = p.nblocks; w.n_valid = it.n_valid;
        w.aux0 = it.rows_valid; w.aux1 = it.out_row0; w.aux2 = it.out_col0; w.aux3 = 0;
        return kWorkOk;
    }
    __device__ static __forceinline__ void store(const GemmParams& p, const GemmWork& w, int row, int, int part, int,
                                                 const float (&acc)[kG_EpiCols], uint8_t*, bool ok) {
        if (!ok || row >= w.aux0) return;
#pragma unroll
        for (int c = 0; c < kG_EpiCols; ++c)
            if (part * kG_EpiCols + c < w.n_valid) p.out[(size_t)(w.aux1 + row) * p.ldo + w.aux2 + part * kG_EpiCols + c] = acc[c];
    }
};

// ------------------------------------------------------------------ MoE prefill policies ----
// Token tiles (built on the device after routing): {expert (-1 = shared expert), start, n_valid, 0}; word 0 of the
// list = number of tiles.  Routed tile: pairs perm[start .. start + n_valid); shared tile: tokens start .. .
constexpr int kTileHeader = 4;

// gate/up: A tile = 64 gate rows | 64 up rows of the same 64 intermediate rows (or 128 up rows when there is no
// gate).  The up half hands its sums to the gate half through shared memory; the activation is quantised to
// Q8_1 (32 consecutive rows = one warp) straight into the down GEMM's token tile.
struct GateUpPolicy {
    __device__ static __forceinline__ int work(const PrefillGemmParams& p, int idx, GemmWork& w) {
        const int n_tiles = __ldcg(p.tiles);
        const int j = idx / p.row_tiles_max, rt = idx - j * p.row_tiles_max;
        if (j >= n_tiles) return kWorkEnd;
        const int4 t = __ldcg(reinterpret_cast<const int4*>(p.tiles + kTileHeader) + j);
        const bool shared = t.x < 0;
        const int row_tiles = shared ? p.row_tiles_shared : p.row_tiles_routed;
        if (rt >= row_tiles) return kWorkSkip;
        const int nb = p.ncols_in / 32;
        w.a_src = (shared ? p.sh_a : p.a_exps + (size_t)t.x * p.stride_a) + (size_t)rt * nb * kG_TileBytes;
        w.b_src = p.b_tiles + (size_t)j * p.b_tile_stride;
        w.nblocks = nb; w.n_valid = t.z;
        w.aux0 = j; w.aux1 = rt; w.aux2 = shared ? 1 : 0; w.aux3 = t.y;
        return kWorkOk;
    }
    __device__ static __forceinline__ void store(const PrefillGemmParams& p, const GemmWork& w, int row, int q, int part, int lane,
                                                 float (&acc)[kG_EpiCols], uint8_t* smem, bool ok) {
        const bool dual = p.act == CHIMERE_ACT_SWIGLU;
        float* xch = reinterpret_cast<float*>(smem);   // [128][129] floats behind the ring
        epilogue_sync();                                // every read-back warp is done with the previous tile's exchange
#pragma unroll
        for (int c = 0; c < kG_EpiCols; ++c) xch[row * 129 + part * kG_EpiCols + c] = acc[c];
        epilogue_sync();
        if (!ok || (dual && q >= 2)) return;
        // this warp's 32 rows form Q8_1 block `blk` of the intermediate; it quantises its half of the token columns
        const int blk = dual ? w.aux1 * 2 + q : w.aux1 * 4 + q;
        if (blk >= (w.aux2 ? p.nblk_shared : p.nblk_routed)) return;   // rows of zero padding behind the last real row
        uint8_t* dst = p.out_tiles + (size_t)w.aux0 * p.out_tile_stride + (size_t)blk * kG_TileBytes;
        const int khalf = lane >> 4, kin = lane & 15;
        const int c_end = min(w.n_valid, part * kG_EpiCols + kG_EpiCols);
        for (int c = part * kG_EpiCols; c < c_end; ++c) {
            const float a = xch[row * 129 + c];
            float v;
            if (dual) v = silu_mul_ref(a, xch[(row + 64) * 129 + c]);
            else { const float r = fmaxf(a, 0.0f); v = r * r; }
            float amax = fabsf(v);
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
            const float d = amax / 127.0f;
            const int8_t qv = (amax == 0.0f) ? (int8_t)0 : (int8_t)roundf(v / d);
            reinterpret_cast<int8_t*>(dst)[khalf * 2048 + (c >> 3) * 128 + (c & 7) * 16 + kin] = qv;
            if (lane == 0) *reinterpret_cast<float*>(dst + 4096 + c * 4) = __half2float(__float2half(d));
        }
        // columns past n_valid: zero quants and scales, so that the down GEMM's unused columns stay finite
        for (int c = max(w.n_valid, part * kG_EpiCols); c < part * kG_EpiCols + kG_EpiCols; ++c) {
            reinterpret_cast<int8_t*>(dst)[khalf * 2048 + (c >> 3) * 128 + (c & 7) * 16 + kin] = 0;
            if (lane == 0) *reinterpret_cast<float*>(dst + 4096 + c * 4) = 0.0f;
        }
    }
};

// down: rows of H; the tile's columns are pairs, written to pair_out[pair row][H]
struct DownPolicy {
    __device__ static __forceinline__ int work(const PrefillGemmParams& p, int idx, GemmWork& w) {
        const int n_tiles = __ldcg(p.tiles);
        const int j = idx / p.row_tiles_max, rt = idx - j * p.row_tiles_max;
        if (j >= n_tiles) return kWorkEnd;
        const int4 t = __ldcg(reinterpret_cast<const int4*>(p.tiles + kTileHeader) + j);
        const bool shared = t.x < 0;
        const int nb = (shared ? p.ncols_in_shared : p.ncols_in) / 32;
        w.a_src = (shared ? p.sh_a : p.a_exps + (size_t)t.x * p.stride_a) + (size_t)rt * nb * kG_TileBytes;
        w.b_src = p.b_tiles + (size_t)j * p.b_tile_stride;
        w.nblocks = nb; w.n_valid = t.z;
        w.aux0 = j; w.aux1 = rt; w.aux2 = shared ? 1 : 0; w.aux3 = t.y;
        return kWorkOk;
    }
    __device__ static __forceinline__ void store(const PrefillGemmParams& p, const GemmWork& w, int row, int, int part, int,
                                                 float (&acc)[kG_EpiCols], uint8_t*, bool ok) {
        if (!ok) return;
        const int h = w.aux1 * 128 + row;
        if (h >= p.H) return;
#pragma unroll
        for (int c = 0; c < kG_EpiCols; ++c) {
            const int col = part * kG_EpiCols + c;
            if (col < w.n_valid) {
                const int prow = w.aux2 ? p.T * p.top_k + w.aux3 + col : __ldcg(p.perm + w.aux3 + col);
                p.pair_out[(size_t)prow * p.H + h] = acc[c];
            }
        }
    }
};

// [rows][cols] int8 + [rows][cols/32] f32 scales -> mma128 tiles (rows padded with zeros to a multiple of 128).
// One thread per (row, block).
__global__ void pack_mma128_kernel(const int8_t* q, const float* scales, uint8_t* out, int rows, int cols) {
    const int nb = cols >> 5;
    const int rows_pad = (rows + 127) & ~127;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)rows_pad * nb) return;
    const int row = (int)(idx % rows_pad), b = (int)(idx / rows_pad);
    const int tile = row >> 7, r = row & 127;
    uint8_t* dst = out + ((size_t)tile * nb + b) * kG_TileBytes;
    uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
    float sc = 0.0f;
    if (row < rows) {
        const uint4* src = reinterpret_cast<const uint4*>(q + (size_t)row * cols + b * 32);
        lo = src[0]; hi = src[1];
        sc = scales[(size_t)row * nb + b];
    }
    *reinterpret_cast<uint4*>(dst + (r >> 3) * 128 + (r & 7) * 16) = lo;          // k 0..15
    *reinterpret_cast<uint4*>(dst + 2048 + (r >> 3) * 128 + (r & 7) * 16) = hi;   // k 16..31
    *reinterpret_cast<float*>(dst + 4096 + r * 4) = sc;
}

cudaError_t launch_pack_mma128(const int8_t* q, const float* scales, uint8_t* out, int rows, int cols, cudaStream_t stream) {
    const int64_t n = (int64_t)((rows + 127) & ~127) * (cols / 32);
    if (n <= 0) return cudaSuccess;
    pack_mma128_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(q, scales, out, rows, cols);
    return cudaGetLastError();
}

// persistent CTAs: one per SM of the current device, or fewer when there are fewer tiles
static int gemm_grid(int n_items) {
    const int n_sm = sm_count();
    return n_items < n_sm ? n_items : n_sm;
}
constexpr size_t kG_RingBytes = (size_t)kG_Stages * kG_StageBytes;
constexpr size_t kG_XchBytes = 128 * 129 * sizeof(float);   // gate/up: where the two halves of a tile meet

cudaError_t launch_gemm_i8_f32(const GemmParams& p_in, int n_items, cudaStream_t stream) {
    if (n_items <= 0) return cudaSuccess;
    GemmParams p = p_in;
    p.n_items = n_items;
    const size_t smem = kG_RingBytes + 1024;
    static bool attr_done[64] = {};
    cudaError_t e = max_smem_once(gemm_i8_kernel<PlainPolicy, GemmParams>, (int)smem, attr_done);
    if (e != cudaSuccess) return e;
    gemm_i8_kernel<PlainPolicy, GemmParams><<<gemm_grid(n_items), kG_Threads, smem, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_prefill_gemm(const PrefillGemmParams& p, bool down, int n_tiles_max, cudaStream_t stream) {
    const int n_items = n_tiles_max * p.row_tiles_max;
    if (n_items <= 0) return cudaSuccess;
    cudaError_t e;
    if (down) {
        const size_t smem = kG_RingBytes + 1024;
        static bool attr_done[64] = {};
        e = max_smem_once(gemm_i8_kernel<DownPolicy, PrefillGemmParams>, (int)smem, attr_done);
        if (e != cudaSuccess) return e;
        gemm_i8_kernel<DownPolicy, PrefillGemmParams><<<gemm_grid(n_items), kG_Threads, smem, stream>>>(p);
    } else {
        const size_t smem = kG_RingBytes + kG_XchBytes + 1024;
        static bool attr_done[64] = {};
        e = max_smem_once(gemm_i8_kernel<GateUpPolicy, PrefillGemmParams>, (int)smem, attr_done);
        if (e != cudaSuccess) return e;
        gemm_i8_kernel<GateUpPolicy, PrefillGemmParams><<<gemm_grid(n_items), kG_Threads, smem, stream>>>(p);
    }
    return cudaGetLastError();
}

// ------------------------------------------------------------------ tensor-pipe probe ----
// What the int8 tensor pipe can do when nothing is read back: every CTA (one per SM) keeps issuing
// tcgen05.mma kind::i8 (M 128, N 128 or 256, K 32) on operands resident in shared memory, accumulating in TMEM,
// with a commit every 64 instructions and a bounded wait on the last one.  Timed from the host with events, this
// is the denominator the prefill numbers are stated against (2 * 128 * N * 32 operations per instruction).
__global__ void __launch_bounds__(128, 1) mma_i8_probe_kernel(int n_mma, int n_cols, int n_acc, int32_t* status) {
    extern __shared__ __align__(1024) uint8_t smem[];   // A: 128 x 32 int8 (4096 B), B: n_cols x 32 int8
    __shared__ __align__(8) uint64_t s_bar[2];   // commit groups alternate between the two
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < (4096 + n_cols * 32) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(smem)[i] = 0x9E3779B9u * (uint32_t)(i + 1 + blockIdx.x * 977);   // any bytes will do
    if (tid == 0) { mbar_init(&s_bar[0], 1); mbar_init(&s_bar[1], 1); mbar_fence_init(); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the operands were written by ordinary stores
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    if (tid == 0) {
        const uint32_t sa = smem_u32(smem), sb = sa + 4096;
        const uint32_t lbo_b = (uint32_t)n_cols * 16u;   // K halves of B are n_cols / 8 row groups of 128 bytes apart
        const uint64_t adesc = smem_desc_kmajor(sa);
        const uint64_t bdesc = (uint64_t)((sb & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_b >> 4) << 16) | ((uint64_t)(128u >> 4) << 32) | (1ull << 46);
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (((uint32_t)n_cols >> 3) << 17) | ((128u >> 4) << 24);
        auto mma = [&](uint32_t d, uint32_t acc) {
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
        };
        // accumulators taken in turn (n_acc of them, n_cols columns each); groups of 64 instructions per commit
        uint32_t dcol[4];
        for (int j = 0; j < 4; ++j) dcol[j] = tmem + (uint32_t)((j % n_acc) * n_cols);
        const int groups = (n_mma + 63) / 64;
        bool ok = true;
        for (int g = 0; g < groups && ok; ++g) {
#pragma unroll 4
            for (int j = 0; j < 64; j += 4) {
                mma(dcol[0], g > 0 || j >= 4 ? 1u : 0u);
                mma(dcol[1], g > 0 || j >= 4 ? 1u : 0u);
                mma(dcol[2], g > 0 || j >= 4 ? 1u : 0u);
                mma(dcol[3], g > 0 || j >= 4 ? 1u : 0u);
            }
            tc_commit(&s_bar[g & 1]);
            // at most two commit groups in flight: wait for the one before the one just issued
            if (g >= 1 && !mbar_wait(&s_bar[(g - 1) & 1], ((g - 1) >> 1) & 1)) { if (status) atomicOr(status, kStatusWaitTimeout); ok = false; }
        }
        if (ok && groups >= 1 && !mbar_wait(&s_bar[(groups - 1) & 1], ((groups - 1) >> 1) & 1) && status) atomicOr(status, kStatusWaitTimeout);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

// Returns the number of CTAs launched (each issues n_mma instructions, rounded up to a multiple of 64), or a negative CUDA error.
int launch_mma_i8_probe(int n_mma, int n_cols, int n_acc, int32_t* status, cudaStream_t stream) {
    const int ctas = gemm_grid(1 << 30);
    const size_t smem = 4096 + (size_t)n_cols * 32 + 1024;
    mma_i8_probe_kernel<<<ctas, 128, smem, stream>>>(n_mma, n_cols, n_acc, status);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ctas : -100 - (int)e;
}

// ------------------------------------------------------------------ prefill plumbing kernels ----
// ggml blocks -> mma128 tiles: int8 values and f32 block scales (IQ3_S: scale = d * (1 + 2*sub-scale), exact in f32).
// dst row of source row r: plain (mode 0), gate half (mode 1: (r/64)*128 + r%64) or up half (mode 2: ... + 64).
// One thread per (row, block); blockIdx.y = expert.
template <int TYPE>
__global__ void pack_mma128_ggml_kernel(const uint8_t* raw, uint8_t* out, int nrows, int ncols, int mode, int64_t raw_stride,
                                        int64_t out_stride, const uint32_t* grid) {
    const int nb = ncols >> 5;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)nrows * nb) return;
    const int r = (int)(idx % nrows), b = (int)(idx / nrows);
    int w[8], mul;
    float dw;
    Unit<TYPE>::load(raw + (size_t)blockIdx.y * raw_stride + (size_t)r * Unit<TYPE>::row_bytes(ncols), b, grid, w, dw, mul);
    if (TYPE == CHIMERE_TYPE_Q4_0) {
#pragma unroll
        for (int g = 0; g < 8; ++g) {   // bytes hold 16 * (nibble - 8): arithmetic shift of every byte
            const int x = w[g];
            w[g] = (int)(((uint32_t)((int8_t)(x) >> 4) & 0xFFu) | (((uint32_t)((int8_t)(x >> 8) >> 4) & 0xFFu) << 8) |
                         (((uint32_t)((int8_t)(x >> 16) >> 4) & 0xFFu) << 16) | (((uint32_t)((int8_t)(x >> 24) >> 4) & 0xFFu) << 24));
        }
    }
    const int dr = mode == 0 ? r : (r >> 6) * 128 + (r & 63) + (mode == 2 ? 64 : 0);
    const int tile = dr >> 7, rr = dr & 127;
    uint8_t* dst = out + (size_t)blockIdx.y * out_stride + ((size_t)tile * nb + b) * kG_TileBytes;
    *reinterpret_cast<uint4*>(dst + (rr >> 3) * 128 + (rr & 7) * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4*>(dst + 2048 + (rr >> 3) * 128 + (rr & 7) * 16) = make_uint4(w[4], w[5], w[6], w[7]);
    *reinterpret_cast<float*>(dst + 4096 + rr * 4) = dw * (float)mul;
}

static __device__ const uint32_t g_iq3s_grid_mma[512] = {
#include "iq3s_grid.inc"
};

cudaError_t launch_pack_mma128_ggml(int type, const void* raw, void* out, int n_mats, int nrows, int ncols, int mode,
                                    int64_t raw_stride, int64_t out_stride, cudaStream_t stream) {
    if (n_mats <= 0) return cudaSuccess;
    const int64_t n = (int64_t)nrows * (ncols / 32);
    const dim3 grid((unsigned)((n + 255) / 256), (unsigned)n_mats);
    const uint32_t* g = nullptr;
    cudaGetSymbolAddress((void**)&g, g_iq3s_grid_mma);
    switch (type) {
        case CHIMERE_TYPE_Q4_0: pack_mma128_ggml_kernel<CHIMERE_TYPE_Q4_0><<<grid, 256, 0, stream>>>((const uint8_t*)raw, (uint8_t*)out, nrows, ncols, mode, raw_stride, out_stride, g); break;
        case CHIMERE_TYPE_Q8_0: pack_mma128_ggml_kernel<CHIMERE_TYPE_Q8_0><<<grid, 256, 0, stream>>>((const uint8_t*)raw, (uint8_t*)out, nrows, ncols, mode, raw_stride, out_stride, g); break;
        case CHIMERE_TYPE_IQ3_S: pack_mma128_ggml_kernel<CHIMERE_TYPE_IQ3_S><<<grid, 256, 0, stream>>>((const uint8_t*)raw, (uint8_t*)out, nrows, ncols, mode, raw_stride, out_stride, g); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// After routing: token tiles for the experts with at least `gemm_min` pairs (and for the shared expert), and the
// GEMV work list rewritten to hold only the smaller experts.  One CTA of 256 threads, thread e = expert e.
// Full tiles (128 pairs) come first and the partly filled ones last, so that the persistent GEMM CTAs, which take
// tiles round-robin, all get a similar mix of expensive and cheap tiles.
__global__ void __launch_bounds__(256) build_tiles_kernel(const int32_t* offsets, const int32_t* perm, int32_t* tiles, int32_t* list,
                                                          int E, int T, int top_k, int has_shared, int gemm_min) {
    __shared__ int scan_f[8], scan_p[8], scan_e[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cnt = tid < E ? offsets[tid + 1] - offsets[tid] : 0, off = tid < E ? offsets[tid] : 0;
    const bool big = cnt >= gemm_min;
    const int nf = big ? cnt / 128 : 0;                   // full tiles
    const int np = big && (cnt % 128) ? 1 : 0;            // the partly filled one
    const int ne = big ? 0 : (cnt + kMaxGroupTokens - 1) / kMaxGroupTokens;
    int jf = nf, jp = np, ie = ne;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, jf, s), b = __shfl_up_sync(0xffffffffu, jp, s), c = __shfl_up_sync(0xffffffffu, ie, s);
        if (lane >= s) { jf += a; jp += b; ie += c; }
    }
    if (lane == 31) { scan_f[warp] = jf; scan_p[warp] = jp; scan_e[warp] = ie; }
    __syncthreads();
    int bf = 0, bp = 0, be = 0, tot_f = 0, tot_p = 0, tot_e = 0;
    for (int w = 0; w < 8; ++w) {
        if (w < warp) { bf += scan_f[w]; bp += scan_p[w]; be += scan_e[w]; }
        tot_f += scan_f[w]; tot_p += scan_p[w]; tot_e += scan_e[w];
    }
    // shared-expert tiles: the full ones in front, its partly filled one with the other partly filled ones
    const int nsh_full = has_shared ? T / 128 : 0, nsh_part = has_shared && (T % 128) ? 1 : 0;
    int4* tv = reinterpret_cast<int4*>(tiles + kTileHeader);
    for (int i = tid; i < nsh_full; i += 256) tv[i] = make_int4(-1, i * 128, 128, 0);
    const int f0 = nsh_full + bf + jf - nf;
    for (int i = 0; i < nf; ++i) tv[f0 + i] = make_int4(tid, off + i * 128, 128, 0);
    const int part0 = nsh_full + tot_f;
    if (tid == 0 && nsh_part) tv[part0] = make_int4(-1, nsh_full * 128, T - nsh_full * 128, 0);
    if (np) tv[part0 + nsh_part + bp + jp - np] = make_int4(tid, off + nf * 128, cnt - nf * 128, 0);
    const int e0 = be + ie - ne;
    for (int i = 0; i < ne; ++i) {
        int* ent = list + kListHeader + kListEntry * (e0 + i);
        const int mm = min(kMaxGroupTokens, cnt - i * kMaxGroupTokens);
        ent[0] = tid; ent[1] = off + i * kMaxGroupTokens; ent[2] = mm; ent[3] = 0;
        for (int j = 0; j < kMaxGroupTokens; ++j) ent[4 + j] = j < mm ? perm[off + i * kMaxGroupTokens + j] : 0;
    }
    if (tid == 0) {
        tiles[0] = nsh_full + nsh_part + tot_f + tot_p; tiles[1] = nsh_full + nsh_part; tiles[2] = tot_f + tot_p; tiles[3] = 0;
        list[0] = tot_e; list[1] = tot_e; list[2] = 0; list[3] = 0;
    }
}

// Token tiles of the gate/up GEMM: the Q8_1 planes of each tile's tokens in mma128 order.
// grid = (max tiles, 16 groups of 8 token slots), 256 threads = 8 slots x 32 chunk lanes: the eight slots of a group
// are the 8 x 16 bytes of one core-matrix row group, so every 128-byte segment of the tile is written whole, and a
// token's 16-byte chunks are read four in a row.
__global__ void __launch_bounds__(256) gather_tiles_kernel(const int32_t* tiles, const int32_t* perm, const int8_t* x_q, const float* x_d,
                                                           int x_d_stride, uint8_t* b_tiles, int64_t b_tile_stride, int H, int top_k) {
    const int j = blockIdx.x, grp = blockIdx.y;
    if (j >= __ldcg(tiles)) return;
    const int4 t = __ldcg(reinterpret_cast<const int4*>(tiles + kTileHeader) + j);
    const int sl = threadIdx.x & 7, lane_ch = threadIdx.x >> 3;
    const int c = grp * 8 + sl;                   // token slot of the tile
    const bool valid = c < t.z;
    const int tok = !valid ? 0 : (t.x < 0 ? t.y + c : __ldcg(perm + t.y + c) / top_k);
    uint8_t* base = b_tiles + (size_t)j * b_tile_stride;
    for (int ch = lane_ch; ch < H / 16; ch += 32) {
        const uint4 v = valid ? __ldcg(reinterpret_cast<const uint4*>(x_q + (size_t)tok * H) + ch) : make_uint4(0, 0, 0, 0);
        const int b = ch >> 1, khalf = ch & 1;
        *reinterpret_cast<uint4*>(base + (size_t)b * kG_TileBytes + khalf * 2048 + grp * 128 + sl * 16) = v;
    }
    for (int b = lane_ch; b < H / 32; b += 32)
        *reinterpret_cast<float*>(base + (size_t)b * kG_TileBytes + 4096 + c * 4) = valid ? __ldcg(x_d + (size_t)tok * x_d_stride + b) : 0.0f;
}

cudaError_t launch_build_tiles(const int32_t* offsets, const int32_t* perm, int32_t* tiles, int32_t* list, int E, int T, int top_k,
                               int has_shared, int gemm_min, cudaStream_t stream) {
    build_tiles_kernel<<<1, 256, 0, stream>>>(offsets, perm, tiles, list, E, T, top_k, has_shared, gemm_min);
    return cudaGetLastError();
}

cudaError_t launch_gather_tiles(const int32_t* tiles, const int32_t* perm, const int8_t* x_q, const float* x_d, int x_d_stride,
                                uint8_t* b_tiles, int64_t b_tile_stride, int H, int top_k, int n_tiles_max, cudaStream_t stream) {
    if (n_tiles_max <= 0) return cudaSuccess;
    gather_tiles_kernel<<<dim3(n_tiles_max, 16), 256, 0, stream>>>(tiles, perm, x_q, x_d, x_d_stride, b_tiles, b_tile_stride, H, top_k);
    return cudaGetLastError();
}


}  // namespace chimere
