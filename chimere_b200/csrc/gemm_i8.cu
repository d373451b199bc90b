// gemm_i8.cu -- block-scaled int8 GEMM on the 5th-generation tensor cores (tcgen05, sm_100a), the
// prefill-size counterpart of the GEMV kernels.
//
// Math per output element:   D[row][tok] = sum over 32-wide blocks b of
//                            sa[row][b] * sb[tok][b] * (sum_i A[row][32b+i] * B[tok][32b+i])
// i.e. exactly the per-block integer dot of the ggml Q8_0 x Q8_1 / Q4_0 x Q8_1 / IQ3_S x Q8_1 kernels
// (chimere-server/src/kernels/gemv_q8_0.rs:230-255, chimere-server/kernels/chimere_kernels.cu:788-862),
// kept as an exact int32 per block and scaled in fp32 -- the integer results are bit-identical to the
// GEMV path; only the order of the fp32 operations differs.
//
// Operands come in the "mma128" layout made for the MMA: per (128-row tile, block b) 4096 bytes of int8
// in the canonical K-major no-swizzle core-matrix order [k half (2)][row group (16)][row (8)][16 bytes]
// followed by 128 f32 scales.  A plain bulk copy of a (tile, block range) lands MMA-ready in shared
// memory: shared-memory descriptor with leading (K) byte offset 2048 and stride (row group) byte offset 128.
//
// CTA = 18 warps, persistent (one CTA per SM), output tiles handed out by an atomic counter:
//   warp 0  takes the next tile index, publishes it to the other warps through a small ring in shared memory, and
//           feeds the operand ring with cp.async.bulk;
//   warp 1  owns TMEM (512 columns = four 128x128 int32 accumulators, used as two pairs) and issues one
//           tcgen05.mma kind::i8 (M 128, N = the tile's token count rounded up to 16, K 32) per block, never
//           accumulating across blocks;
//   warps 2..17 read each block's accumulator back (tcgen05.ld, four warps per TMEM lane quarter, each a quarter of
//           the tile's token columns), convert, scale and add into fp32 registers (thread = output row), then store
//           the tile.  The loads of one piece are in flight while the previous piece is processed, and a pair of
//           accumulators is handed back to the MMA warp as soon as its values are in registers.
// The read-back is what bounds the kernel: per (row, token, block) one integer add and two fused multiply-adds
// against 32 tensor-pipe multiply-adds, i.e. about four times the MMA's own time on the CUDA cores.
// All waits are bounded; a wait that runs out raises a status bit, nothing blocks for good, and the CTA still
// frees its TMEM.
#include "common.cuh"
#include "kernels.h"

namespace chimere {

constexpr int kG_TileBytes = 4096 + 512;     // one (128 x 32) int8 block + 128 f32 scales
constexpr int kG_BlocksPerStage = 4;
constexpr int kG_Stages = 4;
constexpr int kG_StageBytes = 2 * kG_BlocksPerStage * kG_TileBytes;   // A blocks then B blocks
constexpr int kG_EpiWarps = 16;                // four per TMEM lane quarter: each takes a quarter of the tile's token columns
constexpr int kG_EpiCols = 128 / (kG_EpiWarps / 4);   // columns per read-back warp in a full tile
constexpr int kG_Threads = 32 * (2 + kG_EpiWarps);
constexpr int kG_TmemCols = 512;
constexpr int kG_Sched = 4;                    // tile indices in flight between the scheduler and the other warps

__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t saddr) {
    // start address (>>4) | leading byte offset 2048 (>>4) << 16 | stride byte offset 128 (>>4) << 32 | version 1 << 46
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(2048u >> 4) << 16) | ((uint64_t)(128u >> 4) << 32) | (1ull << 46);
}
// D format S32 (2 << 4), A and B signed int8 (1 << 7, 1 << 10), both K-major, N (>> 3 at bit 17), M = 128 (>> 4 at bit 24)
__device__ __forceinline__ uint32_t instr_desc_i8(int n) { return (2u << 4) | (1u << 7) | (1u << 10) | (((uint32_t)n >> 3) << 17) | ((128u >> 4) << 24); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
// TMEM -> registers, thread = lane (row), N consecutive 32-bit columns; no wait: tc_wait_ld() before the values are used
template <int N> __device__ __forceinline__ void tc_ld_nowait(uint32_t taddr, int (&v)[N]);
template <> __device__ __forceinline__ void tc_ld_nowait<32>(uint32_t taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
template <> __device__ __forceinline__ void tc_ld_nowait<16>(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}
template <> __device__ __forceinline__ void tc_ld_nowait<8>(uint32_t taddr, int (&v)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// int32 -> f32 without the conversion unit: |v| <= 32 * 127 * 128 < 2^22, so v + 0x4B400000 read as a float is
// 12582912 + v exactly.  The subtraction of 12582912 is folded into the first scaling step (see block_piece).
constexpr uint32_t kMagicBits = 0x4B400000u;
constexpr float kMagic = 12582912.0f;

struct GemmShared {
    uint64_t full[kG_Stages];        // stage bytes have landed
    uint64_t empty[kG_Stages];       // stage read by the MMAs and by the read-back warps (scales)
    uint64_t tfull[2];               // the two accumulators of a block pair are complete
    uint64_t tempty[2];              // ... have been read back
    uint64_t sfull[kG_Sched];        // a tile index has been published
    uint64_t sempty[kG_Sched];       // ... and taken by the MMA warp and every read-back warp
    uint64_t ebar;                   // meeting point of the read-back warps in an epilogue
    int sched[kG_Sched];
    uint32_t tmem_base;
    int failed;
};

// What a CTA works on: its operands (mma128 tiles), the number of K blocks and of valid token columns.
struct GemmWork {
    const uint8_t* a_src; const uint8_t* b_src;
    int nblocks, n_valid;
    int aux0, aux1, aux2, aux3;   // policy specific
};

// Policy::work() names tile idx: kWorkOk, kWorkSkip (no such tile, go on) or kWorkEnd (nothing at or after idx).
// Policy::store<W>() consumes the fp32 accumulators, thread = row; acc[c] belongs to token column part * W + c.
constexpr int kWorkOk = 0, kWorkSkip = 1, kWorkEnd = 2;

// Meeting point of the read-back warps with a bounded wait (a warp that gave up must not block the others
// for good).  `phase` counts the meetings of this warp; false if the wait ran out.
__device__ __forceinline__ bool epilogue_meet(GemmShared& sh, uint32_t& phase, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive_cta(&sh.ebar);
    const bool ok = mbar_wait(&sh.ebar, phase & 1u);
    ++phase;
    return ok;
}

// two 64-bit words (four floats) from a 32-bit shared address, the same for every lane
__device__ __forceinline__ void lds_2x64(uint32_t a, uint64_t& x, uint64_t& y) { asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(x), "=l"(y) : "r"(a)); }
__device__ __forceinline__ float lds_f32(uint32_t a) { float v; asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a)); return v; }

// One piece of one block: CH accumulator columns of this thread's row, already in registers as int32.
//   acc[c] += (S * sa) * sb[col]      with S * sa = fma(float(S + magic), sa, -magic * sa)
// The addend of the first step is exact when sa has at most 22 significant bits (every ggml scale is an f16 times
// a small integer), so the step rounds S * sa once, like a plain multiplication.  sb: shared address of the token
// scales of the piece's first column (16-byte aligned).
template <int CH>
__device__ __forceinline__ void block_piece(const int (&v)[CH], uint64_t sa2, uint32_t sb, uint64_t* acc2) {
    const uint64_t c2 = mul2(sa2, pack2(__float_as_uint(-kMagic), __float_as_uint(-kMagic)));
#pragma unroll
    for (int g = 0; g < CH / 4; ++g) {
        uint64_t s01, s23;
        lds_2x64(sb + 16u * g, s01, s23);
        const uint64_t u01 = fma2(pack2((uint32_t)v[4 * g + 0] + kMagicBits, (uint32_t)v[4 * g + 1] + kMagicBits), sa2, c2);
        const uint64_t u23 = fma2(pack2((uint32_t)v[4 * g + 2] + kMagicBits, (uint32_t)v[4 * g + 3] + kMagicBits), sa2, c2);
        acc2[2 * g + 0] = fma2(u01, s01, acc2[2 * g + 0]);
        acc2[2 * g + 1] = fma2(u23, s23, acc2[2 * g + 1]);
    }
}

// The read-back of one output tile by one warp: W = CH * NCH token columns per warp, taken in pieces of CH columns.
// Blocks come in pairs (never across a ring stage): one wait per pair, and the pair's TMEM buffers are handed back as
// soon as their values are in registers.  The load of a piece is in flight while the piece before it is processed
// (two register sets in turn); the last piece of a pair is processed under the first load of the next pair.
template <int CH, int NCH>
__device__ __forceinline__ bool readback_tile(GemmShared& sh, uint32_t smem_base, uint32_t tmem, int32_t* status, int nblocks, int q, int part,
                                              int lane, uint32_t& sg, uint32_t& bg, uint64_t* acc2) {
    constexpr int W = CH * NCH;
    constexpr int kLast = (NCH - 1) * CH;        // first column of a block's last piece
    const uint32_t row4 = (uint32_t)(q * 32 + lane) * 4u, col4 = (uint32_t)(part * W) * 4u;
    const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(part * W);
    int va[CH], vb[CH];                          // pieces with an even / odd number within their pair
    uint64_t p_sa2 = 0; uint32_t p_sb = 0;       // scales of the piece waiting in vb
    bool have = false;
    int release_st = -1;                         // ring stage whose scales the waiting piece still needs
    bool ok = true;
    for (int blk = 0; blk < nblocks; ++bg) {
        const int s = blk / kG_BlocksPerStage, j0 = blk - s * kG_BlocksPerStage;
        const int st = (int)((sg + (uint32_t)s) % kG_Stages);
        const int nb_stage = min(kG_BlocksPerStage, nblocks - s * kG_BlocksPerStage);
        const int npair = min(2, nb_stage - j0);
        const int pr = (int)(bg & 1u), tph = (int)((bg >> 1) & 1u);
        if (!mbar_wait(&sh.tfull[pr], (uint32_t)tph)) { if (status) atomicOr(status, kStatusWaitTimeout); sh.failed = 1; ok = false; break; }
        tc_fence_after();
        // shared addresses of block j0's row scales (this thread's row) and token scales (this warp's first column)
        const uint32_t a_sc = smem_base + (uint32_t)(st * kG_StageBytes + j0 * kG_TileBytes + 4096) + row4;
        const uint32_t sb_0 = smem_base + (uint32_t)(st * kG_StageBytes + (kG_BlocksPerStage + j0) * kG_TileBytes + 4096) + col4;
        const float sa_0 = lds_f32(a_sc);
        const uint64_t sa2_0 = pack2(__float_as_uint(sa_0), __float_as_uint(sa_0));
        const uint32_t t0 = trow + (uint32_t)((2 * pr) * 128);
        if (npair == 2) {
            const float sa_1 = lds_f32(a_sc + kG_TileBytes);
            const uint64_t sa2_1 = pack2(__float_as_uint(sa_1), __float_as_uint(sa_1));
            const uint32_t sb_1 = sb_0 + kG_TileBytes;
#pragma unroll
            for (int k = 0; k < 2 * NCH; ++k) {
                const int h = k / NCH, c = k % NCH;
                const uint32_t ta = t0 + (uint32_t)(h * 128 + c * CH);
                if ((k & 1) == 0) tc_ld_nowait<CH>(ta, va); else tc_ld_nowait<CH>(ta, vb);
                if (k == 0) {
                    if (have) {
                        block_piece<CH>(vb, p_sa2, p_sb, acc2 + kLast / 2);
                        if (release_st >= 0) { __syncwarp(); if (lane == 0) mbar_arrive_cta(&sh.empty[release_st]); release_st = -1; }
                    }
                } else {
                    const int hp = (k - 1) / NCH, cp = (k - 1) % NCH;
                    if (((k - 1) & 1) == 0) block_piece<CH>(va, hp ? sa2_1 : sa2_0, (hp ? sb_1 : sb_0) + 4u * cp * CH, acc2 + cp * CH / 2);
                    else block_piece<CH>(vb, hp ? sa2_1 : sa2_0, (hp ? sb_1 : sb_0) + 4u * cp * CH, acc2 + cp * CH / 2);
                }
                tc_wait_ld();
            }
            p_sa2 = sa2_1; p_sb = sb_1 + 4u * kLast; have = true;   // piece 2 * NCH - 1 waits in vb
        } else {
            // an odd last block: no partner to overlap with
            if (have) {
                block_piece<CH>(vb, p_sa2, p_sb, acc2 + kLast / 2);
                if (release_st >= 0) { __syncwarp(); if (lane == 0) mbar_arrive_cta(&sh.empty[release_st]); release_st = -1; }
                have = false;
            }
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                tc_ld_nowait<CH>(t0 + (uint32_t)(c * CH), va);
                tc_wait_ld();
                block_piece<CH>(va, sa2_0, sb_0 + 4u * c * CH, acc2 + c * CH / 2);
            }
        }
        // every value of the pair is in registers: the MMA warp may overwrite its two accumulators
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cta(&sh.tempty[pr]);
        blk += npair;
        if (j0 + npair == nb_stage) {   // the stage's scales are needed until the waiting piece has been processed
            if (have) release_st = st;
            else if (lane == 0) mbar_arrive_cta(&sh.empty[st]);
        }
    }
    if (ok && have) block_piece<CH>(vb, p_sa2, p_sb, acc2 + kLast / 2);
    if (release_st >= 0) { __syncwarp(); if (lane == 0) mbar_arrive_cta(&sh.empty[release_st]); }
    sg += (uint32_t)((nblocks + kG_BlocksPerStage - 1) / kG_BlocksPerStage);
    return ok;
}

// One output tile by one read-back warp: accumulate over the blocks, then hand the sums to the policy's store.
template <class Policy, class Params, int CH, int NCH>
__device__ __forceinline__ bool readback_and_store(const Params& p, int idx, GemmShared& sh, uint32_t smem_base, uint8_t* xch, uint32_t tmem, int q,
                                                   int part, int lane, uint32_t& sg, uint32_t& bg, uint32_t& ephase) {
    constexpr int W = CH * NCH;
    GemmWork item;
    Policy::work(p, idx, item);
    uint64_t acc2[W / 2];
#pragma unroll
    for (int i = 0; i < W / 2; ++i) acc2[i] = 0ull;
    const bool ok = readback_tile<CH, NCH>(sh, smem_base, tmem, p.status, item.nblocks, q, part, lane, sg, bg, acc2);
    float acc[W];
#pragma unroll
    for (int i = 0; i < W / 2; ++i) unpack2(acc2[i], acc[2 * i], acc[2 * i + 1]);
    Policy::work(p, idx, item);   // named again here rather than kept in registers through the read-back
    Policy::template store<W>(p, item, q * 32 + lane, q, part, lane, acc, xch, sh, ephase, ok);
    return ok;
}
template <class Policy, class Params, int CH, int NCH>
__device__ __noinline__ bool readback_and_store_call(const Params& p, int idx, GemmShared& sh, uint32_t smem_base, uint8_t* xch, uint32_t tmem, int q,
                                                     int part, int lane, uint32_t& sg, uint32_t& bg, uint32_t& ephase) {
    return readback_and_store<Policy, Params, CH, NCH>(p, idx, sh, smem_base, xch, tmem, q, part, lane, sg, bg, ephase);
}

template <class Policy, class Params>
__global__ void __launch_bounds__(kG_Threads, 1) gemm_i8_kernel(const Params p, int32_t* tile_counter) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ GemmShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (tid == 0) {
        for (int i = 0; i < kG_Stages; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 1 + kG_EpiWarps); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sh.tfull[i], 1); mbar_init(&sh.tempty[i], kG_EpiWarps); }
        for (int i = 0; i < kG_Sched; ++i) { mbar_init(&sh.sfull[i], 1); mbar_init(&sh.sempty[i], 1 + kG_EpiWarps); }
        mbar_init(&sh.ebar, kG_EpiWarps);
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
        // ------------------------------ tile scheduler + operand producer ------------------------------
        if (lane == 0) {
            uint32_t sg = 0, tn = 0;   // ring stages issued / tile indices published so far
            bool ok = true;
            while (ok) {
                // next tile (heavy tiles have the low indices); a skipped index costs one more atomic
                GemmWork item;
                int idx, ws;
                do { idx = atomicAdd(tile_counter, 1); ws = Policy::work(p, idx, item); } while (ws == kWorkSkip);
                const int slot = (int)(tn % kG_Sched), sph = (int)((tn / kG_Sched) & 1u);
                if (!mbar_wait(&sh.sempty[slot], (uint32_t)(sph ^ 1))) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; break; }
                sh.sched[slot] = ws == kWorkEnd ? -1 : idx;
                mbar_arrive_cta(&sh.sfull[slot]);   // (release: the index is visible to whoever sees the arrival)
                ++tn;
                if (ws == kWorkEnd) break;
                const int nstages = (item.nblocks + kG_BlocksPerStage - 1) / kG_BlocksPerStage;
                for (int s = 0; s < nstages; ++s, ++sg) {
                    const int st = (int)(sg % kG_Stages), ph = (int)((sg / kG_Stages) & 1u);
                    if (!mbar_wait(&sh.empty[st], (uint32_t)(ph ^ 1))) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; ok = false; break; }
                    const int b0 = s * kG_BlocksPerStage, nb = min(kG_BlocksPerStage, item.nblocks - b0);
                    uint8_t* dst = smem + (size_t)st * kG_StageBytes;
                    const uint32_t bytes = (uint32_t)nb * kG_TileBytes;
                    mbar_expect_tx(&sh.full[st], 2 * bytes);
                    bulk_g2s(dst, item.a_src + (size_t)b0 * kG_TileBytes, bytes, &sh.full[st]);
                    bulk_g2s(dst + kG_BlocksPerStage * kG_TileBytes, item.b_src + (size_t)b0 * kG_TileBytes, bytes, &sh.full[st]);
                }
            }
        }
    } else {
        // ------------------------------ MMA issuer (warp 1) and read-back warps (2..17) ------------------------------
        const int q = warp & 3;                      // TMEM lane quarter a read-back warp may read
        const int part = (warp - 2) >> 2;            // which share of the token columns
        uint32_t sg = 0, bg = 0, tn = 0, ephase = 0; // ring stages / block pairs / tiles / epilogue meetings so far
        bool ok = true;
        while (ok) {
            const int slot = (int)(tn % kG_Sched), sph = (int)((tn / kG_Sched) & 1u);
            if (!mbar_wait(&sh.sfull[slot], (uint32_t)sph)) { if (lane == 0) atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; break; }
            const int idx = *reinterpret_cast<volatile int*>(&sh.sched[slot]);
            __syncwarp();
            if (lane == 0) mbar_arrive_cta(&sh.sempty[slot]);
            ++tn;
            if (idx < 0) break;
            GemmWork item;
            Policy::work(p, idx, item);
            const int nblocks = item.nblocks;
            if (warp == 1) {
                if (lane == 0) {
                    const int n_mma = min(128, max(16, (item.n_valid + 15) & ~15));
                    const uint32_t idesc = instr_desc_i8(n_mma);
                    const int nstages = (nblocks + kG_BlocksPerStage - 1) / kG_BlocksPerStage;
                    for (int s = 0; s < nstages && ok; ++s, ++sg) {
                        const int st = (int)(sg % kG_Stages), ph = (int)((sg / kG_Stages) & 1u);
                        if (!mbar_wait(&sh.full[st], (uint32_t)ph)) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; ok = false; break; }
                        tc_fence_after();
                        const int nb = min(kG_BlocksPerStage, nblocks - s * kG_BlocksPerStage);
                        const uint32_t sa = smem_u32(smem + (size_t)st * kG_StageBytes);
                        const uint32_t sb = sa + kG_BlocksPerStage * kG_TileBytes;
                        // two blocks per hand-over: accumulator pair bg & 1 = TMEM buffers 2 * (bg & 1) and + 1
                        for (int j = 0; j < nb; j += 2, ++bg) {
                            const int pr = (int)(bg & 1u), tph = (int)((bg >> 1) & 1u);
                            if (!mbar_wait(&sh.tempty[pr], (uint32_t)(tph ^ 1))) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; ok = false; break; }
                            tc_fence_after();
                            tc_mma_i8(tmem + (2 * pr) * 128, smem_desc_kmajor(sa + j * kG_TileBytes), smem_desc_kmajor(sb + j * kG_TileBytes), idesc);
                            if (j + 1 < nb)
                                tc_mma_i8(tmem + (2 * pr + 1) * 128, smem_desc_kmajor(sa + (j + 1) * kG_TileBytes), smem_desc_kmajor(sb + (j + 1) * kG_TileBytes), idesc);
                            tc_commit(&sh.tfull[pr]);        // both accumulators ready when these MMAs have finished
                        }
                        if (ok) tc_commit(&sh.empty[st]);    // ... and the stage's int8 data is no longer needed
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                continue;
            }
            // ---- read-back: thread = output row; the narrower the tile, the fewer columns per warp ----
            // (full tiles inline; the narrower classes are calls, so that they do not weigh on the registers of this loop)
            const int n_valid = item.n_valid;
            uint8_t* xch = smem + (size_t)kG_Stages * kG_StageBytes;
            if (n_valid > 64) ok = readback_and_store<Policy, Params, 8, 4>(p, idx, sh, smem_u32(smem), xch, tmem, q, part, lane, sg, bg, ephase);
            else if (n_valid > 32) ok = readback_and_store_call<Policy, Params, 8, 2>(p, idx, sh, smem_u32(smem), xch, tmem, q, part, lane, sg, bg, ephase);
            else ok = readback_and_store_call<Policy, Params, 8, 1>(p, idx, sh, smem_u32(smem), xch, tmem, q, part, lane, sg, bg, ephase);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kG_TmemCols) : "memory");
    }
}

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
    template <int W>
    __device__ static __forceinline__ void store(const GemmParams& p, const GemmWork& w, int row, int, int part, int,
                                                 const float (&acc)[W], uint8_t*, GemmShared&, uint32_t&, bool ok) {
        if (!ok || row >= w.aux0) return;
        float* out = p.out + (size_t)(w.aux1 + row) * p.ldo + w.aux2 + part * W;
#pragma unroll
        for (int c = 0; c < W; ++c)
            if (part * W + c < w.n_valid) out[c] = acc[c];
    }
};

// ------------------------------------------------------------------ MoE prefill policies ----
// Token tiles (built on the device after routing): {expert (-1 = shared expert), start, n_valid, 0}; word 0 of the
// list = number of tiles, words 4 and 5 = the tile counters of the two GEMM launches (zero when the list is built).
// Routed tile: pairs perm[start .. start + n_valid); shared tile: tokens start .. .
constexpr int kTileHeader = 8;

// gate/up: A tile = 64 gate rows | 64 up rows of the same 64 intermediate rows (or 128 up rows when there is no
// gate).  The halves meet in shared memory; the activation is quantised to Q8_1 (32 consecutive rows = one warp)
// straight into the down GEMM's token tile.
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
    template <int W>
    __device__ static __forceinline__ void store(const PrefillGemmParams& p, const GemmWork& w, int row, int q, int part, int lane,
                                                 float (&acc)[W], uint8_t* smem, GemmShared& sh, uint32_t& ephase, bool ok) {
        const bool dual = p.act == CHIMERE_ACT_SWIGLU;
        float* xch = reinterpret_cast<float*>(smem);   // [128][129] floats behind the ring
        // every read-back warp is done with the previous tile's exchange
        if (!epilogue_meet(sh, ephase, lane) && lane == 0) atomicOr(p.status, kStatusWaitTimeout);
#pragma unroll
        for (int c = 0; c < W; ++c) xch[row * 129 + part * W + c] = acc[c];
        if (!epilogue_meet(sh, ephase, lane) && lane == 0) atomicOr(p.status, kStatusWaitTimeout);
        if (!ok) return;
        // units of work: (32-row block of the intermediate, token column); a warp takes a unit at a time, lane = row
        const int nrb = dual ? 2 : 4;
        const int ew = (part << 2) | q;                  // this warp's number among the read-back warps
        const int nblk_limit = w.aux2 ? p.nblk_shared : p.nblk_routed;
        const int khalf = lane >> 4, kin = lane & 15;
        for (int u = ew; u < nrb * w.n_valid; u += kG_EpiWarps) {
            const int rb = u % nrb, c = u / nrb;
            const int blk = (dual ? w.aux1 * 2 : w.aux1 * 4) + rb;
            if (blk >= nblk_limit) continue;             // rows of zero padding behind the last real row
            const int r = rb * 32 + lane;
            const float a = xch[r * 129 + c];
            float v;
            if (dual) v = silu_mul_ref(a, xch[(r + 64) * 129 + c]);
            else { const float t = fmaxf(a, 0.0f); v = t * t; }
            float amax = fabsf(v);
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
            const float d = amax / 127.0f;
            const int8_t qv = (amax == 0.0f) ? (int8_t)0 : (int8_t)roundf(v / d);
            uint8_t* dst = p.out_tiles + (size_t)w.aux0 * p.out_tile_stride + (size_t)blk * kG_TileBytes;
            reinterpret_cast<int8_t*>(dst)[khalf * 2048 + (c >> 3) * 128 + (c & 7) * 16 + kin] = qv;
            if (lane == 0) *reinterpret_cast<float*>(dst + 4096 + c * 4) = __half2float(__float2half(d));
        }
        // Token columns past n_valid of the tile are left as they are: the down GEMM never stores them, and every
        // column's sums depend on that column alone.
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
    template <int W>
    __device__ static __forceinline__ void store(const PrefillGemmParams& p, const GemmWork& w, int row, int, int part, int,
                                                 float (&acc)[W], uint8_t*, GemmShared&, uint32_t&, bool ok) {
        if (!ok) return;
        const int h = w.aux1 * 128 + row;
        if (h >= p.H) return;
#pragma unroll
        for (int c = 0; c < W; ++c) {
            const int col = part * W + c;
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

// tile_counter: one int32 of device memory that is zero when the kernel starts (it ends at n_items + the number of CTAs)
cudaError_t launch_gemm_i8_f32(const GemmParams& p_in, int n_items, int32_t* tile_counter, cudaStream_t stream) {
    if (n_items <= 0) return cudaSuccess;
    GemmParams p = p_in;
    p.n_items = n_items;
    const size_t smem = kG_RingBytes + 1024;
    static bool attr_done[64] = {};
    cudaError_t e = max_smem_once(gemm_i8_kernel<PlainPolicy, GemmParams>, (int)smem, attr_done);
    if (e != cudaSuccess) return e;
    gemm_i8_kernel<PlainPolicy, GemmParams><<<gemm_grid(n_items), kG_Threads, smem, stream>>>(p, tile_counter);
    return cudaGetLastError();
}

// The tile list's header words 4 (gate/up) and 5 (down) are the launches' tile counters; build_tiles_kernel zeroes them.
cudaError_t launch_prefill_gemm(const PrefillGemmParams& p, bool down, int n_tiles_max, cudaStream_t stream) {
    const int n_items = n_tiles_max * p.row_tiles_max;
    if (n_items <= 0) return cudaSuccess;
    int32_t* counter = const_cast<int32_t*>(p.tiles) + (down ? 5 : 4);
    cudaError_t e;
    if (down) {
        const size_t smem = kG_RingBytes + 1024;
        static bool attr_done[64] = {};
        e = max_smem_once(gemm_i8_kernel<DownPolicy, PrefillGemmParams>, (int)smem, attr_done);
        if (e != cudaSuccess) return e;
        gemm_i8_kernel<DownPolicy, PrefillGemmParams><<<gemm_grid(n_items), kG_Threads, smem, stream>>>(p, counter);
    } else {
        const size_t smem = kG_RingBytes + kG_XchBytes + 1024;
        static bool attr_done[64] = {};
        e = max_smem_once(gemm_i8_kernel<GateUpPolicy, PrefillGemmParams>, (int)smem, attr_done);
        if (e != cudaSuccess) return e;
        gemm_i8_kernel<GateUpPolicy, PrefillGemmParams><<<gemm_grid(n_items), kG_Threads, smem, stream>>>(p, counter);
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
        tiles[4] = 0; tiles[5] = 0; tiles[6] = 0; tiles[7] = 0;   // the two GEMM launches' tile counters start at zero
        list[0] = tot_e; list[1] = tot_e; list[2] = 0; list[3] = 0;
    }
}

// Token tiles of the gate/up GEMM: the Q8_1 planes of each tile's tokens in mma128 order.
// grid = (max tiles, 16 groups of 8 token slots), 256 threads = 8 slots x 32 chunk lanes: the eight slots of a group
// are the 8 x 16 bytes of one core-matrix row group, so every 128-byte segment of the tile is written whole, and a
// token's 16-byte chunks are read four in a row.
__global__ void __launch_bounds__(256) gather_tiles_kernel(const int32_t* tiles, const int32_t* perm, const int8_t* x_q, int64_t x_q_stride,
                                                           const float* x_d, int x_d_stride, uint8_t* b_tiles, int64_t b_tile_stride, int H,
                                                           int top_k) {
    const int j = blockIdx.x, grp = blockIdx.y;
    if (j >= __ldcg(tiles)) return;
    const int4 t = __ldcg(reinterpret_cast<const int4*>(tiles + kTileHeader) + j);
    const int sl = threadIdx.x & 7, lane_ch = threadIdx.x >> 3;
    const int c = grp * 8 + sl;                   // token slot of the tile
    const bool valid = c < t.z;
    const int tok = !valid ? 0 : (t.x < 0 ? t.y + c : __ldcg(perm + t.y + c) / top_k);
    uint8_t* base = b_tiles + (size_t)j * b_tile_stride;
    for (int ch = lane_ch; ch < H / 16; ch += 32) {
        const uint4 v = valid ? __ldcg(reinterpret_cast<const uint4*>(x_q + (size_t)tok * x_q_stride) + ch) : make_uint4(0, 0, 0, 0);
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

cudaError_t launch_gather_tiles(const int32_t* tiles, const int32_t* perm, const int8_t* x_q, int64_t x_q_stride, const float* x_d,
                                int x_d_stride, uint8_t* b_tiles, int64_t b_tile_stride, int H, int top_k, int n_tiles_max, cudaStream_t stream) {
    if (n_tiles_max <= 0) return cudaSuccess;
    gather_tiles_kernel<<<dim3(n_tiles_max, 16), 256, 0, stream>>>(tiles, perm, x_q, x_q_stride, x_d, x_d_stride, b_tiles, b_tile_stride, H, top_k);
    return cudaGetLastError();
}


}  // namespace chimere
