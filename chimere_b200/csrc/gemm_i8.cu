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
// CTA = 6 warps: warp 0 feeds a shared-memory ring with cp.async.bulk; warp 1 owns TMEM (512 columns =
// four 128x128 int32 accumulators) and issues one tcgen05.mma kind::i8 (M 128, N 128, K 32) per block,
// never accumulating across blocks; warps 2..5 read each block's accumulator back (tcgen05.ld), convert,
// scale and add into fp32 registers (thread = output row), then write the tile.
// All waits are bounded; a wait that runs out raises a status bit and the CTA still frees its TMEM.
#include "common.cuh"
#include "kernels.h"

namespace chimere {

constexpr int kG_TileBytes = 4096 + 512;     // one (128 x 32) int8 block + 128 f32 scales
constexpr int kG_BlocksPerStage = 4;
constexpr int kG_Stages = 3;
constexpr int kG_StageBytes = 2 * kG_BlocksPerStage * kG_TileBytes;   // A blocks then B blocks
constexpr int kG_Threads = 192;
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

struct GemmShared {
    uint64_t full[kG_Stages];        // stage bytes have landed
    uint64_t empty[kG_Stages];       // stage read by the MMAs and by the epilogue (scales)
    uint64_t tfull[4];               // accumulator of a block is complete
    uint64_t tempty[4];              // accumulator has been read back
    uint32_t tmem_base;
    int failed;
};

// One CTA per (row tile, token tile).  a_tiles / b_tiles: mma128 operands; nblocks K blocks.
// out[(row0 + r) * ldo + col0 + c] = D[r][c] for r < rows_valid, c < n_valid.
template <class Epilogue>
__global__ void __launch_bounds__(kG_Threads, 1) gemm_i8_kernel(const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ GemmShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const GemmItem item = p.items[blockIdx.x];
    const uint8_t* a_src = p.a_base + item.a_offset;
    const uint8_t* b_src = p.b_base + item.b_offset;
    const int nblocks = p.nblocks;
    const int nstages_total = (nblocks + kG_BlocksPerStage - 1) / kG_BlocksPerStage;

    if (tid == 0) {
        for (int i = 0; i < kG_Stages; ++i) { mbar_init(&sh.full[i], 1); mbar_init(&sh.empty[i], 1 + 4); }
        for (int i = 0; i < 4; ++i) { mbar_init(&sh.tfull[i], 1); mbar_init(&sh.tempty[i], 4); }
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
            for (int s = 0; s < nstages_total; ++s) {
                const int st = s % kG_Stages, ph = (s / kG_Stages) & 1;
                if (!mbar_wait(&sh.empty[st], ph ^ 1)) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; break; }
                const int b0 = s * kG_BlocksPerStage, nb = min(kG_BlocksPerStage, nblocks - b0);
                uint8_t* dst = smem + (size_t)st * kG_StageBytes;
                const uint32_t bytes = (uint32_t)nb * kG_TileBytes;
                mbar_expect_tx(&sh.full[st], 2 * bytes);
                bulk_g2s(dst, a_src + (size_t)b0 * kG_TileBytes, bytes, &sh.full[st]);
                bulk_g2s(dst + kG_BlocksPerStage * kG_TileBytes, b_src + (size_t)b0 * kG_TileBytes, bytes, &sh.full[st]);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            int blk = 0;
            bool ok = true;
            for (int s = 0; s < nstages_total && ok; ++s) {
                const int st = s % kG_Stages, ph = (s / kG_Stages) & 1;
                if (!mbar_wait(&sh.full[st], ph)) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; ok = false; break; }
                tc_fence_after();
                const int nb = min(kG_BlocksPerStage, nblocks - s * kG_BlocksPerStage);
                const uint32_t sa = smem_u32(smem + (size_t)st * kG_StageBytes);
                const uint32_t sb = sa + kG_BlocksPerStage * kG_TileBytes;
                for (int j = 0; j < nb; ++j, ++blk) {
                    const int buf = blk & 3, tph = (blk >> 2) & 1;
                    if (!mbar_wait(&sh.tempty[buf], tph ^ 1)) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; ok = false; break; }
                    tc_fence_after();
                    tc_mma_i8(tmem + buf * 128, smem_desc_kmajor(sa + j * kG_TileBytes), smem_desc_kmajor(sb + j * kG_TileBytes));
                    tc_commit(&sh.tfull[buf]);       // accumulator ready when this MMA has finished
                }
                tc_commit(&sh.empty[st]);            // ... and the stage's int8 data is no longer needed
            }
        }
    } else {
        // ------------------------------ epilogue: thread = output row ------------------------------
        const int q = warp & 3;                      // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;
        const int nchunks = (item.n_valid + 31) >> 5;
        float acc[128];
#pragma unroll
        for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
        bool ok = true;
        for (int blk = 0; blk < nblocks && ok; ++blk) {
            const int s = blk / kG_BlocksPerStage, j = blk - s * kG_BlocksPerStage;
            const int st = s % kG_Stages;
            const int buf = blk & 3, tph = (blk >> 2) & 1;
            if (!mbar_wait(&sh.tfull[buf], tph)) { atomicOr(p.status, kStatusWaitTimeout); sh.failed = 1; ok = false; break; }
            tc_fence_after();
            const uint8_t* stage = smem + (size_t)st * kG_StageBytes;
            const float sa = *reinterpret_cast<const float*>(stage + j * kG_TileBytes + 4096 + row * 4);
            const float4* sbv = reinterpret_cast<const float4*>(stage + (kG_BlocksPerStage + j) * kG_TileBytes + 4096);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (c < nchunks) {
                    int v[32];
                    tc_ld32(tmem + ((uint32_t)(q * 32) << 16) + buf * 128 + c * 32, v);
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        const float4 sb4 = sbv[c * 8 + g];
                        acc[c * 32 + 4 * g + 0] = fmaf((float)v[4 * g + 0] * sb4.x, sa, acc[c * 32 + 4 * g + 0]);
                        acc[c * 32 + 4 * g + 1] = fmaf((float)v[4 * g + 1] * sb4.y, sa, acc[c * 32 + 4 * g + 1]);
                        acc[c * 32 + 4 * g + 2] = fmaf((float)v[4 * g + 2] * sb4.z, sa, acc[c * 32 + 4 * g + 2]);
                        acc[c * 32 + 4 * g + 3] = fmaf((float)v[4 * g + 3] * sb4.w, sa, acc[c * 32 + 4 * g + 3]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cta(&sh.tempty[buf]);
                if (j == kG_BlocksPerStage - 1 || blk == nblocks - 1) mbar_arrive_cta(&sh.empty[st]);   // scales of the stage read
            }
        }
        if (ok) Epilogue::store(p, item, row, acc);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kG_TmemCols) : "memory");
    }
}

// plain fp32 tile store (primitive test and the down projection's per-pair rows)
struct StoreF32 {
    __device__ static __forceinline__ void store(const GemmParams& p, const GemmItem& it, int row, const float (&acc)[128]) {
        if (row >= it.rows_valid) return;
#pragma unroll
        for (int c = 0; c < 128; ++c)
            if (c < it.n_valid) p.out[(size_t)(it.out_row0 + row) * p.ldo + it.out_col0 + c] = acc[c];
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

cudaError_t launch_gemm_i8_f32(const GemmParams& p, int n_items, cudaStream_t stream) {
    if (n_items <= 0) return cudaSuccess;
    const size_t smem = (size_t)kG_Stages * kG_StageBytes + 1024;
    cudaError_t e = cudaFuncSetAttribute(gemm_i8_kernel<StoreF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    gemm_i8_kernel<StoreF32><<<n_items, kG_Threads, smem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace chimere
