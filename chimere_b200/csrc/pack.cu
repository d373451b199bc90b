// pack.cu -- one-time rewrite of ggml block matrices into the tiled32 layout (see tiled.cuh).
// The rewrite is lossless: chimere_b200_block_sumi_tiled returns the same integers from the
// packed form as chimere_b200_block_sumi does from the ggml form.
#include "common.cuh"
#include "kernels.h"
#include "tiled.cuh"

namespace chimere {

static __device__ const uint32_t g_iq3s_grid_pack[512] = {
#include "iq3s_grid.inc"
};

// One thread per (row, unit); consecutive threads take consecutive rows so the stores coalesce.
// blockIdx.y = matrix index (expert).
template <int TYPE>
__global__ void pack_kernel(const uint8_t* raw, uint8_t* out, int nrows, int ncols, int64_t raw_stride, int64_t out_stride) {
    const int nb = ncols >> 5;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)nrows * nb) return;
    const int row = (int)(idx % nrows), b = (int)(idx / nrows);
    const int tile = row >> 5, lane = row & 31;
    const uint8_t* src_row = raw + (size_t)blockIdx.y * raw_stride + (size_t)row * Unit<TYPE>::row_bytes(ncols);
    uint8_t* dst_tile = out + (size_t)blockIdx.y * out_stride + (size_t)tile * Tiled<TYPE>::tile_bytes(ncols);
    if (TYPE == CHIMERE_TYPE_Q4_0) {
        const uint8_t* blk = src_row + b * 18;
        uint4 v;
        // low nibble: ggml's unsigned n; high nibble: n - 8 in two's complement
        v.x = ld_u32_a2(blk + 2) ^ 0x80808080u;  v.y = ld_u32_a2(blk + 6) ^ 0x80808080u;
        v.z = ld_u32_a2(blk + 10) ^ 0x80808080u; v.w = ld_u32_a2(blk + 14) ^ 0x80808080u;
        uint8_t* d = dst_tile + (size_t)b * 576;
        *reinterpret_cast<uint4*>(d + lane * 16) = v;
        *reinterpret_cast<uint16_t*>(d + 512 + lane * 2) = (uint16_t)ld_u16(blk);
    } else if (TYPE == CHIMERE_TYPE_Q8_0) {
        const uint8_t* blk = src_row + b * 34;
        uint4 lo, hi;
        lo.x = ld_u32_a2(blk + 2);  lo.y = ld_u32_a2(blk + 6);  lo.z = ld_u32_a2(blk + 10); lo.w = ld_u32_a2(blk + 14);
        hi.x = ld_u32_a2(blk + 18); hi.y = ld_u32_a2(blk + 22); hi.z = ld_u32_a2(blk + 26); hi.w = ld_u32_a2(blk + 30);
        uint8_t* d = dst_tile + (size_t)b * 1088;
        *reinterpret_cast<uint4*>(d + lane * 16) = lo;
        *reinterpret_cast<uint4*>(d + 512 + lane * 16) = hi;
        *reinterpret_cast<uint16_t*>(d + 1024 + lane * 2) = (uint16_t)ld_u16(blk);
    } else {
        const uint8_t* blk = src_row + (b >> 3) * 110;
        const int sg = b & 7;
        const uint32_t qh = blk[66 + sg];
        const uint32_t sgn = ld_u32_a2(blk + 74 + sg * 4);
        uint32_t word[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const uint32_t gv = g_iq3s_grid_pack[blk[2 + sg * 8 + g] | (((qh >> g) & 1u) << 8)];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int v = (int)((gv >> (8 * i)) & 0xFFu);         // odd magnitude 1..15
                if ((sgn >> (4 * g + i)) & 1u) v = -v;
                const int e = 4 * g + i;                      // element within the unit
                const int byte = e & 15, hi = e >> 4;
                const int c = (v - 1) >> 1;                   // code -8..7, value = 2c + 1
                const uint32_t code = hi ? ((uint32_t)c & 15u) : (uint32_t)(c + 8);   // high: two's complement; low: offset by 8
                word[byte >> 2] |= code << (8 * (byte & 3) + 4 * hi);
            }
        }
        uint8_t* d = dst_tile + (size_t)(b >> 3) * 4288;
        *reinterpret_cast<uint4*>(d + sg * 512 + lane * 16) = make_uint4(word[0], word[1], word[2], word[3]);
        if (sg == 0) {
            *reinterpret_cast<uint16_t*>(d + 4096 + lane * 2) = (uint16_t)ld_u16(blk);
            *reinterpret_cast<uint32_t*>(d + 4160 + lane * 4) = ld_u32_a2(blk + 106);
        }
    }
}

cudaError_t launch_pack(int type, const void* raw, void* out, int n_mats, int nrows, int ncols, int64_t raw_stride,
                        int64_t out_stride, cudaStream_t stream) {
    if (n_mats <= 0) return cudaSuccess;
    const int64_t n = (int64_t)nrows * (ncols / 32);
    const dim3 grid((unsigned)((n + 255) / 256), (unsigned)n_mats);
    switch (type) {
        case CHIMERE_TYPE_Q4_0: pack_kernel<CHIMERE_TYPE_Q4_0><<<grid, 256, 0, stream>>>((const uint8_t*)raw, (uint8_t*)out, nrows, ncols, raw_stride, out_stride); break;
        case CHIMERE_TYPE_Q8_0: pack_kernel<CHIMERE_TYPE_Q8_0><<<grid, 256, 0, stream>>>((const uint8_t*)raw, (uint8_t*)out, nrows, ncols, raw_stride, out_stride); break;
        case CHIMERE_TYPE_IQ3_S: pack_kernel<CHIMERE_TYPE_IQ3_S><<<grid, 256, 0, stream>>>((const uint8_t*)raw, (uint8_t*)out, nrows, ncols, raw_stride, out_stride); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// Parity tap on the packed form: integer block dots of `nrows` rows against one Q8_1 row.
template <int TYPE>
__global__ void block_sumi_tiled_kernel(const uint8_t* packed, const uint8_t* xq8, int32_t* out, int ncols, int nrows) {
    using TT = Tiled<TYPE>;
    const int nb = ncols >> 5;
    const int ngroups = (nb + kGroupUnits - 1) / kGroupUnits;
    const int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;  // one warp per (tile, group)
    const int lane = threadIdx.x & 31;
    if (gw >= (int64_t)(nrows / 32) * ngroups) return;
    const int tile = (int)(gw / ngroups), grp = (int)(gw % ngroups);
    const int nu = min(kGroupUnits, nb - grp * kGroupUnits);
    typename TT::Regs r;
    TT::load(packed + (size_t)tile * TT::tile_bytes(ncols), grp, lane, nu, r);
#pragma unroll
    for (int u = 0; u < kGroupUnits; ++u) {
        if (u < nu) {
            int w[8];
            TT::decode(r, u, w);
            const int b = grp * kGroupUnits + u;
            const int* qw = reinterpret_cast<const int*>(xq8 + (size_t)b * kQ81Bytes + 4);
            const uint4 q0 = make_uint4((uint32_t)qw[0], (uint32_t)qw[1], (uint32_t)qw[2], (uint32_t)qw[3]);
            const uint4 q1 = make_uint4((uint32_t)qw[4], (uint32_t)qw[5], (uint32_t)qw[6], (uint32_t)qw[7]);
            out[(size_t)(tile * 32 + lane) * nb + b] = unit_dot<TYPE>(w, q0, q1, TT::correction(sum16(q0), sum16(q1)), r, u);
        }
    }
}

cudaError_t launch_block_sumi_tiled(int type, const void* packed, const void* xq8, int32_t* sumi, int ncols, int nrows,
                                    cudaStream_t stream) {
    const int nb = ncols / 32;
    auto run = [&](auto tag) {
        constexpr int TYPE = decltype(tag)::value;
        const int ngroups = (nb + kGroupUnits - 1) / kGroupUnits;
        const int64_t warps = (int64_t)(nrows / 32) * ngroups;
        if (warps > 0)
            block_sumi_tiled_kernel<TYPE><<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>((const uint8_t*)packed, (const uint8_t*)xq8, sumi, ncols, nrows);
    };
    switch (type) {
        case CHIMERE_TYPE_Q4_0: run(std::integral_constant<int, CHIMERE_TYPE_Q4_0>{}); break;
        case CHIMERE_TYPE_Q8_0: run(std::integral_constant<int, CHIMERE_TYPE_Q8_0>{}); break;
        case CHIMERE_TYPE_IQ3_S: run(std::integral_constant<int, CHIMERE_TYPE_IQ3_S>{}); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace chimere
