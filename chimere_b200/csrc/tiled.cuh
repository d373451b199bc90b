// tiled.cuh -- the "tiled32" weight layout and its in-register decode.
//
// ggml blocks are 2-byte aligned records with the scale in front (Q4_0 18 B, Q8_0 34 B, IQ3_S
// 110 B), which forces narrow loads and, for IQ3_S, a codebook lookup plus sign fix-up per four
// weights.  chimere_b200_moe_pack rewrites every matrix once, at load time, into a layout made
// for one warp = 32 consecutive rows, lane = row:
//
//   rows are grouped in tiles of 32; within a tile the data of 32-weight unit b of all 32 rows
//   is contiguous, 16 bytes per row, so a warp-wide 128-bit load is one contiguous 512-byte
//   read and every lane receives whole units of its own row in registers.
//
//   Q4_0  -> per (tile, unit): 512 B nibbles + 64 B f16 scales               (576 B, as before)
//            nibble stored as (n - 8) in two's complement: byte (s << 4) = 16 * (n - 8).
//   Q8_0  -> per (tile, unit): 2 x 512 B int8 + 64 B f16 scales              (1088 B, as before)
//   IQ3_S -> per (tile, super-block of 8 units): 8 x 512 B signed 4-bit codes + 64 B f16 d +
//            128 B sub-block scale nibbles                                   (4288 B, was 3520 B)
//            Each IQ3_S weight is +-(1,3,..,15): sixteen values, i.e. exactly four bits.  Code s
//            (two's complement nibble) stands for 2s + 1; byte (s << 4) | 8 = 8 * (2s + 1).
//            The expansion is lossless: integer block dots are identical to the codebook form.
//
// Within a unit, byte j of a row's 16 bytes holds element j in its low nibble and element j+16
// in its high nibble (the Q4_0 convention), so words 0..3 pair with Q8_1 words 0..3 (low) and
// 4..7 (high).
#pragma once
#include "common.cuh"

namespace chimere {

// Weight loads: read-only, streamed once, so they bypass L1 allocation.
__device__ __forceinline__ uint4 ldg128(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_u16(const uint8_t* p) { return __ldg(reinterpret_cast<const uint16_t*>(p)); }
__device__ __forceinline__ uint32_t ldg_u32(const uint8_t* p) { return __ldg(reinterpret_cast<const uint32_t*>(p)); }
__device__ __forceinline__ void prefetch_l2(const uint8_t* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// Shared-memory loads by 32-bit shared address.
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}

// A "group" is kGroupUnits = 4 consecutive units of the 32 rows of a tile: what one lane decodes
// at a time.  kChunkBytes is the smallest contiguous piece a tile may be cut into when it is
// streamed in slabs (an IQ3_S super-block keeps its scales behind its eight units).
constexpr int kGroupUnits = 4;

template <int TYPE> struct Tiled;

template <> struct Tiled<CHIMERE_TYPE_Q4_0> {
    static constexpr int kUnitBytes = 576, kChunkBytes = 4 * 576, kGroupsPerChunk = 1;
    static constexpr bool kGroupScale = false;   // one scale per unit
    struct Regs { uint4 v[4]; uint32_t d[4]; };
    __host__ __device__ static int64_t tile_bytes(int ncols) { return (int64_t)(ncols / 32) * kUnitBytes; }
    __device__ static __forceinline__ void load(const uint8_t* tile, int grp, int lane, int nu, Regs& r) {
        const uint8_t* g = tile + (size_t)grp * (kGroupUnits * kUnitBytes);
#pragma unroll
        for (int u = 0; u < kGroupUnits; ++u)
            if (u < nu) { r.v[u] = ldg128(g + u * kUnitBytes + lane * 16); r.d[u] = ldg_u16(g + u * kUnitBytes + 512 + lane * 2); }
    }
    __device__ static __forceinline__ void prefetch(const uint8_t* tile, int grp, int lane, int nu) {
        const uint8_t* g = tile + (size_t)grp * (kGroupUnits * kUnitBytes);
#pragma unroll
        for (int u = 0; u < kGroupUnits; ++u)
            if (u < nu) prefetch_l2(g + u * kUnitBytes + lane * 16);
    }
    // the same group from a copy of the tile in shared memory (shared address `tile`)
    __device__ static __forceinline__ void loads(uint32_t tile, int grp, int lane, int nu, Regs& r) {
        const uint32_t g = tile + (uint32_t)grp * (kGroupUnits * kUnitBytes);
#pragma unroll
        for (int u = 0; u < kGroupUnits; ++u)
            if (u < nu) { r.v[u] = lds128(g + u * kUnitBytes + lane * 16); r.d[u] = lds16(g + u * kUnitBytes + 512 + lane * 2); }
    }
    static constexpr int kChunkUnits = 4;
    __host__ __device__ static uint32_t unit_offset(int u) { return (uint32_t)u * kUnitBytes; }   // u: a chunk boundary or the row's end
    __device__ static __forceinline__ void decode(const Regs& r, int u, int (&w)[8]) {
        const uint32_t x[4] = {r.v[u].x, r.v[u].y, r.v[u].z, r.v[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { w[j] = (int)((x[j] << 4) & 0xF0F0F0F0u); w[4 + j] = (int)(x[j] & 0xF0F0F0F0u); }
    }
    __device__ static __forceinline__ int finish(int s, const Regs&, int, int) { return s >> 4; }
    __device__ static __forceinline__ float dscale(const Regs& r, int u) { return h2f(r.d[u]); }
};

template <> struct Tiled<CHIMERE_TYPE_IQ3_S> {
    static constexpr int kSuperBytes = 4288, kChunkBytes = 4288, kGroupsPerChunk = 2;
    static constexpr bool kGroupScale = true;    // one f16 d per super-block: the same for the four units of a group
    struct Regs { uint4 v[4]; uint32_t d; uint32_t sc; };
    __host__ __device__ static int64_t tile_bytes(int ncols) { return (int64_t)(ncols / 256) * kSuperBytes; }
    __device__ static __forceinline__ void load(const uint8_t* tile, int grp, int lane, int nu, Regs& r) {
        const uint8_t* g = tile + (size_t)(grp >> 1) * kSuperBytes;
        const int u0 = (grp & 1) * 4;
#pragma unroll
        for (int u = 0; u < kGroupUnits; ++u)
            if (u < nu) r.v[u] = ldg128(g + (u0 + u) * 512 + lane * 16);
        r.d = ldg_u16(g + 4096 + lane * 2);
        r.sc = ldg_u32(g + 4160 + lane * 4) >> (16 * (grp & 1));   // this half's four scale nibbles
    }
    __device__ static __forceinline__ void prefetch(const uint8_t* tile, int grp, int lane, int nu) {
        const uint8_t* g = tile + (size_t)(grp >> 1) * kSuperBytes;
        const int u0 = (grp & 1) * 4;
#pragma unroll
        for (int u = 0; u < kGroupUnits; ++u)
            if (u < nu) prefetch_l2(g + (u0 + u) * 512 + lane * 16);
    }
    __device__ static __forceinline__ void loads(uint32_t tile, int grp, int lane, int nu, Regs& r) {
        const uint32_t g = tile + (uint32_t)(grp >> 1) * kSuperBytes;
        const int u0 = (grp & 1) * 4;
#pragma unroll
        for (int u = 0; u < kGroupUnits; ++u)
            if (u < nu) r.v[u] = lds128(g + (u0 + u) * 512 + lane * 16);
        r.d = lds16(g + 4096 + lane * 2);
        r.sc = lds32(g + 4160 + lane * 4) >> (16 * (grp & 1));
    }
    static constexpr int kChunkUnits = 8;
    __host__ __device__ static uint32_t unit_offset(int u) { return (uint32_t)(u >> 3) * kSuperBytes; }
    __device__ static __forceinline__ void decode(const Regs& r, int u, int (&w)[8]) {
        const uint32_t x[4] = {r.v[u].x, r.v[u].y, r.v[u].z, r.v[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            w[j] = (int)(((x[j] << 4) & 0xF0F0F0F0u) | 0x08080808u);
            w[4 + j] = (int)((x[j] & 0xF0F0F0F0u) | 0x08080808u);
        }
    }
    // dp4a result = 8 * sum(+-magnitude * q); times the sub-block factor 1 + 2*scale (chimere_kernels.cu:860)
    __device__ static __forceinline__ int finish(int s, const Regs& r, int u, int) {
        return (s >> 3) * (int)(1u + 2u * ((r.sc >> (4 * u)) & 15u));
    }
    __device__ static __forceinline__ float dscale(const Regs& r, int) { return h2f(r.d); }
};

template <> struct Tiled<CHIMERE_TYPE_Q8_0> {
    static constexpr int kUnitBytes = 1088, kChunkBytes = 4 * 1088, kGroupsPerChunk = 1;
    static constexpr bool kGroupScale = false;
    struct Regs { uint4 v[8]; uint32_t d[4]; };
    __host__ __device__ static int64_t tile_bytes(int ncols) { return (int64_t)(ncols / 32) * kUnitBytes; }
    __device__ static __forceinline__ void load(const uint8_t* tile, int grp, int lane, int nu, Regs& r) {
        const uint8_t* g = tile + (size_t)grp * (kGroupUnits * kUnitBytes);
#pragma unroll
        for (int u = 0; u < kGroupUnits; ++u)
            if (u < nu) {
                r.v[2 * u] = ldg128(g + u * kUnitBytes + lane * 16);
                r.v[2 * u + 1] = ldg128(g + u * kUnitBytes + 512 + lane * 16);
                r.d[u] = ldg_u16(g + u * kUnitBytes + 1024 + lane * 2);
            }
    }
    __device__ static __forceinline__ void prefetch(const uint8_t* tile, int grp, int lane, int nu) {
        const uint8_t* g = tile + (size_t)grp * (kGroupUnits * kUnitBytes);
#pragma unroll
        for (int u = 0; u < kGroupUnits; ++u)
            if (u < nu) { prefetch_l2(g + u * kUnitBytes + lane * 16); prefetch_l2(g + u * kUnitBytes + 512 + lane * 16); }
    }
    __device__ static __forceinline__ void loads(uint32_t tile, int grp, int lane, int nu, Regs& r) {
        const uint32_t g = tile + (uint32_t)grp * (kGroupUnits * kUnitBytes);
#pragma unroll
        for (int u = 0; u < kGroupUnits; ++u)
            if (u < nu) {
                r.v[2 * u] = lds128(g + u * kUnitBytes + lane * 16);
                r.v[2 * u + 1] = lds128(g + u * kUnitBytes + 512 + lane * 16);
                r.d[u] = lds16(g + u * kUnitBytes + 1024 + lane * 2);
            }
    }
    static constexpr int kChunkUnits = 4;
    __host__ __device__ static uint32_t unit_offset(int u) { return (uint32_t)u * kUnitBytes; }
    __device__ static __forceinline__ void decode(const Regs& r, int u, int (&w)[8]) {
        w[0] = (int)r.v[2 * u].x; w[1] = (int)r.v[2 * u].y; w[2] = (int)r.v[2 * u].z; w[3] = (int)r.v[2 * u].w;
        w[4] = (int)r.v[2 * u + 1].x; w[5] = (int)r.v[2 * u + 1].y; w[6] = (int)r.v[2 * u + 1].z; w[7] = (int)r.v[2 * u + 1].w;
    }
    __device__ static __forceinline__ int finish(int s, const Regs&, int, int) { return s; }
    __device__ static __forceinline__ float dscale(const Regs& r, int u) { return h2f(r.d[u]); }
};

// bytes of one matrix [nrows][ncols] in tiled32 form (nrows a multiple of 32)
__host__ __device__ inline int64_t tiled_matrix_bytes(int type, int nrows, int ncols) {
    const int64_t tiles = nrows / 32;
    switch (type) {
        case CHIMERE_TYPE_Q4_0: return tiles * Tiled<CHIMERE_TYPE_Q4_0>::tile_bytes(ncols);
        case CHIMERE_TYPE_Q8_0: return tiles * Tiled<CHIMERE_TYPE_Q8_0>::tile_bytes(ncols);
        case CHIMERE_TYPE_IQ3_S: return tiles * Tiled<CHIMERE_TYPE_IQ3_S>::tile_bytes(ncols);
        default: return -1;
    }
}

}  // namespace chimere
