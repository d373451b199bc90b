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
//   Q8_0  -> per (tile, unit): 2 x 512 B int8 + 64 B f16 scales              (1088 B, as before)
//   IQ3_S -> per (tile, super-block of 8 units): 8 x 512 B 4-bit codes + 64 B f16 d +
//            128 B sub-block scale nibbles                                   (4288 B, was 3520 B)
//            Each IQ3_S weight is +-(1,3,..,15): sixteen values, i.e. exactly four bits: code s in
//            -8..7 stands for 2s + 1.  The expansion is lossless: integer block dots are
//            identical to the codebook form.
//
// Within a unit, byte j of a row's 16 bytes holds element j in its low nibble and element j+16
// in its high nibble (the Q4_0 convention), so words 0..3 pair with Q8_1 words 0..3 (low) and
// 4..7 (high).  The two nibbles are stored differently so that neither needs a shift before dp4a:
//   low nibble  = code + 8, unsigned 0..15 (for Q4_0 that is ggml's own nibble): x & 0x0F0F0F0F is an
//                 unsigned byte vector;  sum(code * q) = sum(nibble * q) - 8 * sum(q)
//   high nibble = code in two's complement: x & 0xF0F0F0F0 is the signed byte vector 16 * code
// The terms in sum(q) depend on the activations only; whoever stages a token's Q8_1 block computes
// them once per (token, unit) as the "correction" word that a dp4a accumulator starts from.
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

// dp4a with unsigned bytes in a and signed bytes in b
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}

// Per type, besides the loads:
//   decode(r, u, w)        w[0..3]: low-nibble words (elements 0..15), w[4..7]: high-nibble words (16..31)
//   kLowUnsigned           w[0..3] are unsigned byte vectors (dp4a_us), else signed
//   kCorrLow               the correction word starts the low accumulator (else the high one)
//   correction(s_lo, s_hi) from the sums of a token's quants 0..15 and 16..31 of the unit
//   finish(sl, sh, r, u)   the integer block dot from the two accumulators
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
    static constexpr bool kLowUnsigned = true, kCorrLow = true;
    __device__ static __forceinline__ void decode(const Regs& r, int u, int (&w)[8]) {
        const uint32_t x[4] = {r.v[u].x, r.v[u].y, r.v[u].z, r.v[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { w[j] = (int)(x[j] & 0x0F0F0F0Fu); w[4 + j] = (int)(x[j] & 0xF0F0F0F0u); }
    }
    __host__ __device__ static __forceinline__ int correction(int s_lo, int) { return -8 * s_lo; }
    __device__ static __forceinline__ int finish(int sl, int sh, const Regs&, int) { return sl + (sh >> 4); }
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
    static constexpr bool kLowUnsigned = true, kCorrLow = false;
    __device__ static __forceinline__ void decode(const Regs& r, int u, int (&w)[8]) {
        const uint32_t x[4] = {r.v[u].x, r.v[u].y, r.v[u].z, r.v[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { w[j] = (int)(x[j] & 0x0F0F0F0Fu); w[4 + j] = (int)(x[j] & 0xF0F0F0F0u); }
    }
    // weight = 2*code + 1.  Low half: sum((2n - 15) q) = 2*sl - 15*s_lo; high half: sum((2c + 1) q) = sh/8 + s_hi with
    // sh = sum(16c * q).  The correction 8*(s_hi - 15*s_lo) starts sh, so the block dot is 2*sl + (sh >> 3), exactly;
    // times the sub-block factor 1 + 2*scale (chimere_kernels.cu:860).
    __host__ __device__ static __forceinline__ int correction(int s_lo, int s_hi) { return 8 * (s_hi - 15 * s_lo); }
    __device__ static __forceinline__ int finish(int sl, int sh, const Regs& r, int u) {
        return (2 * sl + (sh >> 3)) * (int)(1u + 2u * ((r.sc >> (4 * u)) & 15u));
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
    static constexpr bool kLowUnsigned = false, kCorrLow = true;
    __host__ __device__ static __forceinline__ int correction(int, int) { return 0; }
    __device__ static __forceinline__ int finish(int sl, int sh, const Regs&, int) { return sl + sh; }
    __device__ static __forceinline__ float dscale(const Regs& r, int u) { return h2f(r.d[u]); }
};

// One unit against one token: q0 / q1 = the token's quants 0..15 / 16..31 of the unit, corr = its correction word.
template <int TYPE>
__device__ __forceinline__ int unit_dot(const int (&w)[8], const uint4& q0, const uint4& q1, int corr, const typename Tiled<TYPE>::Regs& r, int u) {
    using TT = Tiled<TYPE>;
    int sl = TT::kCorrLow ? corr : 0, sh = TT::kCorrLow ? 0 : corr;   // two independent chains
    if (TT::kLowUnsigned) {
        sl = dp4a_us((uint32_t)w[0], (int)q0.x, sl); sh = __dp4a(w[4], (int)q1.x, sh);
        sl = dp4a_us((uint32_t)w[1], (int)q0.y, sl); sh = __dp4a(w[5], (int)q1.y, sh);
        sl = dp4a_us((uint32_t)w[2], (int)q0.z, sl); sh = __dp4a(w[6], (int)q1.z, sh);
        sl = dp4a_us((uint32_t)w[3], (int)q0.w, sl); sh = __dp4a(w[7], (int)q1.w, sh);
    } else {
        sl = __dp4a(w[0], (int)q0.x, sl); sh = __dp4a(w[4], (int)q1.x, sh);
        sl = __dp4a(w[1], (int)q0.y, sl); sh = __dp4a(w[5], (int)q1.y, sh);
        sl = __dp4a(w[2], (int)q0.z, sl); sh = __dp4a(w[6], (int)q1.z, sh);
        sl = __dp4a(w[3], (int)q0.w, sl); sh = __dp4a(w[7], (int)q1.w, sh);
    }
    return TT::finish(sl, sh, r, u);
}
// sums of sixteen int8 held in a uint4
__device__ __forceinline__ int sum16(const uint4& x) {
    int s = __dp4a((int)x.x, 0x01010101, 0);
    s = __dp4a((int)x.y, 0x01010101, s);
    s = __dp4a((int)x.z, 0x01010101, s);
    return __dp4a((int)x.w, 0x01010101, s);
}

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
