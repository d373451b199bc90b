// common.cuh -- device helpers shared by the MoE kernels (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/chimere_b200_moe.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "this library is written for sm_100a only"
#endif

namespace chimere {

constexpr int kQ81Bytes = 36;
constexpr int kMaxGroupTokens = 8;   // tokens one GEMV work entry carries
constexpr int kSharedGroupTokens = 2;  // ... for the shared expert (every token uses it): smaller entries balance the grid
// Decode-size batches give every token its own shared-expert entry: the kernels stage one token per pass there, and
// a second pass in the same CTA is a longer chain than a second CTA reading the shared matrices from L2.
__host__ __device__ inline int shared_group_tokens(int T) { return T <= 8 ? 1 : kSharedGroupTokens; }
constexpr int kMaxTopK = 8;
constexpr int kMaxExperts = 256;

// Work list the routing kernel leaves for the grouped GEMV kernels: word 0 = number of entries, word 1 = routed
// entries, word 2 = shared-expert entries; entries start at word 4, kListEntry words each:
// { expert id (-1 = shared expert), start, m, 0, pair row of token 0 .. 7 }.  Routed entry: pairs
// perm[start .. start+m) (the pair rows repeat them so a kernel needs no second look-up); shared entry:
// tokens start .. start+m, pair rows T*top_k + token.  The shared expert's entries come first: they carry the
// most tokens and should start early.
constexpr int kListHeader = 4;
constexpr int kListEntry = 12;

// status bits a kernel may raise in the workspace status word
constexpr int kStatusWaitTimeout = 1;

__device__ __forceinline__ float h2f(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }
__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }
// 32-bit load from an address that is only 2-byte aligned (ggml blocks are 2-byte aligned).
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t* p) { return ld_u16(p) | (ld_u16(p + 2) << 16); }

// PTX prmt in its default mode: selector nibble bit 3 replicates the sign bit of the chosen byte.
// (__byte_perm documents only the low three selector bits, so the instruction is spelled out.)
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier + bulk async copy (global -> shared), no multicast -------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cta(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// dst and src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Bounded wait on phase `parity`; false if the limit ran out (caller raises a status bit).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok = 0;
    for (int it = 0; it < (1 << 22) && !ok; ++it) {
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    }
    return ok != 0;
}

// ---- two fp32 lanes in one 64-bit register (sm_100 has two-wide fp32 add / mul / fma, each lane rounded like the scalar form) ----
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi)); return r; }
__device__ __forceinline__ uint64_t pack2f(float lo, float hi) { return pack2(__float_as_uint(lo), __float_as_uint(hi)); }
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) { uint64_t d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d; }
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) { uint64_t d; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b)); return d; }

// Counter increment that publishes this thread's (and, behind a CTA barrier, its CTA's) earlier writes and makes the
// writes published by the other arrivals visible: release and acquire in the one instruction, instead of a fence on
// either side of a relaxed atomic.  Returns the old value.
__device__ __forceinline__ int atom_add_acq_rel_gpu(int* p, int v) {
    int old;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}

// ---- programmatic dependent launch ---------------------------------------------------------
// A kernel launched with the programmatic-serialization attribute may start while its predecessor in the
// stream still runs; griddep_wait() blocks until that predecessor has completed and its writes are visible
// (a no-op for a normally launched kernel).  griddep_launch() lets the successor's CTAs start once every CTA
// of this grid has called it or exited.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- per-type decode of one 32-weight unit into eight int8x4 words -----------------------
// Unit b of a row = 32 consecutive weights (a Q4_0 / Q8_0 block, or sub-block b%8 of IQ3_S
// super-block b/8).  load() returns the signed int8 weights packed four per word such that
// finish(sum_g dp4a(w[g], q8word[g]), mul) is the integer block dot (Q4_0 words carry 16x the weight,
// IQ3_S units a per-sub-block multiplier `mul`).
template <int TYPE> struct Unit;

template <> struct Unit<CHIMERE_TYPE_Q8_0> {
    static constexpr int kBlockBytes = 34, kBlockElems = 32;
    __device__ static __forceinline__ int64_t row_bytes(int ncols) { return (int64_t)(ncols >> 5) * 34; }
    __device__ static __forceinline__ void load(const uint8_t* row, int b, const uint32_t*, int (&w)[8], float& dw, int& mul) {
        const uint8_t* blk = row + b * 34;
        dw = h2f(ld_u16(blk));
        mul = 1;
#pragma unroll
        for (int g = 0; g < 8; ++g) w[g] = (int)ld_u32_a2(blk + 2 + 4 * g);
    }
    __device__ static __forceinline__ int finish(int sumi, int mul) { (void)mul; return sumi; }
};

template <> struct Unit<CHIMERE_TYPE_Q4_0> {
    static constexpr int kBlockBytes = 18, kBlockElems = 32;
    __device__ static __forceinline__ int64_t row_bytes(int ncols) { return (int64_t)(ncols >> 5) * 18; }
    // byte = ((nibble ^ 8) << 4) read as int8 = 16 * (nibble - 8); the dot comes out times 16.
    __device__ static __forceinline__ void load(const uint8_t* row, int b, const uint32_t*, int (&w)[8], float& dw, int& mul) {
        const uint8_t* blk = row + b * 18;
        dw = h2f(ld_u16(blk));
        mul = 1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t t = ld_u32_a2(blk + 2 + 4 * j) ^ 0x88888888u;
            w[j] = (int)((t << 4) & 0xF0F0F0F0u);   // low nibbles: elements 4j .. 4j+3
            w[4 + j] = (int)(t & 0xF0F0F0F0u);      // high nibbles: elements 16+4j ..
        }
    }
    __device__ static __forceinline__ int finish(int sumi, int mul) { (void)mul; return sumi >> 4; }
};

template <> struct Unit<CHIMERE_TYPE_IQ3_S> {
    static constexpr int kBlockBytes = 110, kBlockElems = 256;
    __device__ static __forceinline__ int64_t row_bytes(int ncols) { return (int64_t)(ncols >> 8) * 110; }
    // Layout of the 110-byte super-block: d f16 @0, qs[64] @2, qh[8] @66, signs[32] @74, scales[4] @106.
    __device__ static __forceinline__ void load(const uint8_t* row, int b, const uint32_t* grid, int (&w)[8], float& dw, int& mul) {
        const uint8_t* blk = row + (b >> 3) * 110;
        const int sg = b & 7;
        dw = h2f(ld_u16(blk));
        const uint32_t q0 = ld_u32_a2(blk + 2 + sg * 8), q1 = ld_u32_a2(blk + 6 + sg * 8);
        const uint32_t qh = blk[66 + sg];
        const uint32_t sgn = ld_u32_a2(blk + 74 + sg * 4);
        const uint32_t scb = blk[106 + (sg >> 1)];
        mul = 1 + 2 * (int)((scb >> ((sg & 1) * 4)) & 15u);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const uint32_t qsb = ((g < 4 ? q0 : q1) >> (8 * (g & 3))) & 0xFFu;
            const uint32_t gv = grid[qsb | (((qh >> g) & 1u) << 8)];
            // 4 sign bits -> bit 7 of each byte -> 0xFF/0x00 byte mask; -m = (m ^ 0xFF) + 1 never
            // carries out of its byte because every magnitude is >= 1.
            const uint32_t t7 = (((sgn >> (4 * g)) & 15u) * 0x10204080u) & 0x80808080u;
            const uint32_t mask = prmt(t7, 0u, 0xBA98u);
            w[g] = (int)((gv ^ mask) + (t7 >> 7));
        }
    }
    __device__ static __forceinline__ int finish(int sumi, int mul) { return sumi * mul; }
};

template <int TYPE>
__device__ __forceinline__ int unit_sumi(const int (&w)[8], int mul, const int* q8words) {
    int s = 0;
#pragma unroll
    for (int g = 0; g < 8; ++g) s = __dp4a(w[g], q8words[g], s);
    return Unit<TYPE>::finish(s, mul);
}

// Sigmoid and SiLU exactly as the reference spells them (chimere_kernels.cu:1545, scratch_pool.rs:272).
__device__ __forceinline__ float sigmoid_ref(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float silu_mul_ref(float g, float u) { float s = g / (1.0f + expf(-g)); return s * u; }

}  // namespace chimere
