// gemv.cu -- memory-bound grouped GEMV kernels of the decode path, on raw ggml blocks.
//
//   gate_up_kernel : per work entry (one expert, up to 8 tokens) and 32-row tile: gate and up rows
//                    against the tokens' Q8_1 input, SwiGLU (or relu^2), Q8_1 of the 32 results.
//                    Replaces moe_ffn.rs:1206-1323 (batched gate GEMV, batched up GEMV,
//                    silu_mul, batched Q8_1) and the shared expert's first half (:1597-1700).
//   down_kernel    : per work entry and row tile of H: down rows against the entry's Q8_1
//                    intermediates; the CTA that completes a token's last contribution for a row
//                    tile adds them up in slot order with the routing weights and the sigmoid-gated
//                    shared expert.  Replaces moe_ffn.rs:1325-1384 and :1700-1766.
//   mmvq_kernel    : the same tile code behind the legacy operator entries
//                    (ffi/ggml_cuda_gemv.cu:105-116, 243-279).
//
// A CTA first asks the copy engine for its whole weight tile (cp.async.bulk, 8-row pieces, one
// mbarrier each), stages the activations as an int8 plane + f32 scale plane while the weights
// are in flight, and every warp starts on a piece as soon as that piece has landed.
#include "common.cuh"
#include "kernels.h"

namespace chimere {

static __device__ const uint32_t g_iq3s_grid[512] = {
#include "iq3s_grid.inc"
};

constexpr int kThreads = 256;
constexpr int kPieceRows = 8;

__device__ __forceinline__ uint32_t align16(uint32_t v) { return (v + 15u) & ~15u; }

// Copy `bytes` from global `src` to shared `dst` and signal `bar` (initialised with count 1).
// Bulk copy when source and size are 16-byte aligned, otherwise 2-byte loads by all threads.
// Must be called by every thread of the CTA (it synchronises on the slow path).
__device__ __forceinline__ void stage_piece(uint8_t* dst, const uint8_t* src, uint32_t bytes, uint64_t* bar, int tid) {
    const bool fast = (((uintptr_t)src | bytes) & 15u) == 0;
    if (fast) {
        if (tid == 0) {
            mbar_expect_tx(bar, bytes);
            bulk_g2s(dst, src, bytes, bar);
        }
    } else {
        for (uint32_t i = 2u * tid; i < bytes; i += 2u * kThreads)
            *reinterpret_cast<uint16_t*>(dst + i) = *reinterpret_cast<const uint16_t*>(src + i);
        __syncthreads();
        if (tid == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
    }
}

// Q8_1 rows (36-byte blocks) -> int8 plane aq[i][ncols] and f32 scale plane ad[i][nb].
__device__ __forceinline__ void stage_q8(const uint8_t* const* rows, int m, int nb, int ncols, int8_t* aq, float* ad, int tid) {
    for (int i = 0; i < m; ++i) {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(rows[i]);  // 36-byte blocks: 9 words
        uint32_t* dq = reinterpret_cast<uint32_t*>(aq + (size_t)i * ncols);
        for (int wd = tid; wd < nb * 9; wd += kThreads) {
            const int b = wd / 9, r = wd - b * 9;
            const uint32_t v = __ldcg(src + wd);
            if (r == 0) ad[i * nb + b] = h2f(v & 0xFFFFu);
            else dq[b * 8 + (r - 1)] = v;
        }
    }
}

// One row against up to 8 tokens: lane l8 of the row's 8 lanes takes units l8, l8+8, ...
template <int TYPE>
__device__ __forceinline__ void row_dot(const uint8_t* rowp, int l8, int nb, int ncols, const int8_t* aq, const float* ad,
                                        int m, const uint32_t* grid, float (&acc)[kMaxGroupTokens]) {
    for (int b = l8; b < nb; b += 8) {
        int w[8], mul;
        float dw;
        Unit<TYPE>::load(rowp, b, grid, w, dw, mul);
#pragma unroll
        for (int i = 0; i < kMaxGroupTokens; ++i) {
            if (i < m) {
                const int4* q = reinterpret_cast<const int4*>(aq + (size_t)i * ncols + b * 32);
                const int4 q0 = q[0], q1 = q[1];
                const int qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                const int s = unit_sumi<TYPE>(w, mul, qw);
                acc[i] = fmaf(dw * ad[i * nb + b], (float)s, acc[i]);
            }
        }
    }
}

__device__ __forceinline__ void reduce8(float (&acc)[kMaxGroupTokens], int m) {
#pragma unroll
    for (int i = 0; i < kMaxGroupTokens; ++i) {
        if (i < m) {
            acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 1);
            acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 2);
            acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 4);
        }
    }
}

struct SmemPlan {
    uint32_t grid, bars, aq, ad, misc, w0, w1, total;
};
__host__ __device__ inline SmemPlan plan_smem(int ncols, int tile_rows, int64_t row_bytes, bool dual) {
    SmemPlan s;
    uint32_t o = 0;
    s.grid = o; o += 2048;
    s.bars = o; o += 64;
    s.aq = o; o += (uint32_t)kMaxGroupTokens * ncols;
    s.ad = o; o += (uint32_t)kMaxGroupTokens * (ncols / 32) * 4;
    s.misc = o; o += kMaxGroupTokens * 32 * 4 + 64;
    o = (o + 127u) & ~127u;
    s.w0 = o; o += (uint32_t)(tile_rows * row_bytes + 16);
    o = (o + 127u) & ~127u;
    s.w1 = o; if (dual) o += (uint32_t)(tile_rows * row_bytes + 16);
    s.total = o;
    return s;
}

// ------------------------------------------------------------------ gate / up stage --------
// grid = (ceil(max(F, F_s) / 32), max entries).  An instance handles the entries whose weight
// type is TYPE and returns at once for the others.
template <int TYPE>
__global__ void __launch_bounds__(kThreads) gate_up_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ const uint8_t* s_rows[kMaxGroupTokens];
    __shared__ int s_out_row[kMaxGroupTokens];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_entries = __ldcg(p.group_list);
    if ((int)blockIdx.y >= n_entries) return;
    const int* ent = p.group_list + kListHeader + kListEntry * blockIdx.y;
    const int expert = __ldcg(ent), start = __ldcg(ent + 1), m = __ldcg(ent + 2);
    const bool shared = expert < 0;
    if ((shared ? p.type_shared : p.type_routed) != TYPE) return;
    const int nrows = shared ? p.nrows_shared : p.nrows_routed;
    const int r0 = blockIdx.x * 32;
    if (r0 >= nrows) return;
    const bool dual = p.act == CHIMERE_ACT_SWIGLU;
    const int ncols = p.H, nb = ncols >> 5;
    const int64_t rb = Unit<TYPE>::row_bytes(ncols);
    const SmemPlan sp = plan_smem(ncols, 32, rb, dual);
    uint32_t* grid_s = reinterpret_cast<uint32_t*>(smem + sp.grid);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + sp.bars);
    int8_t* aq = reinterpret_cast<int8_t*>(smem + sp.aq);
    float* ad = reinterpret_cast<float*>(smem + sp.ad);
    float* inter = reinterpret_cast<float*>(smem + sp.misc);  // [8][32]
    uint8_t* wa = smem + sp.w0;
    uint8_t* wb = smem + sp.w1;

    const uint8_t* src_a = (shared ? p.sh_b : p.w_b + (size_t)expert * p.stride_b) + (size_t)r0 * rb;          // up
    const uint8_t* src_b = dual ? (shared ? p.sh_a : p.w_a + (size_t)expert * p.stride_a) + (size_t)r0 * rb : nullptr;  // gate

    if (tid == 0) {
        for (int c = 0; c < 4; ++c) mbar_init(bars + c, dual ? 2 : 1);
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t piece = (uint32_t)(kPieceRows * rb);
    for (int c = 0; c < 4; ++c) {
        stage_piece(wa + c * piece, src_a + (size_t)c * piece, piece, bars + c, tid);
        if (dual) stage_piece(wb + c * piece, src_b + (size_t)c * piece, piece, bars + c, tid);
    }
    if (TYPE == CHIMERE_TYPE_IQ3_S)
        for (int i = tid; i < 512; i += kThreads) grid_s[i] = g_iq3s_grid[i];

    // Q8_1 input rows of the entry's tokens
    if (tid < m) {
        int t, orow;
        if (shared) { t = start + tid; orow = p.T * p.top_k + t; }
        else { const int q = __ldcg(p.perm + start + tid); t = q / p.top_k; orow = q; }
        s_rows[tid] = p.in_q8 + (size_t)t * p.in_stride;
        s_out_row[tid] = orow;
    }
    __syncthreads();
    stage_q8(s_rows, m, nb, ncols, aq, ad, tid);
    __syncthreads();

    // rows 4*warp .. 4*warp+3 of the tile live in piece warp/2
    if (!mbar_wait(bars + (warp >> 1), 0)) atomicOr(p.status, kStatusWaitTimeout);
    const int row = 4 * warp + (lane >> 3), l8 = lane & 7;
    float au[kMaxGroupTokens], ag[kMaxGroupTokens];
#pragma unroll
    for (int i = 0; i < kMaxGroupTokens; ++i) { au[i] = 0.0f; ag[i] = 0.0f; }
    row_dot<TYPE>(wa + (size_t)row * rb, l8, nb, ncols, aq, ad, m, grid_s, au);
    if (dual) row_dot<TYPE>(wb + (size_t)row * rb, l8, nb, ncols, aq, ad, m, grid_s, ag);
    reduce8(au, m);
    if (dual) reduce8(ag, m);
    if (l8 == 0) {
#pragma unroll
        for (int i = 0; i < kMaxGroupTokens; ++i) {
            if (i < m) {
                float v;
                if (dual) v = silu_mul_ref(ag[i], au[i]);
                else { const float r = fmaxf(au[i], 0.0f); v = r * r; }
                inter[i * 32 + row] = v;
            }
        }
    }
    __syncthreads();
    // Q8_1 of the 32 results of each token (same rule as the input rows): warp i takes token i
    if (warp < m) {
        uint8_t* out = p.inter_q8 + (size_t)s_out_row[warp] * p.inter_stride + (size_t)blockIdx.x * kQ81Bytes;
        const float v = inter[warp * 32 + lane];
        float amax = fabsf(v), sum = v;
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
            sum += __shfl_xor_sync(0xffffffffu, sum, s);
        }
        const float d = amax / 127.0f;
        const int8_t q = (amax == 0.0f) ? (int8_t)0 : (int8_t)roundf(v / d);
        reinterpret_cast<int8_t*>(out)[4 + lane] = q;
        if (lane == 0) *reinterpret_cast<__half2*>(out) = __halves2half2(__float2half(d), __float2half(sum));
    }
}

// ------------------------------------------------------------------ down stage / plain -----
// PLAIN = false: work-list driven; writes pair_out rows and combines them per token.
// PLAIN = true : slot driven (legacy operator entries): blockIdx.y = slot, expert id from ids,
//                output y[slot][row].
struct PlainParams {
    const uint8_t* w; const uint8_t* xq8; float* y; const int* ids;
    int ncols, nrows; int64_t expert_stride, input_stride;
};

template <int TYPE, bool PLAIN>
__global__ void __launch_bounds__(kThreads) down_kernel(const GemvParams p, const PlainParams pp, int tile_rows) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ const uint8_t* s_rows[kMaxGroupTokens];
    __shared__ int s_out_row[kMaxGroupTokens];
    __shared__ int s_tok[kMaxGroupTokens];
    __shared__ int s_done[kMaxGroupTokens];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int expert, start, m, nrows, ncols;
    bool shared = false;
    if (PLAIN) {
        expert = pp.ids ? pp.ids[blockIdx.y] : 0; start = blockIdx.y; m = 1; nrows = pp.nrows; ncols = pp.ncols;
    } else {
        const int n_entries = __ldcg(p.group_list);
        if ((int)blockIdx.y >= n_entries) return;
        const int* ent = p.group_list + kListHeader + kListEntry * blockIdx.y;
        expert = __ldcg(ent); start = __ldcg(ent + 1); m = __ldcg(ent + 2);
        shared = expert < 0;
        if ((shared ? p.type_shared : p.type_routed) != TYPE) return;
        nrows = shared ? p.nrows_shared : p.nrows_routed;
        ncols = shared ? p.ncols_shared : p.ncols_routed;
    }
    const int r0 = blockIdx.x * tile_rows;
    if (r0 >= nrows) return;
    const int rows_here = min(tile_rows, nrows - r0);
    const int nb = ncols >> 5;
    const int64_t rb = Unit<TYPE>::row_bytes(ncols);
    const SmemPlan sp = plan_smem(ncols, tile_rows, rb, false);
    uint32_t* grid_s = reinterpret_cast<uint32_t*>(smem + sp.grid);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + sp.bars);
    int8_t* aq = reinterpret_cast<int8_t*>(smem + sp.aq);
    float* ad = reinterpret_cast<float*>(smem + sp.ad);
    uint8_t* wt = smem + sp.w0;

    const uint8_t* wsrc = PLAIN ? pp.w + (size_t)expert * pp.expert_stride
                                : (shared ? p.sh_a : p.w_a + (size_t)expert * p.stride_a);
    wsrc += (size_t)r0 * rb;
    const int npieces = (rows_here + kPieceRows - 1) / kPieceRows;
    if (tid == 0) {
        for (int c = 0; c < npieces; ++c) mbar_init(bars + c, 1);
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t piece = (uint32_t)(kPieceRows * rb);
    for (int c = 0; c < npieces; ++c) {
        const uint32_t bytes = (uint32_t)(min(kPieceRows, rows_here - c * kPieceRows) * rb);
        stage_piece(wt + c * piece, wsrc + (size_t)c * piece, bytes, bars + c, tid);
    }
    if (TYPE == CHIMERE_TYPE_IQ3_S)
        for (int i = tid; i < 512; i += kThreads) grid_s[i] = g_iq3s_grid[i];

    if (tid < m) {
        if (PLAIN) {
            s_rows[0] = pp.xq8 + (size_t)start * pp.input_stride;
        } else {
            int t, irow;
            if (shared) { t = start + tid; irow = p.T * p.top_k + t; }
            else { irow = __ldcg(p.perm + start + tid); t = irow / p.top_k; }
            s_rows[tid] = p.in_q8 + (size_t)irow * p.in_stride;
            s_out_row[tid] = irow;
            s_tok[tid] = t;
        }
    }
    __syncthreads();
    stage_q8(s_rows, m, nb, ncols, aq, ad, tid);
    __syncthreads();

    const int l8 = lane & 7;
    for (int rr = 4 * warp; rr < rows_here; rr += 32) {
        if (!mbar_wait(bars + (rr >> 3), 0) && p.status) atomicOr(p.status, kStatusWaitTimeout);
        const int row = rr + (lane >> 3);
        const bool valid = row < rows_here;
        float acc[kMaxGroupTokens];
#pragma unroll
        for (int i = 0; i < kMaxGroupTokens; ++i) acc[i] = 0.0f;
        if (valid) row_dot<TYPE>(wt + (size_t)row * rb, l8, nb, ncols, aq, ad, m, grid_s, acc);
        reduce8(acc, m);
        if (valid && l8 == 0) {
            if (PLAIN) {
                pp.y[(size_t)blockIdx.y * nrows + r0 + row] = acc[0];
            } else {
#pragma unroll
                for (int i = 0; i < kMaxGroupTokens; ++i)
                    if (i < m) p.pair_out[(size_t)s_out_row[i] * p.H + r0 + row] = acc[i];
            }
        }
    }
    if (PLAIN) return;

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
    const int k = p.top_k, H = p.H;
    for (int i = 0; i < m; ++i) {
        if (!s_done[i]) continue;
        const int t = s_tok[i];
        for (int r = tid; r < rows_here; r += kThreads) {
            const int h = r0 + r;
            // weighted_combine_kernel (chimere_kernels.cu:1551-1565): slots in ascending order
            float sum = 0.0f;
            for (int j = 0; j < k; ++j)
                sum = fmaf(p.topk_w[(size_t)t * k + j], __ldcg(p.pair_out + ((size_t)t * k + j) * H + h), sum);
            if (p.nrows_shared > 0) {
                // sigmoid_gate_add_kernel (scratch_pool.rs:266-277): shared * sigmoid(logit) + routed
                const float sh = __ldcg(p.pair_out + ((size_t)p.T * k + t) * H + h);
                if (p.sh_gate_logit) sum = fmaf(sh, sigmoid_ref(__ldcg(p.sh_gate_logit + t)), sum);
                else sum = sh + sum;
            }
            p.y[(size_t)t * H + h] = sum;
        }
    }
}

// ------------------------------------------------------------------ small kernels ----------
// Parity tap: exact integer dot of every (row, 32-wide block) against one Q8_1 row.
template <int TYPE>
__global__ void block_sumi_kernel(const uint8_t* w, const uint8_t* xq8, int32_t* out, int ncols, int nrows) {
    const int nb = ncols >> 5;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)nrows * nb) return;
    const int r = (int)(idx / nb), b = (int)(idx - (int64_t)r * nb);
    int wv[8], mul;
    float dw;
    Unit<TYPE>::load(w + (size_t)r * Unit<TYPE>::row_bytes(ncols), b, g_iq3s_grid, wv, dw, mul);
    int qw[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) qw[g] = *reinterpret_cast<const int*>(xq8 + (size_t)b * kQ81Bytes + 4 + 4 * g);
    out[idx] = unit_sumi<TYPE>(wv, mul, qw);
}

// Q8_1 of `batch` rows of ncols floats; output rows of ncols_padded/32 blocks, tail blocks zero.
// One warp per block.  quantize_row_q8_1_cuda as called from ffi/ggml_cuda_gemv.cu:184-194,393-404.
__global__ void quantize_q8_1_kernel(const float* x, uint8_t* out, int64_t ncols, int64_t ncols_padded, int batch) {
    const int lane = threadIdx.x & 31;
    const int64_t nbp = ncols_padded >> 5;
    const int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (gw >= nbp * batch) return;
    const int64_t row = gw / nbp, b = gw - row * nbp;
    const int64_t col = b * 32 + lane;
    const float xi = (col < ncols) ? x[row * ncols + col] : 0.0f;
    float amax = fabsf(xi), sum = xi;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
        sum += __shfl_xor_sync(0xffffffffu, sum, s);
    }
    const float d = amax / 127.0f;
    const int8_t q = (amax == 0.0f) ? (int8_t)0 : (int8_t)roundf(xi / d);
    uint8_t* o = out + (row * nbp + b) * kQ81Bytes;
    reinterpret_cast<int8_t*>(o)[4 + lane] = q;
    if (lane == 0) *reinterpret_cast<__half2*>(o) = __halves2half2(__float2half(d), __float2half(sum));
}

// y = x / sqrt(mean(x^2) + eps), one CTA per row.
__global__ void rmsnorm_kernel(const float* x, float* y, int H, float eps) {
    __shared__ float s_part[32];
    const float* xr = x + (size_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += s_part[w];
    const float inv = 1.0f / sqrtf(tot / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) y[(size_t)blockIdx.x * H + i] = xr[i] * inv;
}

// residual += hidden; normed = residual / sqrt(mean(residual^2) + eps) * weight, one CTA of 256 per token row.
// fused_add_residual_rmsnorm (chimere-server/src/kernels/fused_ops.rs:91-140) for T rows at once, in its order:
// thread i sums the squares of elements i, i+256, ... (one fused multiply-add each), the 256 sums meet in a tree
// of strides 128 .. 1, and every element is scaled as (residual * inv_rms) * weight.
__global__ void __launch_bounds__(256) add_residual_rmsnorm_kernel(const float* hidden, float* residual, const float* weight, float* normed,
                                                                   int H, float eps) {
    __shared__ float s_sum[256];
    griddep_wait();                       // the rows may come from the previous kernel of the stream
    if (threadIdx.x == 0) griddep_launch();
    const int tid = threadIdx.x;
    const float* h = hidden + (size_t)blockIdx.x * H;
    float* r = residual + (size_t)blockIdx.x * H;
    float sum_sq = 0.0f;
    for (int i = tid; i < H; i += 256) {
        const float val = h[i] + r[i];
        r[i] = val;
        sum_sq = fmaf(val, val, sum_sq);
    }
    s_sum[tid] = sum_sq;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (tid < s) s_sum[tid] += s_sum[tid + s];
        __syncthreads();
    }
    const float rms = sqrtf(s_sum[0] / (float)H + eps);
    const float inv_rms = 1.0f / rms;
    for (int i = tid; i < H; i += 256) normed[(size_t)blockIdx.x * H + i] = r[i] * inv_rms * weight[i];
}

cudaError_t launch_add_residual_rmsnorm(const float* hidden, float* residual, const float* weight, float* normed, int T, int H, float eps,
                                        cudaStream_t stream) {
    if (T <= 0) return cudaSuccess;
    return launch_pdl(add_residual_rmsnorm_kernel, dim3(T), 256, 0, stream, hidden, residual, weight, normed, H, eps);
}

// ------------------------------------------------------------------ launchers --------------
constexpr int kSmemCap = 200 * 1024;

template <typename K>
static cudaError_t set_smem(K kernel, size_t bytes) {
    if (bytes > (size_t)kSmemCap) return cudaErrorInvalidValue;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemCap);
}

static int64_t host_row_bytes(int type, int ncols) {
    switch (type) {
        case CHIMERE_TYPE_Q4_0: return (int64_t)(ncols / 32) * 18;
        case CHIMERE_TYPE_Q8_0: return (int64_t)(ncols / 32) * 34;
        case CHIMERE_TYPE_IQ3_S: return (int64_t)(ncols / 256) * 110;
        default: return -1;
    }
}

template <int TYPE>
static cudaError_t launch_gate_up_t(const GemvParams& p, int max_entries, cudaStream_t stream) {
    const bool dual = p.act == CHIMERE_ACT_SWIGLU;
    const size_t smem = plan_smem(p.H, 32, host_row_bytes(TYPE, p.H), dual).total;
    cudaError_t e = set_smem(gate_up_kernel<TYPE>, smem);
    if (e != cudaSuccess) return e;
    const int tiles = (max(p.nrows_routed, p.nrows_shared) + 31) / 32;
    gate_up_kernel<TYPE><<<dim3(tiles, max_entries), kThreads, smem, stream>>>(p);
    return cudaGetLastError();
}

static cudaError_t dispatch_gate_up(int type, const GemvParams& p, int max_entries, cudaStream_t stream) {
    switch (type) {
        case CHIMERE_TYPE_Q4_0: return launch_gate_up_t<CHIMERE_TYPE_Q4_0>(p, max_entries, stream);
        case CHIMERE_TYPE_Q8_0: return launch_gate_up_t<CHIMERE_TYPE_Q8_0>(p, max_entries, stream);
        case CHIMERE_TYPE_IQ3_S: return launch_gate_up_t<CHIMERE_TYPE_IQ3_S>(p, max_entries, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gate_up(const GemvParams& p, int max_entries, cudaStream_t stream) {
    cudaError_t e = dispatch_gate_up(p.type_routed, p, max_entries, stream);
    if (e == cudaSuccess && p.nrows_shared > 0 && p.type_shared != p.type_routed)
        e = dispatch_gate_up(p.type_shared, p, max_entries, stream);
    return e;
}

// Output rows per CTA of the down stage: as many (<= 64, multiple of 8) as keep the weight tile
// under 48 KiB, so that several CTAs share an SM.
int down_tile_rows(int type_routed, int ncols_routed, int type_shared, int ncols_shared) {
    int64_t rb = host_row_bytes(type_routed, ncols_routed);
    if (ncols_shared > 0) rb = max(rb, host_row_bytes(type_shared, ncols_shared));
    int rows = 64;
    while (rows > 8 && rows * rb > 48 * 1024) rows >>= 1;
    return rows;
}

template <int TYPE>
static cudaError_t launch_down_t(const GemvParams& p, int max_entries, cudaStream_t stream) {
    size_t smem = 0;
    if (p.type_routed == TYPE) smem = plan_smem(p.ncols_routed, p.tile_rows, host_row_bytes(TYPE, p.ncols_routed), false).total;
    if (p.nrows_shared > 0 && p.type_shared == TYPE)
        smem = max(smem, (size_t)plan_smem(p.ncols_shared, p.tile_rows, host_row_bytes(TYPE, p.ncols_shared), false).total);
    cudaError_t e = set_smem(down_kernel<TYPE, false>, smem);
    if (e != cudaSuccess) return e;
    down_kernel<TYPE, false><<<dim3(p.n_row_tiles, max_entries), kThreads, smem, stream>>>(p, PlainParams{}, p.tile_rows);
    return cudaGetLastError();
}

static cudaError_t dispatch_down(int type, const GemvParams& p, int max_entries, cudaStream_t stream) {
    switch (type) {
        case CHIMERE_TYPE_Q4_0: return launch_down_t<CHIMERE_TYPE_Q4_0>(p, max_entries, stream);
        case CHIMERE_TYPE_Q8_0: return launch_down_t<CHIMERE_TYPE_Q8_0>(p, max_entries, stream);
        case CHIMERE_TYPE_IQ3_S: return launch_down_t<CHIMERE_TYPE_IQ3_S>(p, max_entries, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_down(const GemvParams& p, int max_entries, cudaStream_t stream) {
    cudaError_t e = dispatch_down(p.type_routed, p, max_entries, stream);
    if (e == cudaSuccess && p.nrows_shared > 0 && p.type_shared != p.type_routed)
        e = dispatch_down(p.type_shared, p, max_entries, stream);
    return e;
}

template <int TYPE>
static cudaError_t launch_mmvq_t(const PlainParams& pp, int nslots, cudaStream_t stream) {
    const int64_t rb = host_row_bytes(TYPE, pp.ncols);
    int rows = 64;
    while (rows > 8 && rows * rb > 48 * 1024) rows >>= 1;
    const size_t smem = plan_smem(pp.ncols, rows, rb, false).total;
    cudaError_t e = set_smem(down_kernel<TYPE, true>, smem);
    if (e != cudaSuccess) return e;
    GemvParams p{};
    down_kernel<TYPE, true><<<dim3((pp.nrows + rows - 1) / rows, nslots), kThreads, smem, stream>>>(p, pp, rows);
    return cudaGetLastError();
}

cudaError_t launch_mmvq(int wtype, const void* w, const void* xq8, float* y, const int* ids, int ncols, int nrows,
                        int64_t expert_stride, int64_t input_stride, int nslots, cudaStream_t stream) {
    PlainParams pp{(const uint8_t*)w, (const uint8_t*)xq8, y, ids, ncols, nrows, expert_stride, input_stride};
    if (nslots <= 0 || nrows <= 0) return cudaSuccess;
    switch (wtype) {
        case CHIMERE_TYPE_Q4_0: return launch_mmvq_t<CHIMERE_TYPE_Q4_0>(pp, nslots, stream);
        case CHIMERE_TYPE_Q8_0: return launch_mmvq_t<CHIMERE_TYPE_Q8_0>(pp, nslots, stream);
        case CHIMERE_TYPE_IQ3_S: return launch_mmvq_t<CHIMERE_TYPE_IQ3_S>(pp, nslots, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_block_sumi(int wtype, const void* w, const void* xq8, int32_t* sumi, int ncols, int nrows,
                              cudaStream_t stream) {
    const int64_t n = (int64_t)nrows * (ncols / 32);
    if (n <= 0) return cudaSuccess;
    const dim3 grid((unsigned)((n + 255) / 256));
    switch (wtype) {
        case CHIMERE_TYPE_Q4_0: block_sumi_kernel<CHIMERE_TYPE_Q4_0><<<grid, 256, 0, stream>>>((const uint8_t*)w, (const uint8_t*)xq8, sumi, ncols, nrows); break;
        case CHIMERE_TYPE_Q8_0: block_sumi_kernel<CHIMERE_TYPE_Q8_0><<<grid, 256, 0, stream>>>((const uint8_t*)w, (const uint8_t*)xq8, sumi, ncols, nrows); break;
        case CHIMERE_TYPE_IQ3_S: block_sumi_kernel<CHIMERE_TYPE_IQ3_S><<<grid, 256, 0, stream>>>((const uint8_t*)w, (const uint8_t*)xq8, sumi, ncols, nrows); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_quantize_q8_1(const float* x, void* out, int64_t ncols, int64_t ncols_padded, int batch,
                                 cudaStream_t stream) {
    const int64_t warps = (ncols_padded / 32) * batch;
    if (warps <= 0) return cudaSuccess;
    quantize_q8_1_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(x, (uint8_t*)out, ncols, ncols_padded, batch);
    return cudaGetLastError();
}

cudaError_t launch_rmsnorm(const float* x, float* y, int T, int H, float eps, cudaStream_t stream) {
    if (T <= 0) return cudaSuccess;
    rmsnorm_kernel<<<T, 256, 0, stream>>>(x, y, H, eps);
    return cudaGetLastError();
}

}  // namespace chimere
