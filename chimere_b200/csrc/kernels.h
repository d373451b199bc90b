// kernels.h -- parameter blocks and launchers shared by the .cu files of the library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace chimere {

// layout of the workspace's integer scratch ("counters"); everything returns to zero after a call
constexpr int kCtrRouteAll = 0;    // token tiles whose top-k is done
constexpr int kCtrSpare = 4;       // [4] unused, kept zero
constexpr int kCtrRouteTile = 16;  // [ceil(max_T/8)] row tiles done per token tile
// the combine counters follow at ws-specific offset (one per token and output row tile)

struct RouteParams {
    int T, H, E, top_k, route_mode, has_shared;
    int idx_stride;             // permute only: distance in int32 between consecutive ids (0 or 1 = dense)
    int list_mode;              // 0: work list for routed + shared entries; 1: shared-expert entries only (expert-parallel home
                                // rank); 2: an empty list (the prefill path builds its own from offsets and perm)
    float route_scale;
    const float* x;             // [T][H]
    const float* router_w;      // [E][H]
    const float* router_bias;   // [E] or null
    const float* shexp_gate_w;  // [H] or null
    float* router_logits;       // [T][E]
    float* sh_gate_logit;       // [T]
    int32_t* topk_idx;          // [T][k]
    float* topk_w;              // [T][k]
    uint8_t* x_q8;              // [T][H/32][36]
    int8_t* x_soa_q;            // [T][H] the same quants as a plane
    float* x_soa_d;             // [T][x_soa_d_stride] the same scales (f16-rounded) as f32
    int x_soa_d_stride;
    int32_t* perm;              // [T*k]
    int32_t* offsets;           // [E+1]
    int32_t* group_list;
    int32_t* counters;
    int32_t* status;            // workspace status word (may be null): a bounded wait that ran out raises a bit here
    int32_t* wait_flags;        // dispatch step alone (expert-parallel owner): counters of the peer-store exchange to wait for first
    int wait_n, wait_expect;    // ... `wait_n` of them, each has to reach `wait_expect`; they are taken down again (null = none)
    int32_t* dispatch_scratch;  // zeroed scratch for the dispatch of large batches: ceil(T*top_k / 128) * 256 + 260 ints, left
                                // zeroed again; null = always sort in one CTA
};

// Grouped GEMV over work entries (see common.cuh for the list layout).
struct GemvParams {
    int T, top_k, H;
    int ncols_routed, ncols_shared;  // input width: H, H for gate/up; F, F_s for down
    int nrows_routed, nrows_shared;  // output rows per expert: F, F_s for gate/up; H, H for down
    int act;                     // CHIMERE_ACT_* (gate/up stage)
    int type_routed, type_shared;
    const int32_t* group_list;
    const int32_t* perm;
    // weights
    const uint8_t* w_a;          // gate (or null) / down
    const uint8_t* w_b;          // up
    int64_t stride_a, stride_b;  // bytes per routed expert
    const uint8_t* sh_a;         // shared-expert gate (or null) / down
    const uint8_t* sh_b;         // shared-expert up
    // input: Q8_1 rows
    const uint8_t* in_q8;        // gate/up: x_q8 [T]; down: inter_q8 [pairs]
    int64_t in_stride;           // bytes per input row
    // gate/up output
    uint8_t* inter_q8;           // [T*k + T][inter_stride]
    int64_t inter_stride;
    // down output + combine
    float* pair_out;             // [T*k + T][H]
    const float* topk_w;         // [T][k]
    const float* sh_gate_logit;  // [T] or null
    float* y;                    // [T][H]
    int32_t* combine_ctr;        // [T][row tiles]
    int tile_rows;               // down stage: output rows per CTA (multiple of 8, <= 64)
    int n_row_tiles;             // down stage: ceil(H / tile_rows)
    // tiled path: the same Q8_1 rows as planes (int8 values / f32 scales), input and gate-up output
    const int8_t* in_soa_q; int64_t in_soa_q_stride;   // bytes per row
    const float* in_soa_d; int64_t in_soa_d_stride;     // floats per row
    int8_t* out_soa_q; int64_t out_soa_q_stride;
    float* out_soa_d; int64_t out_soa_d_stride;
    int32_t* status;
    int no_combine;              // down stage: only write the per-pair rows (the caller combines)
    int few_tokens;              // T counts row slots that are mostly empty (fixed-size expert-parallel exchange): size the
                                 // kernels as for a decode batch whatever T says
};

cudaError_t launch_route(const RouteParams& p, cudaStream_t stream);
// dispatch permutation + work list from p.topk_idx alone (no routing, no shared entries)
cudaError_t launch_permute(const RouteParams& p, cudaStream_t stream);
// y[t][h] = sum_j w[t][j] * rows[t*k+j][h] (+ shared[t][h] * sigmoid(logit[t]) or + shared[t][h])
cudaError_t launch_ep_finish(const float* rows, const int32_t* slot, const float* topk_w, const float* shared_rows, const float* sh_logit,
                             float* y, int T, int H, int k, cudaStream_t stream);
// fixed-size dispatch: fill send[world*cap][row_bytes] with the pairs of each destination rank in pair order
// exact-size dispatch: send row j = the pair perm[j] (pairs sorted by expert, hence by owner rank), slot[pair] = j
cudaError_t launch_ep_pack_sorted(const int32_t* perm, const int32_t* topk_idx, const int8_t* x_q, const float* x_d, int d_stride, uint8_t* send,
                                  int32_t* slot, int T, int k, int H, int experts_per_rank, int row_bytes, cudaStream_t stream);
cudaError_t launch_ep_pack(const int32_t* topk_idx, const int8_t* x_q, const float* x_d, int d_stride, uint8_t* send, int32_t* slot,
                           int T, int k, int H, int experts_per_rank, int world, int cap, int row_bytes, cudaStream_t stream);
// expert-parallel exchange by peer stores (decode-size batches); see router.cu
cudaError_t launch_ep_pack_p2p(const int32_t* topk_idx, const float* topk_w, const int8_t* x_q, const float* x_d, int d_stride,
                               uint8_t* const* peer_recv, int32_t* const* peer_flags, int rank, int T, int k, int H,
                               int experts_per_rank, int world, int cap, int row_bytes, cudaStream_t stream);
cudaError_t launch_ep_wait_flags(int32_t* flags, int n, int expect, int32_t* status, cudaStream_t stream);
cudaError_t launch_ep_return_p2p(const float* pair_rows, const uint8_t* recv, int row_bytes, int tail_off, float* const* peer_back,
                                 int32_t* const* peer_flags, int rank, int world, int T, int cap, int H, cudaStream_t stream);
cudaError_t launch_ep_finish_p2p(const float* back, int32_t* flags, int world, const float* shared_rows, const float* sh_logit, float* y,
                                 int T, int H, int32_t* ctr, int32_t* status, cudaStream_t stream);
cudaError_t launch_gate_up(const GemvParams& p, int max_entries, cudaStream_t stream);
cudaError_t launch_down(const GemvParams& p, int max_entries, cudaStream_t stream);

// Plain batched GEMV (legacy operator entries): y[slot][row] = W[ids[slot]][row] . xq8[slot].
cudaError_t launch_mmvq(int wtype, const void* w, const void* xq8, float* y, const int* ids, int ncols, int nrows,
                        int64_t expert_stride, int64_t input_stride, int nslots, cudaStream_t stream);
// K-quant rows (CHIMERE_TYPE_Q4_K / Q5_K / Q6_K) against one Q8_1 row: y[nrows] = W . x_q8
cudaError_t launch_mmvq_kquant(int wtype, const void* w, const void* xq8, float* y, int ncols, int nrows, cudaStream_t stream);
// ... `n_inputs` Q8_1 rows x_stride bytes apart, outputs y_stride floats apart; mode 0 store, 1 add, 2 add sigmoid(logit[t]) * v;
// w2 / y2 (optional): a second matrix against the same inputs in the same launch; chained: programmatic launch
cudaError_t launch_mmvq_kquant_batched(int wtype, const void* w, const void* w2, const void* xq8, int64_t x_stride, float* y, float* y2,
                                       int64_t y_stride, int n_inputs, int ncols, int nrows, int mode, const float* logit, bool chained,
                                       cudaStream_t stream);
// out[t] (Q8_1 blocks, out_stride bytes apart) = Q8_1(silu(g[t]) * u[t]) or, without g, Q8_1(relu(u[t])^2); rows in_stride floats apart
cudaError_t launch_act_q8_1(const float* g, const float* u, int64_t in_stride, void* out, int64_t out_stride, int T, int F, cudaStream_t stream);
cudaError_t launch_block_sumi(int wtype, const void* w, const void* xq8, int32_t* sumi, int ncols, int nrows,
                              cudaStream_t stream);
cudaError_t launch_quantize_q8_1(const float* x, void* out, int64_t ncols, int64_t ncols_padded, int batch,
                                 cudaStream_t stream);
cudaError_t launch_rmsnorm(const float* x, float* y, int T, int H, float eps, cudaStream_t stream);
cudaError_t launch_add_residual_rmsnorm(const float* hidden, float* residual, const float* weight, float* normed, int T, int H, float eps,
                                        cudaStream_t stream);
// routing trace: ids as bytes [T][k] for the drafter tooling, and (optional) per-expert pair counts added into load[E]
cudaError_t launch_routing_trace(const int32_t* topk_idx, uint8_t* trace, int32_t* load, int T, int k, int E, cudaStream_t stream);
int down_tile_rows(int type_routed, int ncols_routed, int type_shared, int ncols_shared);

// block-scaled int8 GEMM on tcgen05 (gemm_i8.cu); operands in the mma128 layout
struct GemmItem { int64_t a_offset, b_offset; int n_valid, rows_valid, out_row0, out_col0; };
struct GemmParams {
    const uint8_t* a_base; const uint8_t* b_base;   // mma128 tiles; an item's operands start at base + offset
    const GemmItem* items;
    int n_items;
    int nblocks;                                    // 32-wide K blocks
    float* out; int64_t ldo;                        // f32 output, row pitch in floats
    int32_t* status;
};
cudaError_t launch_gemm_i8_f32(const GemmParams& p, int n_items, int32_t* tile_counter, cudaStream_t stream);
int launch_mma_i8_probe(int n_mma, int n_cols, int n_acc, int32_t* status, cudaStream_t stream);

// MoE prefill on the GEMM: token tiles built on the device, weights in mma128 form
struct PrefillGemmParams {
    const int32_t* tiles;            // tile list (word 0 = count, words 4 / 5 = tile counters of the gate/up / down launch, tiles from word 8)
    const int32_t* perm;
    const uint8_t* a_exps; int64_t stride_a;   // routed experts' mma128 matrices
    const uint8_t* sh_a;                       // shared expert's
    const uint8_t* b_tiles; int64_t b_tile_stride;   // token tiles (input)
    uint8_t* out_tiles; int64_t out_tile_stride;     // gate/up: token tiles of the down GEMM (output)
    float* pair_out;                                 // down: per-pair rows [pairs][H]
    int row_tiles_routed, row_tiles_shared, row_tiles_max;
    int nblk_routed, nblk_shared;    // gate/up: 32-row blocks of the intermediate (F / 32, F_s / 32); blocks beyond are padding
    int ncols_in, ncols_in_shared;   // K of the routed / shared matrices
    int act, T, top_k, H;
    int32_t* status;
};
cudaError_t launch_prefill_gemm(const PrefillGemmParams& p, bool down, int n_tiles_max, cudaStream_t stream);
cudaError_t launch_pack_mma128_ggml(int type, const void* raw, void* out, int n_mats, int nrows, int ncols, int mode,
                                    int64_t raw_stride, int64_t out_stride, cudaStream_t stream);
cudaError_t launch_build_tiles(const int32_t* offsets, const int32_t* perm, int32_t* tiles, int32_t* list, int E, int T, int top_k,
                               int has_shared, int gemm_min, cudaStream_t stream);
cudaError_t launch_gather_tiles(const int32_t* tiles, const int32_t* perm, const int8_t* x_q, int64_t x_q_stride, const float* x_d,
                                int x_d_stride, uint8_t* b_tiles, int64_t b_tile_stride, int H, int top_k, int n_tiles_max, cudaStream_t stream);
cudaError_t launch_pack_mma128(const int8_t* q, const float* scales, uint8_t* out, int rows, int cols, cudaStream_t stream);

// tiled32 layout (tiled.cuh): pack, kernels on packed weights, parity tap
struct TiledGeomHost { int wk, wr; };  // warps along K x row tiles per CTA (wk * wr = 8)
TiledGeomHost tiled_gate_up_geom(int type_routed, int type_shared, int H, bool has_shared);
TiledGeomHost tiled_down_geom(int type_routed, int F, int type_shared, int F_s, int T);
cudaError_t launch_pack(int type, const void* raw, void* out, int n_mats, int nrows, int ncols, int64_t raw_stride,
                        int64_t out_stride, cudaStream_t stream);
cudaError_t launch_gate_up_tiled(const GemvParams& p, int max_entries, cudaStream_t stream);
cudaError_t launch_down_tiled(const GemvParams& p, int max_entries, cudaStream_t stream);
cudaError_t launch_block_sumi_tiled(int type, const void* packed, const void* xq8, int32_t* sumi, int ncols, int nrows,
                                    cudaStream_t stream);

// cudaFuncSetAttribute(max dynamic shared memory) once per kernel and device instead of on every launch.
// `done` is a static array owned by the calling launcher (one per kernel instantiation).
template <typename K>
inline cudaError_t max_smem_once(K kernel, int bytes, bool (&done)[64]) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done[dev] = true;
    return e;
}

// Number of SMs of the current device (cached per device).
inline int sm_count() {
    static int n_sm_of[64] = {};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = -1;
    if (dev >= 0 && n_sm_of[dev]) return n_sm_of[dev];
    if (dev < 0 || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0) n_sm_of[dev] = n;
    return n;
}

// Launch with programmatic stream serialization: the grid may start while the previous kernel of the stream is
// still running; the kernels call griddep_wait() before they touch what that kernel writes.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, int threads, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace chimere
