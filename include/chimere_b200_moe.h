/* chimere_b200_moe.h -- C ABI of the B200 (sm_100a) quantized MoE feed-forward library.
 *
 * Two groups of entry points:
 *
 *  1. Legacy operator entries.  Same names, argument order and meaning as the reference's
 *     FFI layer (chimere-server/ffi/ggml_cuda_gemv.cu, Rust declarations in
 *     chimere-server/src/kernels/ggml_gpu.rs:101-240), so the Rust wrappers link unchanged.
 *     They return void and report nothing, exactly like the reference.
 *
 *  2. Layer-level entries (chimere_b200_moe_*).  One call replaces the launch sequence of
 *     forward_moe_cudarc_with_cache (chimere-server/src/qwen35_model/moe_ffn.rs:1094-1766):
 *     router GEMV, softmax/top-k, Q8_1 quantization, batched gate/up GEMVs, SwiGLU,
 *     re-quantization, batched down GEMV, weighted combine, shared expert and sigmoid gate,
 *     for T tokens at once.  They return int: 0 = ok, <0 = argument error found on the host
 *     before anything was launched.
 *
 * Conventions (both groups): every pointer named dev / d_* is device memory owned by the
 * caller; the library never allocates, frees or keeps device memory; all work is enqueued on
 * the stream passed in (NULL = legacy default stream); no entry synchronises the host unless
 * its comment says so.  Quantized weights use the ggml block layouts unchanged
 * (Q4_0 18 B / 32, Q8_0 34 B / 32, IQ3_S 110 B / 256; sizes as in
 * chimere-server/src/gguf_loader.rs:161-193), row-major, experts contiguous.
 */
#ifndef CHIMERE_B200_MOE_H
#define CHIMERE_B200_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef __DRIVER_TYPES_H__
typedef struct CUstream_st* cudaStream_t;
#endif

/* ggml tensor-type ids of the weight formats this path supports. */
enum { CHIMERE_TYPE_Q4_0 = 2, CHIMERE_TYPE_Q8_0 = 8, CHIMERE_TYPE_IQ3_S = 21,
       /* K-quant super-blocks: plain GEMV entries (chimere_mmvq_q4k / _q5k / _q6k) only, not a chimere_moe_layer weight type */
       CHIMERE_TYPE_Q4_K = 12, CHIMERE_TYPE_Q5_K = 13, CHIMERE_TYPE_Q6_K = 14 };
/* Router variants. */
enum { CHIMERE_ROUTE_SOFTMAX_RENORM = 0,  /* softmax over E, top-k on probabilities, renormalise (chimere_kernels.cu:1150-1223) */
       CHIMERE_ROUTE_SIGMOID_NORM_SCALE = 1 /* sigmoid scores, top-k, normalise to sum 1, multiply by route_scale (Nemotron-H style) */ };
/* Expert activation. */
enum { CHIMERE_ACT_SWIGLU = 0,  /* silu(gate x) * (up x)   (fused_ops.rs:34-45) */
       CHIMERE_ACT_RELU2 = 1    /* relu(up x)^2, no gate matrix */ };

/* Weight layouts.  GGML: the blocks exactly as the GGUF file holds them.  TILED32: the library's own
 * lossless rearrangement made once by chimere_b200_moe_pack (32-row tiles, 16 bytes per row and
 * 32-weight unit, IQ3_S expanded from codebook indices to signed 4-bit codes); the layer-level
 * entries run several times faster on it. */
enum { CHIMERE_LAYOUT_GGML = 0, CHIMERE_LAYOUT_TILED32 = 1 };

/* One MoE layer: dimensions, modes and device pointers.  Mirrors MoeWeightsRaw
 * (chimere-server/src/qwen35_model/compute_graph.rs:1000-1049).  For the CPU oracle the same
 * struct is used with host pointers. */
typedef struct chimere_moe_layer {
    int32_t H;            /* hidden size (multiple of 256 for IQ3_S inputs, of 32 otherwise) */
    int32_t E;            /* routed experts (<= 256) */
    int32_t F;            /* routed expert width */
    int32_t F_s;          /* shared expert width, 0 = no shared expert */
    int32_t top_k;        /* experts per token (<= 8) */
    int32_t route_mode;   /* CHIMERE_ROUTE_* */
    int32_t act;          /* CHIMERE_ACT_* */
    float   route_scale;  /* multiplier on the normalised weights (1.0 for softmax mode) */
    int32_t type_gate, type_up, type_down;          /* routed expert weight types */
    int32_t type_sh_gate, type_sh_up, type_sh_down; /* shared expert weight types */
    int32_t layout;       /* CHIMERE_LAYOUT_* of the nine expert matrices below */
    int32_t reserved;
    const float* router_w;     /* f32 [E][H] row-major */
    const float* router_bias;  /* f32 [E] added to the logits before scoring, or NULL */
    const float* shexp_gate_w; /* f32 [H]: shared expert scaled by sigmoid(x . w), or NULL = scale 1 */
    const void*  gate_exps;    /* [E][F rows][H cols] quant blocks; NULL when act == RELU2 */
    const void*  up_exps;      /* [E][F rows][H cols] */
    const void*  down_exps;    /* [E][H rows][F cols] */
    int64_t stride_gate, stride_up, stride_down;    /* bytes per expert */
    const void*  sh_gate;      /* [F_s rows][H cols]; NULL when act == RELU2 */
    const void*  sh_up;        /* [F_s rows][H cols] */
    const void*  sh_down;      /* [H rows][F_s cols] */
} chimere_moe_layer;

/* Scratch of one stream.  Mirrors GgmlGpuBuffers::with_moe
 * (chimere-server/src/kernels/ggml_gpu.rs:358-406): allocated once by the caller, reused by
 * every call, not re-entrant.  All members point into the caller's arena; they stay readable
 * after a call and are the parity taps (routing indices, permutation, Q8_1 bytes). */
typedef struct chimere_moe_workspace {
    int32_t max_T;          /* capacity in tokens */
    int32_t reserved0;
    int32_t* topk_idx;      /* [T][top_k] expert ids, descending score */
    float*   topk_w;        /* [T][top_k] combine weights */
    float*   router_logits; /* [T][E] (after bias) */
    float*   sh_gate_logit; /* [T] x . shexp_gate_w */
    uint8_t* x_q8;          /* [T][H/32] Q8_1 blocks (36 B) of the input rows */
    int32_t* perm;          /* [T*top_k] pair ids t*top_k+j sorted by expert (stable) */
    int32_t* offsets;       /* [E+1] start of each expert's pairs in perm */
    int32_t* group_list;    /* work list of the grouped GEMV kernels, built on the device */
    int32_t* counters;      /* small integer scratch; zero between calls */
    uint8_t* inter_q8;      /* [(T*top_k + T)] rows of F_max/32 Q8_1 blocks (row stride rounded up to 16 B) */
    float*   pair_out;      /* [(T*top_k + T)][H] down-projection rows before the combine */
    int8_t*  x_q;           /* [T][H] the quants of x_q8 as a plane */
    float*   x_d;           /* [T][ceil4(H/32)] the scales of x_q8 (f16-rounded) as f32 */
    int8_t*  inter_q;       /* [(T*top_k + T)][F_max] the quants of inter_q8 as a plane */
    float*   inter_d;       /* [(T*top_k + T)][ceil4(F_max/32)] the scales of inter_q8 as f32 */
    void*    prefill_arena; /* staging for the grouped int8 GEMM path */
    size_t   prefill_bytes;
    int32_t* status;        /* device status word: 0 = ok */
} chimere_moe_workspace;

/* ---------------------------------------------------------------- layer-level entries ---- */

/* Bytes of device memory a workspace for up to max_T tokens needs. */
size_t chimere_b200_moe_workspace_bytes(const chimere_moe_layer* w, int max_T);

/* Carve `ws` out of the caller's device arena (`bytes` >= workspace_bytes, 256-byte aligned)
 * and zero what must start at zero (enqueued on `stream`).  Returns 0, or <0 on bad arguments. */
int chimere_b200_moe_workspace_init(chimere_moe_workspace* ws, void* d_arena, size_t bytes,
                                    const chimere_moe_layer* w, int max_T, cudaStream_t stream);

/* Bytes of device memory the TILED32 copy of the layer's expert matrices needs (0 on bad arguments). */
size_t chimere_b200_moe_pack_bytes(const chimere_moe_layer* raw);

/* One-time, load-side: rewrite the expert matrices of `raw` (layout GGML) into `d_arena`
 * (256-byte aligned, >= pack_bytes) and fill `packed` with a copy of `raw` that points at the
 * rewritten matrices (layout TILED32; router tensors are shared with `raw`).  The caller may free the
 * GGML expert matrices afterwards.  F, F_s and H must be multiples of 32. */
int chimere_b200_moe_pack(const chimere_moe_layer* raw, void* d_arena, size_t bytes,
                          chimere_moe_layer* packed, cudaStream_t stream);

/* The same rewrite for one matrix [nrows][ncols] (nrows % 32 == 0), and its size. */
size_t chimere_b200_packed_matrix_bytes(int wtype, int nrows, int ncols);
int chimere_b200_pack_matrix(int wtype, const void* d_raw, void* d_out, int nrows, int ncols,
                             cudaStream_t stream);

/* y[T][H] = MoE(x[T][H]).  Replaces moe_ffn.rs:1094-1766 for T tokens.  x, y: device f32.
 * Capturable in a CUDA graph: no allocation, no host synchronisation, no device-to-host copy. */
int chimere_b200_moe_forward(const chimere_moe_layer* w, const float* d_x, float* d_y, int T,
                             chimere_moe_workspace* ws, cudaStream_t stream);

/* Same, with HOST buffers: copies x in, runs the layer, copies y out, all on `stream`, and
 * waits for the stream.  h_x / h_y should be pinned.  d_x / d_y are caller-provided staging.
 * When h_y is pinned (cudaHostAlloc / cudaHostRegister) the last kernel stores the result straight into it and d_y
 * is not used; pageable memory goes through d_y and a copy. */
int chimere_b200_moe_forward_host(const chimere_moe_layer* w, const float* h_x, float* h_y, int T,
                                  float* d_x, float* d_y, chimere_moe_workspace* ws,
                                  cudaStream_t stream);

/* Routing only: fills ws->router_logits, topk_idx, topk_w, sh_gate_logit, x_q8
 * (moe_ffn.rs:1094-1126 + 1185-1204 + 1736-1746). */
int chimere_b200_moe_route(const chimere_moe_layer* w, const float* d_x, int T,
                           chimere_moe_workspace* ws, cudaStream_t stream);

/* Routing for callers that cannot provide scratch memory and cannot allocate any: a serving process
 * that handed all device memory to its own pool at start-up, or code running where cudaMalloc is not
 * allowed.  Same computation as chimere_b200_moe_route, but the scratch is a fixed array inside the
 * library (about 680 KiB per GPU, held from the moment the library is loaded on that GPU until the
 * process exits) and the results go to the caller's buffers: d_topk_idx [T][top_k] int32 and
 * d_topk_w [T][top_k] f32.  Limits: T <= 64 tokens, H <= 4096, E <= 256, top_k <= 8; anything larger
 * returns -7 (malformed descriptions -- null pointers, non-positive sizes, H not a multiple of 32 --
 * return -1 / -2 as everywhere else).  The first call on each device looks the array's address up
 * (cudaGetSymbolAddress): make that call outside any stream capture; a first call made while `stream`
 * is being captured returns -8 and does nothing.  All calls on a device share the array, so calls that overlap on the GPU
 * race; run them on one stream or order them yourself.  No cudaMalloc / cudaFree, here or below.
 * This entry has no counterpart in the reference. */
int chimere_b200_moe_route_noalloc(const chimere_moe_layer* w, const float* d_x, int T,
                                   int32_t* d_topk_idx, float* d_topk_w, cudaStream_t stream);

/* The fused expert up/gate operator on its own: for every (token, selected expert) pair and the
 * shared expert, act(gate . x, up . x) quantized to Q8_1 into ws->inter_q8.  Needs the routing
 * results of chimere_b200_moe_route in `ws`.  Replaces moe_ffn.rs:1206-1323 (batched gate GEMV,
 * batched up GEMV, silu_mul, batched Q8_1) and :1597-1700 for the shared expert. */
int chimere_b200_moe_gate_up(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws,
                             cudaStream_t stream);

/* Down projections of ws->inter_q8, routing-weighted combine in slot order, sigmoid-gated shared
 * expert; writes y[T][H].  Replaces moe_ffn.rs:1325-1384 and :1700-1766. */
int chimere_b200_moe_down_combine(const chimere_moe_layer* w, float* d_y, int T,
                                  chimere_moe_workspace* ws, cudaStream_t stream);

/* Dispatch permutation from ws->topk_idx: stable counting sort of the pairs (t, j) by expert id
 * into ws->perm / ws->offsets.  The reference has no token permutation (it loops tokens,
 * compute_graph.rs:1787-1808); this is the canonical order the grouped kernels use. */
int chimere_b200_moe_permute(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws,
                             cudaStream_t stream);

/* ------------------------------------------------------------ expert-parallel pieces ------ */
/* Experts sharded over several GPUs (contiguous ranges), router and shared expert replicated.  The
 * reference is single-GPU (no collective anywhere in its sources); these four entries are the local
 * steps either side of the two all-to-all exchanges, which the host runs with NCCL.  All need the
 * TILED32 layout.
 *
 * Home rank of a token:   route_home -> [send Q8_1 planes of the routed pairs] ... shared_expert ...
 *                         [receive the pairs' expert rows] -> ep_finish
 * Owner rank of experts:  [receive planes + local expert ids into ws->x_q, ws->x_d, ws->topk_idx]
 *                         -> experts -> [send ws->pair_out rows back]                              */

/* Router, top-k and Q8_1 as chimere_b200_moe_route, but the work list holds only the shared expert. */
int chimere_b200_moe_route_home(const chimere_moe_layer* w, const float* d_x, int T,
                                chimere_moe_workspace* ws, cudaStream_t stream);
/* Shared expert of the T routed tokens: rows land in ws->pair_out[T*top_k + t]. */
int chimere_b200_moe_shared_expert(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws,
                                   cudaStream_t stream);
/* n_rows (token, expert) pairs whose Q8_1 planes sit in ws->x_q / ws->x_d and whose local expert ids sit in
 * ws->topk_idx[n_rows]; w_local describes the local shard (E = local experts, top_k = 1, F_s = 0).
 * Expert outputs (down . act(gate/up . x), unweighted) land in ws->pair_out[row][H]. */
int chimere_b200_moe_experts(const chimere_moe_layer* w_local, int n_rows, chimere_moe_workspace* ws,
                             cudaStream_t stream);
/* The same with the rows where a fixed-size exchange left them: row r = [H int8][ceil4(H/32) f32][int32 local
 * expert id], row_bytes a multiple of 16; id -1 = no pair in this row (it costs nothing). */
int chimere_b200_moe_experts_packed(const chimere_moe_layer* w_local, int n_rows, const void* d_rows,
                                    int row_bytes, chimere_moe_workspace* ws, cudaStream_t stream);
/* Home rank, fixed-size dispatch: fills d_send[world*cap][row_bytes] (rows in the format above; slot d*cap + i =
 * i-th pair, in pair order, whose expert lives on rank d) and d_slot[T*top_k] = the slot of every pair.
 * cap >= T*top_k.  Needs the results of route_home in `ws`. */
int chimere_b200_moe_ep_pack(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws, void* d_send,
                             int32_t* d_slot, int experts_per_rank, int world, int cap, int row_bytes,
                             cudaStream_t stream);
/* y[t] = sum_j topk_w[t][j] * row(t, j) (slot order) + sigmoid-gated shared row, where row(t, j) is
 * d_rows[d_slot[t*top_k + j]] or, with d_slot == NULL, d_rows[t*top_k + j]. */
int chimere_b200_moe_ep_finish(const chimere_moe_layer* w, const float* d_rows, const int32_t* d_slot, int T,
                               chimere_moe_workspace* ws, float* d_y, cudaStream_t stream);

/* The same step with the two exchanges done by the kernels themselves: rows and partial sums are written straight into the
 * peers' buffers (memory of the other GPUs of the node mapped into this process, e.g. by CUDA IPC; plain stores over
 * NVLink, no collective call, no multicast), and one counter per (buffer, source rank), raised by the writers behind their
 * stores and taken down by the reader, tells the reader that a call's rows are complete.  For decode-size batches, where two collective launches per layer cost more than the expert products.
 *   row          = [H int8][ceil4(H/32) f32][int32 local expert id | -1][int32 token][f32 routing weight], row_bytes % 16 == 0
 *   d_peer_recv  = device array of `world` pointers: rank r's receive buffer [world * cap][row_bytes]
 *   d_peer_flags = device array of `world` pointers: rank r's counters [world] for that buffer (zero at start)
 *   d_peer_back  = device array of `world` pointers: rank r's return buffer f32 [world][T][H]
 *   d_ctr        = one int of this rank's scratch, zero at start (ep_finish_p2p; the other entries ignore it)
 * Home rank: route_home -> ep_pack_p2p -> shared_expert -> ep_finish_p2p.
 * Owner rank: ep_wait -> experts_packed on its own receive buffer (or experts_packed_p2p, which does both) -> ep_return_p2p, which adds up,
 * per (home rank, token), the routing-weighted expert rows in slot order and stores the sums in the home rank's return
 * buffer; ep_finish_p2p waits for the return flags and adds the owners' sums in rank order.  The result differs from
 * the single-GPU layer only in the order of those fp32 additions.  All waits are bounded (status word of `ws`).
 * The reference is single-GPU: these entries have no counterpart there. */
int chimere_b200_moe_ep_pack_p2p(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws, void* const* d_peer_recv,
                                 int32_t* const* d_peer_flags, int32_t* d_ctr, int rank, int experts_per_rank, int world, int cap,
                                 int row_bytes, cudaStream_t stream);
int chimere_b200_moe_ep_wait(int32_t* d_flags, int world, int cap, chimere_moe_workspace* ws, cudaStream_t stream);
/* experts_packed with the wait folded into its first kernel: waits for `cap` arrivals from each of the `world` source ranks on
 * d_flags, takes the counters down, then runs the experts on the received rows. */
int chimere_b200_moe_experts_packed_p2p(const chimere_moe_layer* w_local, int n_rows, const void* d_rows, int row_bytes,
                                        int32_t* d_flags, int world, int cap, chimere_moe_workspace* ws, cudaStream_t stream);
int chimere_b200_moe_ep_return_p2p(const chimere_moe_layer* w_local, chimere_moe_workspace* ws_owner, const void* d_rows, int row_bytes,
                                   float* const* d_peer_back, int32_t* const* d_peer_flags, int32_t* d_ctr, int rank, int world, int T,
                                   int cap, cudaStream_t stream);
int chimere_b200_moe_ep_finish_p2p(const chimere_moe_layer* w, const float* d_back, int32_t* d_flags, int world, int T,
                                   chimere_moe_workspace* ws, float* d_y, int32_t* d_ctr, cudaStream_t stream);

/* Parity tap: integer block dot products.  For `nrows` weight rows of type `wtype` with `ncols`
 * columns and one Q8_1 input row, writes sumi[nrows][ncols/32] (int32): the exact integer sum of
 * each 32-wide block (for IQ3_S including the (1 + 2*scale) factor, chimere_kernels.cu:860). */
int chimere_b200_block_sumi(int wtype, const void* d_w, const void* d_xq8, int32_t* d_sumi,
                            int ncols, int nrows, cudaStream_t stream);

/* The same tap on a TILED32 matrix; the integers must equal those of the GGML form. */
int chimere_b200_block_sumi_tiled(int wtype, const void* d_packed, const void* d_xq8,
                                  int32_t* d_sumi, int ncols, int nrows, cudaStream_t stream);

/* ------------------------------------------------- block-scaled int8 GEMM (tensor cores) ---- */
/* The prefill-size primitive: out[rows][tokens] (f32, row-major) with
 *   out[r][t] = sum over 32-wide blocks b of sa[r][b] * sb[t][b] * (int8 dot of block b of row r and token t),
 * on tcgen05 kind::i8 MMAs (one per block, int32 accumulators in TMEM read back and scaled per block) -- the
 * block arithmetic of the reference's Q8_0 x Q8_1 dot (src/kernels/gemv_q8_0.rs:230-255) for many tokens at
 * once.  The reference has no prefill kernel of its own (it loops tokens, compute_graph.rs:1787-1808).
 * Operands are int8 matrices [rows][cols] / [tokens][cols] with f32 block scales, rewritten by
 * chimere_b200_pack_mma128 into the MMA's shared-memory order.  The scales of the rows (d_a) must have at most 22
 * significant bits -- every ggml scale, an f16 times a small integer, has -- for the per-block scaling to round once.
 * d_items: scratch for ceil(rows/128) * ceil(tokens/128) * 32 + 256 bytes.  This entry synchronises the stream once
 * (it stages its tile list). */
size_t chimere_b200_mma128_bytes(int rows, int cols);
int chimere_b200_pack_mma128(const int8_t* d_q, const float* d_scales, void* d_out, int rows, int cols,
                             cudaStream_t stream);
int chimere_b200_gemm_i8(const void* d_a, const void* d_b, int rows, int tokens, int cols, float* d_out,
                         void* d_items, int32_t* d_status, cudaStream_t stream);

/* Measurement aid: what the int8 tensor pipe of this GPU sustains with no read-back.  One CTA per SM issues n_mma (a
 * multiple of 64) tcgen05.mma kind::i8 instructions (M 128, N n_cols = 128 or 256, K 32) on operands resident in
 * shared memory, into n_acc accumulators taken in turn (n_acc * n_cols <= 512 TMEM columns).
 * Returns the number of CTAs launched (operations = CTAs * n_mma * 2 * 128 * n_cols * 32), or < 0 on error; the
 * caller times the stream.  d_status (may be NULL): raised if a bounded wait ran out.  No counterpart in the
 * reference (it has no tensor-core kernel). */
int chimere_b200_mma_i8_probe(int n_mma, int n_cols, int n_acc, int32_t* d_status, cudaStream_t stream);

/* ------------------------------------------------------------ prefill-size batches -------- */
/* For many tokens per call the expert products run as grouped block-scaled int8 GEMMs on the tensor cores
 * (the primitive above): experts with at least 8 routed tokens and the shared expert go to the GEMM, the rest
 * stay on the GEMV kernels.  The GEMM needs a second weight copy in its own layout (int8 values + f32 block
 * scales, gate and up rows interleaved per 64 rows): about 1.06x the Q8_0 bytes, 2x Q4_0, 2.3x IQ3_S. */
typedef struct chimere_moe_prefill_weights {
    const void* gu_exps;   int64_t stride_gu;     /* routed: gate|up tiles */
    const void* down_exps; int64_t stride_down;
    const void* sh_gu;     const void* sh_down;   /* shared expert */
    int32_t rows_per_gu_tile;                     /* 64 with a gate matrix, 128 without */
    int32_t reserved;
} chimere_moe_prefill_weights;

size_t chimere_b200_moe_pack_prefill_bytes(const chimere_moe_layer* raw);
/* raw: layout GGML.  H a multiple of 128; with a gate matrix F and F_s multiples of 64; without one any
 * multiple of 32 (a last, partly filled 128-row tile is padded with zero rows). */
int chimere_b200_moe_pack_prefill(const chimere_moe_layer* raw, void* d_arena, size_t bytes,
                                  chimere_moe_prefill_weights* out, cudaStream_t stream);
/* Extra scratch the prefill path needs for up to max_T tokens; pass it with ws->prefill_arena / prefill_bytes. */
size_t chimere_b200_moe_prefill_bytes(const chimere_moe_layer* w, int max_T);
/* y = MoE(x) like chimere_b200_moe_forward; `w` TILED32 (used for the small experts), `pw` its GEMM copy. */
int chimere_b200_moe_forward_prefill(const chimere_moe_layer* w, const chimere_moe_prefill_weights* pw,
                                     const float* d_x, float* d_y, int T, chimere_moe_workspace* ws,
                                     cudaStream_t stream);

/* The step in front of the layer in both of the reference's callers, and the layer, in one call:
 *   residual[t] += hidden[t];  normed[t] = residual[t] / sqrt(mean(residual[t]^2) + eps) * norm_weight;  y = MoE(normed)
 * fused_add_residual_rmsnorm (src/kernels/fused_ops.rs:91-140) followed by forward_moe_cudarc_with_cache, as called at
 * src/qwen35_model/compute_graph.rs:2063-2069, for T rows.  d_residual is updated in place; the normalised rows stay
 * inside the workspace.  pw: NULL = the decode kernels, else the prefill path (w must then be TILED32).  Same capture
 * rules as chimere_b200_moe_forward (src/qwen35_model/cuda_graph.rs:12-31: no allocation, no host synchronisation). */
int chimere_b200_moe_forward_residual_norm(const chimere_moe_layer* w, const chimere_moe_prefill_weights* pw,
                                           const float* d_hidden, float* d_residual, const float* d_norm_weight, float eps,
                                           float* d_y, int T, chimere_moe_workspace* ws, cudaStream_t stream);

/* Routing trace for the drafter tooling: the expert ids of the last routing in `ws` as d_trace[T][top_k] bytes, slots
 * in descending-score order -- the layout in which chimere-dflash/extract/target_daemon.cpp:18-23 stores the
 * "ffn_moe_topk-{L}" tensor of each captured layer.  d_expert_load (optional, int32 [E]): the number of pairs each
 * expert received is added to it (the per-expert load metric the reference logs, moe_ffn.rs:120-131). */
int chimere_b200_moe_routing_trace(const chimere_moe_layer* w, int T, const chimere_moe_workspace* ws, uint8_t* d_trace,
                                   int32_t* d_expert_load, cudaStream_t stream);

/* Expert-parallel owner rank, prefill-size batches: as chimere_b200_moe_experts (planes in ws->x_q / ws->x_d, local expert
 * ids in ws->topk_idx[n_rows], results in ws->pair_out[row][H]), with the local experts that received at least 8 rows on the
 * grouped GEMM.  pw_local: the GEMM copy of the local shard (chimere_b200_moe_pack_prefill of the shard); ws needs the
 * prefill arena.  No counterpart in the reference (single GPU, no prefill kernel). */
int chimere_b200_moe_experts_prefill(const chimere_moe_layer* w_local, const chimere_moe_prefill_weights* pw_local, int n_rows,
                                     chimere_moe_workspace* ws, cudaStream_t stream);
/* Expert-parallel home rank, prefill-size batches: chimere_b200_moe_shared_expert on the grouped GEMM.  pw: a GEMM copy that
 * holds the shared expert's matrices; ws needs the prefill arena.  Overwrites the work list of the routing call. */
int chimere_b200_moe_shared_expert_prefill(const chimere_moe_layer* w, const chimere_moe_prefill_weights* pw, int T,
                                           chimere_moe_workspace* ws, cudaStream_t stream);
/* The same on rows that lie where an exchange left them (the row format of chimere_b200_moe_ep_pack). */
int chimere_b200_moe_experts_packed_prefill(const chimere_moe_layer* w_local, const chimere_moe_prefill_weights* pw_local,
                                            int n_rows, const void* d_rows, int row_bytes, chimere_moe_workspace* ws,
                                            cudaStream_t stream);
/* Exact-size dispatch for a prefill-size batch: after chimere_b200_moe_route_home, ws->perm lists the T * top_k pairs sorted
 * by expert, i.e. grouped by owner rank (the ranks own contiguous expert ranges; ws->offsets[r * experts_per_rank] is
 * the first row for rank r).  Row j of d_send = pair perm[j] in the packed row format, d_slot[pair] = j.  The caller sends
 * the rank ranges with one all-to-all of exact sizes. */
int chimere_b200_moe_ep_pack_sorted(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws, void* d_send, int32_t* d_slot,
                                    int experts_per_rank, int row_bytes, cudaStream_t stream);

/* RMSNorm with unit weight over rows of length H: y = x / sqrt(mean(x^2) + eps). Used between
 * stacked layers. */
int chimere_b200_rmsnorm(const float* d_x, float* d_y, int T, int H, float eps, cudaStream_t stream);

/* Library/ABI version and the compute capability it was built for (100 = sm_100a). */
int chimere_b200_abi_version(void);
int chimere_b200_built_for_sm(void);

/* --------------------------------------------------------- legacy operator entries ------- */
/* Each replaces the function of the same name in chimere-server/ffi/ggml_cuda_gemv.cu. */

/* ggml_cuda_gemv.cu:184-194.  out needs pad(ncols,512)/32*36 bytes; blocks past ncols are zero. */
void chimere_quantize_q8_1(const float* input, void* output, int64_t ncols, int64_t ncols_padded,
                           cudaStream_t stream);
/* ggml_cuda_gemv.cu:393-404.  `batch` rows, output row stride = ncols_padded/32*36 bytes. */
void chimere_quantize_q8_1_batched(const float* input, void* output, int64_t ncols,
                                   int64_t ncols_padded, int batch, cudaStream_t stream);
/* ggml_cuda_gemv.cu:105-116 / 150-160: y[nrows] = W[nrows][ncols] . x_q8 */
void chimere_mmvq_iq3s(const void* weights, const void* input_q8, float* output, int ncols,
                       int nrows, int nrows_y_padded, cudaStream_t stream);
void chimere_mmvq_q8_0(const void* weights, const void* input_q8, float* output, int ncols,
                       int nrows, int nrows_y_padded, cudaStream_t stream);
/* New, same shape as the two above, for Q4_0 experts. */
void chimere_mmvq_q4_0(const void* weights, const void* input_q8, float* output, int ncols,
                       int nrows, int nrows_y_padded, cudaStream_t stream);
/* ggml_cuda_gemv.cu:322-352 (Rust declarations src/kernels/ggml_gpu.rs:173-193, call sites :933, :972): quantize the
 * f32 input row to Q8_1 into q8_scratch (ncols_padded / 32 * 36 bytes, ncols_padded = pad(ncols, 512); blocks past
 * ncols are zero), then y[nrows] = W . x_q8.  The Q4_0 variant is new, same shape. */
void chimere_mmvq_iq3s_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows,
                           int ncols_padded, void* q8_scratch, cudaStream_t stream);
void chimere_mmvq_q8_0_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows,
                           int ncols_padded, void* q8_scratch, cudaStream_t stream);
void chimere_mmvq_q4_0_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows,
                           int ncols_padded, void* q8_scratch, cudaStream_t stream);
/* ggml_cuda_gemv.cu:118-131, 147-172 and :302-321, 353-391 (Rust declarations src/kernels/ggml_gpu.rs:113-151, 162-216): the
 * K-quant matrices of the production files (the shared expert is Q5_K there, moe_ffn.rs:1597-1650).  ncols a multiple of
 * 256.  y = sum over 32-weight sub-blocks of d*d8*sc*dot - dmin*m*s8 (Q4_K, Q5_K) or d*d8*(sc_a*dot_a + sc_b*dot_b) (Q6_K). */
void chimere_mmvq_q5k(const void* weights, const void* input_q8, float* output, int ncols, int nrows, int nrows_y_padded,
                      cudaStream_t stream);
void chimere_mmvq_q4k(const void* weights, const void* input_q8, float* output, int ncols, int nrows, int nrows_y_padded,
                      cudaStream_t stream);
void chimere_mmvq_q6k(const void* weights, const void* input_q8, float* output, int ncols, int nrows, int nrows_y_padded,
                      cudaStream_t stream);
void chimere_mmvq_q5k_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows, int ncols_padded,
                          void* q8_scratch, cudaStream_t stream);
void chimere_mmvq_q4k_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows, int ncols_padded,
                          void* q8_scratch, cudaStream_t stream);
void chimere_mmvq_q6k_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows, int ncols_padded,
                          void* q8_scratch, cudaStream_t stream);
/* ggml_cuda_gemv.cu:243-279: top_k expert GEMVs in one launch, expert ids read on the device.
 * input_stride = 0: one shared Q8_1 input; otherwise bytes between the per-slot inputs. */
void chimere_mmvq_iq3s_batched(const void* all_weights, const void* input_q8, float* output,
                               const int* expert_ids, int ncols, int nrows, int nrows_y_padded,
                               int64_t expert_stride, int64_t input_stride, int top_k,
                               cudaStream_t stream);
/* New, same shape, for Q4_0 and Q8_0 experts. */
void chimere_mmvq_q4_0_batched(const void* all_weights, const void* input_q8, float* output,
                               const int* expert_ids, int ncols, int nrows, int nrows_y_padded,
                               int64_t expert_stride, int64_t input_stride, int top_k,
                               cudaStream_t stream);
void chimere_mmvq_q8_0_batched(const void* all_weights, const void* input_q8, float* output,
                               const int* expert_ids, int ncols, int nrows, int nrows_y_padded,
                               int64_t expert_stride, int64_t input_stride, int top_k,
                               cudaStream_t stream);
/* ggml_cuda_gemv.cu:196-209 */
int chimere_q8_1_block_bytes(void);   /* 36 */
int chimere_q8_1_block_elems(void);   /* 32 */
int chimere_matrix_row_padding(void); /* 512 */

/* ------------------------------------------------------------------------------------------------------------------
 * GGUF ingestion for this path (host side).  Replaces, for the MoE tensors, the reference's file parser
 * (src/gguf_loader.rs:286-455: header, metadata, tensor infos, data offset) and the per-layer tensor look-up of
 * compute_graph.rs:992-999, 1400-1500.  Tensor bytes are handed over as they lie in the file (the raw ggml blocks the
 * pack entries above take).  Errors: -1 bad argument, -2 shapes that do not fit, -9 I/O, -10 not a GGUF v2/v3 file or a
 * truncated one, -11 no such tensor / key. */
typedef struct chimere_gguf chimere_gguf;
typedef struct {
    int32_t ggml_type;     /* ggml type id (0 F32, 2 Q4_0, 8 Q8_0, 12-14 Q4_K/Q5_K/Q6_K, 21 IQ3_S, ...) */
    int32_t n_dims;
    int64_t dims[4];       /* innermost first, 1 beyond n_dims */
    int64_t file_offset;   /* absolute */
    int64_t nbytes;        /* -1: a type whose block size is not known here */
} chimere_gguf_tensor;
typedef struct {
    chimere_gguf_tensor router, gate_exps, up_exps, down_exps, sh_gate, sh_up, sh_down, sh_gate_proj;
    int32_t has_gate, has_shared, has_shared_gate, has_shared_gate_proj;
    int32_t H, E, F, F_s;
} chimere_gguf_moe_layer;
int chimere_b200_gguf_open(const char* path, chimere_gguf** out);
void chimere_b200_gguf_close(chimere_gguf* g);
int64_t chimere_b200_gguf_n_tensors(const chimere_gguf* g);
/* name of tensor i into buf (truncated to buflen - 1); returns its full length */
int chimere_b200_gguf_tensor_name(const chimere_gguf* g, int64_t i, char* buf, int buflen);
int chimere_b200_gguf_find(const chimere_gguf* g, const char* name, chimere_gguf_tensor* out);
/* the tensor's bytes into host memory (pinned, if an upload follows) */
int chimere_b200_gguf_read(const chimere_gguf* g, const chimere_gguf_tensor* t, void* dst, int64_t dst_bytes);
/* integer-valued metadata (any integer width, bool), e.g. "<arch>.expert_count", "<arch>.expert_used_count" */
int chimere_b200_gguf_meta_u64(const chimere_gguf* g, const char* key, uint64_t* out);
int chimere_b200_gguf_meta_str(const chimere_gguf* g, const char* key, char* buf, int buflen);
/* blk.<layer>.ffn_gate_inp / ffn_{gate,up,down}_exps / ffn_{gate,up,down}_shexp / ffn_gate_inp_shexp, shapes checked */
int chimere_b200_gguf_moe_layer(const chimere_gguf* g, int layer, chimere_gguf_moe_layer* out);

#ifdef __cplusplus
}
#endif
#endif /* CHIMERE_B200_MOE_H */
