// abi.cu -- host side of the library: the C ABI declared in include/chimere_b200_moe.h.
//
// The layer-level entries are the C++ counterpart of the reference's Rust orchestration
// (forward_moe_cudarc_with_cache, chimere-server/src/qwen35_model/moe_ffn.rs:1081-1768, and its
// scratch owner GgmlGpuBuffers, src/kernels/ggml_gpu.rs:292-407): they validate, lay the
// caller's arena out, and enqueue three kernels per call.  Nothing here allocates device
// memory or synchronises, except chimere_b200_moe_forward_host which waits for its stream.
#include <cstdio>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "kernels.h"
#include "tiled.cuh"

using namespace chimere;

namespace {

inline size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

inline bool type_ok(int t) { return t == CHIMERE_TYPE_Q4_0 || t == CHIMERE_TYPE_Q8_0 || t == CHIMERE_TYPE_IQ3_S; }
inline int type_cols_multiple(int t) { return t == CHIMERE_TYPE_IQ3_S ? 256 : 32; }

inline bool kquant_type(int t) { return t == CHIMERE_TYPE_Q4_K || t == CHIMERE_TYPE_Q5_K || t == CHIMERE_TYPE_Q6_K; }
// A layer whose shared expert is kept in K-quant super-blocks (the production files: Q5_K, moe_ffn.rs:1597-1650).  Its routed
// experts run as a layer without a shared expert; the shared expert follows as plain GEMVs on the raw blocks
// (kshared_chain below), which is how the reference runs it (three GEMV calls, an activation, the sigmoid-gated add).
inline bool kshared(const chimere_moe_layer* w) { return w && w->F_s > 0 && kquant_type(w->type_sh_up); }
inline chimere_moe_layer routed_only(const chimere_moe_layer* w) {
    chimere_moe_layer r = *w;
    r.F_s = 0; r.sh_gate = nullptr; r.sh_up = nullptr; r.sh_down = nullptr;
    r.type_sh_gate = r.type_sh_up = r.type_sh_down = 0;
    return r;   // (keeps shexp_gate_w: the router still computes the gate logit)
}

int validate_layer(const chimere_moe_layer* w) {
    if (!w) return -1;
    if (kshared(w)) {
        const bool dual_k = w->act == CHIMERE_ACT_SWIGLU;
        if (!kquant_type(w->type_sh_down) || (dual_k && !kquant_type(w->type_sh_gate))) return -3;
        if (w->H % 256 || w->F_s % 256) return -2;
        if (!w->sh_up || !w->sh_down || (dual_k && !w->sh_gate)) return -1;
        // the shared expert's f32 rows and Q8_1 intermediates borrow the routed pairs' areas of the workspace
        if (2 * (int64_t)w->F_s > (int64_t)w->top_k * w->H || (int64_t)w->F_s > (int64_t)w->top_k * w->F) return -2;
        const chimere_moe_layer r = routed_only(w);
        return validate_layer(&r);
    }
    if (w->H <= 0 || w->E <= 0 || w->E > kMaxExperts || w->F <= 0 || w->F_s < 0) return -2;
    if (w->top_k <= 0 || w->top_k > kMaxTopK || w->top_k > w->E) return -2;
    if (w->H % 32 || w->F % 32 || w->F_s % 32) return -2;
    if (w->layout != CHIMERE_LAYOUT_GGML && w->layout != CHIMERE_LAYOUT_TILED32) return -2;
    if (w->layout == CHIMERE_LAYOUT_TILED32 && w->H % 128) return -2;   // Q8_1 input rows must be 16-byte multiples
    if (w->route_mode != CHIMERE_ROUTE_SOFTMAX_RENORM && w->route_mode != CHIMERE_ROUTE_SIGMOID_NORM_SCALE) return -2;
    if (w->act != CHIMERE_ACT_SWIGLU && w->act != CHIMERE_ACT_RELU2) return -2;
    const bool dual = w->act == CHIMERE_ACT_SWIGLU;
    if (!type_ok(w->type_up) || !type_ok(w->type_down) || (dual && !type_ok(w->type_gate))) return -3;
    if (dual && w->type_gate != w->type_up) return -3;  // gate and up rows are streamed by one kernel instance
    if (w->H % type_cols_multiple(w->type_up) || w->F % type_cols_multiple(w->type_down)) return -2;
    if (!w->router_w || !w->up_exps || !w->down_exps || (dual && !w->gate_exps)) return -1;
    if (w->F_s > 0) {
        if (!type_ok(w->type_sh_up) || !type_ok(w->type_sh_down) || (dual && !type_ok(w->type_sh_gate))) return -3;
        if (dual && w->type_sh_gate != w->type_sh_up) return -3;
        if (w->H % type_cols_multiple(w->type_sh_up) || w->F_s % type_cols_multiple(w->type_sh_down)) return -2;
        if (!w->sh_up || !w->sh_down || (dual && !w->sh_gate)) return -1;
    }
    return 0;
}

struct Layout {
    size_t topk_idx, topk_w, logits, sh_logit, x_q8, perm, offsets, group_list, counters, inter_q8, pair_out, status, total;
    size_t x_q, x_d, inter_q, inter_d;
    int x_d_stride, inter_d_stride, Fmax;
    int max_entries, n_row_tiles, tile_rows, n_counters;
    int n_row_tiles_tiled;
    size_t inter_stride;
};

int max_entries_for(const chimere_moe_layer* w, int T) {
    const int P = T * w->top_k;
    return (w->E < P ? w->E : P) + P / kMaxGroupTokens + (w->F_s > 0 ? (T + shared_group_tokens(T) - 1) / shared_group_tokens(T) : 0);
}
// The same bound when the ids come from the library's own top-k (distinct within a token): an expert's pairs are cut into
// entries of kMaxGroupTokens, so with at most that many tokens no expert needs a second entry.  Sizes launch grids only.
int routed_entries_for(const chimere_moe_layer* w, int T) {
    const int P = T * w->top_k;
    const int extra = T <= kMaxGroupTokens ? 0 : P / kMaxGroupTokens;
    return (w->E < P ? w->E : P) + extra + (w->F_s > 0 ? (T + shared_group_tokens(T) - 1) / shared_group_tokens(T) : 0);
}

Layout make_layout(const chimere_moe_layer* w, int T) {
    if (kshared(w)) { const chimere_moe_layer r = routed_only(w); return make_layout(&r, T); }
    Layout L{};
    const int k = w->top_k, H = w->H, E = w->E;
    const int Fmax = w->F > w->F_s ? w->F : w->F_s;
    const size_t pairs = (size_t)T * k + (w->F_s > 0 ? T : 0);
    L.max_entries = max_entries_for(w, T);   // T = the workspace's capacity; a smaller batch may need a few more entries
    if (T > 8 && max_entries_for(w, 8) > L.max_entries) L.max_entries = max_entries_for(w, 8);   // (one-token shared entries up to T = 8)
    L.tile_rows = down_tile_rows(w->type_down, w->F, w->type_sh_down, w->F_s);
    L.n_row_tiles = (H + L.tile_rows - 1) / L.tile_rows;
    L.n_row_tiles_tiled = (H + 31) / 32;   // counters for the finest row tiling any batch size may choose
    const int max_tiles = L.n_row_tiles > L.n_row_tiles_tiled ? L.n_row_tiles : L.n_row_tiles_tiled;
    L.n_counters = kCtrRouteTile + (T + 7) / 8 + T * max_tiles;
    L.inter_stride = ((size_t)(Fmax / 32) * kQ81Bytes + 15) & ~(size_t)15;   // rows start on 16-byte boundaries (bulk copies)
    size_t o = 0;
    L.topk_idx = o; o += up256((size_t)T * k * 4);
    L.topk_w = o; o += up256((size_t)T * k * 4);
    L.logits = o; o += up256((size_t)T * E * 4);
    L.sh_logit = o; o += up256((size_t)T * 4);
    L.x_q8 = o; o += up256((size_t)T * (H / 32) * kQ81Bytes);
    L.perm = o; o += up256((size_t)T * k * 4);
    L.offsets = o; o += up256((size_t)(E + 1) * 4);
    L.group_list = o; o += up256((size_t)(kListHeader + kListEntry * L.max_entries) * 4);
    L.counters = o; o += up256((size_t)L.n_counters * 4);
    L.inter_q8 = o; o += up256(pairs * L.inter_stride);
    L.pair_out = o; o += up256(pairs * H * 4);
    L.Fmax = Fmax;
    L.x_d_stride = (H / 32 + 3) & ~3;
    L.inter_d_stride = (Fmax / 32 + 3) & ~3;
    L.x_q = o; o += up256((size_t)T * H);
    L.x_d = o; o += up256((size_t)T * L.x_d_stride * 4);
    L.inter_q = o; o += up256(pairs * Fmax);
    L.inter_d = o; o += up256(pairs * L.inter_d_stride * 4);
    L.status = o; o += 256;
    L.total = o;
    return L;
}

int cuda_rc(cudaError_t e) { return e == cudaSuccess ? 0 : -100 - (int)e; }

}  // namespace

extern "C" {

int chimere_b200_abi_version(void) { return 1; }
int chimere_b200_built_for_sm(void) { return 100; }

size_t chimere_b200_moe_workspace_bytes(const chimere_moe_layer* w, int max_T) {
    if (validate_layer(w) != 0 || max_T <= 0) return 0;
    return make_layout(w, max_T).total;
}

int chimere_b200_moe_workspace_init(chimere_moe_workspace* ws, void* d_arena, size_t bytes, const chimere_moe_layer* w,
                                    int max_T, cudaStream_t stream) {
    if (!ws || !d_arena) return -1;
    int rc = validate_layer(w);
    if (rc) return rc;
    if (max_T <= 0) return -2;
    if ((uintptr_t)d_arena & 255) return -5;
    const Layout L = make_layout(w, max_T);
    if (bytes < L.total) return -4;
    uint8_t* base = (uint8_t*)d_arena;
    std::memset(ws, 0, sizeof(*ws));
    ws->max_T = max_T;
    ws->topk_idx = (int32_t*)(base + L.topk_idx);
    ws->topk_w = (float*)(base + L.topk_w);
    ws->router_logits = (float*)(base + L.logits);
    ws->sh_gate_logit = (float*)(base + L.sh_logit);
    ws->x_q8 = base + L.x_q8;
    ws->perm = (int32_t*)(base + L.perm);
    ws->offsets = (int32_t*)(base + L.offsets);
    ws->group_list = (int32_t*)(base + L.group_list);
    ws->counters = (int32_t*)(base + L.counters);
    ws->inter_q8 = base + L.inter_q8;
    ws->pair_out = (float*)(base + L.pair_out);
    ws->x_q = (int8_t*)(base + L.x_q);
    ws->x_d = (float*)(base + L.x_d);
    ws->inter_q = (int8_t*)(base + L.inter_q);
    ws->inter_d = (float*)(base + L.inter_d);
    ws->status = (int32_t*)(base + L.status);
    cudaError_t e = cudaMemsetAsync(ws->counters, 0, (size_t)L.n_counters * 4, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(ws->status, 0, 256, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(ws->group_list, 0, (size_t)(kListHeader + kListEntry * L.max_entries) * 4, stream);
    return cuda_rc(e);
}

static RouteParams route_params(const chimere_moe_layer* w, const float* d_x, int T, chimere_moe_workspace* ws, bool keep_gate_vector = false) {
    RouteParams p{};
    p.T = T; p.H = w->H; p.E = w->E; p.top_k = w->top_k; p.route_mode = w->route_mode;
    p.has_shared = w->F_s > 0;
    p.route_scale = w->route_scale;
    p.x = d_x; p.router_w = w->router_w; p.router_bias = w->router_bias;
    p.shexp_gate_w = (w->F_s > 0 || keep_gate_vector) ? w->shexp_gate_w : nullptr;
    p.router_logits = ws->router_logits; p.sh_gate_logit = ws->sh_gate_logit;
    p.topk_idx = ws->topk_idx; p.topk_w = ws->topk_w; p.x_q8 = ws->x_q8;
    p.perm = ws->perm; p.offsets = ws->offsets; p.group_list = ws->group_list; p.counters = ws->counters;
    p.x_soa_q = ws->x_q; p.x_soa_d = ws->x_d; p.x_soa_d_stride = (w->H / 32 + 3) & ~3;
    p.status = ws->status;
    // the dispatch of a large batch counts in the memory of the down stage's combine counters (zero between the stages'
    // uses, and large enough from a few dozen tokens on)
    const Layout L = make_layout(w, ws->max_T);
    const size_t combine_ints = (size_t)L.n_counters - kCtrRouteTile - (ws->max_T + 7) / 8;
    const size_t need = (size_t)((T * w->top_k + 127) / 128) * 256 + 260;
    p.dispatch_scratch = need <= combine_ints ? ws->counters + kCtrRouteTile + (ws->max_T + 7) / 8 : nullptr;
    return p;
}

static int check_call(const chimere_moe_layer* w, const void* a, const void* b, int T, const chimere_moe_workspace* ws,
                      bool allow_kquant_shared = false) {
    int rc = validate_layer(w);
    if (rc) return rc;
    if (kshared(w) && !allow_kquant_shared) return -6;   // only the whole-layer entries take a K-quant shared expert
    if (!a || !b || !ws || !ws->counters) return -1;
    if (T <= 0 || T > ws->max_T) return -2;
    return 0;
}

int chimere_b200_moe_route(const chimere_moe_layer* w, const float* d_x, int T, chimere_moe_workspace* ws,
                           cudaStream_t stream) {
    int rc = check_call(w, d_x, d_x, T, ws);
    if (rc) return rc;
    return cuda_rc(launch_route(route_params(w, d_x, T, ws), stream));
}

static int kshared_chain(const chimere_moe_layer* w, int T, float* d_y, chimere_moe_workspace* ws, cudaStream_t stream);
static GemvParams gate_up_params(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws, const Layout& L);
static GemvParams down_params(const chimere_moe_layer* w, float* d_y, int T, chimere_moe_workspace* ws, const Layout& L);

int chimere_b200_moe_permute(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws, cudaStream_t stream) {
    // The routing launch already leaves perm / offsets / the work list behind; this entry is for callers
    // that write ws->topk_idx themselves.  It runs only the dispatch step (no shared-expert entries).
    int rc = check_call(w, ws, ws, T, ws);
    if (rc) return rc;
    RouteParams p = route_params(w, nullptr, T, ws);
    p.has_shared = 0;
    return cuda_rc(launch_permute(p, stream));
}

// ---------------------------------------------------------------- expert-parallel pieces ----
int chimere_b200_moe_route_home(const chimere_moe_layer* w, const float* d_x, int T, chimere_moe_workspace* ws,
                                cudaStream_t stream) {
    int rc = check_call(w, d_x, d_x, T, ws);
    if (rc) return rc;
    RouteParams p = route_params(w, d_x, T, ws);
    p.list_mode = 1;   // work list: shared-expert entries only; the routed pairs go to their owners
    return cuda_rc(launch_route(p, stream));
}

int chimere_b200_moe_shared_expert(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws, cudaStream_t stream) {
    int rc = check_call(w, ws, ws, T, ws);
    if (rc) return rc;
    if (w->layout != CHIMERE_LAYOUT_TILED32) return -2;
    if (w->F_s <= 0) return 0;
    const Layout L = make_layout(w, ws->max_T);
    const int max_entries = (T + shared_group_tokens(T) - 1) / shared_group_tokens(T);   // the home rank's list holds nothing else
    cudaError_t e = launch_gate_up_tiled(gate_up_params(w, T, ws, L), max_entries, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    GemvParams g = down_params(w, nullptr, T, ws, L);
    g.no_combine = 1;
    return cuda_rc(launch_down_tiled(g, max_entries, stream));
}

static int run_experts(const chimere_moe_layer* w_local, int n_rows, const void* d_packed, int row_bytes, chimere_moe_workspace* ws,
                       cudaStream_t stream, int32_t* wait_flags = nullptr, int wait_n = 0, int wait_expect = 0) {
    if (n_rows == 0) return 0;
    int rc = check_call(w_local, ws, ws, n_rows, ws);
    if (rc) return rc;
    if (w_local->layout != CHIMERE_LAYOUT_TILED32 || w_local->top_k != 1 || w_local->F_s != 0) return -2;
    const int ds = (w_local->H / 32 + 3) & ~3;
    if (d_packed && (row_bytes % 16 || row_bytes < w_local->H + 4 * ds + 4)) return -2;
    RouteParams p = route_params(w_local, nullptr, n_rows, ws);
    p.has_shared = 0;
    if (d_packed) {   // ids sit behind the planes of every packed row
        p.topk_idx = (int32_t*)((uint8_t*)d_packed + w_local->H + 4 * ds);
        p.idx_stride = row_bytes / 4;
    }
    p.wait_flags = wait_flags; p.wait_n = wait_n; p.wait_expect = wait_expect;
    cudaError_t e = launch_permute(p, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    const Layout L = make_layout(w_local, ws->max_T);
    const int max_entries = max_entries_for(w_local, n_rows);
    GemvParams gu = gate_up_params(w_local, n_rows, ws, L);
    if (d_packed) {
        gu.in_soa_q = (const int8_t*)d_packed; gu.in_soa_q_stride = row_bytes;
        gu.in_soa_d = (const float*)((const uint8_t*)d_packed + w_local->H); gu.in_soa_d_stride = row_bytes / 4;
        gu.few_tokens = 1;   // a fixed-size exchange: most of the n_rows slots carry no pair
    }
    e = launch_gate_up_tiled(gu, max_entries, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    GemvParams g = down_params(w_local, nullptr, n_rows, ws, L);
    g.no_combine = 1;
    g.few_tokens = d_packed ? 1 : 0;
    return cuda_rc(launch_down_tiled(g, max_entries, stream));
}

int chimere_b200_moe_experts(const chimere_moe_layer* w_local, int n_rows, chimere_moe_workspace* ws, cudaStream_t stream) {
    return run_experts(w_local, n_rows, nullptr, 0, ws, stream);
}

int chimere_b200_moe_experts_packed(const chimere_moe_layer* w_local, int n_rows, const void* d_rows, int row_bytes,
                                    chimere_moe_workspace* ws, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    if (!d_rows) return -1;
    return run_experts(w_local, n_rows, d_rows, row_bytes, ws, stream);
}

int chimere_b200_moe_experts_packed_p2p(const chimere_moe_layer* w_local, int n_rows, const void* d_rows, int row_bytes, int32_t* d_flags,
                                        int world, int cap, chimere_moe_workspace* ws, cudaStream_t stream) {
    if (!d_rows || !d_flags) return -1;
    if (world <= 0 || world > 32 || cap <= 0) return -2;
    return run_experts(w_local, n_rows, d_rows, row_bytes, ws, stream, d_flags, world, cap);
}

int chimere_b200_moe_ep_pack(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws, void* d_send, int32_t* d_slot,
                             int experts_per_rank, int world, int cap, int row_bytes, cudaStream_t stream) {
    int rc = check_call(w, d_send, d_slot, T, ws);
    if (rc) return rc;
    const int ds = (w->H / 32 + 3) & ~3;
    if (experts_per_rank <= 0 || world <= 0 || world * experts_per_rank != w->E || cap < T * w->top_k) return -2;
    if (row_bytes % 16 || row_bytes < w->H + 4 * ds + 4 || w->H % 16) return -2;
    return cuda_rc(launch_ep_pack(ws->topk_idx, ws->x_q, ws->x_d, ds, (uint8_t*)d_send, d_slot, T, w->top_k, w->H, experts_per_rank,
                                  world, cap, row_bytes, stream));
}

int chimere_b200_moe_ep_finish(const chimere_moe_layer* w, const float* d_rows, const int32_t* d_slot, int T,
                               chimere_moe_workspace* ws, float* d_y, cudaStream_t stream) {
    int rc = check_call(w, d_rows, d_y, T, ws);
    if (rc) return rc;
    const float* shared_rows = w->F_s > 0 ? ws->pair_out + (size_t)T * w->top_k * w->H : nullptr;
    const float* logit = (w->F_s > 0 && w->shexp_gate_w) ? ws->sh_gate_logit : nullptr;
    return cuda_rc(launch_ep_finish(d_rows, d_slot, ws->topk_w, shared_rows, logit, d_y, T, w->H, w->top_k, stream));
}

// ---- exchange by peer stores (decode-size batches) ----
int chimere_b200_moe_ep_pack_p2p(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws, void* const* d_peer_recv,
                                 int32_t* const* d_peer_flags, int32_t* d_ctr, int rank, int experts_per_rank, int world, int cap,
                                 int row_bytes, cudaStream_t stream) {
    int rc = check_call(w, d_peer_recv, d_peer_flags, T, ws);
    if (rc) return rc;
    if (!d_ctr) return -1;
    const int ds = (w->H / 32 + 3) & ~3;
    if (experts_per_rank <= 0 || world <= 0 || world * experts_per_rank != w->E || cap < T * w->top_k || rank < 0 || rank >= world) return -2;
    if (row_bytes % 16 || row_bytes < w->H + 4 * ds + 12 || w->H % 16) return -2;
    (void)d_ctr;
    return cuda_rc(launch_ep_pack_p2p(ws->topk_idx, ws->topk_w, ws->x_q, ws->x_d, ds, (uint8_t* const*)d_peer_recv, d_peer_flags, rank, T,
                                      w->top_k, w->H, experts_per_rank, world, cap, row_bytes, stream));
}

int chimere_b200_moe_ep_wait(int32_t* d_flags, int world, int cap, chimere_moe_workspace* ws, cudaStream_t stream) {
    if (!d_flags || !ws) return -1;
    if (world <= 0 || world > 32 || cap <= 0) return -2;
    return cuda_rc(launch_ep_wait_flags(d_flags, world, cap, ws->status, stream));
}

int chimere_b200_moe_ep_return_p2p(const chimere_moe_layer* w_local, chimere_moe_workspace* ws_owner, const void* d_rows, int row_bytes,
                                   float* const* d_peer_back, int32_t* const* d_peer_flags, int32_t* d_ctr, int rank, int world, int T, int cap,
                                   cudaStream_t stream) {
    if (!w_local || !ws_owner || !ws_owner->pair_out || !d_rows || !d_peer_back || !d_peer_flags || !d_ctr) return -1;
    const int ds = (w_local->H / 32 + 3) & ~3;
    if (world <= 0 || rank < 0 || rank >= world || T <= 0 || cap <= 0 || world * cap > ws_owner->max_T) return -2;
    if (row_bytes % 16 || row_bytes < w_local->H + 4 * ds + 12) return -2;
    (void)d_ctr;
    return cuda_rc(launch_ep_return_p2p(ws_owner->pair_out, (const uint8_t*)d_rows, row_bytes, w_local->H + 4 * ds, d_peer_back, d_peer_flags,
                                        rank, world, T, cap, w_local->H, stream));
}

int chimere_b200_moe_ep_finish_p2p(const chimere_moe_layer* w, const float* d_back, int32_t* d_flags, int world, int T,
                                   chimere_moe_workspace* ws, float* d_y, int32_t* d_ctr, cudaStream_t stream) {
    int rc = check_call(w, d_back, d_y, T, ws);
    if (rc) return rc;
    if (!d_flags || !d_ctr) return -1;
    if (world <= 0 || world > 32) return -2;
    const float* shared_rows = w->F_s > 0 ? ws->pair_out + (size_t)T * w->top_k * w->H : nullptr;
    const float* logit = (w->F_s > 0 && w->shexp_gate_w) ? ws->sh_gate_logit : nullptr;
    return cuda_rc(launch_ep_finish_p2p(d_back, d_flags, world, shared_rows, logit, d_y, T, w->H, d_ctr, ws->status, stream));
}

static GemvParams gate_up_params(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws, const Layout& L) {
    GemvParams g{};
    g.T = T; g.top_k = w->top_k; g.H = w->H;
    g.act = w->act;
    g.group_list = ws->group_list; g.perm = ws->perm;
    g.status = ws->status;
    g.ncols_routed = w->H; g.ncols_shared = w->H;
    g.nrows_routed = w->F; g.nrows_shared = w->F_s;
    g.type_routed = w->type_up; g.type_shared = w->type_sh_up;
    g.w_a = (const uint8_t*)w->gate_exps; g.w_b = (const uint8_t*)w->up_exps;
    g.stride_a = w->stride_gate; g.stride_b = w->stride_up;
    g.sh_a = (const uint8_t*)w->sh_gate; g.sh_b = (const uint8_t*)w->sh_up;
    g.in_q8 = ws->x_q8; g.in_stride = (int64_t)(w->H / 32) * kQ81Bytes;
    g.inter_q8 = ws->inter_q8; g.inter_stride = (int64_t)L.inter_stride;
    g.in_soa_q = ws->x_q; g.in_soa_q_stride = w->H; g.in_soa_d = ws->x_d; g.in_soa_d_stride = L.x_d_stride;
    g.out_soa_q = ws->inter_q; g.out_soa_q_stride = L.Fmax; g.out_soa_d = ws->inter_d; g.out_soa_d_stride = L.inter_d_stride;
    return g;
}

static GemvParams down_params(const chimere_moe_layer* w, float* d_y, int T, chimere_moe_workspace* ws, const Layout& L) {
    GemvParams g{};
    g.T = T; g.top_k = w->top_k; g.H = w->H;
    g.act = w->act;
    g.group_list = ws->group_list; g.perm = ws->perm;
    g.status = ws->status;
    g.ncols_routed = w->F; g.ncols_shared = w->F_s;
    g.nrows_routed = w->H; g.nrows_shared = w->F_s > 0 ? w->H : 0;
    g.type_routed = w->type_down; g.type_shared = w->type_sh_down;
    g.w_a = (const uint8_t*)w->down_exps; g.stride_a = w->stride_down;
    g.sh_a = (const uint8_t*)w->sh_down;
    g.in_q8 = ws->inter_q8; g.in_stride = (int64_t)L.inter_stride;
    g.in_soa_q = ws->inter_q; g.in_soa_q_stride = L.Fmax; g.in_soa_d = ws->inter_d; g.in_soa_d_stride = L.inter_d_stride;
    g.pair_out = ws->pair_out; g.topk_w = ws->topk_w;
    g.sh_gate_logit = (w->F_s > 0 && w->shexp_gate_w) ? ws->sh_gate_logit : nullptr;
    g.y = d_y;
    g.combine_ctr = ws->counters + kCtrRouteTile + (ws->max_T + 7) / 8;
    g.tile_rows = L.tile_rows;
    g.n_row_tiles = (w->layout == CHIMERE_LAYOUT_TILED32)
                        ? (w->H + 32 * tiled_down_geom(w->type_down, w->F, w->type_sh_down, w->F_s, T).wr - 1) /
                              (32 * tiled_down_geom(w->type_down, w->F, w->type_sh_down, w->F_s, T).wr)
                        : L.n_row_tiles;
    return g;
}

static cudaError_t run_gate_up(const chimere_moe_layer* w, const GemvParams& g, int max_entries, cudaStream_t stream) {
    return w->layout == CHIMERE_LAYOUT_TILED32 ? launch_gate_up_tiled(g, max_entries, stream) : launch_gate_up(g, max_entries, stream);
}
static cudaError_t run_down(const chimere_moe_layer* w, const GemvParams& g, int max_entries, cudaStream_t stream) {
    return w->layout == CHIMERE_LAYOUT_TILED32 ? launch_down_tiled(g, max_entries, stream) : launch_down(g, max_entries, stream);
}

// ---- tiled32 packing ----
struct PackPlan { size_t gate, up, down, sh_gate, sh_up, sh_down, total; int64_t sg, su, sd; };
static PackPlan pack_plan(const chimere_moe_layer* w) {
    PackPlan P{};
    const bool dual = w->act == CHIMERE_ACT_SWIGLU;
    size_t o = 0;
    P.su = tiled_matrix_bytes(w->type_up, w->F, w->H);
    P.sg = dual ? tiled_matrix_bytes(w->type_gate, w->F, w->H) : 0;
    P.sd = tiled_matrix_bytes(w->type_down, w->H, w->F);
    P.gate = o; o += up256((size_t)P.sg * w->E);
    P.up = o; o += up256((size_t)P.su * w->E);
    P.down = o; o += up256((size_t)P.sd * w->E);
    if (w->F_s > 0) {
        P.sh_gate = o; o += dual ? up256((size_t)tiled_matrix_bytes(w->type_sh_gate, w->F_s, w->H)) : 0;
        P.sh_up = o; o += up256((size_t)tiled_matrix_bytes(w->type_sh_up, w->F_s, w->H));
        P.sh_down = o; o += up256((size_t)tiled_matrix_bytes(w->type_sh_down, w->H, w->F_s));
    }
    P.total = o;
    return P;
}

size_t chimere_b200_moe_pack_bytes(const chimere_moe_layer* raw) {
    if (validate_layer(raw) != 0 || raw->layout != CHIMERE_LAYOUT_GGML) return 0;
    if (kshared(raw)) { const chimere_moe_layer r = routed_only(raw); return pack_plan(&r).total; }
    return pack_plan(raw).total;
}

int chimere_b200_moe_pack(const chimere_moe_layer* raw, void* d_arena, size_t bytes, chimere_moe_layer* packed,
                          cudaStream_t stream) {
    int rc = validate_layer(raw);
    if (rc) return rc;
    if (!d_arena || !packed) return -1;
    if (kshared(raw)) {   // the routed experts are re-tiled; the K-quant shared matrices stay where and as they are
        const chimere_moe_layer r = routed_only(raw);
        rc = chimere_b200_moe_pack(&r, d_arena, bytes, packed, stream);
        if (rc) return rc;
        packed->F_s = raw->F_s; packed->sh_gate = raw->sh_gate; packed->sh_up = raw->sh_up; packed->sh_down = raw->sh_down;
        packed->type_sh_gate = raw->type_sh_gate; packed->type_sh_up = raw->type_sh_up; packed->type_sh_down = raw->type_sh_down;
        return 0;
    }
    if (raw->layout != CHIMERE_LAYOUT_GGML) return -2;
    if ((uintptr_t)d_arena & 255) return -5;
    const PackPlan P = pack_plan(raw);
    if (bytes < P.total) return -4;
    const bool dual = raw->act == CHIMERE_ACT_SWIGLU;
    uint8_t* base = (uint8_t*)d_arena;
    *packed = *raw;
    packed->layout = CHIMERE_LAYOUT_TILED32;
    cudaError_t e = cudaSuccess;
    if (dual) {
        e = launch_pack(raw->type_gate, raw->gate_exps, base + P.gate, raw->E, raw->F, raw->H, raw->stride_gate, P.sg, stream);
        packed->gate_exps = base + P.gate; packed->stride_gate = P.sg;
    }
    if (e == cudaSuccess) e = launch_pack(raw->type_up, raw->up_exps, base + P.up, raw->E, raw->F, raw->H, raw->stride_up, P.su, stream);
    packed->up_exps = base + P.up; packed->stride_up = P.su;
    if (e == cudaSuccess) e = launch_pack(raw->type_down, raw->down_exps, base + P.down, raw->E, raw->H, raw->F, raw->stride_down, P.sd, stream);
    packed->down_exps = base + P.down; packed->stride_down = P.sd;
    if (raw->F_s > 0) {
        if (dual) {
            if (e == cudaSuccess) e = launch_pack(raw->type_sh_gate, raw->sh_gate, base + P.sh_gate, 1, raw->F_s, raw->H, 0, 0, stream);
            packed->sh_gate = base + P.sh_gate;
        }
        if (e == cudaSuccess) e = launch_pack(raw->type_sh_up, raw->sh_up, base + P.sh_up, 1, raw->F_s, raw->H, 0, 0, stream);
        packed->sh_up = base + P.sh_up;
        if (e == cudaSuccess) e = launch_pack(raw->type_sh_down, raw->sh_down, base + P.sh_down, 1, raw->H, raw->F_s, 0, 0, stream);
        packed->sh_down = base + P.sh_down;
    }
    return cuda_rc(e);
}

size_t chimere_b200_packed_matrix_bytes(int wtype, int nrows, int ncols) {
    if (!type_ok(wtype) || nrows <= 0 || nrows % 32 || ncols <= 0 || ncols % type_cols_multiple(wtype)) return 0;
    return (size_t)tiled_matrix_bytes(wtype, nrows, ncols);
}

int chimere_b200_pack_matrix(int wtype, const void* d_raw, void* d_out, int nrows, int ncols, cudaStream_t stream) {
    if (!d_raw || !d_out) return -1;
    if (!type_ok(wtype)) return -3;
    if (nrows <= 0 || nrows % 32 || ncols <= 0 || ncols % type_cols_multiple(wtype)) return -2;
    return cuda_rc(launch_pack(wtype, d_raw, d_out, 1, nrows, ncols, 0, 0, stream));
}

int chimere_b200_block_sumi_tiled(int wtype, const void* d_packed, const void* d_xq8, int32_t* d_sumi, int ncols, int nrows,
                                  cudaStream_t stream) {
    if (!d_packed || !d_xq8 || !d_sumi) return -1;
    if (!type_ok(wtype)) return -3;
    if (ncols <= 0 || nrows < 0 || nrows % 32 || ncols % type_cols_multiple(wtype)) return -2;
    return cuda_rc(launch_block_sumi_tiled(wtype, d_packed, d_xq8, d_sumi, ncols, nrows, stream));
}

int chimere_b200_moe_gate_up(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws, cudaStream_t stream) {
    int rc = check_call(w, ws, ws, T, ws);
    if (rc) return rc;
    const Layout L = make_layout(w, ws->max_T);
    return cuda_rc(run_gate_up(w, gate_up_params(w, T, ws, L), max_entries_for(w, T), stream));
}

int chimere_b200_moe_down_combine(const chimere_moe_layer* w, float* d_y, int T, chimere_moe_workspace* ws,
                                  cudaStream_t stream) {
    int rc = check_call(w, d_y, d_y, T, ws);
    if (rc) return rc;
    const Layout L = make_layout(w, ws->max_T);
    return cuda_rc(run_down(w, down_params(w, d_y, T, ws, L), max_entries_for(w, T), stream));
}

int chimere_b200_moe_forward(const chimere_moe_layer* w, const float* d_x, float* d_y, int T, chimere_moe_workspace* ws,
                             cudaStream_t stream) {
    int rc = check_call(w, d_x, d_y, T, ws, true);
    if (rc) return rc;
    const bool ks = kshared(w);
    const chimere_moe_layer wr_ = ks ? routed_only(w) : *w;
    const chimere_moe_layer* wr = &wr_;
    const Layout L = make_layout(wr, ws->max_T);
    const int max_entries = routed_entries_for(wr, T);
    cudaError_t e = launch_route(route_params(wr, d_x, T, ws, ks), stream);
    if (e != cudaSuccess) return cuda_rc(e);
    e = run_gate_up(wr, gate_up_params(wr, T, ws, L), max_entries, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    e = run_down(wr, down_params(wr, d_y, T, ws, L), max_entries, stream);
    if (e != cudaSuccess || !ks) return cuda_rc(e);
    return kshared_chain(w, T, d_y, ws, stream);
}

int chimere_b200_moe_forward_host(const chimere_moe_layer* w, const float* h_x, float* h_y, int T, float* d_x, float* d_y,
                                  chimere_moe_workspace* ws, cudaStream_t stream) {
    if (!h_x || !h_y) return -1;
    int rc = check_call(w, d_x, d_y, T, ws, true);
    if (rc) return rc;
    const size_t bytes = (size_t)T * w->H * sizeof(float);
    cudaError_t e = cudaMemcpyAsync(d_x, h_x, bytes, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    // A pinned result buffer is addressable from the device under a pointer of its own: the last kernel then stores y
    // straight into host memory and the copy back (a second trip through the copy engine, serial behind the kernels) is
    // not needed.  Pageable memory, or a K-quant shared expert (whose last step reads y back), takes the staged copy.
    float* y_dev = d_y;
    cudaPointerAttributes attr{};
    if (!kshared(w) && cudaPointerGetAttributes(&attr, h_y) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer)
        y_dev = static_cast<float*>(attr.devicePointer);
    else
        (void)cudaGetLastError();   // (an unregistered pointer leaves an error behind on older runtimes)
    rc = chimere_b200_moe_forward(w, d_x, y_dev, T, ws, stream);
    if (rc) return rc;
    if (y_dev == d_y) {
        e = cudaMemcpyAsync(h_y, d_y, bytes, cudaMemcpyDeviceToHost, stream);
        if (e != cudaSuccess) return cuda_rc(e);
    }
    return cuda_rc(cudaStreamSynchronize(stream));
}

int chimere_b200_block_sumi(int wtype, const void* d_w, const void* d_xq8, int32_t* d_sumi, int ncols, int nrows,
                            cudaStream_t stream) {
    if (!d_w || !d_xq8 || !d_sumi) return -1;
    if (!type_ok(wtype)) return -3;
    if (ncols <= 0 || nrows < 0 || ncols % type_cols_multiple(wtype)) return -2;
    return cuda_rc(launch_block_sumi(wtype, d_w, d_xq8, d_sumi, ncols, nrows, stream));
}

// ---------------------------------------------------------------- tcgen05 block-scaled GEMM --
size_t chimere_b200_mma128_bytes(int rows, int cols) {
    if (rows <= 0 || cols <= 0 || cols % 32) return 0;
    return (size_t)((rows + 127) / 128) * (cols / 32) * (4096 + 512);
}

int chimere_b200_pack_mma128(const int8_t* d_q, const float* d_scales, void* d_out, int rows, int cols, cudaStream_t stream) {
    if (!d_q || !d_scales || !d_out) return -1;
    if (rows <= 0 || cols <= 0 || cols % 32) return -2;
    return cuda_rc(launch_pack_mma128(d_q, d_scales, (uint8_t*)d_out, rows, cols, stream));
}

int chimere_b200_gemm_i8(const void* d_a, const void* d_b, int rows, int tokens, int cols, float* d_out, void* d_items,
                         int32_t* d_status, cudaStream_t stream) {
    if (!d_a || !d_b || !d_out || !d_items || !d_status) return -1;
    if (rows <= 0 || tokens <= 0 || cols <= 0 || cols % 32) return -2;
    const int rt = (rows + 127) / 128, tt = (tokens + 127) / 128, nb = cols / 32;
    std::vector<GemmItem> items;
    for (int i = 0; i < rt; ++i)
        for (int j = 0; j < tt; ++j) {
            GemmItem it{};
            it.a_offset = (int64_t)i * nb * (4096 + 512);
            it.b_offset = (int64_t)j * nb * (4096 + 512);
            it.n_valid = tokens - j * 128 < 128 ? tokens - j * 128 : 128;
            it.rows_valid = rows - i * 128 < 128 ? rows - i * 128 : 128;
            it.out_row0 = i * 128; it.out_col0 = j * 128;
            items.push_back(it);
        }
    cudaError_t e = cudaMemcpyAsync(d_items, items.data(), items.size() * sizeof(GemmItem), cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    int32_t* counter = (int32_t*)((uint8_t*)d_items + items.size() * sizeof(GemmItem));   // the tile counter sits behind the list
    e = cudaMemsetAsync(counter, 0, 256, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    e = cudaStreamSynchronize(stream);   // the host vector goes away; this entry is a test primitive, not the hot path
    if (e != cudaSuccess) return cuda_rc(e);
    GemmParams p{};
    p.a_base = (const uint8_t*)d_a; p.b_base = (const uint8_t*)d_b; p.items = (const GemmItem*)d_items; p.nblocks = nb;
    p.out = d_out; p.ldo = tokens; p.status = d_status;
    return cuda_rc(launch_gemm_i8_f32(p, (int)items.size(), counter, stream));
}

int chimere_b200_mma_i8_probe(int n_mma, int n_cols, int n_acc, int32_t* d_status, cudaStream_t stream) {
    if (n_mma <= 0 || n_mma % 64 || (n_cols != 128 && n_cols != 256) || n_acc < 1 || n_acc * n_cols > 512) return -2;
    return launch_mma_i8_probe(n_mma, n_cols, n_acc, d_status, stream);
}

// ---------------------------------------------------------------- prefill path ----
namespace {
constexpr int kGemmMin = 8;           // pairs an expert needs to go to the GEMM (a partly filled tile costs the read-back
                                      // warps only its own columns; eight tokens on the GEMV kernels cost eight passes of dp4a)
constexpr size_t kMmaTile = 4096 + 512;
int n_tiles_max_for(const chimere_moe_layer* w, int T) {
    const int P = T * w->top_k;
    int big = P / kGemmMin; if (big > w->E) big = w->E;
    return P / 128 + big + (w->F_s > 0 ? (T + 127) / 128 : 0) + 1;
}
struct PrefillPlan { size_t gu, down, sh_gu, sh_down, total; int64_t sgu, sdown; int rows_per_tile; };
PrefillPlan prefill_plan(const chimere_moe_layer* w) {
    PrefillPlan P{};
    const bool dual = w->act == CHIMERE_ACT_SWIGLU;
    P.rows_per_tile = dual ? 64 : 128;
    const size_t nbH = w->H / 32;
    P.sgu = (int64_t)((w->F + P.rows_per_tile - 1) / P.rows_per_tile) * nbH * kMmaTile;   // a last, partly filled row tile is zero-padded
    P.sdown = (int64_t)(w->H / 128) * (w->F / 32) * kMmaTile;
    size_t o = 0;
    P.gu = o; o += up256((size_t)P.sgu * w->E);
    P.down = o; o += up256((size_t)P.sdown * w->E);
    if (w->F_s > 0) {
        P.sh_gu = o; o += up256((size_t)((w->F_s + P.rows_per_tile - 1) / P.rows_per_tile) * nbH * kMmaTile);
        P.sh_down = o; o += up256((size_t)(w->H / 128) * (w->F_s / 32) * kMmaTile);
    }
    P.total = o;
    return P;
}
int prefill_dims_ok(const chimere_moe_layer* w) {
    // gated experts: 64 gate rows and their 64 up rows share a tile; ungated ones may end in a partly filled tile
    const int rpt = w->act == CHIMERE_ACT_SWIGLU ? 64 : 32;
    if (w->H % 128 || w->F % rpt || w->F_s % rpt) return 0;
    return 1;
}
struct PrefillArena { size_t tiles, bx, b2, total; int64_t bx_stride, b2_stride; int n_tiles_max; };
PrefillArena prefill_arena(const chimere_moe_layer* w, int T) {
    PrefillArena A{};
    A.n_tiles_max = n_tiles_max_for(w, T);
    const int Fmax = w->F > w->F_s ? w->F : w->F_s;
    A.bx_stride = (int64_t)(w->H / 32) * kMmaTile;
    A.b2_stride = (int64_t)(Fmax / 32) * kMmaTile;
    size_t o = 0;
    A.tiles = o; o += up256((size_t)(8 + 4 * A.n_tiles_max) * 4);
    A.bx = o; o += up256((size_t)A.n_tiles_max * A.bx_stride);
    A.b2 = o; o += up256((size_t)A.n_tiles_max * A.b2_stride);
    A.total = o;
    return A;
}
}  // namespace

size_t chimere_b200_moe_pack_prefill_bytes(const chimere_moe_layer* raw) {
    if (validate_layer(raw) != 0) return 0;
    if (kshared(raw)) { const chimere_moe_layer r = routed_only(raw); return chimere_b200_moe_pack_prefill_bytes(&r); }
    if (raw->layout != CHIMERE_LAYOUT_GGML || !prefill_dims_ok(raw)) return 0;
    return prefill_plan(raw).total;
}

int chimere_b200_moe_pack_prefill(const chimere_moe_layer* raw, void* d_arena, size_t bytes, chimere_moe_prefill_weights* out,
                                  cudaStream_t stream) {
    int rc = validate_layer(raw);
    if (rc) return rc;
    if (!d_arena || !out) return -1;
    if (kshared(raw)) { const chimere_moe_layer r = routed_only(raw); return chimere_b200_moe_pack_prefill(&r, d_arena, bytes, out, stream); }
    if (raw->layout != CHIMERE_LAYOUT_GGML || !prefill_dims_ok(raw)) return -2;
    if ((uintptr_t)d_arena & 255) return -5;
    const PrefillPlan P = prefill_plan(raw);
    if (bytes < P.total) return -4;
    const bool dual = raw->act == CHIMERE_ACT_SWIGLU;
    uint8_t* base = (uint8_t*)d_arena;
    cudaError_t e = cudaSuccess;
    if (raw->F % P.rows_per_tile || raw->F_s % P.rows_per_tile) e = cudaMemsetAsync(base, 0, P.total, stream);   // zero rows and scales behind the last real row
    if (dual && e == cudaSuccess) e = launch_pack_mma128_ggml(raw->type_gate, raw->gate_exps, base + P.gu, raw->E, raw->F, raw->H, 1, raw->stride_gate, P.sgu, stream);
    if (e == cudaSuccess) e = launch_pack_mma128_ggml(raw->type_up, raw->up_exps, base + P.gu, raw->E, raw->F, raw->H, dual ? 2 : 0, raw->stride_up, P.sgu, stream);
    if (e == cudaSuccess) e = launch_pack_mma128_ggml(raw->type_down, raw->down_exps, base + P.down, raw->E, raw->H, raw->F, 0, raw->stride_down, P.sdown, stream);
    if (raw->F_s > 0) {
        if (dual && e == cudaSuccess) e = launch_pack_mma128_ggml(raw->type_sh_gate, raw->sh_gate, base + P.sh_gu, 1, raw->F_s, raw->H, 1, 0, 0, stream);
        if (e == cudaSuccess) e = launch_pack_mma128_ggml(raw->type_sh_up, raw->sh_up, base + P.sh_gu, 1, raw->F_s, raw->H, dual ? 2 : 0, 0, 0, stream);
        if (e == cudaSuccess) e = launch_pack_mma128_ggml(raw->type_sh_down, raw->sh_down, base + P.sh_down, 1, raw->H, raw->F_s, 0, 0, 0, stream);
    }
    out->gu_exps = base + P.gu; out->stride_gu = P.sgu;
    out->down_exps = base + P.down; out->stride_down = P.sdown;
    out->sh_gu = raw->F_s > 0 ? base + P.sh_gu : nullptr;
    out->sh_down = raw->F_s > 0 ? base + P.sh_down : nullptr;
    out->rows_per_gu_tile = P.rows_per_tile; out->reserved = 0;
    return cuda_rc(e);
}

size_t chimere_b200_moe_prefill_bytes(const chimere_moe_layer* w, int max_T) {
    if (validate_layer(w) != 0 || max_T <= 0) return 0;
    if (kshared(w)) { const chimere_moe_layer r = routed_only(w); return chimere_b200_moe_prefill_bytes(&r, max_T); }
    if (!prefill_dims_ok(w)) return 0;
    return prefill_arena(w, max_T).total;
}

// The K-quant shared expert of `w` for T tokens whose Q8_1 rows (ws->x_q8) and gate logits (ws->sh_gate_logit) the router
// left behind, added to d_y: up (and gate) GEMVs, activation + Q8_1, down GEMV with the sigmoid-gated add.  The f32 rows
// borrow ws->pair_out and the intermediates ws->inter_q8: the routed part of the call is done with both by then.
static int kshared_chain(const chimere_moe_layer* w, int T, float* d_y, chimere_moe_workspace* ws, cudaStream_t stream) {
    const bool dual = w->act == CHIMERE_ACT_SWIGLU;
    const int64_t x_stride = (int64_t)(w->H / 32) * kQ81Bytes, i_stride = (int64_t)(w->F_s / 32) * kQ81Bytes;
    float* up = ws->pair_out;
    float* gate = dual ? ws->pair_out + (size_t)T * w->F_s : nullptr;
    // gate and up share a launch when they have the same type; the three (or four) kernels are chained programmatically
    const bool one = dual && w->type_sh_gate == w->type_sh_up;
    cudaError_t e = launch_mmvq_kquant_batched(w->type_sh_up, w->sh_up, one ? w->sh_gate : nullptr, ws->x_q8, x_stride, up, one ? gate : nullptr,
                                               w->F_s, T, w->H, w->F_s, 0, nullptr, true, stream);
    if (e == cudaSuccess && dual && !one)
        e = launch_mmvq_kquant_batched(w->type_sh_gate, w->sh_gate, nullptr, ws->x_q8, x_stride, gate, nullptr, w->F_s, T, w->H, w->F_s, 0, nullptr,
                                       true, stream);
    if (e == cudaSuccess) e = launch_act_q8_1(gate, up, w->F_s, ws->inter_q8, i_stride, T, w->F_s, stream);
    if (e == cudaSuccess)
        e = launch_mmvq_kquant_batched(w->type_sh_down, w->sh_down, nullptr, ws->inter_q8, i_stride, d_y, nullptr, w->H, T, w->F_s, w->H,
                                       w->shexp_gate_w ? 2 : 1, w->shexp_gate_w ? ws->sh_gate_logit : nullptr, true, stream);
    return cuda_rc(e);
}

// The expert products of a prefill-size batch whose routing (ws->offsets, ws->perm) and Q8_1 planes (ws->x_q, ws->x_d) are
// in place: token tiles for the experts with at least kGemmMin pairs (and the shared expert, if any) on the grouped GEMM,
// the rest on the GEMV kernels; per-pair rows land in ws->pair_out.
static int prefill_gemms(const chimere_moe_layer* w, const chimere_moe_prefill_weights* pw, int T, chimere_moe_workspace* ws, uint8_t* base,
                         const PrefillArena& A, int32_t* tiles, int n_tiles_max, cudaStream_t stream);
static int prefill_experts(const chimere_moe_layer* w, const chimere_moe_prefill_weights* pw, int T, chimere_moe_workspace* ws,
                           cudaStream_t stream, const void* d_packed = nullptr, int row_bytes = 0) {
    if (!pw || !ws->prefill_arena) return -1;
    if (w->layout != CHIMERE_LAYOUT_TILED32 || !prefill_dims_ok(w)) return -2;
    const PrefillArena A = prefill_arena(w, ws->max_T);
    if (ws->prefill_bytes < A.total || ((uintptr_t)ws->prefill_arena & 255)) return -4;
    uint8_t* base = (uint8_t*)ws->prefill_arena;
    int32_t* tiles = (int32_t*)(base + A.tiles);
    const Layout L = make_layout(w, ws->max_T);
    const int n_tiles_max = n_tiles_max_for(w, T);
    cudaError_t e = launch_build_tiles(ws->offsets, ws->perm, tiles, ws->group_list, w->E, T, w->top_k, w->F_s > 0, kGemmMin, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    // the rows' Q8_1 planes: the workspace's, or (expert-parallel owner) the received packed rows in place
    const int8_t* xq = d_packed ? (const int8_t*)d_packed : ws->x_q;
    const float* xd = d_packed ? (const float*)((const uint8_t*)d_packed + w->H) : ws->x_d;
    const int64_t xq_stride = d_packed ? row_bytes : w->H;
    const int xd_stride = d_packed ? row_bytes / 4 : L.x_d_stride;
    e = launch_gather_tiles(tiles, ws->perm, xq, xq_stride, xd, xd_stride, base + A.bx, A.bx_stride, w->H, w->top_k, n_tiles_max, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    // the small experts: GEMV kernels on the rewritten work list, per-pair rows only
    // (the shared expert is not on this list: the kernels are sized for the routed matrices alone)
    // every expert on this list has fewer than kGemmMin <= kMaxGroupTokens pairs, i.e. one entry; the grid is sized for that,
    // not for the worst case of the all-GEMV path
    static_assert(kGemmMin <= kMaxGroupTokens, "a small expert must fit one work entry");
    const int max_entries = w->E < T * w->top_k ? w->E : T * w->top_k;
    GemvParams gu = gate_up_params(w, T, ws, L);
    gu.nrows_shared = 0; gu.ncols_shared = 0; gu.sh_a = nullptr; gu.sh_b = nullptr;
    if (d_packed) { gu.in_soa_q = xq; gu.in_soa_q_stride = xq_stride; gu.in_soa_d = xd; gu.in_soa_d_stride = xd_stride; }
    e = launch_gate_up_tiled(gu, max_entries, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    GemvParams dn = down_params(w, nullptr, T, ws, L);
    dn.no_combine = 1;
    dn.nrows_shared = 0; dn.ncols_shared = 0; dn.sh_a = nullptr; dn.sh_b = nullptr;
    e = launch_down_tiled(dn, max_entries, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    // the large experts and the shared expert: grouped GEMMs
    return prefill_gemms(w, pw, T, ws, base, A, tiles, n_tiles_max, stream);
}

// The two grouped GEMM launches over the token tiles in `tiles` (gate/up with the fused activation and Q8_1 step, then down).
static int prefill_gemms(const chimere_moe_layer* w, const chimere_moe_prefill_weights* pw, int T, chimere_moe_workspace* ws, uint8_t* base,
                         const PrefillArena& A, int32_t* tiles, int n_tiles_max, cudaStream_t stream) {
    cudaError_t e;
    PrefillGemmParams g{};
    g.tiles = tiles; g.perm = ws->perm; g.status = ws->status;
    g.act = w->act; g.T = T; g.top_k = w->top_k; g.H = w->H;
    g.a_exps = (const uint8_t*)pw->gu_exps; g.stride_a = pw->stride_gu; g.sh_a = (const uint8_t*)pw->sh_gu;
    g.b_tiles = base + A.bx; g.b_tile_stride = A.bx_stride;
    g.out_tiles = base + A.b2; g.out_tile_stride = A.b2_stride;
    g.row_tiles_routed = (w->F + pw->rows_per_gu_tile - 1) / pw->rows_per_gu_tile;
    g.row_tiles_shared = (w->F_s + pw->rows_per_gu_tile - 1) / pw->rows_per_gu_tile;
    g.nblk_routed = w->F / 32; g.nblk_shared = w->F_s / 32;
    g.row_tiles_max = g.row_tiles_routed > g.row_tiles_shared ? g.row_tiles_routed : g.row_tiles_shared;
    g.ncols_in = w->H; g.ncols_in_shared = w->H;
    e = launch_prefill_gemm(g, false, n_tiles_max, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    g.a_exps = (const uint8_t*)pw->down_exps; g.stride_a = pw->stride_down; g.sh_a = (const uint8_t*)pw->sh_down;
    g.b_tiles = base + A.b2; g.b_tile_stride = A.b2_stride;
    g.out_tiles = nullptr; g.pair_out = ws->pair_out;
    g.row_tiles_routed = g.row_tiles_shared = g.row_tiles_max = w->H / 128;
    g.ncols_in = w->F; g.ncols_in_shared = w->F_s;
    return cuda_rc(launch_prefill_gemm(g, true, n_tiles_max, stream));
}

int chimere_b200_moe_forward_prefill(const chimere_moe_layer* w, const chimere_moe_prefill_weights* pw, const float* d_x, float* d_y,
                                     int T, chimere_moe_workspace* ws, cudaStream_t stream) {
    int rc = check_call(w, d_x, d_y, T, ws, true);
    if (rc) return rc;
    if (!pw || !ws->prefill_arena) return -1;
    const bool ks = kshared(w);   // (a K-quant shared expert runs as GEMVs per token behind the routed part, at any batch size)
    const chimere_moe_layer wr_ = ks ? routed_only(w) : *w;
    const chimere_moe_layer* wr = &wr_;
    if (wr->layout != CHIMERE_LAYOUT_TILED32 || !prefill_dims_ok(wr)) return -2;
    RouteParams rp = route_params(wr, d_x, T, ws, ks);
    rp.list_mode = 2;   // no work entries from the router: the tile builder writes the list of the small experts
    cudaError_t e = launch_route(rp, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    rc = prefill_experts(wr, pw, T, ws, stream);
    if (rc) return rc;
    // routing-weighted sum of every token's pair rows in slot order + the sigmoid-gated shared expert
    const float* shared_rows = wr->F_s > 0 ? ws->pair_out + (size_t)T * wr->top_k * wr->H : nullptr;
    const float* logit = (wr->F_s > 0 && wr->shexp_gate_w) ? ws->sh_gate_logit : nullptr;
    e = launch_ep_finish(ws->pair_out, nullptr, ws->topk_w, shared_rows, logit, d_y, T, wr->H, wr->top_k, stream);
    if (e != cudaSuccess || !ks) return cuda_rc(e);
    return kshared_chain(w, T, d_y, ws, stream);
}

// Expert-parallel owner rank, prefill-size: as chimere_b200_moe_experts, with the large local experts on the grouped GEMM.
int chimere_b200_moe_experts_prefill(const chimere_moe_layer* w_local, const chimere_moe_prefill_weights* pw_local, int n_rows,
                                     chimere_moe_workspace* ws, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    int rc = check_call(w_local, ws, ws, n_rows, ws);
    if (rc) return rc;
    if (w_local->layout != CHIMERE_LAYOUT_TILED32 || w_local->top_k != 1 || w_local->F_s != 0) return -2;
    RouteParams p = route_params(w_local, nullptr, n_rows, ws);
    p.has_shared = 0;
    p.list_mode = 2;
    cudaError_t e = launch_permute(p, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    return prefill_experts(w_local, pw_local, n_rows, ws, stream);
}

// Expert-parallel home rank, prefill-size: the shared expert of this rank's T tokens on the grouped GEMM (token tiles of
// the shared expert only), per-token rows into ws->pair_out[T * top_k + t] as chimere_b200_moe_shared_expert leaves them.
int chimere_b200_moe_shared_expert_prefill(const chimere_moe_layer* w, const chimere_moe_prefill_weights* pw, int T, chimere_moe_workspace* ws,
                                           cudaStream_t stream) {
    int rc = check_call(w, ws, ws, T, ws);
    if (rc) return rc;
    if (w->F_s <= 0) return 0;
    if (!pw || !pw->sh_gu || !pw->sh_down || !ws->prefill_arena) return -1;
    if (w->layout != CHIMERE_LAYOUT_TILED32 || !prefill_dims_ok(w)) return -2;
    const PrefillArena A = prefill_arena(w, ws->max_T);
    if (ws->prefill_bytes < A.total || ((uintptr_t)ws->prefill_arena & 255)) return -4;
    uint8_t* base = (uint8_t*)ws->prefill_arena;
    int32_t* tiles = (int32_t*)(base + A.tiles);
    const Layout L = make_layout(w, ws->max_T);
    const int n_tiles = (T + 127) / 128;
    // no routed expert gets a tile (E = 0): the list holds the shared expert's token tiles alone
    cudaError_t e = launch_build_tiles(ws->offsets, ws->perm, tiles, ws->group_list, 0, T, w->top_k, 1, kGemmMin, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    e = launch_gather_tiles(tiles, ws->perm, ws->x_q, w->H, ws->x_d, L.x_d_stride, base + A.bx, A.bx_stride, w->H, w->top_k, n_tiles, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    return prefill_gemms(w, pw, T, ws, base, A, tiles, n_tiles, stream);
}

// ... with the rows where an exchange left them: packed rows [H int8][d_stride f32][int32 local expert id] (see ep_pack).
int chimere_b200_moe_experts_packed_prefill(const chimere_moe_layer* w_local, const chimere_moe_prefill_weights* pw_local, int n_rows,
                                            const void* d_rows, int row_bytes, chimere_moe_workspace* ws, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    if (!d_rows) return -1;
    int rc = check_call(w_local, ws, ws, n_rows, ws);
    if (rc) return rc;
    if (w_local->layout != CHIMERE_LAYOUT_TILED32 || w_local->top_k != 1 || w_local->F_s != 0) return -2;
    const int ds = (w_local->H / 32 + 3) & ~3;
    if (row_bytes % 16 || row_bytes < w_local->H + 4 * ds + 4) return -2;
    RouteParams p = route_params(w_local, nullptr, n_rows, ws);
    p.has_shared = 0;
    p.list_mode = 2;
    p.topk_idx = (int32_t*)((uint8_t*)d_rows + w_local->H + 4 * ds);
    p.idx_stride = row_bytes / 4;
    cudaError_t e = launch_permute(p, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    return prefill_experts(w_local, pw_local, n_rows, ws, stream, d_rows, row_bytes);
}

int chimere_b200_moe_ep_pack_sorted(const chimere_moe_layer* w, int T, chimere_moe_workspace* ws, void* d_send, int32_t* d_slot,
                                    int experts_per_rank, int row_bytes, cudaStream_t stream) {
    int rc = check_call(w, d_send, d_slot, T, ws);
    if (rc) return rc;
    const int ds = (w->H / 32 + 3) & ~3;
    if (experts_per_rank <= 0 || row_bytes % 16 || row_bytes < w->H + 4 * ds + 4) return -2;
    return cuda_rc(launch_ep_pack_sorted(ws->perm, ws->topk_idx, ws->x_q, ws->x_d, ds, (uint8_t*)d_send, d_slot, T, w->top_k, w->H,
                                         experts_per_rank, row_bytes, stream));
}

int chimere_b200_moe_forward_residual_norm(const chimere_moe_layer* w, const chimere_moe_prefill_weights* pw, const float* d_hidden,
                                           float* d_residual, const float* d_norm_weight, float eps, float* d_y, int T,
                                           chimere_moe_workspace* ws, cudaStream_t stream) {
    int rc = check_call(w, d_hidden, d_y, T, ws, true);
    if (rc) return rc;
    if (!d_residual || !d_norm_weight || !ws->pair_out) return -1;
    // the normalised rows live in the first T rows of the per-pair output area until the router and the Q8_1 step have
    // read them; the down stage writes that area only afterwards
    float* normed = ws->pair_out;
    cudaError_t e = launch_add_residual_rmsnorm(d_hidden, d_residual, d_norm_weight, normed, T, w->H, eps, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    return pw ? chimere_b200_moe_forward_prefill(w, pw, normed, d_y, T, ws, stream) : chimere_b200_moe_forward(w, normed, d_y, T, ws, stream);
}

int chimere_b200_moe_routing_trace(const chimere_moe_layer* w, int T, const chimere_moe_workspace* ws, uint8_t* d_trace,
                                   int32_t* d_expert_load, cudaStream_t stream) {
    if (!w || !ws || !ws->topk_idx || !d_trace) return -1;
    if (T <= 0 || T > ws->max_T || w->top_k <= 0 || w->top_k > kMaxTopK || w->E <= 0 || w->E > kMaxExperts) return -2;
    return cuda_rc(launch_routing_trace(ws->topk_idx, d_trace, d_expert_load, T, w->top_k, w->E, stream));
}

int chimere_b200_rmsnorm(const float* d_x, float* d_y, int T, int H, float eps, cudaStream_t stream) {
    if (!d_x || !d_y) return -1;
    if (T < 0 || H <= 0) return -2;
    return cuda_rc(launch_rmsnorm(d_x, d_y, T, H, eps, stream));
}

// ---------------------------------------------------------------- legacy operator entries --
void chimere_quantize_q8_1(const float* input, void* output, int64_t ncols, int64_t ncols_padded, cudaStream_t stream) {
    launch_quantize_q8_1(input, output, ncols, ncols_padded, 1, stream);
}
void chimere_quantize_q8_1_batched(const float* input, void* output, int64_t ncols, int64_t ncols_padded, int batch,
                                   cudaStream_t stream) {
    launch_quantize_q8_1(input, output, ncols, ncols_padded, batch, stream);
}
void chimere_mmvq_iq3s(const void* weights, const void* input_q8, float* output, int ncols, int nrows, int, cudaStream_t stream) {
    launch_mmvq(CHIMERE_TYPE_IQ3_S, weights, input_q8, output, nullptr, ncols, nrows, 0, 0, 1, stream);
}
void chimere_mmvq_q8_0(const void* weights, const void* input_q8, float* output, int ncols, int nrows, int, cudaStream_t stream) {
    launch_mmvq(CHIMERE_TYPE_Q8_0, weights, input_q8, output, nullptr, ncols, nrows, 0, 0, 1, stream);
}
void chimere_mmvq_q4_0(const void* weights, const void* input_q8, float* output, int ncols, int nrows, int, cudaStream_t stream) {
    launch_mmvq(CHIMERE_TYPE_Q4_0, weights, input_q8, output, nullptr, ncols, nrows, 0, 0, 1, stream);
}
// Fused quantize + GEMV from an f32 input row (ffi/ggml_cuda_gemv.cu:322-352): Q8_1 of the input into the caller's
// scratch (pad(ncols, 512) / 32 * 36 bytes, blocks past ncols zero), then the GEMV above on that scratch.
static void mmvq_f32(int wtype, const void* weights, const float* input_f32, float* output, int ncols, int nrows, int ncols_padded,
                     void* q8_scratch, cudaStream_t stream) {
    launch_quantize_q8_1(input_f32, q8_scratch, ncols, ncols_padded, 1, stream);
    launch_mmvq(wtype, weights, q8_scratch, output, nullptr, ncols, nrows, 0, 0, 1, stream);
}
void chimere_mmvq_iq3s_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows, int ncols_padded,
                           void* q8_scratch, cudaStream_t stream) {
    mmvq_f32(CHIMERE_TYPE_IQ3_S, weights, input_f32, output, ncols, nrows, ncols_padded, q8_scratch, stream);
}
void chimere_mmvq_q8_0_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows, int ncols_padded,
                           void* q8_scratch, cudaStream_t stream) {
    mmvq_f32(CHIMERE_TYPE_Q8_0, weights, input_f32, output, ncols, nrows, ncols_padded, q8_scratch, stream);
}
void chimere_mmvq_q4_0_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows, int ncols_padded,
                           void* q8_scratch, cudaStream_t stream) {
    mmvq_f32(CHIMERE_TYPE_Q4_0, weights, input_f32, output, ncols, nrows, ncols_padded, q8_scratch, stream);
}
void chimere_mmvq_q5k(const void* weights, const void* input_q8, float* output, int ncols, int nrows, int, cudaStream_t stream) {
    launch_mmvq_kquant(CHIMERE_TYPE_Q5_K, weights, input_q8, output, ncols, nrows, stream);
}
void chimere_mmvq_q4k(const void* weights, const void* input_q8, float* output, int ncols, int nrows, int, cudaStream_t stream) {
    launch_mmvq_kquant(CHIMERE_TYPE_Q4_K, weights, input_q8, output, ncols, nrows, stream);
}
void chimere_mmvq_q6k(const void* weights, const void* input_q8, float* output, int ncols, int nrows, int, cudaStream_t stream) {
    launch_mmvq_kquant(CHIMERE_TYPE_Q6_K, weights, input_q8, output, ncols, nrows, stream);
}
static void mmvq_kquant_f32(int wtype, const void* weights, const float* input_f32, float* output, int ncols, int nrows, int ncols_padded,
                            void* q8_scratch, cudaStream_t stream) {
    launch_quantize_q8_1(input_f32, q8_scratch, ncols, ncols_padded, 1, stream);
    launch_mmvq_kquant(wtype, weights, q8_scratch, output, ncols, nrows, stream);
}
void chimere_mmvq_q5k_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows, int ncols_padded,
                          void* q8_scratch, cudaStream_t stream) {
    mmvq_kquant_f32(CHIMERE_TYPE_Q5_K, weights, input_f32, output, ncols, nrows, ncols_padded, q8_scratch, stream);
}
void chimere_mmvq_q4k_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows, int ncols_padded,
                          void* q8_scratch, cudaStream_t stream) {
    mmvq_kquant_f32(CHIMERE_TYPE_Q4_K, weights, input_f32, output, ncols, nrows, ncols_padded, q8_scratch, stream);
}
void chimere_mmvq_q6k_f32(const void* weights, const float* input_f32, float* output, int ncols, int nrows, int ncols_padded,
                          void* q8_scratch, cudaStream_t stream) {
    mmvq_kquant_f32(CHIMERE_TYPE_Q6_K, weights, input_f32, output, ncols, nrows, ncols_padded, q8_scratch, stream);
}
void chimere_mmvq_iq3s_batched(const void* all_weights, const void* input_q8, float* output, const int* expert_ids, int ncols,
                               int nrows, int, int64_t expert_stride, int64_t input_stride, int top_k, cudaStream_t stream) {
    launch_mmvq(CHIMERE_TYPE_IQ3_S, all_weights, input_q8, output, expert_ids, ncols, nrows, expert_stride, input_stride, top_k, stream);
}
void chimere_mmvq_q4_0_batched(const void* all_weights, const void* input_q8, float* output, const int* expert_ids, int ncols,
                               int nrows, int, int64_t expert_stride, int64_t input_stride, int top_k, cudaStream_t stream) {
    launch_mmvq(CHIMERE_TYPE_Q4_0, all_weights, input_q8, output, expert_ids, ncols, nrows, expert_stride, input_stride, top_k, stream);
}
void chimere_mmvq_q8_0_batched(const void* all_weights, const void* input_q8, float* output, const int* expert_ids, int ncols,
                               int nrows, int, int64_t expert_stride, int64_t input_stride, int top_k, cudaStream_t stream) {
    launch_mmvq(CHIMERE_TYPE_Q8_0, all_weights, input_q8, output, expert_ids, ncols, nrows, expert_stride, input_stride, top_k, stream);
}
int chimere_q8_1_block_bytes(void) { return kQ81Bytes; }
int chimere_q8_1_block_elems(void) { return 32; }
int chimere_matrix_row_padding(void) { return 512; }

}  // extern "C"
