// C-ABI entry points (include/fp8w8a16_b200.h): argument validation, algorithm choice, workspace
// carve-up and kernel launches.  No allocation, no host synchronisation (except device_status).
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <new>

#include "common.cuh"
#include "align.cuh"
#include "ep.h"
#include "gemm_tc.h"

namespace w8a16 {

// ---- error plumbing ------------------------------------------------------------------------------
static thread_local char t_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
    return code;
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

static std::atomic<unsigned long long> g_variants[FP8W8A16_NUM_VARIANTS];
void count_variant(int v) { g_variants[v].fetch_add(1, std::memory_order_relaxed); }

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// ---- kernels defined in the other translation units -------------------------------------------------
int launch_e4m3_to_fp16(const uint8_t* in, __half* out, int64_t n, cudaStream_t st);
int launch_e4m3_to_fp16_scaled(const uint8_t* in, const __half* scales, __half* out, int64_t n, int64_t group, cudaStream_t st);
int launch_dequant_block(const uint8_t* w, const void* scales, int scale_dtype, __half* out, int N, int K, int block_h,
                         int block_w, cudaStream_t st);
int launch_add_rmsnorm(const __half* x, const __half* residual, const __half* weight, float eps, __half* out, __half* residual_out,
                       int M, int N, cudaStream_t st);
size_t gemv_workspace_bytes(int M, int N, int K);
int launch_gemv(const __half* x, const uint8_t* w, const void* scales, int scale_dtype, __half* out, int M, int N, int K,
                int block_h, int block_w, void* workspace, size_t workspace_bytes, cudaStream_t st);
int launch_topk_softmax(const void* logits, int logits_dtype, int M, int E, int topk, int renorm, int* ids, float* weights,
                        cudaStream_t st);
int launch_router_topk(const __half* x, const void* gate, int gate_dtype, int M, int E, int H, int topk, int renorm, int shared_id,
                       float routed_scale, int* ids, float* weights, float* logits_out, cudaStream_t st);
int launch_align(const void* ids, int ids_are_i64, int R, const int* expert_map, int n_global, int E, int bt, int* counts,
                 int* offsets, int* tile_offsets, int* sorted_route, int* inv_pos, cudaStream_t st, const __half* x = nullptr,
                 const float* topk_w = nullptr, int topk = 1, int H = 0, int weight_on_input = 0, __half* x_sorted = nullptr,
                 float* w_sorted = nullptr);
int launch_gather(const __half* x, const int* sorted_route, const float* topk_w, int R, int topk, int H, int weight_on_input,
                  __half* x_sorted, float* w_sorted, cudaStream_t st, const int* n_valid = nullptr, int pad_rows = 0);
int launch_combine(const __half* y_sorted, const int* inv_pos, int M, int topk, int H, __half* out, cudaStream_t st);

namespace {

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int dense_token_tile(int M);

size_t tc_dense_workspace_bytes(int M, int N, int K) {
    (void)N;
    (void)K;
    return tc_workspace_bytes(dense_token_tile(M), false);
}

// Token tile of the tensor-core GEMM for a dense problem of M tokens: the next of 16 / 32 / 64 / 128 at or above M, 256 beyond.
int dense_token_tile(int M) { return tc_pick_bt(M); }

// Largest token count served by the CUDA-core GEMV under ALGO_AUTO (the reference has the same kind of
// knob, _COALESCED_GEMV_M_MAX, src/fp8_w8a16_sm70/vllm_serve.py:1063-1072).  Default 1: measured on B200 the
// tensor-core kernel is faster from two tokens on.  FP8W8A16_GEMV_MAX_M=0..4 overrides it.
int gemv_max_m() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("FP8W8A16_GEMV_MAX_M");
        int x = e ? atoi(e) : 1;
        v = x < 0 ? 0 : (x > 4 ? 4 : x);
    }
    return v;
}

int check_common(const void* x, const void* w, const void* scales, const void* out, int M, int N, int K, int block_h,
                 int block_w, int scale_dtype) {
    W8A16_REQUIRE(M >= 0 && N >= 0 && K >= 0, FP8W8A16_ERR_INVALID, "negative dimension M=%d N=%d K=%d", M, N, K);
    if (M == 0 || N == 0) return 0;
    W8A16_REQUIRE(x && w && scales && out, FP8W8A16_ERR_INVALID, "null pointer argument");
    W8A16_REQUIRE(block_w == 128, FP8W8A16_ERR_UNSUPPORTED, "block_w must be 128 (got %d)", block_w);
    W8A16_REQUIRE(block_h >= 1, FP8W8A16_ERR_INVALID, "block_h must be >= 1 (got %d)", block_h);
    W8A16_REQUIRE(K > 0 && K % 16 == 0, FP8W8A16_ERR_UNSUPPORTED, "K must be a positive multiple of 16 (got %d)", K);
    W8A16_REQUIRE(scale_dtype == FP8W8A16_SCALE_F16 || scale_dtype == FP8W8A16_SCALE_F32, FP8W8A16_ERR_INVALID,
                  "unknown scale dtype %d", scale_dtype);
    W8A16_REQUIRE(aligned16(x) && aligned16(w), FP8W8A16_ERR_INVALID, "x and w must be 16-byte aligned");
    return 0;
}

int linear_tc(const __half* x, const uint8_t* w, const void* scales, int scale_dtype, __half* out, int M, int N, int K,
              int block_h, void* workspace, size_t workspace_bytes, cudaStream_t st, const ArParams* ar = nullptr,
              const __half* residual = nullptr) {
    const int bt = dense_token_tile(M), bk = tc_block_k(bt, false);
    const int token_tiles = (M + bt - 1) / bt;
    const int64_t tiles = (int64_t)((N + 127) / 128) * token_tiles;
    const size_t need = tc_workspace_bytes(bt, false);
    W8A16_REQUIRE(workspace != nullptr && workspace_bytes >= need, FP8W8A16_ERR_WORKSPACE,
                  "linear: workspace too small (%zu < %zu bytes)", workspace_bytes, need);
    TcLaunch L;
    memset(&L, 0, sizeof(L));
    L.p.M = M;
    L.p.N = N;
    L.p.K = K;
    L.p.w_rows_per_expert = N;
    L.p.pair_offset = 0;
    L.p.scales = scales;
    L.p.scale_dtype = scale_dtype;
    L.p.block_h = block_h;
    L.p.Kb = (K + 127) / 128;
    L.p.scale_expert_stride = 0;
    L.p.num_experts = 1;
    L.p.out = out;
    L.p.ldo = N;
    L.p.residual = residual;
    L.p.n_token_tiles = token_tiles;
    // many tiles per CTA: whole tiles cost < 12 % in the last wave and need no partial-tile traffic
    L.p.no_split = (tiles > (int64_t)tc_max_tiles_with_tickets() || tiles >= 8ll * tc_grid(bt, false)) ? 1 : 0;
    L.p.tickets = reinterpret_cast<unsigned int*>(workspace);
    L.p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kTicketBytes);
    L.w = w;
    L.x = x;
    L.w_total_rows = N;
    L.max_units = tiles * ((K + bk - 1) / bk);
    W8A16_REQUIRE(L.max_units < (1ll << 31), FP8W8A16_ERR_UNSUPPORTED, "linear: problem too large for 32-bit work indices");
    L.p.cluster_size = tc_cluster_size(tiles, (K + bk - 1) / bk, bt, false);
    L.cluster_tiles = tiles;
    if (ar != nullptr && ar->world > 1) {
        W8A16_REQUIRE(N % 4 == 0, FP8W8A16_ERR_UNSUPPORTED, "linear_allreduce: N must be a multiple of 4 (got %d)", N);
        W8A16_REQUIRE((int64_t)M * N <= ar->part_elems, FP8W8A16_ERR_UNSUPPORTED,
                      "linear_allreduce: M*N = %lld exceeds the communicator's buffer of %lld elements", (long long)M * N,
                      (long long)ar->part_elems);
        L.ar = *ar;
        L.ar.out = out;
        count_variant(FP8W8A16_VARIANT_FUSED_ALLREDUCE);
    }
    count_variant(L.p.cluster_size > 1 ? FP8W8A16_VARIANT_TC_CLUSTER
                                       : (L.p.no_split ? FP8W8A16_VARIANT_TC_TILES : FP8W8A16_VARIANT_TC_STREAMK));
    return tc_launch(L, bt, false, st);
}

// Token tile of the grouped GEMMs: twice the average rows per expert, rounded up to a tile size (measured on B200: the
// best choice at every batch; 16 / 32 cover decode), at most 128 because the paired gate/up kernel keeps two accumulators.
int token_tile_for(int R, int E) {
    const int avg = (R + E - 1) / E;
    int bt = tc_pick_bt(2 * avg);
    if (bt > 128) bt = 128;
    return bt;
}

int token_tiles_upper_bound(int R, int E, int bt) { return (R < E ? R : E) + R / bt; }

int grouped_gemm(const __half* x_sorted, const uint8_t* w, const void* scales, int scale_dtype, __half* out,
                 const float* row_weight, const int* offsets, const int* tile_offsets, int R, int E, int N, int K,
                 int block_h, int paired, int bt, void* workspace, size_t workspace_bytes, cudaStream_t st) {
    if (R == 0 || N == 0) return 0;
    const int bk = tc_block_k(bt, paired != 0);
    const int rows_w = paired ? 2 * N : N;
    const int64_t tiles_ub = (int64_t)token_tiles_upper_bound(R, E, bt) * ((N + 127) / 128);
    const size_t need = tc_workspace_bytes(bt, paired != 0);
    W8A16_REQUIRE(workspace != nullptr && workspace_bytes >= need, FP8W8A16_ERR_WORKSPACE,
                  "moe_grouped_gemm: workspace too small (%zu < %zu bytes)", workspace_bytes, need);
    TcLaunch L;
    memset(&L, 0, sizeof(L));
    L.p.M = R;
    L.p.N = N;
    L.p.K = K;
    L.p.w_rows_per_expert = rows_w;
    L.p.pair_offset = paired ? N : 0;
    L.p.scales = scales;
    L.p.scale_dtype = scale_dtype;
    L.p.block_h = block_h;
    L.p.Kb = (K + 127) / 128;
    L.p.scale_expert_stride = (int64_t)((rows_w + block_h - 1) / block_h) * L.p.Kb;
    L.p.expert_offsets = offsets;
    L.p.tile_offsets = tile_offsets;
    L.p.num_experts = E;
    L.p.out = out;
    L.p.ldo = N;
    L.p.row_weight = row_weight;
    L.p.activation = paired;
    L.p.n_token_tiles = 0;
    // Whole tiles instead of stream-K when a tile is only a few K blocks long and there are at least two per CTA (the MoE
    // down projection: K = I): splitting such a tile over two CTAs costs a partial-tile round trip and a ticket per tile,
    // more than the last-wave imbalance of at most one short tile.
    const int total_kb = (K + bk - 1) / bk;
    const bool short_tiles = total_kb <= 8 && tiles_ub >= 2ll * tc_grid(bt, paired != 0);
    L.p.no_split = (tiles_ub > (int64_t)tc_max_tiles_with_tickets() || short_tiles) ? 1 : 0;
    L.p.tickets = reinterpret_cast<unsigned int*>(workspace);
    L.p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kTicketBytes);
    L.w = w;
    L.x = x_sorted;
    L.w_total_rows = (int64_t)E * rows_w;
    L.max_units = tiles_ub * ((K + bk - 1) / bk);
    W8A16_REQUIRE(L.max_units < (1ll << 31), FP8W8A16_ERR_UNSUPPORTED, "moe_grouped_gemm: problem too large for 32-bit work indices");
    L.p.cluster_size = tc_cluster_size(tiles_ub, (K + bk - 1) / bk, bt, paired != 0);
    L.cluster_tiles = tiles_ub;
    count_variant(paired ? FP8W8A16_VARIANT_GROUPED_PAIRED : FP8W8A16_VARIANT_GROUPED);
    return tc_launch(L, bt, paired != 0, st);
}

// Workspace of the whole MoE layer.
struct MoeLayout {
    size_t counts, offsets, tile_offsets, sorted_route, inv_pos, w_sorted, x_sorted, h_sorted, y_sorted, gemm_ws, total;
    size_t gemm_ws_bytes;
    int bt;
};

// Scratch of the grouped pipeline over R routed rows with token tile bt.
MoeLayout moe_layout_rows(int R, int E, int H, int I, int bt) {
    MoeLayout L;
    L.bt = bt;
    size_t o = kTicketBytes;  // the grouped GEMMs' ticket header sits at the very start
    // the GEMM scratch (tickets + partials) must be one contiguous block: header first, partials
    // right after it; the bookkeeping arrays follow the partials.
    const size_t a13 = tc_workspace_bytes(L.bt, true), a2 = tc_workspace_bytes(L.bt, false);
    L.gemm_ws = 0;
    L.gemm_ws_bytes = align_up(a13 > a2 ? a13 : a2, 256);
    o = L.gemm_ws_bytes;
    auto take = [&o](size_t bytes) {
        const size_t at = o;
        o += align_up(bytes, 256);
        return at;
    };
    L.counts = take((size_t)E * 4);
    L.offsets = take((size_t)(E + 1) * 4);
    L.tile_offsets = take((size_t)(E + 1) * 4);
    L.sorted_route = take((size_t)R * 4);
    L.inv_pos = take((size_t)R * 4);
    L.w_sorted = take((size_t)R * 4);
    L.x_sorted = take((size_t)R * H * 2);
    L.h_sorted = take((size_t)R * I * 2);
    L.y_sorted = take((size_t)R * H * 2);
    L.total = o;
    return L;
}

MoeLayout moe_layout(int M, int topk, int E, int H, int I) {
    const int R = M * topk;
    return moe_layout_rows(R, E, H, I, token_tile_for(R > 0 ? R : 1, E));
}

// ---- expert-parallel exchange buffer (see ep.cu) ---------------------------------------------------------------
struct Ep {
    EpGeom g;
    int device, max_tokens, topk, n_global;
    size_t bytes, off_dest_map;
    bool ipc_opened[kEpMaxWorld];
};

// Workspace of one expert-parallel call: the grouped pipeline over world * cap_call received rows first (its ticket
// header must sit at the start of the workspace), then the receive lists, then the dispatch plan.
struct EpLayout {
    MoeLayout moe;
    size_t counts_in, d_counts, d_offsets, d_tiles, d_sorted, d_inv, total;
    int cap_call, rows_in;
};

EpLayout ep_layout(const Ep& e, int M, int M_max, int E_local, int I) {
    EpLayout L;
    L.cap_call = M_max * e.topk;
    L.rows_in = e.g.world * L.cap_call;
    // about as many rows arrive as leave: size the token tile for M * topk rows over the local experts
    const int r_est = (M > 0 ? M : 1) * e.topk;
    L.moe = moe_layout_rows(L.rows_in, E_local, e.g.H, I, token_tile_for(r_est, E_local));
    size_t o = L.moe.total;
    auto take = [&o](size_t bytes) {
        const size_t at = o;
        o += align_up(bytes, 256);
        return at;
    };
    L.counts_in = take(kEpMaxWorld * 4);
    const int R = M * e.topk;
    L.d_counts = take(kEpMaxWorld * 4);
    L.d_offsets = take((kEpMaxWorld + 1) * 4);
    L.d_tiles = take((kEpMaxWorld + 1) * 4);
    L.d_sorted = take((size_t)(R > 0 ? R : 1) * 4);
    L.d_inv = take((size_t)(R > 0 ? R : 1) * 4);
    L.total = o;
    return L;
}


// ---- peer-memory communicator of the fused row-parallel GEMM + all-reduce ---------------------------------
// One cudaMalloc per rank with the same layout on every rank: control words, the rank's own FP16 staging buffer, and
// the inbox [2 parities][world sources][part_elems / 2] of 8-byte packets the peers store into.
struct Comm {
    int rank, world, device;
    unsigned int timeout_ms;
    int64_t part_elems;
    size_t part_off, inbox_off, bytes;
    char* base[kArMaxWorld];     // base[rank] is the local allocation, the others are the peers' mappings
    bool ipc_opened[kArMaxWorld];
};

int comm_params(const Comm* c, ArParams* ar) {
    memset(ar, 0, sizeof(*ar));
    ar->world = c->world;
    ar->rank = c->rank;
    ar->timeout_ms = c->timeout_ms;
    ar->part_elems = c->part_elems;
    ar->ctrl = reinterpret_cast<unsigned int*>(c->base[c->rank]);
    ar->part = reinterpret_cast<__half*>(c->base[c->rank] + c->part_off);
    for (int r = 0; r < c->world; ++r) {
        W8A16_REQUIRE(c->base[r] != nullptr, FP8W8A16_ERR_INVALID, "comm: rank %d is not attached", r);
        ar->inbox[r] = reinterpret_cast<uint2*>(c->base[r] + c->inbox_off);
    }
    return 0;
}

}  // namespace
}  // namespace w8a16

using namespace w8a16;

extern "C" {

int fp8w8a16_version(void) { return 100; }

const char* fp8w8a16_last_error(void) { return t_err; }

uint64_t fp8w8a16_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int fp8w8a16_variant_counts(uint64_t* counts, int n) {
    for (int i = 0; counts != nullptr && i < n && i < FP8W8A16_NUM_VARIANTS; ++i)
        counts[i] = g_variants[i].load(std::memory_order_relaxed);
    return FP8W8A16_NUM_VARIANTS;
}

int fp8w8a16_device_status(int* status, int reset) {
    W8A16_REQUIRE(status != nullptr, FP8W8A16_ERR_INVALID, "device_status: null status pointer");
    W8A16_CUDA(cudaDeviceSynchronize());
    int a = 0, b = 0;
    int rc = tc_read_status(&a, reset);
    if (rc) return rc;
    rc = ep_read_status(&b, reset);
    if (rc) return rc;
    *status = a | b;
    return 0;
}

int fp8w8a16_e4m3_to_fp16(const uint8_t* w, uint16_t* out, int64_t n, void* stream) {
    W8A16_REQUIRE(n >= 0, FP8W8A16_ERR_INVALID, "e4m3_to_fp16: negative n");
    W8A16_REQUIRE(n == 0 || (w && out), FP8W8A16_ERR_INVALID, "e4m3_to_fp16: null pointer");
    count_variant(FP8W8A16_VARIANT_DEQUANT);
    return launch_e4m3_to_fp16(w, reinterpret_cast<__half*>(out), n, (cudaStream_t)stream);
}

int fp8w8a16_e4m3_to_fp16_scaled(const uint8_t* w, const uint16_t* scales_f16, uint16_t* out, int64_t n,
                                 int64_t group_size, void* stream) {
    W8A16_REQUIRE(n >= 0 && group_size > 0, FP8W8A16_ERR_INVALID, "e4m3_to_fp16_scaled: n=%lld group=%lld", (long long)n,
                  (long long)group_size);
    W8A16_REQUIRE(n == 0 || (w && out && scales_f16), FP8W8A16_ERR_INVALID, "e4m3_to_fp16_scaled: null pointer");
    count_variant(FP8W8A16_VARIANT_DEQUANT);
    return launch_e4m3_to_fp16_scaled(w, reinterpret_cast<const __half*>(scales_f16), reinterpret_cast<__half*>(out), n,
                                      group_size, (cudaStream_t)stream);
}

int fp8w8a16_dequant_block_scaled(const uint8_t* w, const void* scales, int scale_dtype, uint16_t* out, int N, int K,
                                  int block_h, int block_w, void* stream) {
    W8A16_REQUIRE(N >= 0 && K >= 0, FP8W8A16_ERR_INVALID, "dequant_block_scaled: negative dimension");
    W8A16_REQUIRE(block_h >= 1 && block_w >= 1, FP8W8A16_ERR_INVALID, "dequant_block_scaled: block %dx%d", block_h, block_w);
    W8A16_REQUIRE(scale_dtype == FP8W8A16_SCALE_F16 || scale_dtype == FP8W8A16_SCALE_F32, FP8W8A16_ERR_INVALID,
                  "dequant_block_scaled: unknown scale dtype %d", scale_dtype);
    W8A16_REQUIRE((N == 0 || K == 0) || (w && scales && out), FP8W8A16_ERR_INVALID, "dequant_block_scaled: null pointer");
    count_variant(FP8W8A16_VARIANT_DEQUANT);
    return launch_dequant_block(w, scales, scale_dtype, reinterpret_cast<__half*>(out), N, K, block_h, block_w,
                                (cudaStream_t)stream);
}

size_t fp8w8a16_linear_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return kTicketBytes;
    const size_t a = gemv_workspace_bytes(M, N, K);
    const size_t b = tc_dense_workspace_bytes(M, N, K);
    return a > b ? a : b;
}

int fp8w8a16_linear(const uint16_t* x, const uint8_t* w, const void* scales, int scale_dtype, uint16_t* out, int M,
                    int N, int K, int block_h, int block_w, int algo, void* workspace, size_t workspace_bytes,
                    void* stream) {
    int rc = check_common(x, w, scales, out, M, N, K, block_h, block_w, scale_dtype);
    if (rc) return rc;
    if (M == 0 || N == 0) return 0;
    const __half* xh = reinterpret_cast<const __half*>(x);
    __half* oh = reinterpret_cast<__half*>(out);
    cudaStream_t st = (cudaStream_t)stream;
    if (algo == FP8W8A16_ALGO_AUTO) algo = (M <= gemv_max_m()) ? FP8W8A16_ALGO_GEMV : FP8W8A16_ALGO_TC;
    switch (algo) {
        case FP8W8A16_ALGO_GEMV:
            count_variant(FP8W8A16_VARIANT_GEMV);
            return launch_gemv(xh, w, scales, scale_dtype, oh, M, N, K, block_h, block_w, workspace, workspace_bytes, st);
        case FP8W8A16_ALGO_TC:
            return linear_tc(xh, w, scales, scale_dtype, oh, M, N, K, block_h, workspace, workspace_bytes, st);
    }
    return fail(FP8W8A16_ERR_INVALID, "linear: unknown algo %d", algo);
}

int fp8w8a16_linear_residual(const uint16_t* x, const uint8_t* w, const void* scales, int scale_dtype, const uint16_t* residual,
                             uint16_t* out, int M, int N, int K, int block_h, int block_w, void* workspace, size_t workspace_bytes,
                             void* stream) {
    int rc = check_common(x, w, scales, out, M, N, K, block_h, block_w, scale_dtype);
    if (rc) return rc;
    if (M == 0 || N == 0) return 0;
    W8A16_REQUIRE(residual != nullptr, FP8W8A16_ERR_INVALID, "linear_residual: null residual");
    return linear_tc(reinterpret_cast<const __half*>(x), w, scales, scale_dtype, reinterpret_cast<__half*>(out), M, N, K, block_h,
                     workspace, workspace_bytes, (cudaStream_t)stream, nullptr, reinterpret_cast<const __half*>(residual));
}

int fp8w8a16_add_rmsnorm(const uint16_t* x, const uint16_t* residual, const uint16_t* weight, float eps, uint16_t* out,
                         uint16_t* residual_out, int M, int N, void* stream) {
    W8A16_REQUIRE(M >= 0 && N >= 0, FP8W8A16_ERR_INVALID, "add_rmsnorm: negative dimension");
    if (M == 0 || N == 0) return 0;
    W8A16_REQUIRE(x && weight && out, FP8W8A16_ERR_INVALID, "add_rmsnorm: null pointer");
    W8A16_REQUIRE(N % 8 == 0 && aligned16(x) && aligned16(weight) && aligned16(out) && aligned16(residual) && aligned16(residual_out),
                  FP8W8A16_ERR_UNSUPPORTED, "add_rmsnorm: N must be a multiple of 8 and all pointers 16-byte aligned");
    W8A16_REQUIRE(residual == nullptr || residual_out != nullptr, FP8W8A16_ERR_INVALID, "add_rmsnorm: residual given without residual_out");
    return launch_add_rmsnorm(reinterpret_cast<const __half*>(x), reinterpret_cast<const __half*>(residual),
                              reinterpret_cast<const __half*>(weight), eps, reinterpret_cast<__half*>(out),
                              reinterpret_cast<__half*>(residual_out), M, N, (cudaStream_t)stream);
}

int fp8w8a16_moe_topk_softmax(const void* logits, int logits_dtype, int M, int E, int topk, int renormalize,
                              int32_t* topk_ids, float* topk_weights, void* stream) {
    W8A16_REQUIRE(M >= 0, FP8W8A16_ERR_INVALID, "moe_topk_softmax: negative M");
    W8A16_REQUIRE(M == 0 || (logits && topk_ids && topk_weights), FP8W8A16_ERR_INVALID, "moe_topk_softmax: null pointer");
    return launch_topk_softmax(logits, logits_dtype, M, E, topk, renormalize, topk_ids, topk_weights, (cudaStream_t)stream);
}

int fp8w8a16_moe_router_topk(const uint16_t* x, const void* gate_weight, int gate_dtype, int M, int E, int H, int topk,
                             int renormalize, int shared_expert_id, float routed_scale, int32_t* topk_ids, float* topk_weights,
                             float* logits, void* stream) {
    W8A16_REQUIRE(M >= 0, FP8W8A16_ERR_INVALID, "moe_router_topk: negative M");
    W8A16_REQUIRE(M == 0 || (x && gate_weight && topk_ids && topk_weights), FP8W8A16_ERR_INVALID, "moe_router_topk: null pointer");
    W8A16_REQUIRE(M == 0 || (aligned16(x) && aligned16(gate_weight)), FP8W8A16_ERR_INVALID, "moe_router_topk: x and gate_weight must be 16-byte aligned");
    return launch_router_topk(reinterpret_cast<const __half*>(x), gate_weight, gate_dtype, M, E, H, topk, renormalize,
                              shared_expert_id, routed_scale, topk_ids, topk_weights, logits, (cudaStream_t)stream);
}

int fp8w8a16_moe_token_tile(int R, int num_local_experts) {
    if (R <= 0 || num_local_experts <= 0) return 16;
    return token_tile_for(R, num_local_experts);
}

int fp8w8a16_moe_align(const void* topk_ids, int ids_are_i64, int R, const int32_t* expert_map, int n_global_experts,
                       int num_local_experts, int token_tile, int32_t* counts, int32_t* offsets, int32_t* tile_offsets,
                       int32_t* sorted_route, int32_t* inv_pos, void* stream) {
    W8A16_REQUIRE(R >= 0, FP8W8A16_ERR_INVALID, "moe_align: negative R");
    W8A16_REQUIRE(token_tile >= 1, FP8W8A16_ERR_INVALID, "moe_align: token_tile=%d", token_tile);
    W8A16_REQUIRE(counts && offsets && tile_offsets, FP8W8A16_ERR_INVALID, "moe_align: null output pointer");
    W8A16_REQUIRE(R == 0 || (topk_ids && sorted_route && inv_pos), FP8W8A16_ERR_INVALID, "moe_align: null pointer");
    return launch_align(topk_ids, ids_are_i64, R, expert_map, n_global_experts, num_local_experts, token_tile, counts, offsets,
                        tile_offsets, sorted_route, inv_pos, (cudaStream_t)stream);
}

size_t fp8w8a16_moe_grouped_gemm_workspace_bytes(int R, int num_local_experts, int N, int K, int paired, int token_tile) {
    (void)R;
    (void)num_local_experts;
    (void)N;
    (void)K;
    return tc_workspace_bytes(token_tile, paired != 0);
}

int fp8w8a16_moe_grouped_gemm(const uint16_t* x_sorted, const uint8_t* w, const void* scales, int scale_dtype,
                              uint16_t* out, const float* row_weight, const int32_t* offsets,
                              const int32_t* tile_offsets, int R, int num_local_experts, int N, int K, int block_h,
                              int paired, int token_tile, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_common(x_sorted, w, scales, out, R, N, K, block_h, 128, scale_dtype);
    if (rc) return rc;
    W8A16_REQUIRE(num_local_experts >= 1, FP8W8A16_ERR_INVALID, "moe_grouped_gemm: num_local_experts=%d", num_local_experts);
    W8A16_REQUIRE(token_tile == 16 || token_tile == 32 || token_tile == 64 || token_tile == 128 || token_tile == 256,
                  FP8W8A16_ERR_INVALID, "moe_grouped_gemm: token_tile=%d not in {16,32,64,128,256}", token_tile);
    W8A16_REQUIRE(R == 0 || (offsets && tile_offsets), FP8W8A16_ERR_INVALID, "moe_grouped_gemm: null route table");
    W8A16_REQUIRE(paired >= 0 && paired <= 2, FP8W8A16_ERR_INVALID, "moe_grouped_gemm: paired=%d not in {0,1,2}", paired);
    return grouped_gemm(reinterpret_cast<const __half*>(x_sorted), w, scales, scale_dtype, reinterpret_cast<__half*>(out),
                        row_weight, offsets, tile_offsets, R, num_local_experts, N, K, block_h, paired, token_tile, workspace,
                        workspace_bytes, (cudaStream_t)stream);
}

int fp8w8a16_moe_gather(const uint16_t* x, const int32_t* sorted_route, const float* topk_weights, int R, int topk,
                        int H, int weight_on_input, uint16_t* x_sorted, float* w_sorted, void* stream) {
    W8A16_REQUIRE(R >= 0 && topk >= 1 && H >= 0, FP8W8A16_ERR_INVALID, "moe_gather: R=%d topk=%d H=%d", R, topk, H);
    W8A16_REQUIRE(R == 0 || (x && sorted_route && topk_weights && x_sorted && w_sorted), FP8W8A16_ERR_INVALID,
                  "moe_gather: null pointer");
    return launch_gather(reinterpret_cast<const __half*>(x), sorted_route, topk_weights, R, topk, H, weight_on_input,
                         reinterpret_cast<__half*>(x_sorted), w_sorted, (cudaStream_t)stream);
}

int fp8w8a16_moe_combine(const uint16_t* y_sorted, const int32_t* inv_pos, int M, int topk, int H, uint16_t* out,
                         void* stream) {
    W8A16_REQUIRE(M >= 0 && topk >= 1 && H >= 0, FP8W8A16_ERR_INVALID, "moe_combine: M=%d topk=%d H=%d", M, topk, H);
    W8A16_REQUIRE(M == 0 || (y_sorted && inv_pos && out), FP8W8A16_ERR_INVALID, "moe_combine: null pointer");
    return launch_combine(reinterpret_cast<const __half*>(y_sorted), inv_pos, M, topk, H, reinterpret_cast<__half*>(out),
                          (cudaStream_t)stream);
}

size_t fp8w8a16_moe_workspace_bytes(int M, int topk, int num_local_experts, int H, int I) {
    if (M <= 0 || topk <= 0 || num_local_experts <= 0 || H <= 0 || I <= 0) return kTicketBytes;
    return moe_layout(M, topk, num_local_experts, H, I).total;
}

int fp8w8a16_moe_forward(const uint16_t* x, const void* topk_ids, int ids_are_i64, const float* topk_weights,
                         const int32_t* expert_map, int n_global_experts, const uint8_t* w13, const void* s13,
                         const uint8_t* w2, const void* s2, int scale_dtype, uint16_t* out, int M, int topk,
                         int num_local_experts, int H, int I, int block_h, int weight_on_input, int activation,
                         void* workspace, size_t workspace_bytes, void* stream) {
    W8A16_REQUIRE(M >= 0 && topk >= 1 && num_local_experts >= 1 && H > 0 && I > 0, FP8W8A16_ERR_INVALID,
                  "moe_forward: M=%d topk=%d E=%d H=%d I=%d", M, topk, num_local_experts, H, I);
    if (M == 0) return 0;
    W8A16_REQUIRE(x && topk_ids && topk_weights && w13 && s13 && w2 && s2 && out, FP8W8A16_ERR_INVALID,
                  "moe_forward: null pointer");
    W8A16_REQUIRE(H % 16 == 0 && I % 16 == 0, FP8W8A16_ERR_UNSUPPORTED,
                  "moe_forward: hidden %d and intermediate %d must be multiples of 16", H, I);
    W8A16_REQUIRE(block_h >= 1, FP8W8A16_ERR_INVALID, "moe_forward: block_h=%d", block_h);
    W8A16_REQUIRE(activation == FP8W8A16_ACT_SILU || activation == FP8W8A16_ACT_GELU, FP8W8A16_ERR_UNSUPPORTED,
                  "moe_forward: activation %d is not SiLU (1) or GELU (2)", activation);
    W8A16_REQUIRE((int64_t)M * topk < (1ll << 30), FP8W8A16_ERR_UNSUPPORTED, "moe_forward: too many routed rows");
    const int E = num_local_experts, R = M * topk;
    const MoeLayout L = moe_layout(M, topk, E, H, I);
    W8A16_REQUIRE(workspace != nullptr && workspace_bytes >= L.total, FP8W8A16_ERR_WORKSPACE,
                  "moe_forward: workspace too small (%zu < %zu bytes)", workspace_bytes, L.total);
    W8A16_REQUIRE(aligned16(workspace) && aligned16(x) && aligned16(out), FP8W8A16_ERR_INVALID,
                  "moe_forward: x, out and workspace must be 16-byte aligned");
    char* ws = reinterpret_cast<char*>(workspace);
    int* counts = reinterpret_cast<int*>(ws + L.counts);
    int* offsets = reinterpret_cast<int*>(ws + L.offsets);
    int* tile_offsets = reinterpret_cast<int*>(ws + L.tile_offsets);
    int* sorted_route = reinterpret_cast<int*>(ws + L.sorted_route);
    int* inv_pos = reinterpret_cast<int*>(ws + L.inv_pos);
    float* w_sorted = reinterpret_cast<float*>(ws + L.w_sorted);
    __half* x_sorted = reinterpret_cast<__half*>(ws + L.x_sorted);
    __half* h_sorted = reinterpret_cast<__half*>(ws + L.h_sorted);
    __half* y_sorted = reinterpret_cast<__half*>(ws + L.y_sorted);
    cudaStream_t st = (cudaStream_t)stream;

    int rc;
    if (R <= kFuseRows) {
        // few rows: the CTA that builds the route table gathers them too
        rc = launch_align(topk_ids, ids_are_i64, R, expert_map, n_global_experts, E, L.bt, counts, offsets, tile_offsets, sorted_route,
                          inv_pos, st, reinterpret_cast<const __half*>(x), topk_weights, topk, H, weight_on_input, x_sorted, w_sorted);
        if (rc) return rc;
    } else {
        rc = launch_align(topk_ids, ids_are_i64, R, expert_map, n_global_experts, E, L.bt, counts, offsets, tile_offsets, sorted_route,
                          inv_pos, st);
        if (rc) return rc;
        rc = launch_gather(reinterpret_cast<const __half*>(x), sorted_route, topk_weights, R, topk, H, weight_on_input, x_sorted,
                           w_sorted, st);
        if (rc) return rc;
    }
    rc = grouped_gemm(x_sorted, w13, s13, scale_dtype, h_sorted, nullptr, offsets, tile_offsets, R, E, I, H, block_h, activation, L.bt,
                      ws + L.gemm_ws, L.gemm_ws_bytes, st);
    if (rc) return rc;
    rc = grouped_gemm(h_sorted, w2, s2, scale_dtype, y_sorted, w_sorted, offsets, tile_offsets, R, E, H, I, block_h, 0, L.bt,
                      ws + L.gemm_ws, L.gemm_ws_bytes, st);
    if (rc) return rc;
    return launch_combine(y_sorted, inv_pos, M, topk, H, reinterpret_cast<__half*>(out), st);
}

// ---- fused row-parallel linear + all-reduce over peer memory ---------------------------------------------
struct fp8w8a16_comm {
    w8a16::Comm c;
};

int fp8w8a16_comm_create(int rank, int world, int64_t max_out_elems, unsigned int timeout_ms, fp8w8a16_comm** comm) {
    W8A16_REQUIRE(comm != nullptr, FP8W8A16_ERR_INVALID, "comm_create: null output pointer");
    *comm = nullptr;
    W8A16_REQUIRE(world >= 2 && world <= kArMaxWorld && rank >= 0 && rank < world, FP8W8A16_ERR_INVALID,
                  "comm_create: rank %d of world %d (2..%d ranks supported)", rank, world, kArMaxWorld);
    W8A16_REQUIRE(max_out_elems > 0 && max_out_elems <= (1ll << 32), FP8W8A16_ERR_INVALID, "comm_create: max_out_elems=%lld",
                  (long long)max_out_elems);
    fp8w8a16_comm* h = new (std::nothrow) fp8w8a16_comm();
    W8A16_REQUIRE(h != nullptr, FP8W8A16_ERR_CUDA, "comm_create: out of host memory");
    Comm& c = h->c;
    memset(&c, 0, sizeof(c));
    c.rank = rank;
    c.world = world;
    c.timeout_ms = timeout_ms ? timeout_ms : 2000u;
    c.part_elems = (max_out_elems + 127) / 128 * 128;
    c.part_off = 256;
    c.inbox_off = align_up(c.part_off + (size_t)c.part_elems * sizeof(__half), 256);
    c.bytes = c.inbox_off + 2 * (size_t)world * (size_t)c.part_elems * 4;   // 8 bytes per pair of FP16 values
    cudaError_t e = cudaGetDevice(&c.device);
    void* base = nullptr;
    if (e == cudaSuccess) e = cudaMalloc(&base, c.bytes);
    if (e == cudaSuccess) e = cudaMemset(base, 0, c.bytes);
    if (e != cudaSuccess) {
        if (base) cudaFree(base);
        delete h;
        return fail(FP8W8A16_ERR_CUDA, "comm_create: %s", cudaGetErrorString(e));
    }
    c.base[rank] = reinterpret_cast<char*>(base);
    *comm = h;
    return 0;
}

int fp8w8a16_comm_export(const fp8w8a16_comm* comm, void* handle) {
    W8A16_REQUIRE(comm && handle, FP8W8A16_ERR_INVALID, "comm_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == FP8W8A16_COMM_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t hd;
    W8A16_CUDA(cudaIpcGetMemHandle(&hd, comm->c.base[comm->c.rank]));
    memcpy(handle, &hd, sizeof(hd));
    return 0;
}

int fp8w8a16_comm_attach(fp8w8a16_comm* comm, int peer, const void* handle) {
    W8A16_REQUIRE(comm && handle, FP8W8A16_ERR_INVALID, "comm_attach: null pointer");
    Comm& c = comm->c;
    W8A16_REQUIRE(peer >= 0 && peer < c.world && peer != c.rank, FP8W8A16_ERR_INVALID, "comm_attach: bad peer %d", peer);
    W8A16_REQUIRE(c.base[peer] == nullptr, FP8W8A16_ERR_INVALID, "comm_attach: peer %d is already attached", peer);
    cudaIpcMemHandle_t hd;
    memcpy(&hd, handle, sizeof(hd));
    void* ptr = nullptr;
    W8A16_CUDA(cudaIpcOpenMemHandle(&ptr, hd, cudaIpcMemLazyEnablePeerAccess));
    c.base[peer] = reinterpret_cast<char*>(ptr);
    c.ipc_opened[peer] = true;
    return 0;
}

int fp8w8a16_comm_attach_ptr(fp8w8a16_comm* comm, int peer, void* peer_base) {
    W8A16_REQUIRE(comm && peer_base, FP8W8A16_ERR_INVALID, "comm_attach_ptr: null pointer");
    Comm& c = comm->c;
    W8A16_REQUIRE(peer >= 0 && peer < c.world && peer != c.rank, FP8W8A16_ERR_INVALID, "comm_attach_ptr: bad peer %d", peer);
    W8A16_REQUIRE(c.base[peer] == nullptr, FP8W8A16_ERR_INVALID, "comm_attach_ptr: peer %d is already attached", peer);
    c.base[peer] = reinterpret_cast<char*>(peer_base);
    c.ipc_opened[peer] = false;
    return 0;
}

void* fp8w8a16_comm_base(const fp8w8a16_comm* comm) { return comm ? comm->c.base[comm->c.rank] : nullptr; }

size_t fp8w8a16_comm_bytes(const fp8w8a16_comm* comm) { return comm ? comm->c.bytes : 0; }

int fp8w8a16_comm_reset(fp8w8a16_comm* comm, void* stream) {
    W8A16_REQUIRE(comm != nullptr, FP8W8A16_ERR_INVALID, "comm_reset: null communicator");
    Comm& c = comm->c;
    char* base = c.base[c.rank];
    W8A16_REQUIRE(base != nullptr, FP8W8A16_ERR_INVALID, "comm_reset: communicator has no local buffer");
    cudaStream_t st = (cudaStream_t)stream;
    // control words (launch number, CTAs-done counter), then every packet of both inbox parities: a stale packet whose
    // tag equals a launch number that is about to be reused would otherwise be taken for a fresh one
    W8A16_CUDA(cudaMemsetAsync(base, 0, c.part_off, st));
    W8A16_CUDA(cudaMemsetAsync(base + c.inbox_off, 0, c.bytes - c.inbox_off, st));
    return 0;
}

int fp8w8a16_comm_destroy(fp8w8a16_comm* comm) {
    if (comm == nullptr) return 0;
    Comm& c = comm->c;
    for (int r = 0; r < c.world; ++r)
        if (r != c.rank && c.base[r] != nullptr && c.ipc_opened[r]) cudaIpcCloseMemHandle(c.base[r]);
    if (c.base[c.rank] != nullptr) cudaFree(c.base[c.rank]);
    delete comm;
    return 0;
}

int fp8w8a16_linear_allreduce_residual(fp8w8a16_comm* comm, const uint16_t* x, const uint8_t* w, const void* scales, int scale_dtype,
                                       const uint16_t* residual, uint16_t* out, int M, int N, int K, int block_h, int block_w,
                                       void* workspace, size_t workspace_bytes, void* stream) {
    W8A16_REQUIRE(comm != nullptr, FP8W8A16_ERR_INVALID, "linear_allreduce: null communicator");
    int rc = check_common(x, w, scales, out, M, N, K, block_h, block_w, scale_dtype);
    if (rc) return rc;
    if (M == 0 || N == 0) return 0;
    W8A16_REQUIRE(residual == nullptr || aligned16(residual), FP8W8A16_ERR_INVALID, "linear_allreduce: residual must be 16-byte aligned");
    ArParams ar;
    rc = comm_params(&comm->c, &ar);
    if (rc) return rc;
    return linear_tc(reinterpret_cast<const __half*>(x), w, scales, scale_dtype, reinterpret_cast<__half*>(out), M, N, K,
                     block_h, workspace, workspace_bytes, (cudaStream_t)stream, &ar, reinterpret_cast<const __half*>(residual));
}

int fp8w8a16_linear_allreduce(fp8w8a16_comm* comm, const uint16_t* x, const uint8_t* w, const void* scales, int scale_dtype,
                              uint16_t* out, int M, int N, int K, int block_h, int block_w, void* workspace,
                              size_t workspace_bytes, void* stream) {
    return fp8w8a16_linear_allreduce_residual(comm, x, w, scales, scale_dtype, nullptr, out, M, N, K, block_h, block_w, workspace,
                                              workspace_bytes, stream);
}

// ---- expert-parallel MoE over peer memory ------------------------------------------------------------------------
struct fp8w8a16_ep {
    w8a16::Ep e;
};

int fp8w8a16_ep_create(int rank, int world, int max_tokens, int topk, int hidden, int n_global_experts, unsigned int timeout_ms,
                       fp8w8a16_ep** ep) {
    W8A16_REQUIRE(ep != nullptr, FP8W8A16_ERR_INVALID, "ep_create: null output pointer");
    *ep = nullptr;
    W8A16_REQUIRE(world >= 1 && world <= kEpMaxWorld && rank >= 0 && rank < world, FP8W8A16_ERR_INVALID,
                  "ep_create: rank %d of world %d (1..%d ranks supported)", rank, world, kEpMaxWorld);
    W8A16_REQUIRE(max_tokens >= 1 && topk >= 1 && (int64_t)max_tokens * topk <= (1 << 24), FP8W8A16_ERR_INVALID,
                  "ep_create: max_tokens=%d topk=%d", max_tokens, topk);
    W8A16_REQUIRE(hidden >= 8 && hidden % 8 == 0, FP8W8A16_ERR_UNSUPPORTED, "ep_create: hidden size %d must be a multiple of 8", hidden);
    W8A16_REQUIRE(n_global_experts >= world && n_global_experts % world == 0, FP8W8A16_ERR_INVALID,
                  "ep_create: %d experts do not divide over %d ranks", n_global_experts, world);
    fp8w8a16_ep* h = new (std::nothrow) fp8w8a16_ep();
    W8A16_REQUIRE(h != nullptr, FP8W8A16_ERR_CUDA, "ep_create: out of host memory");
    Ep& e = h->e;
    memset(&e, 0, sizeof(e));
    EpGeom& g = e.g;
    g.world = world;
    g.rank = rank;
    g.H = hidden;
    g.cap = max_tokens * topk;
    g.experts_per_rank = n_global_experts / world;
    g.timeout_ms = timeout_ms ? timeout_ms : 2000u;
    e.max_tokens = max_tokens;
    e.topk = topk;
    e.n_global = n_global_experts;
    size_t o = 0;
    auto take = [&o](size_t bytes) {
        const size_t at = o;
        o += align_up(bytes, 256);
        return at;
    };
    const size_t slots = (size_t)world * g.cap;
    g.off_ctrl = (int64_t)take(256);
    g.off_hdr = (int64_t)take(kEpMaxWorld * 8);
    g.off_rflag = (int64_t)take(kEpMaxWorld * 8);
    e.off_dest_map = take((size_t)n_global_experts * 4);
    g.off_meta_e = (int64_t)take(slots * 4);
    g.off_meta_j = (int64_t)take(slots * 4);
    g.off_meta_w = (int64_t)take(slots * 4);
    g.off_rows = (int64_t)take(slots * hidden * 2);
    g.off_ret = (int64_t)take((size_t)g.cap * hidden * 2);
    e.bytes = o;
    cudaError_t ce = cudaGetDevice(&e.device);
    void* base = nullptr;
    if (ce == cudaSuccess) ce = cudaMalloc(&base, e.bytes);
    if (ce == cudaSuccess) ce = cudaMemset(base, 0, e.bytes);
    if (ce == cudaSuccess) {
        // expert -> owning rank (contiguous partition): the "expert map" the destination route table is built with
        int* host_map = new (std::nothrow) int[n_global_experts];
        if (host_map == nullptr) {
            ce = cudaErrorMemoryAllocation;
        } else {
            for (int x = 0; x < n_global_experts; ++x) host_map[x] = x / g.experts_per_rank;
            ce = cudaMemcpy(reinterpret_cast<char*>(base) + e.off_dest_map, host_map, (size_t)n_global_experts * 4, cudaMemcpyHostToDevice);
            delete[] host_map;
        }
    }
    if (ce != cudaSuccess) {
        if (base) cudaFree(base);
        delete h;
        return fail(FP8W8A16_ERR_CUDA, "ep_create: %s", cudaGetErrorString(ce));
    }
    g.base[rank] = reinterpret_cast<char*>(base);
    *ep = h;
    return 0;
}

int fp8w8a16_ep_export(const fp8w8a16_ep* ep, void* handle) {
    W8A16_REQUIRE(ep && handle, FP8W8A16_ERR_INVALID, "ep_export: null pointer");
    cudaIpcMemHandle_t hd;
    W8A16_CUDA(cudaIpcGetMemHandle(&hd, ep->e.g.base[ep->e.g.rank]));
    memcpy(handle, &hd, sizeof(hd));
    return 0;
}

int fp8w8a16_ep_attach(fp8w8a16_ep* ep, int peer, const void* handle) {
    W8A16_REQUIRE(ep && handle, FP8W8A16_ERR_INVALID, "ep_attach: null pointer");
    Ep& e = ep->e;
    W8A16_REQUIRE(peer >= 0 && peer < e.g.world && peer != e.g.rank, FP8W8A16_ERR_INVALID, "ep_attach: bad peer %d", peer);
    W8A16_REQUIRE(e.g.base[peer] == nullptr, FP8W8A16_ERR_INVALID, "ep_attach: peer %d is already attached", peer);
    cudaIpcMemHandle_t hd;
    memcpy(&hd, handle, sizeof(hd));
    void* ptr = nullptr;
    W8A16_CUDA(cudaIpcOpenMemHandle(&ptr, hd, cudaIpcMemLazyEnablePeerAccess));
    e.g.base[peer] = reinterpret_cast<char*>(ptr);
    e.ipc_opened[peer] = true;
    return 0;
}

int fp8w8a16_ep_attach_ptr(fp8w8a16_ep* ep, int peer, void* peer_base) {
    W8A16_REQUIRE(ep && peer_base, FP8W8A16_ERR_INVALID, "ep_attach_ptr: null pointer");
    Ep& e = ep->e;
    W8A16_REQUIRE(peer >= 0 && peer < e.g.world && peer != e.g.rank, FP8W8A16_ERR_INVALID, "ep_attach_ptr: bad peer %d", peer);
    W8A16_REQUIRE(e.g.base[peer] == nullptr, FP8W8A16_ERR_INVALID, "ep_attach_ptr: peer %d is already attached", peer);
    e.g.base[peer] = reinterpret_cast<char*>(peer_base);
    e.ipc_opened[peer] = false;
    return 0;
}

void* fp8w8a16_ep_base(const fp8w8a16_ep* ep) { return ep ? ep->e.g.base[ep->e.g.rank] : nullptr; }

size_t fp8w8a16_ep_bytes(const fp8w8a16_ep* ep) { return ep ? ep->e.bytes : 0; }

int fp8w8a16_ep_reset(fp8w8a16_ep* ep, void* stream) {
    W8A16_REQUIRE(ep != nullptr, FP8W8A16_ERR_INVALID, "ep_reset: null handle");
    Ep& e = ep->e;
    // call number, kernel counters, headers and return flags; the row buffers need no clearing (they are only read
    // up to a count that a fresh header announces)
    W8A16_CUDA(cudaMemsetAsync(e.g.base[e.g.rank], 0, e.off_dest_map, (cudaStream_t)stream));
    return 0;
}

int fp8w8a16_ep_destroy(fp8w8a16_ep* ep) {
    if (ep == nullptr) return 0;
    Ep& e = ep->e;
    for (int r = 0; r < e.g.world; ++r)
        if (r != e.g.rank && e.g.base[r] != nullptr && e.ipc_opened[r]) cudaIpcCloseMemHandle(e.g.base[r]);
    if (e.g.base[e.g.rank] != nullptr) cudaFree(e.g.base[e.g.rank]);
    delete ep;
    return 0;
}

static int ep_check_call(const fp8w8a16_ep* ep, int M, int M_max, const char* what) {
    W8A16_REQUIRE(ep != nullptr, FP8W8A16_ERR_INVALID, "%s: null handle", what);
    const Ep& e = ep->e;
    for (int r = 0; r < e.g.world; ++r)
        W8A16_REQUIRE(e.g.base[r] != nullptr, FP8W8A16_ERR_INVALID, "%s: rank %d is not attached", what, r);
    W8A16_REQUIRE(M >= 0 && M <= M_max && M_max >= 1 && M_max <= e.max_tokens, FP8W8A16_ERR_INVALID,
                  "%s: M=%d, largest batch of the call %d, buffer built for %d tokens per rank", what, M, M_max, e.max_tokens);
    return 0;
}

size_t fp8w8a16_ep_workspace_bytes(const fp8w8a16_ep* ep, int M, int M_max, int num_local_experts, int I) {
    if (ep == nullptr || M < 0 || M_max < 1 || num_local_experts < 1 || I < 1) return kTicketBytes;
    return ep_layout(ep->e, M, M_max, num_local_experts, I).total;
}

int fp8w8a16_ep_dispatch(fp8w8a16_ep* ep, const uint16_t* x, const void* topk_ids, int ids_are_i64, const float* topk_weights,
                         int M, int M_max, int num_local_experts, int I, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = ep_check_call(ep, M, M_max, "ep_dispatch");
    if (rc) return rc;
    const Ep& e = ep->e;
    W8A16_REQUIRE(M == 0 || (x && topk_ids && topk_weights), FP8W8A16_ERR_INVALID, "ep_dispatch: null pointer");
    W8A16_REQUIRE(M == 0 || aligned16(x), FP8W8A16_ERR_INVALID, "ep_dispatch: x must be 16-byte aligned");
    const EpLayout L = ep_layout(e, M, M_max, num_local_experts, I);
    W8A16_REQUIRE(workspace != nullptr && workspace_bytes >= L.total, FP8W8A16_ERR_WORKSPACE,
                  "ep_dispatch: workspace too small (%zu < %zu bytes)", workspace_bytes, L.total);
    char* ws = reinterpret_cast<char*>(workspace);
    cudaStream_t st = (cudaStream_t)stream;
    const int R = M * e.topk;
    int* d_offsets = reinterpret_cast<int*>(ws + L.d_offsets);
    int* d_sorted = reinterpret_cast<int*>(ws + L.d_sorted);
    const int* dest_map = reinterpret_cast<const int*>(e.g.base[e.g.rank] + e.off_dest_map);
    if (R <= kFuseRows)   // few rows: route table, stores and headers in one launch
        return launch_ep_send_small(reinterpret_cast<const __half*>(x), topk_ids, ids_are_i64, topk_weights, dest_map, e.n_global,
                                    reinterpret_cast<int*>(ws + L.d_counts), d_offsets, reinterpret_cast<int*>(ws + L.d_tiles), d_sorted,
                                    reinterpret_cast<int*>(ws + L.d_inv), R, e.topk, L.cap_call, e.g, st);
    // route table by destination rank: the align kernel with the expert -> rank map as its expert map
    rc = launch_align(topk_ids, ids_are_i64, R, dest_map, e.n_global, e.g.world, 1,
                      reinterpret_cast<int*>(ws + L.d_counts), d_offsets, reinterpret_cast<int*>(ws + L.d_tiles), d_sorted,
                      reinterpret_cast<int*>(ws + L.d_inv), st);
    if (rc) return rc;
    return launch_ep_send(reinterpret_cast<const __half*>(x), topk_ids, ids_are_i64, topk_weights, d_sorted, d_offsets, R, e.topk, L.cap_call,
                          e.g, st);
}

int fp8w8a16_ep_experts(fp8w8a16_ep* ep, const uint8_t* w13, const void* s13, const uint8_t* w2, const void* s2, int scale_dtype,
                        int M, int M_max, int num_local_experts, int I, int block_h, int activation, void* workspace,
                        size_t workspace_bytes, void* stream) {
    int rc = ep_check_call(ep, M, M_max, "ep_experts");
    if (rc) return rc;
    const Ep& e = ep->e;
    const int H = e.g.H, E = num_local_experts;
    W8A16_REQUIRE(w13 && s13 && w2 && s2, FP8W8A16_ERR_INVALID, "ep_experts: null pointer");
    W8A16_REQUIRE(E == e.g.experts_per_rank, FP8W8A16_ERR_INVALID, "ep_experts: %d local experts, the buffer was built for %d", E,
                  e.g.experts_per_rank);
    W8A16_REQUIRE(H % 16 == 0 && I > 0 && I % 16 == 0, FP8W8A16_ERR_UNSUPPORTED, "ep_experts: hidden %d and intermediate %d must be multiples of 16", H, I);
    W8A16_REQUIRE(block_h >= 1, FP8W8A16_ERR_INVALID, "ep_experts: block_h=%d", block_h);
    W8A16_REQUIRE(activation == FP8W8A16_ACT_SILU || activation == FP8W8A16_ACT_GELU, FP8W8A16_ERR_UNSUPPORTED,
                  "ep_experts: activation %d is not SiLU (1) or GELU (2)", activation);
    W8A16_REQUIRE(scale_dtype == FP8W8A16_SCALE_F16 || scale_dtype == FP8W8A16_SCALE_F32, FP8W8A16_ERR_INVALID, "ep_experts: unknown scale dtype %d", scale_dtype);
    const EpLayout L = ep_layout(e, M, M_max, E, I);
    W8A16_REQUIRE(workspace != nullptr && workspace_bytes >= L.total && aligned16(workspace), FP8W8A16_ERR_WORKSPACE,
                  "ep_experts: workspace too small or misaligned (%zu < %zu bytes)", workspace_bytes, L.total);
    char* ws = reinterpret_cast<char*>(workspace);
    cudaStream_t st = (cudaStream_t)stream;
    const MoeLayout& ML = L.moe;
    int* counts_in = reinterpret_cast<int*>(ws + L.counts_in);
    int* counts = reinterpret_cast<int*>(ws + ML.counts);
    int* offsets = reinterpret_cast<int*>(ws + ML.offsets);
    int* tile_offsets = reinterpret_cast<int*>(ws + ML.tile_offsets);
    int* sorted_route = reinterpret_cast<int*>(ws + ML.sorted_route);
    int* inv_pos = reinterpret_cast<int*>(ws + ML.inv_pos);
    float* w_sorted = reinterpret_cast<float*>(ws + ML.w_sorted);
    __half* x_sorted = reinterpret_cast<__half*>(ws + ML.x_sorted);
    __half* h_sorted = reinterpret_cast<__half*>(ws + ML.h_sorted);
    __half* y_sorted = reinterpret_cast<__half*>(ws + ML.y_sorted);
    const char* mine = e.g.base[e.g.rank];
    const int Rin = L.rows_in;
    // header wait and route table of the received rows in one launch; a small inbox is gathered by the same CTA
    const int fuse_gather = Rin <= kFuseRows ? 1 : 0;
    rc = launch_ep_recv_align(L.cap_call, counts_in, E, ML.bt, counts, offsets, tile_offsets, sorted_route, inv_pos, fuse_gather, x_sorted,
                              w_sorted, e.g, st);
    if (rc) return rc;
    if (!fuse_gather) {
        // every received row is one route of its own (top-1 view of the inbox); its weight came with it
        rc = launch_gather(reinterpret_cast<const __half*>(mine + e.g.off_rows), sorted_route,
                           reinterpret_cast<const float*>(mine + e.g.off_meta_w), Rin, 1, H, 0, x_sorted, w_sorted, st, offsets + E, ML.bt);
        if (rc) return rc;
    }
    rc = grouped_gemm(x_sorted, w13, s13, scale_dtype, h_sorted, nullptr, offsets, tile_offsets, Rin, E, I, H, block_h, activation, ML.bt,
                      ws + ML.gemm_ws, ML.gemm_ws_bytes, st);
    if (rc) return rc;
    rc = grouped_gemm(h_sorted, w2, s2, scale_dtype, y_sorted, w_sorted, offsets, tile_offsets, Rin, E, H, I, block_h, 0, ML.bt,
                      ws + ML.gemm_ws, ML.gemm_ws_bytes, st);
    if (rc) return rc;
    return launch_ep_return(y_sorted, inv_pos, counts_in, L.cap_call, e.g, st);
}

int fp8w8a16_ep_combine(fp8w8a16_ep* ep, const void* topk_ids, int ids_are_i64, uint16_t* out, int M, void* stream) {
    int rc = ep_check_call(ep, M, M > 0 ? M : 1, "ep_combine");
    if (rc) return rc;
    W8A16_REQUIRE(M == 0 || (topk_ids && out && aligned16(out)), FP8W8A16_ERR_INVALID, "ep_combine: null or misaligned pointer");
    return launch_ep_combine(topk_ids, ids_are_i64, M, ep->e.topk, reinterpret_cast<__half*>(out), ep->e.g, (cudaStream_t)stream);
}

int fp8w8a16_ep_moe_forward(fp8w8a16_ep* ep, const uint16_t* x, const void* topk_ids, int ids_are_i64, const float* topk_weights,
                            const uint8_t* w13, const void* s13, const uint8_t* w2, const void* s2, int scale_dtype, uint16_t* out,
                            int M, int M_max, int num_local_experts, int I, int block_h, int activation, void* workspace,
                            size_t workspace_bytes, void* stream) {
    int rc = fp8w8a16_ep_dispatch(ep, x, topk_ids, ids_are_i64, topk_weights, M, M_max, num_local_experts, I, workspace, workspace_bytes, stream);
    if (rc) return rc;
    rc = fp8w8a16_ep_experts(ep, w13, s13, w2, s2, scale_dtype, M, M_max, num_local_experts, I, block_h, activation, workspace,
                             workspace_bytes, stream);
    if (rc) return rc;
    return fp8w8a16_ep_combine(ep, topk_ids, ids_are_i64, out, M, stream);
}

}  // extern "C"
