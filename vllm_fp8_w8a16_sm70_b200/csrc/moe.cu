// Device-side routing and bookkeeping kernels of the MoE layer.  Nothing here synchronises with
// the host, so the whole layer can be captured in a CUDA graph.
//
//   topk_softmax : router logits -> top-k expert ids + weights (what vLLM's fused_topk hands to the
//                  reference's MoE apply, src/fp8_w8a16_sm70/vllm_serve.py:2175).
//   align        : expert_map remap (vllm_serve.py:2237-2243), per-expert counts, offsets, token-tile
//                  table and a STABLE expert-sorted permutation of the routed rows (the reference's
//                  sync-free route table: compressed_tensors_v100.py:776-784).
//   gather       : activations -> expert-sorted rows (reference: index_select, vllm_serve.py:1862).
//   combine      : weighted expert outputs -> one row per token (reference: index_add_, :1990).
#include <cuda_bf16.h>

#include "common.cuh"
#include "align.cuh"

namespace w8a16 {

namespace {

// ------------------------------------------------------------------------------------------------
// top-k softmax: one warp per token.  Selection is on the logits (ties -> lowest expert index);
// the weights are the fp32 softmax probabilities of the selected experts, optionally renormalised.
// ------------------------------------------------------------------------------------------------
constexpr int kMaxPerLane = 32;  // experts <= 1024

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Top-k softmax of one row of logits by one warp: fp32 softmax, k picks in descending order of logit, ties to the
// lowest expert index, weights = the picks' probabilities (optionally renormalised to sum to one).
template <typename T, int PER_LANE>
__device__ __forceinline__ void topk_row(const T* row, int E, int topk, int renorm, int* ids, float* weights, int lane) {
    float v[PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int e = i * 32 + lane;
        v[i] = e < E ? to_f32<T>(row[e]) : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) sum += (i * 32 + lane < E) ? expf(v[i] - mx) : 0.f;
    sum = warp_sum(sum);

    uint32_t taken = 0;  // bit i: this lane's i-th expert already selected
    float wsel = 0.f;    // lane t keeps the weight of the t-th pick
    int isel = 0;
    float wtot = 0.f;
    for (int t = 0; t < topk; ++t) {
        float best = -INFINITY;
        int best_e = 0x7FFFFFFF;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int e = i * 32 + lane;
            if (e < E && !((taken >> i) & 1u) && (v[i] > best)) {  // ascending e inside a lane: strict > keeps the lowest index
                best = v[i];
                best_e = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const int oe = __shfl_xor_sync(0xFFFFFFFFu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) {
                best = ob;
                best_e = oe;
            }
        }
        if (best_e != 0x7FFFFFFF && (best_e & 31) == lane) taken |= 1u << (best_e >> 5);
        const float pw = expf(best - mx) / sum;
        wtot += pw;
        if (lane == (t & 31)) {
            wsel = pw;
            isel = best_e;
        }
        if ((t & 31) == 31 || t == topk - 1) {  // flush up to 32 picks
            const int t0 = t & ~31;
            if (t0 + lane <= t) {
                ids[t0 + lane] = isel;
                weights[t0 + lane] = wsel;
            }
        }
    }
    if (renorm) {
        __syncwarp();
        for (int t = lane; t < topk; t += 32) weights[t] /= wtot;
    }
}

template <typename T, int PER_LANE>
__global__ void __launch_bounds__(128) k_topk_softmax(const T* __restrict__ logits, int M, int E, int topk, int renorm,
                                                      int* __restrict__ ids, float* __restrict__ weights) {
    pdl_trigger();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M) return;
    topk_row<T, PER_LANE>(logits + (int64_t)warp * E, E, topk, renorm, ids + (int64_t)warp * topk, weights + (int64_t)warp * topk, lane);
}

// Router: gate GEMV + top-k softmax in one kernel, one CTA per token.  logit[e] = sum_h x[h] * Wg[e, h] in fp32 (x FP16,
// gate weight FP16 / BF16 / fp32 as the model keeps it), then the same selection code as k_topk_softmax on the fp32 logits.
template <typename W, int PER_LANE>
__global__ void __launch_bounds__(256) k_router_topk(const __half* __restrict__ x, const W* __restrict__ gate, int M, int E, int H,
                                                     int topk, int renorm, int shared_id, float routed_scale,
                                                     int* __restrict__ ids, float* __restrict__ weights,
                                                     float* __restrict__ logits_out) {
    extern __shared__ __align__(16) unsigned char smem_router[];
    __half* sx = reinterpret_cast<__half*>(smem_router);                         // [H]
    float* sl = reinterpret_cast<float*>(smem_router + (size_t)H * sizeof(__half));  // [E]
    pdl_trigger();
    pdl_wait();
    const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x * 8; i < H; i += 256 * 8)
        *reinterpret_cast<uint4*>(sx + i) = *reinterpret_cast<const uint4*>(x + (int64_t)m * H + i);
    __syncthreads();
    for (int e = warp; e < E; e += 8) {
        const W* wr = gate + (int64_t)e * H;
        float acc = 0.f;
        for (int i = lane * 8; i < H; i += 32 * 8) {
            float wv[8];
            if (sizeof(W) == 2) {
                const uint4 q = *reinterpret_cast<const uint4*>(wr + i);
                const W* h8 = reinterpret_cast<const W*>(&q);
#pragma unroll
                for (int j = 0; j < 8; ++j) wv[j] = to_f32<W>(h8[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) wv[j] = to_f32<W>(wr[i + j]);
            }
            const uint4 xq = *reinterpret_cast<const uint4*>(sx + i);
            const __half* x8 = reinterpret_cast<const __half*>(&xq);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = fmaf(__half2float(x8[j]), wv[j], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            sl[e] = acc;
            if (logits_out != nullptr) logits_out[(int64_t)m * E + e] = acc;
        }
    }
    __syncthreads();
    if (warp == 0) {
        // row stride of the outputs: the picks, plus one fixed slot when a shared expert rides along as expert `shared_id`
        const int ld = topk + (shared_id >= 0 ? 1 : 0);
        int* my_ids = ids + (int64_t)m * ld;
        float* my_w = weights + (int64_t)m * ld;
        topk_row<float, PER_LANE>(sl, E, topk, renorm, my_ids, my_w, lane);
        __syncwarp();
        if (routed_scale != 1.0f)
            for (int t = lane; t < topk; t += 32) my_w[t] *= routed_scale;
        if (shared_id >= 0 && lane == 0) {
            my_ids[topk] = shared_id;
            my_w[topk] = 1.0f;
        }
    }
}

// The same router for decode batches, spread over a thread-block cluster per token: with one CTA per token a single SM
// would read the whole gate matrix (1 MiB at 128 experts x 4096: ~50 us); here every CTA of the cluster computes a
// share of the experts and stores its logits straight into the shared memory of the cluster's first CTA (distributed
// shared memory), which then selects.  Same arithmetic per logit, same selection code: identical results.
constexpr int kRouterCluster = 8;

template <typename W, int PER_LANE>
__global__ void __launch_bounds__(256) k_router_topk_cluster(const __half* __restrict__ x, const W* __restrict__ gate, int M, int E, int H,
                                                             int topk, int renorm, int shared_id, float routed_scale,
                                                             int* __restrict__ ids, float* __restrict__ weights,
                                                             float* __restrict__ logits_out) {
    extern __shared__ __align__(16) unsigned char smem_router[];
    __half* sx = reinterpret_cast<__half*>(smem_router);                         // [H]
    float* sl = reinterpret_cast<float*>(smem_router + (size_t)H * sizeof(__half));  // [E] (used in the cluster's first CTA)
    pdl_trigger();
    pdl_wait();
    uint32_t rank, nranks;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(nranks));
    const int m = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x * 8; i < H; i += 256 * 8)
        *reinterpret_cast<uint4*>(sx + i) = *reinterpret_cast<const uint4*>(x + (int64_t)m * H + i);
    __syncthreads();
    uint32_t sl0;   // the first CTA's logit array, as a cluster-wide shared-memory address
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(sl0) : "r"((uint32_t)__cvta_generic_to_shared(sl)), "r"(0u));
    for (int e = (int)rank * 8 + warp; e < E; e += 8 * (int)nranks) {
        const W* wr = gate + (int64_t)e * H;
        float acc = 0.f;
        for (int i = lane * 8; i < H; i += 32 * 8) {
            float wv[8];
            if (sizeof(W) == 2) {
                const uint4 q = *reinterpret_cast<const uint4*>(wr + i);
                const W* h8 = reinterpret_cast<const W*>(&q);
#pragma unroll
                for (int j = 0; j < 8; ++j) wv[j] = to_f32<W>(h8[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) wv[j] = to_f32<W>(wr[i + j]);
            }
            const uint4 xq = *reinterpret_cast<const uint4*>(sx + i);
            const __half* x8 = reinterpret_cast<const __half*>(&xq);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = fmaf(__half2float(x8[j]), wv[j], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(sl0 + (uint32_t)e * 4u), "f"(acc) : "memory");
            if (logits_out != nullptr) logits_out[(int64_t)m * E + e] = acc;
        }
    }
    // every CTA's logits are in the first CTA's shared memory once the whole cluster has passed this barrier
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    if (rank == 0 && warp == 0) {
        const int ld = topk + (shared_id >= 0 ? 1 : 0);
        int* my_ids = ids + (int64_t)m * ld;
        float* my_w = weights + (int64_t)m * ld;
        topk_row<float, PER_LANE>(sl, E, topk, renorm, my_ids, my_w, lane);
        __syncwarp();
        if (routed_scale != 1.0f)
            for (int t = lane; t < topk; t += 32) my_w[t] *= routed_scale;
        if (shared_id >= 0 && lane == 0) {
            my_ids[topk] = shared_id;
            my_w[topk] = 1.0f;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// align: one CTA.  Stable counting sort of the routed rows by local expert id (align.cuh).  With `x` given (small
// problems) the same CTA then gathers the rows, one warp per sorted position, and the gather kernel is not launched.
// ------------------------------------------------------------------------------------------------
template <typename IdT>
__global__ void __launch_bounds__(kAlignThreads)
k_align(const IdT* __restrict__ ids, int R, const int* __restrict__ expert_map, int n_global, int E, int bt,
        int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ tile_offsets,
        int* __restrict__ sorted_route, int* __restrict__ inv_pos, const __half* __restrict__ x, const float* __restrict__ topk_w,
        int topk, int H, int weight_on_input, __half* __restrict__ x_sorted, float* __restrict__ w_sorted) {
    pdl_trigger();
    extern __shared__ int sm[];
    for (int i = threadIdx.x; i < kAlignWarps * E; i += kAlignThreads) sm[i] = 0;
    pdl_wait();   // the expert ids come from the previous kernel
    __syncthreads();
    align_core([&](int i) { return local_expert(ids, i, expert_map, n_global, E); }, R, E, bt, counts, offsets, tile_offsets,
               sorted_route, inv_pos, sm);
    if (x != nullptr) {
        __syncthreads();   // sorted_route is complete
        for (int pos = threadIdx.x >> 5; pos < R; pos += kAlignWarps)
            gather_row(x, sorted_route[pos], topk_w, topk, H, weight_on_input, x_sorted, w_sorted, pos, threadIdx.x & 31);
    }
}

// ------------------------------------------------------------------------------------------------
// gather: x_sorted[pos] = x[route / topk] (optionally x route weight), w_sorted[pos] = weight[route].
// One warp per sorted row, 16-byte copies.  Rows past the valid count are zero-filled so that the
// token tiles of the grouped GEMM never read uninitialised memory.  When most of the R slots are known to be empty (the
// expert-parallel inbox: R is a capacity), `n_valid` points at the valid-row count and only `pad_rows` rows past it
// - what the last token tile can reach - are zero-filled.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_gather(const __half* __restrict__ x, const int* __restrict__ sorted_route, const float* __restrict__ topk_w, int R,
         int topk, int H, int weight_on_input, __half* __restrict__ x_sorted, float* __restrict__ w_sorted,
         const int* __restrict__ n_valid, int pad_rows) {
    pdl_trigger();
    pdl_wait();
    const int pos = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (pos >= R) return;
    if (n_valid != nullptr && pos >= *n_valid + pad_rows) return;
    gather_row(x, sorted_route[pos], topk_w, topk, H, weight_on_input, x_sorted, w_sorted, pos, lane);
}

// ------------------------------------------------------------------------------------------------
// combine: out[token] = sum over the token's routes of y_sorted[inv_pos[route]] (already weighted),
// summed in fp32 in route order, rounded once.  One CTA per token.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_combine(const __half* __restrict__ y_sorted, const int* __restrict__ inv_pos, int topk, int H, __half* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int token = blockIdx.x;
    extern __shared__ int s_pos[];
    for (int j = threadIdx.x; j < topk; j += blockDim.x) s_pos[j] = inv_pos[(int64_t)token * topk + j];
    __syncthreads();
    const int vecs = H >> 3;
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = 0.f;
        // eight routes' rows are requested together (one L2 round trip per batch instead of one per route); the sum
        // still runs in route order
        for (int j0 = 0; j0 < topk; j0 += 8) {
            uint4 v[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const int pos = (j0 + t < topk) ? s_pos[j0 + t] : -1;
                v[t] = pos >= 0 ? __ldg(reinterpret_cast<const uint4*>(y_sorted + (int64_t)pos * H) + i) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const __half2* h = reinterpret_cast<const __half2*>(&v[t]);   // +0 for a dropped route: exact
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float2 f = __half22float2(h[c]);
                    acc[2 * c] += f.x;
                    acc[2 * c + 1] += f.y;
                }
            }
        }
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int c = 0; c < 4; ++c) oh[c] = __floats2half2_rn(acc[2 * c], acc[2 * c + 1]);
        reinterpret_cast<uint4*>(out + (int64_t)token * H)[i] = o;
    }
}

template <typename T>
int launch_topk_t(const T* logits, int M, int E, int topk, int renorm, int* ids, float* weights, cudaStream_t st) {
    const int per_lane = (E + 31) / 32;
    const unsigned blocks = (unsigned)((M + 3) / 4);
    cudaError_t le = cudaSuccess;
#define W8A16_TOPK(PL) le = launch_pdl(k_topk_softmax<T, PL>, dim3(blocks), dim3(128), 0, st, logits, M, E, topk, renorm, ids, weights)
    if (per_lane <= 1) W8A16_TOPK(1);
    else if (per_lane <= 2) W8A16_TOPK(2);
    else if (per_lane <= 4) W8A16_TOPK(4);
    else if (per_lane <= 8) W8A16_TOPK(8);
    else if (per_lane <= 16) W8A16_TOPK(16);
    else W8A16_TOPK(32);
#undef W8A16_TOPK
    return finish_launch(le, "moe_topk_softmax");
}

}  // namespace

int launch_topk_softmax(const void* logits, int logits_dtype, int M, int E, int topk, int renorm, int* ids, float* weights,
                        cudaStream_t st) {
    W8A16_REQUIRE(E >= 1 && E <= 32 * kMaxPerLane, FP8W8A16_ERR_UNSUPPORTED, "topk_softmax: E=%d out of range [1,1024]", E);
    W8A16_REQUIRE(topk >= 1 && topk <= E, FP8W8A16_ERR_INVALID, "topk_softmax: topk=%d must be in [1,E=%d]", topk, E);
    if (M == 0) return 0;
    switch (logits_dtype) {
        case FP8W8A16_DTYPE_F32: return launch_topk_t(reinterpret_cast<const float*>(logits), M, E, topk, renorm, ids, weights, st);
        case FP8W8A16_DTYPE_F16: return launch_topk_t(reinterpret_cast<const __half*>(logits), M, E, topk, renorm, ids, weights, st);
        case FP8W8A16_DTYPE_BF16: return launch_topk_t(reinterpret_cast<const __nv_bfloat16*>(logits), M, E, topk, renorm, ids, weights, st);
    }
    return fail(FP8W8A16_ERR_INVALID, "topk_softmax: unknown logits dtype %d", logits_dtype);
}

namespace {
template <typename W, int PL>
cudaError_t launch_router_cluster(const __half* x, const W* gate, int M, int E, int H, int topk, int renorm, int shared_id,
                                  float routed_scale, int* ids, float* weights, float* logits_out, size_t smem, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kRouterCluster, (unsigned)M);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = kRouterCluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, k_router_topk_cluster<W, PL>, x, gate, M, E, H, topk, renorm, shared_id, routed_scale, ids, weights, logits_out);
}

template <typename W>
int launch_router_t(const __half* x, const W* gate, int M, int E, int H, int topk, int renorm, int shared_id, float routed_scale,
                    int* ids, float* weights, float* logits_out, cudaStream_t st) {
    const int per_lane = (E + 31) / 32;
    const size_t smem = (size_t)H * sizeof(__half) + (size_t)E * sizeof(float);
    cudaError_t le = cudaSuccess;
    // Decode batches (few tokens, enough experts to share out): a cluster of CTAs per token.  Large batches already fill the
    // machine with one CTA per token.  65535 bounds the y dimension of a grid.
    const bool clustered = E >= 8 * kRouterCluster && M <= 512 && M <= 65535 && smem <= 48 * 1024;
#define W8A16_ROUTER(PL)                                                                                                                   \
    le = clustered ? launch_router_cluster<W, PL>(x, gate, M, E, H, topk, renorm, shared_id, routed_scale, ids, weights, logits_out, smem, st) \
                   : launch_pdl(k_router_topk<W, PL>, dim3((unsigned)M), dim3(256), smem, st, x, gate, M, E, H, topk, renorm, shared_id, routed_scale, ids, weights, logits_out)
    if (per_lane <= 1) W8A16_ROUTER(1);
    else if (per_lane <= 2) W8A16_ROUTER(2);
    else if (per_lane <= 4) W8A16_ROUTER(4);
    else if (per_lane <= 8) W8A16_ROUTER(8);
    else W8A16_ROUTER(16);
#undef W8A16_ROUTER
    return finish_launch(le, "moe_router_topk");
}
}  // namespace

int launch_router_topk(const __half* x, const void* gate, int gate_dtype, int M, int E, int H, int topk, int renorm, int shared_id,
                       float routed_scale, int* ids, float* weights, float* logits_out, cudaStream_t st) {
    W8A16_REQUIRE(E >= 1 && E <= 512, FP8W8A16_ERR_UNSUPPORTED, "moe_router_topk: E=%d out of range [1,512]", E);
    W8A16_REQUIRE(topk >= 1 && topk <= E, FP8W8A16_ERR_INVALID, "moe_router_topk: topk=%d must be in [1,E=%d]", topk, E);
    W8A16_REQUIRE(H >= 8 && H % 8 == 0 && H <= 16384, FP8W8A16_ERR_UNSUPPORTED, "moe_router_topk: hidden size %d must be a multiple of 8, at most 16384", H);
    if (M == 0) return 0;
    switch (gate_dtype) {
        case FP8W8A16_DTYPE_F32: return launch_router_t(x, reinterpret_cast<const float*>(gate), M, E, H, topk, renorm, shared_id, routed_scale, ids, weights, logits_out, st);
        case FP8W8A16_DTYPE_F16: return launch_router_t(x, reinterpret_cast<const __half*>(gate), M, E, H, topk, renorm, shared_id, routed_scale, ids, weights, logits_out, st);
        case FP8W8A16_DTYPE_BF16: return launch_router_t(x, reinterpret_cast<const __nv_bfloat16*>(gate), M, E, H, topk, renorm, shared_id, routed_scale, ids, weights, logits_out, st);
    }
    return fail(FP8W8A16_ERR_INVALID, "moe_router_topk: unknown gate weight dtype %d", gate_dtype);
}

// With `x` given the align CTA also gathers the rows (callers do that for R <= kFuseRows and then skip launch_gather).
int launch_align(const void* ids, int ids_are_i64, int R, const int* expert_map, int n_global, int E, int bt, int* counts,
                 int* offsets, int* tile_offsets, int* sorted_route, int* inv_pos, cudaStream_t st, const __half* x,
                 const float* topk_w, int topk, int H, int weight_on_input, __half* x_sorted, float* w_sorted) {
    W8A16_REQUIRE(E >= 1 && E <= 1024, FP8W8A16_ERR_UNSUPPORTED, "moe_align: E=%d out of range [1,1024]", E);
    W8A16_REQUIRE(x == nullptr || (H % 8 == 0 && topk >= 1 && topk_w && x_sorted && w_sorted), FP8W8A16_ERR_INVALID,
                  "moe_align: fused gather needs H %% 8 == 0 (got %d), topk >= 1 and the gather buffers", H);
    const size_t smem = align_smem_bytes(E);
    // Above 48 KiB (E > ~370) the kernel's dynamic shared-memory limit has to be raised.  The attribute belongs to the
    // (function, device) pair and a later call may need more than an earlier one: remember the largest value set per device.
    static int set_bytes[2][64] = {};
    int dev = 0;
    W8A16_CUDA(cudaGetDevice(&dev));
    const int which = ids_are_i64 ? 1 : 0;
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || (int)smem > set_bytes[which][dev])) {
        if (ids_are_i64) W8A16_CUDA(cudaFuncSetAttribute(k_align<long long>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        else W8A16_CUDA(cudaFuncSetAttribute(k_align<int>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) set_bytes[which][dev] = (int)smem;
    }
    cudaError_t le;
    if (ids_are_i64)
        le = launch_pdl(k_align<long long>, dim3(1), dim3(kAlignThreads), smem, st, reinterpret_cast<const long long*>(ids), R, expert_map,
                        n_global, E, bt, counts, offsets, tile_offsets, sorted_route, inv_pos, x, topk_w, topk, H, weight_on_input,
                        x_sorted, w_sorted);
    else
        le = launch_pdl(k_align<int>, dim3(1), dim3(kAlignThreads), smem, st, reinterpret_cast<const int*>(ids), R, expert_map, n_global,
                        E, bt, counts, offsets, tile_offsets, sorted_route, inv_pos, x, topk_w, topk, H, weight_on_input, x_sorted,
                        w_sorted);
    return finish_launch(le, "moe_align");
}

int launch_gather(const __half* x, const int* sorted_route, const float* topk_w, int R, int topk, int H, int weight_on_input,
                  __half* x_sorted, float* w_sorted, cudaStream_t st, const int* n_valid, int pad_rows) {
    W8A16_REQUIRE(H % 8 == 0, FP8W8A16_ERR_UNSUPPORTED, "moe_gather: hidden size %d must be a multiple of 8", H);
    if (R == 0) return 0;
    return finish_launch(launch_pdl(k_gather, dim3((unsigned)((R + 7) / 8)), dim3(256), 0, st, x, sorted_route, topk_w, R, topk, H,
                                    weight_on_input, x_sorted, w_sorted, n_valid, pad_rows), "moe_gather");
}

int launch_combine(const __half* y_sorted, const int* inv_pos, int M, int topk, int H, __half* out, cudaStream_t st) {
    W8A16_REQUIRE(H % 8 == 0, FP8W8A16_ERR_UNSUPPORTED, "moe_combine: hidden size %d must be a multiple of 8", H);
    if (M == 0) return 0;
    return finish_launch(launch_pdl(k_combine, dim3((unsigned)M), dim3(256), topk * sizeof(int), st, y_sorted, inv_pos, topk, H, out),
                         "moe_combine");
}

}  // namespace w8a16
