// Route-table construction and row gathering shared by the single-GPU MoE layer (moe.cu) and the expert-parallel
// exchange kernels (ep.cu): a stable counting sort of routed rows by a small integer key (local expert, or destination
// rank), done by ONE CTA, and the copy of one routed row by one warp.
#pragma once
#include "common.cuh"

namespace w8a16 {

constexpr int kAlignThreads = 1024;
constexpr int kAlignWarps = kAlignThreads / 32;
// Up to this many rows, the CTA that built the route table also moves the rows (gather, or the stores into the peers'
// inboxes): one SM copies 16 rows of 4 KiB in about a microsecond, less than the launch boundary it saves; at 64 rows the
// copy already costs more than the launch (measured: the layer at 8 tokens x top-8 got 5 us slower).
constexpr int kFuseRows = 16;

inline size_t align_smem_bytes(int E) { return ((size_t)kAlignWarps * E + E + 1) * sizeof(int); }

template <typename IdT>
__device__ __forceinline__ int local_expert(const IdT* ids, int i, const int* expert_map, int n_global, int E) {
    long long g = (long long)ids[i];
    if (g < 0) return -1;
    if (expert_map != nullptr) {
        if (g >= n_global) return -1;
        g = expert_map[g];
    }
    return (g >= 0 && g < E) ? (int)g : -1;
}

// Stable counting sort of routes 0..R-1 by key(i) in [0, E) (-1 = dropped), by all kAlignThreads threads of one CTA.
// `sm` is dynamic shared memory of align_smem_bytes(E) whose first kAlignWarps * E words are ZERO on entry (and a
// __syncthreads() has been passed since they were zeroed).  Writes counts[E], offsets[E + 1], tile_offsets[E + 1]
// (token tiles of `bt` rows per key), sorted_route[R] (route index per sorted position, -1 past the valid rows) and
// inv_pos[R] (sorted position per route, -1 if dropped).  Returns the number of valid rows; the caller must pass a
// __syncthreads() before other threads of the CTA read what this wrote to global memory.
template <typename KeyFn>
__device__ __forceinline__ int align_core(KeyFn key, int R, int E, int bt, int* __restrict__ counts, int* __restrict__ offsets,
                                          int* __restrict__ tile_offsets, int* __restrict__ sorted_route, int* __restrict__ inv_pos,
                                          int* sm) {
    int* warp_hist = sm;                       // [kAlignWarps][E] -> later: running placement cursor
    int* s_off = sm + kAlignWarps * E;         // [E + 1]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // contiguous segment of routes per warp, walked in order 32 at a time
    const int per_warp = ((R + kAlignWarps - 1) / kAlignWarps + 31) & ~31;
    const int seg_begin = min(R, warp * per_warp), seg_end = min(R, seg_begin + per_warp);
    for (int base = seg_begin; base < seg_end; base += 32) {
        const int i = base + lane;
        const int e = i < seg_end ? key(i) : -1;
        if (e >= 0) atomicAdd(&warp_hist[warp * E + e], 1);
    }
    __syncthreads();
    // per key: total count; turn per-warp counts into an exclusive prefix over warps
    for (int e = tid; e < E; e += kAlignThreads) {
        int run = 0;
        for (int w = 0; w < kAlignWarps; ++w) {
            const int c = warp_hist[w * E + e];
            warp_hist[w * E + e] = run;
            run += c;
        }
        counts[e] = run;
        s_off[e] = run;  // counts for now
    }
    __syncthreads();
    if (warp == 0) {
        // exclusive scan of the counts (rows) and of ceil(count / bt) (token tiles) by one warp: every
        // lane scans a contiguous run of keys, the lane totals are scanned with shuffles
        const int per_lane = (E + 31) / 32;
        const int e0 = min(E, lane * per_lane), e1 = min(E, e0 + per_lane);
        int rows = 0, tiles = 0;
        for (int e = e0; e < e1; ++e) {
            const int c = s_off[e];
            rows += c;
            tiles += (c + bt - 1) / bt;
        }
        int rows_incl = rows, tiles_incl = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int a = __shfl_up_sync(0xFFFFFFFFu, rows_incl, o);
            const int b = __shfl_up_sync(0xFFFFFFFFu, tiles_incl, o);
            if (lane >= o) {
                rows_incl += a;
                tiles_incl += b;
            }
        }
        int run = rows_incl - rows, trun = tiles_incl - tiles;
        for (int e = e0; e < e1; ++e) {
            const int c = s_off[e];
            s_off[e] = run;
            offsets[e] = run;
            tile_offsets[e] = trun;
            run += c;
            trun += (c + bt - 1) / bt;
        }
        if (lane == 31) {
            s_off[E] = rows_incl;
            offsets[E] = rows_incl;
            tile_offsets[E] = tiles_incl;
        }
    }
    __syncthreads();
    const int n_valid = s_off[E];
    for (int base = seg_begin; base < seg_end; base += 32) {
        const int i = base + lane;
        const int e = i < seg_end ? key(i) : -1;
        const unsigned peers = __match_any_sync(0xFFFFFFFFu, e);
        if (e >= 0) {
            const int rank = __popc(peers & ((1u << lane) - 1u));
            const int cur = warp_hist[warp * E + e];
            const int pos = s_off[e] + cur + rank;
            sorted_route[pos] = i;
            inv_pos[i] = pos;
            __syncwarp(peers);
            if (rank == 0) warp_hist[warp * E + e] = cur + __popc(peers);
        } else if (i < seg_end) {
            inv_pos[i] = -1;
        }
        __syncwarp();
    }
    for (int i = n_valid + tid; i < R; i += kAlignThreads) sorted_route[i] = -1;
    return n_valid;
}

// One warp copies routed row `route` (token route / topk of x) to sorted position `pos`: x_sorted[pos] = x[route / topk]
// (optionally x route weight, in FP16 as the reference does: vllm_serve.py:1868-1870), w_sorted[pos] = weight[route];
// route < 0 zero-fills the row so that the token tiles of the grouped GEMM never read uninitialised memory.
__device__ __forceinline__ void gather_row(const __half* __restrict__ x, int route, const float* __restrict__ topk_w, int topk, int H,
                                           int weight_on_input, __half* __restrict__ x_sorted, float* __restrict__ w_sorted, int pos,
                                           int lane) {
    uint4* dst = reinterpret_cast<uint4*>(x_sorted + (int64_t)pos * H);
    const int vecs = H >> 3;
    if (route < 0) {
        for (int i = lane; i < vecs; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
        if (lane == 0) w_sorted[pos] = 0.f;
        return;
    }
    const float wt = topk_w[route];
    const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)(route / topk) * H);
    if (!weight_on_input) {
        int i = lane;
        for (; i + 96 < vecs; i += 128) {   // four 16-byte loads in flight per lane
            const uint4 a = __ldg(src + i), b = __ldg(src + i + 32), c = __ldg(src + i + 64), d = __ldg(src + i + 96);
            dst[i] = a;
            dst[i + 32] = b;
            dst[i + 64] = c;
            dst[i + 96] = d;
        }
        for (; i < vecs; i += 32) dst[i] = __ldg(src + i);
        if (lane == 0) w_sorted[pos] = wt;
    } else {
        const __half w16 = __float2half_rn(wt);
        const __half2 w2 = __halves2half2(w16, w16);
        for (int i = lane; i < vecs; i += 32) {
            uint4 v = __ldg(src + i);
            __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __hmul2(h[j], w2);
            dst[i] = v;
        }
        if (lane == 0) w_sorted[pos] = 1.f;
    }
}

}  // namespace w8a16
