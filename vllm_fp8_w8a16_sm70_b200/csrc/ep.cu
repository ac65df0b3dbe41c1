// Expert-parallel token exchange over peer memory (NVLink): device-side dispatch and combine of a routed MoE layer
// whose experts are partitioned over the ranks.  No NCCL, no host synchronisation, no split sizes read back: the
// counts travel as a fixed-size header, every region has a fixed capacity, and each step is an ordinary kernel on
// the caller's stream, so the whole layer can be captured in a CUDA graph.
//
// One call, seen from rank s (source of tokens) and rank q (owner of experts):
//   send     s: route table by DESTINATION rank (the align kernel with an expert -> rank map), then every routed row is
//               stored straight into q's inbox region [s] (plain 16-byte peer stores) with its local expert id, its
//               route index at the source and its route weight; when all rows of the grid have been stored, a header
//               {count, call number} per destination follows (system-scope fence before it).  Up to kFuseRows routed
//               rows, one CTA does all of it in one launch.
//   receive  q: ONE CTA waits - bounded - for the header of every source and sorts the received slots by local expert
//               (a slot past its source's count is dropped; a small inbox is gathered into expert order by the same CTA);
//               the ordinary grouped pipeline (gather -> gate/up GEMM with the activation -> down GEMM x route weight)
//               runs on those rows.
//   return   q: every finished row is stored into its source's return buffer at the row of its route index; a flag per
//               source follows when all rows are stored.
//   combine  s: waits - bounded - for the flag of every expert owner, then sums each token's routes in route order
//               (fp32, one rounding), exactly as the single-GPU combine does.
// Buffers are single: a source can only start call n + 1 after it has received every owner's return flag of call n,
// which an owner sends after it has finished reading call n's inbox.
//
// The reference has no counterpart: it tolerates expert parallelism through expert_map and a later reduce
// (src/fp8_w8a16_sm70/vllm_serve.py:2237-2243); the oracle of this path is the single-GPU layer.
#include "common.cuh"
#include "align.cuh"
#include "ep.h"

namespace w8a16 {

__device__ int g_ep_status = 0;   // sticky: 256 = a header did not arrive in time, 512 = a return flag did not

namespace {

__device__ __forceinline__ unsigned long long ep_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint2 ld_flag(const uint2* p) {
    uint2 v;
    asm volatile("ld.acquire.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_flag(uint2* p, uint32_t a, uint32_t b) {
    asm volatile("st.release.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// Waits until the flag's second word equals `epoch`; gives up after the limit.  Returns the first word, or -1.
__device__ __forceinline__ int wait_flag(const uint2* p, uint32_t epoch, unsigned long long limit_ns, int code) {
    uint2 v = ld_flag(p);
    if (v.y == epoch) return (int)v.x;
    const unsigned long long t0 = ep_now_ns();
    uint32_t spins = 0;
    for (;;) {
        v = ld_flag(p);
        if (v.y == epoch) return (int)v.x;
        if ((++spins & 0x3Fu) == 0u && ep_now_ns() - t0 > limit_ns) {
            atomicOr(&g_ep_status, code);
            return -1;
        }
        __nanosleep(64);
    }
}

// All stores of the grid are done: the last CTA to get here runs `publish`.  Every thread's stores are ordered before
// its CTA's arrival by a system-scope fence; the last CTA's fence after observing every arrival orders all of them
// before whatever `publish` stores.
template <typename F>
__device__ __forceinline__ void grid_done_then(unsigned int* counter, F publish) {
    __threadfence_system();
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(counter, 1u);
        s_last = (prev == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        publish();
        if (threadIdx.x == 0) *counter = 0u;
    }
}

__device__ __forceinline__ uint32_t call_number(const EpGeom& g) {
    return *reinterpret_cast<volatile unsigned int*>(g.base[g.rank] + g.off_ctrl) + 1u;
}
__device__ __forceinline__ unsigned int* ctrl_word(const EpGeom& g, int i) {
    return reinterpret_cast<unsigned int*>(g.base[g.rank] + g.off_ctrl) + i;
}

template <typename T>
__device__ __forceinline__ int64_t read_id(const void* ids, int64_t i) {
    return (int64_t)reinterpret_cast<const T*>(ids)[i];
}

// ---- send ------------------------------------------------------------------------------------------------
// One warp stores destination-sorted route `pos` (route index `route` at this rank) into its owner's inbox.
__device__ __forceinline__ void send_row(const __half* __restrict__ x, const void* __restrict__ topk_ids, int ids_are_i64,
                                         const float* __restrict__ topk_w, const int* dest_offsets, int pos, int route, int topk,
                                         int cap_call, const EpGeom& g, int lane) {
    const int H = g.H, P = g.world, s = g.rank;
    int q = 0;
    while (q + 1 < P && dest_offsets[q + 1] <= pos) ++q;     // at most 8 ranks
    const int i = pos - dest_offsets[q];
    if (i >= cap_call) return;
    char* peer = g.base[q];
    const int64_t slot = (int64_t)s * cap_call + i;
    const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)(route / topk) * H);
    uint4* dst = reinterpret_cast<uint4*>(peer + g.off_rows) + slot * (H >> 3);
    const int vecs = H >> 3;
    int v = lane;
    for (; v + 96 < vecs; v += 128) {
        const uint4 a = __ldg(src + v), b = __ldg(src + v + 32), c = __ldg(src + v + 64), d = __ldg(src + v + 96);
        dst[v] = a;
        dst[v + 32] = b;
        dst[v + 64] = c;
        dst[v + 96] = d;
    }
    for (; v < vecs; v += 32) dst[v] = __ldg(src + v);
    if (lane == 0) {
        const int64_t e = ids_are_i64 ? read_id<long long>(topk_ids, route) : read_id<int>(topk_ids, route);
        reinterpret_cast<int*>(peer + g.off_meta_e)[slot] = (int)(e - (int64_t)q * g.experts_per_rank);
        reinterpret_cast<int*>(peer + g.off_meta_j)[slot] = route;
        reinterpret_cast<float*>(peer + g.off_meta_w)[slot] = topk_w[route];
    }
}

// one warp per destination-sorted route; the route table comes from the align kernel
__global__ void __launch_bounds__(256)
k_ep_send(const __half* __restrict__ x, const void* __restrict__ topk_ids, int ids_are_i64, const float* __restrict__ topk_w,
          const int* __restrict__ sorted_route, const int* __restrict__ dest_offsets, int R, int topk, int cap_call, const EpGeom g) {
    pdl_trigger();
    pdl_wait();
    const uint32_t epoch = call_number(g);
    const int P = g.world, s = g.rank;
    const int pos = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int route = pos < R ? sorted_route[pos] : -1;
    if (route >= 0) send_row(x, topk_ids, ids_are_i64, topk_w, dest_offsets, pos, route, topk, cap_call, g, lane);
    grid_done_then(ctrl_word(g, 1), [&]() {
        if ((int)threadIdx.x < P) {
            const int q = threadIdx.x;
            int cnt = dest_offsets[q + 1] - dest_offsets[q];
            if (cnt > cap_call) cnt = cap_call;
            st_flag(reinterpret_cast<uint2*>(g.base[q] + g.off_hdr) + s, (uint32_t)cnt, epoch);
        }
    });
}

// Small batches: ONE CTA builds the route table by destination rank (align.cuh, key = owner of the route's expert), stores
// the rows and publishes the headers - one launch instead of two.
template <typename IdT>
__global__ void __launch_bounds__(kAlignThreads)
k_ep_send_small(const __half* __restrict__ x, const IdT* __restrict__ topk_ids, const float* __restrict__ topk_w,
                const int* __restrict__ dest_map, int n_global, int* __restrict__ counts, int* __restrict__ offsets,
                int* __restrict__ tile_offsets, int* __restrict__ sorted_route, int* __restrict__ inv_pos, int R, int topk,
                int cap_call, const EpGeom g) {
    pdl_trigger();
    extern __shared__ int sm[];
    const int P = g.world, s = g.rank;
    for (int i = threadIdx.x; i < kAlignWarps * P; i += kAlignThreads) sm[i] = 0;
    pdl_wait();
    __syncthreads();
    align_core([&](int i) { return local_expert(topk_ids, i, dest_map, n_global, P); }, R, P, 1, counts, offsets, tile_offsets,
               sorted_route, inv_pos, sm);
    __syncthreads();   // sorted_route and the offsets are complete
    const uint32_t epoch = call_number(g);
    const int* s_off = sm + kAlignWarps * P;   // exclusive row offsets per destination, [P] = number of valid rows
    const int n_valid = s_off[P];
    for (int pos = threadIdx.x >> 5; pos < n_valid; pos += kAlignWarps)
        send_row(x, topk_ids, sizeof(IdT) == 8, topk_w, s_off, pos, sorted_route[pos], topk, cap_call, g, threadIdx.x & 31);
    __threadfence_system();   // every thread's peer stores before the CTA-wide barrier ...
    __syncthreads();
    if ((int)threadIdx.x < P) {
        __threadfence_system();   // ... and all of them before this thread's header
        const int q = threadIdx.x;
        int cnt = s_off[q + 1] - s_off[q];
        if (cnt > cap_call) cnt = cap_call;
        st_flag(reinterpret_cast<uint2*>(g.base[q] + g.off_hdr) + s, (uint32_t)cnt, epoch);
    }
}

// ---- receive -------------------------------------------------------------------------------------------
// Receive and local route table in ONE CTA: waits for the headers, then sorts the received slots by local expert
// (align.cuh; a slot past its source's count, or with an expert id out of range, is dropped) and - for small inboxes -
// gathers the rows into expert order too, so that the separate receive, align and gather launches are not needed.
__global__ void __launch_bounds__(kAlignThreads)
k_ep_recv_align(int cap_call, int* __restrict__ counts_in, int E, int bt, int* __restrict__ counts, int* __restrict__ offsets,
                int* __restrict__ tile_offsets, int* __restrict__ sorted_route, int* __restrict__ inv_pos, int fuse_gather,
                __half* __restrict__ x_sorted, float* __restrict__ w_sorted, const EpGeom g) {
    pdl_trigger();
    extern __shared__ int sm[];
    int* s_cnt = sm + kAlignWarps * E + E + 1;   // [kEpMaxWorld]
    for (int i = threadIdx.x; i < kAlignWarps * E; i += kAlignThreads) sm[i] = 0;
    pdl_wait();
    const uint32_t epoch = call_number(g);
    const char* mine = g.base[g.rank];
    if ((int)threadIdx.x < g.world) {
        const int c = wait_flag(reinterpret_cast<const uint2*>(mine + g.off_hdr) + threadIdx.x, epoch,
                                (unsigned long long)g.timeout_ms * 1000000ull, 256);
        s_cnt[threadIdx.x] = c < 0 ? 0 : min(c, cap_call);     // a source that never arrived contributes nothing
        counts_in[threadIdx.x] = s_cnt[threadIdx.x];
    }
    __syncthreads();
    const int* meta_e = reinterpret_cast<const int*>(mine + g.off_meta_e);
    const int total = g.world * cap_call;
    const int n_valid = align_core(
        [&](int idx) {
            const int s = idx / cap_call, i = idx - s * cap_call;
            if (i >= s_cnt[s]) return -1;
            const int e = __ldcg(meta_e + idx);
            return (e < 0 || e >= E) ? -1 : e;
        },
        total, E, bt, counts, offsets, tile_offsets, sorted_route, inv_pos, sm);
    if (fuse_gather) {
        __syncthreads();   // sorted_route is complete
        // every received row is one route of its own (top-1 view of the inbox); rows up to the end of the last token tile
        // are zero-filled
        const int rows = min(total, n_valid + bt);
        const __half* rows_in = reinterpret_cast<const __half*>(mine + g.off_rows);
        const float* w_in = reinterpret_cast<const float*>(mine + g.off_meta_w);
        for (int pos = threadIdx.x >> 5; pos < rows; pos += kAlignWarps)
            gather_row(rows_in, sorted_route[pos], w_in, 1, g.H, 0, x_sorted, w_sorted, pos, threadIdx.x & 31);
    }
}

// ---- return: one warp per received slot -----------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_ep_return(const __half* __restrict__ y_sorted, const int* __restrict__ inv_pos, const int* __restrict__ counts_in, int cap_call,
            const EpGeom g) {
    pdl_trigger();
    pdl_wait();
    const uint32_t epoch = call_number(g);
    const int H = g.H, P = g.world;
    const int idx = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (idx < P * cap_call) {
        const int s = idx / cap_call, i = idx - s * cap_call;
        const int pos = i < counts_in[s] ? inv_pos[idx] : -1;
        if (pos >= 0) {
            const int j = __ldcg(reinterpret_cast<const int*>(g.base[g.rank] + g.off_meta_j) + idx);   // route index at the source
            if (j >= 0 && j < g.cap) {
                const uint4* src = reinterpret_cast<const uint4*>(y_sorted + (int64_t)pos * H);
                uint4* dst = reinterpret_cast<uint4*>(g.base[s] + g.off_ret) + (int64_t)j * (H >> 3);
                const int vecs = H >> 3;
                int v = lane;
                for (; v + 96 < vecs; v += 128) {
                    const uint4 a = __ldcg(src + v), b = __ldcg(src + v + 32), c = __ldcg(src + v + 64), d = __ldcg(src + v + 96);
                    dst[v] = a;
                    dst[v + 32] = b;
                    dst[v + 64] = c;
                    dst[v + 96] = d;
                }
                for (; v < vecs; v += 32) dst[v] = __ldcg(src + v);
            }
        }
    }
    grid_done_then(ctrl_word(g, 2), [&]() {
        if ((int)threadIdx.x < P) st_flag(reinterpret_cast<uint2*>(g.base[threadIdx.x] + g.off_rflag) + g.rank, 0u, epoch);
    });
}

// ---- combine: one CTA per token ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
k_ep_combine(const void* __restrict__ topk_ids, int ids_are_i64, int topk, __half* __restrict__ out, const EpGeom g) {
    pdl_trigger();
    pdl_wait();
    const uint32_t epoch = call_number(g);
    const int H = g.H, token = blockIdx.x;
    const char* mine = g.base[g.rank];
    __shared__ int s_bad;
    extern __shared__ int s_row[];
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
    if ((int)threadIdx.x < g.world) {
        if (wait_flag(reinterpret_cast<const uint2*>(mine + g.off_rflag) + threadIdx.x, epoch,
                      (unsigned long long)g.timeout_ms * 1000000ull, 512) < 0)
            s_bad = 1;
    }
    for (int j = threadIdx.x; j < topk; j += blockDim.x) {
        const int64_t r = (int64_t)token * topk + j;
        const int64_t e = ids_are_i64 ? read_id<long long>(topk_ids, r) : read_id<int>(topk_ids, r);
        s_row[j] = (e >= 0 && e < (int64_t)g.experts_per_rank * g.world && r < g.cap) ? (int)r : -1;
    }
    __syncthreads();
    const bool bad = s_bad != 0;       // an owner never answered: write zeros rather than whatever the buffer holds
    const uint4* ret = reinterpret_cast<const uint4*>(mine + g.off_ret);
    const int vecs = H >> 3;
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = 0.f;
        for (int j0 = 0; j0 < topk; j0 += 8) {
            uint4 v[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const int row = (j0 + t < topk && !bad) ? s_row[j0 + t] : -1;
                v[t] = row >= 0 ? __ldcg(ret + (int64_t)row * vecs + i) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const __half2* h = reinterpret_cast<const __half2*>(&v[t]);
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
    // the call is over on this rank when its last CTA has summed its token: advance the call number
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int prev = atomicAdd(ctrl_word(g, 3), 1u);
        if (prev == gridDim.x - 1) {
            *ctrl_word(g, 3) = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned int*>(ctrl_word(g, 0)) = epoch;
        }
    }
}

// an empty local batch still has to close the call (its peers wait for nothing from it, but the call number must advance)
__global__ void k_ep_advance(const EpGeom g) {
    pdl_trigger();
    pdl_wait();
    const uint32_t epoch = call_number(g);
    // the flags of this call must have arrived before the next call may reuse the buffers
    if ((int)threadIdx.x < g.world)
        wait_flag(reinterpret_cast<const uint2*>(g.base[g.rank] + g.off_rflag) + threadIdx.x, epoch,
                  (unsigned long long)g.timeout_ms * 1000000ull, 512);
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile unsigned int*>(ctrl_word(g, 0)) = epoch;
}

}  // namespace

int launch_ep_send(const __half* x, const void* topk_ids, int ids_are_i64, const float* topk_w, const int* sorted_route,
                   const int* dest_offsets, int R, int topk, int cap_call, const EpGeom& g, cudaStream_t st) {
    // at least one CTA even for an empty batch: the headers (count 0) must still go out
    const unsigned grid = (unsigned)((R > 0 ? R : 1) + 7) / 8;
    return finish_launch(launch_pdl(k_ep_send, dim3(grid), dim3(256), 0, st, x, topk_ids, ids_are_i64, topk_w, sorted_route, dest_offsets,
                                    R, topk, cap_call, g), "ep_send");
}

int launch_ep_send_small(const __half* x, const void* topk_ids, int ids_are_i64, const float* topk_w, const int* dest_map, int n_global,
                         int* counts, int* offsets, int* tile_offsets, int* sorted_route, int* inv_pos, int R, int topk, int cap_call,
                         const EpGeom& g, cudaStream_t st) {
    const size_t smem = align_smem_bytes(g.world);
    cudaError_t le;
    if (ids_are_i64)
        le = launch_pdl(k_ep_send_small<long long>, dim3(1), dim3(kAlignThreads), smem, st, x, reinterpret_cast<const long long*>(topk_ids),
                        topk_w, dest_map, n_global, counts, offsets, tile_offsets, sorted_route, inv_pos, R, topk, cap_call, g);
    else
        le = launch_pdl(k_ep_send_small<int>, dim3(1), dim3(kAlignThreads), smem, st, x, reinterpret_cast<const int*>(topk_ids), topk_w,
                        dest_map, n_global, counts, offsets, tile_offsets, sorted_route, inv_pos, R, topk, cap_call, g);
    return finish_launch(le, "ep_send_small");
}

int launch_ep_recv_align(int cap_call, int* counts_in, int E, int bt, int* counts, int* offsets, int* tile_offsets, int* sorted_route,
                         int* inv_pos, int fuse_gather, __half* x_sorted, float* w_sorted, const EpGeom& g, cudaStream_t st) {
    W8A16_REQUIRE(E >= 1 && E <= 1024, FP8W8A16_ERR_UNSUPPORTED, "ep_recv_align: E=%d out of range [1,1024]", E);
    const size_t smem = align_smem_bytes(E) + kEpMaxWorld * sizeof(int);
    static int set_bytes[64] = {};
    int dev = 0;
    W8A16_CUDA(cudaGetDevice(&dev));
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || (int)smem > set_bytes[dev])) {
        W8A16_CUDA(cudaFuncSetAttribute(k_ep_recv_align, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (dev >= 0 && dev < 64) set_bytes[dev] = (int)smem;
    }
    return finish_launch(launch_pdl(k_ep_recv_align, dim3(1), dim3(kAlignThreads), smem, st, cap_call, counts_in, E, bt, counts, offsets,
                                    tile_offsets, sorted_route, inv_pos, fuse_gather, x_sorted, w_sorted, g), "ep_recv_align");
}

int launch_ep_return(const __half* y_sorted, const int* inv_pos, const int* counts_in, int cap_call, const EpGeom& g, cudaStream_t st) {
    const int total = g.world * cap_call;
    const unsigned grid = (unsigned)((total > 0 ? total : 1) + 7) / 8;
    return finish_launch(launch_pdl(k_ep_return, dim3(grid), dim3(256), 0, st, y_sorted, inv_pos, counts_in, cap_call, g), "ep_return");
}

int launch_ep_combine(const void* topk_ids, int ids_are_i64, int M, int topk, __half* out, const EpGeom& g, cudaStream_t st) {
    if (M == 0) return finish_launch(launch_pdl(k_ep_advance, dim3(1), dim3(32), 0, st, g), "ep_advance");
    return finish_launch(launch_pdl(k_ep_combine, dim3((unsigned)M), dim3(256), (size_t)topk * sizeof(int), st, topk_ids, ids_are_i64, topk,
                                    out, g), "ep_combine");
}

int ep_read_status(int* out, int reset) {
    int v = 0;
    W8A16_CUDA(cudaMemcpyFromSymbol(&v, g_ep_status, sizeof(int)));
    if (reset && v != 0) {
        const int zero = 0;
        W8A16_CUDA(cudaMemcpyToSymbol(g_ep_status, &zero, sizeof(int)));
    }
    *out = v;
    return 0;
}

}  // namespace w8a16
