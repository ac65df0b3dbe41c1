// Decode GEMV for 1..4 tokens: C[m,n] = sum_k A[m,k] * cvt(W[n,k]) * S[n/bh, k/128]
//
// HBM-bound on the FP8 weight stream.  One warp owns R = 4 consecutive weight rows and one K range;
// a lane reads 16 weight bytes per row per step (a warp covers 512 contiguous bytes of each row with
// one 16-byte load per lane), so 4 independent 16-byte loads per lane are in flight per step and the
// activations are fetched once per step for all 4 rows.  Dequant happens in registers (hardware
// cvt.rn.f16x2.e4m3x2), products are accumulated in fp32 (fma.rn.f32.f16) per 16-element run and multiplied by the block (or channel) scale once per
// run, the lanes are reduced with warp shuffles.  K is split into ranges; partial sums go to an fp32
// workspace and the LAST warp to arrive for a row group (ticket counter) adds them in fixed split
// order, so the result does not depend on scheduling.
//
// Replaces the reference's decode kernels fp8_w8a16_gemv_coalesced / _coalesced_m / gemm_a3
// (src/fp8_w8a16_sm70/fp8_dequant.cu:622-786, 535-594).
#include "common.cuh"

namespace w8a16 {

namespace {

constexpr int kRows = 4;               // weight rows per warp
constexpr int kWarps = 8;              // warps per CTA
constexpr int kThreads = kWarps * 32;
constexpr int kStep = 512;             // K elements one warp covers per step

// 16 E4M3 bytes (uint4) times 16 FP16 activations (8 packed pairs per token) -> fp32 dot products.
// Weights are converted with the hardware cvt (exact) and multiplied in fma.rn.f32.f16; the block
// scale is applied by the caller once per 16-element run.
template <int M>
__device__ __forceinline__ void dot16(const uint4& q, const uint32_t (&xh)[M][8], float (&part)[M]) {
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        uint32_t w01, w23;
        e4m3x4_cvt(words[t], w01, w23);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            fma2_f32_f16(part[m], w01, xh[m][2 * t]);
            fma2_f32_f16(part[m], w23, xh[m][2 * t + 1]);
        }
    }
}

// One warp per unit = (group of 4 weight rows, K range); warps stride over the units (persistent grid),
// so the last wave is as fine as one unit.  Two 512-element steps are issued back to back: eight 16-byte
// weight loads per lane are in flight before the first conversion starts.
template <int M>
__global__ void __launch_bounds__(kThreads)
k_gemv(const __half* __restrict__ x, const uint8_t* __restrict__ w, const void* __restrict__ scales, int scale_dtype,
       __half* __restrict__ out, float* __restrict__ partial, unsigned int* __restrict__ tickets, int N, int K,
       int block_h, int Kb, int k_chunk, int splits, int row_groups) {
    pdl_trigger();   // let the next kernel of the stream begin launching
    pdl_wait();      // the activations (and the workspace) come from earlier kernels
    const int lane = threadIdx.x & 31;
    const int gwarp = (blockIdx.x * kThreads + threadIdx.x) >> 5;
    const int total_warps = (gridDim.x * kThreads) >> 5;
    const int total_units = row_groups * splits;
    const bool one_scale = (block_h % kRows) == 0;  // all 4 rows share the scale-grid row

    for (int unit = gwarp; unit < total_units; unit += total_warps) {
        const int rg = unit / splits, split = unit - rg * splits;
        const int row0 = rg * kRows;
        const int k_begin = split * k_chunk;
        const int k_end = min(K, k_begin + k_chunk);

        float acc[kRows][M];
#pragma unroll
        for (int r = 0; r < kRows; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) acc[r][m] = 0.f;

        const uint8_t* wrow[kRows];
        int srow[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int n = min(row0 + r, N - 1);  // clamp: out-of-range rows are computed and dropped
            wrow[r] = w + (int64_t)n * K;
            srow[r] = (n / block_h) * Kb;
        }

        for (int k = k_begin + lane * 16; k < k_end; k += 2 * kStep) {
            const bool two = (k + kStep) < k_end;
            const int k2 = two ? k + kStep : k;   // a missing second step re-reads the first with zero weights
            uint4 q[2][kRows];
#pragma unroll
            for (int r = 0; r < kRows; ++r) q[0][r] = __ldcs(reinterpret_cast<const uint4*>(wrow[r] + k));
#pragma unroll
            for (int r = 0; r < kRows; ++r)
                q[1][r] = two ? __ldcs(reinterpret_cast<const uint4*>(wrow[r] + k2)) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int kk = h == 0 ? k : k2;
                uint32_t xh[M][8];
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const uint4 a0 = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)m * K + kk));
                    const uint4 a1 = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)m * K + kk) + 1);
                    xh[m][0] = a0.x; xh[m][1] = a0.y; xh[m][2] = a0.z; xh[m][3] = a0.w;
                    xh[m][4] = a1.x; xh[m][5] = a1.y; xh[m][6] = a1.z; xh[m][7] = a1.w;
                }
                const int kb = kk >> 7;
                float sc[kRows];
                if (one_scale) {
                    const float s0 = __half2float(load_scale_h(scales, srow[0] + kb, scale_dtype));
#pragma unroll
                    for (int r = 0; r < kRows; ++r) sc[r] = s0;
                } else {
#pragma unroll
                    for (int r = 0; r < kRows; ++r) sc[r] = __half2float(load_scale_h(scales, srow[r] + kb, scale_dtype));
                }
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    float part[M];
#pragma unroll
                    for (int m = 0; m < M; ++m) part[m] = 0.f;
                    dot16<M>(q[h][r], xh, part);
#pragma unroll
                    for (int m = 0; m < M; ++m) acc[r][m] = fmaf(sc[r], part[m], acc[r][m]);
                }
            }
        }

#pragma unroll
        for (int r = 0; r < kRows; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]);

        if (splits == 1) {
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < kRows; ++r)
                    if (row0 + r < N)
#pragma unroll
                        for (int m = 0; m < M; ++m) out[(int64_t)m * N + row0 + r] = __float2half_rn(acc[r][m]);
            }
            continue;
        }

        // split-K: publish this warp's partial sums; the last warp to arrive for the row group adds the
        // splits in ascending order (deterministic) and leaves the ticket at zero for the next launch.
        unsigned int ticket = 0;
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < kRows; ++r)
                if (row0 + r < N)
#pragma unroll
                    for (int m = 0; m < M; ++m) __stcg(&partial[((int64_t)split * M + m) * N + row0 + r], acc[r][m]);
            __threadfence();
            ticket = atomicAdd(&tickets[rg], 1u);
        }
        ticket = __shfl_sync(0xFFFFFFFFu, ticket, 0);
        if (ticket != (unsigned)(splits - 1)) continue;
        __threadfence();
        if (lane < kRows * M) {
            const int m = lane / kRows, n = row0 + (lane - m * kRows);
            if (n < N) {
                float v = 0.f;
                for (int sp = 0; sp < splits; ++sp) v += __ldcg(&partial[((int64_t)sp * M + m) * N + n]);
                out[(int64_t)m * N + n] = __float2half_rn(v);
            }
        }
        if (lane == 0) tickets[rg] = 0u;
    }
}

constexpr int kMaxTicketGroups = (int)(kTicketBytes / sizeof(unsigned int));

int gemv_grid_ctas() { return sm_count() * 3; }

// CTAs of k_gemv<M> that fit on one SM (register-limited), asked from the runtime once per M.
int resident_ctas_per_sm(int m) {
    static int cached[5] = {0, 0, 0, 0, 0};
    if (cached[m] == 0) {
        int n = 0;
        cudaError_t e = cudaErrorUnknown;
        switch (m) {
            case 1: e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k_gemv<1>, kThreads, 0); break;
            case 2: e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k_gemv<2>, kThreads, 0); break;
            case 3: e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k_gemv<3>, kThreads, 0); break;
            default: e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k_gemv<4>, kThreads, 0); break;
        }
        cached[m] = (e == cudaSuccess && n > 0) ? n : 2;
    }
    return cached[m];
}

}  // namespace

// K range of one unit for a GEMV over [N,K] (a multiple of the 512-element step; the number of splits follows from it).
// All units are the same size and the warps of the resident grid take them in waves, so a launch lasts about
// ceil(units / warps) * k_chunk elements per warp: the candidate with the smallest such product wins (every unit at least
// 2048 elements long; a split costs a partial-sum round trip, so ties go to fewer splits).
int gemv_pick_chunk(int N, int K) {
    const int row_groups = (N + kRows - 1) / kRows;
    const int k_full = (K + kStep - 1) / kStep * kStep;
    if (row_groups > kMaxTicketGroups) return k_full;   // more row groups than ticket counters: no split (already plenty of units)
    const int64_t warps = (int64_t)gemv_grid_ctas() * kWarps;
    int max_s = K / (4 * kStep);
    if (max_s > 32) max_s = 32;
    if (max_s < 1) max_s = 1;
    int best_chunk = k_full;
    int64_t best_cost = -1;
    for (int s = 1; s <= max_s; ++s) {
        const int chunk = ((K + s - 1) / s + kStep - 1) / kStep * kStep;
        const int splits = (K + chunk - 1) / chunk;
        const int64_t units = (int64_t)row_groups * splits;
        const int64_t waves = (units + warps - 1) / warps;
        const int64_t cost = waves * chunk + (splits > 1 ? 64 * splits : 0);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best_chunk = chunk;
        }
    }
    return best_chunk;
}

int gemv_pick_splits(int N, int K) {
    const int chunk = gemv_pick_chunk(N, K);
    return (K + chunk - 1) / chunk;
}

size_t gemv_workspace_bytes(int M, int N, int K) {
    const int splits = gemv_pick_splits(N, K);
    const int mm = M < 4 ? M : 4;
    const size_t partial = splits > 1 ? (size_t)splits * mm * N * sizeof(float) : 0;
    return kTicketBytes + ((partial + 255) & ~(size_t)255);
}

// Workspace layout: ticket counters in the first kTicketBytes (zero on entry, left at zero on
// exit), fp32 partial sums after them (no initialisation needed).
int launch_gemv(const __half* x, const uint8_t* w, const void* scales, int scale_dtype, __half* out, int M, int N,
                int K, int block_h, int block_w, void* workspace, size_t workspace_bytes, cudaStream_t st) {
    W8A16_REQUIRE(block_w == 128, FP8W8A16_ERR_UNSUPPORTED, "gemv: block_w must be 128 (got %d)", block_w);
    W8A16_REQUIRE(K % 16 == 0, FP8W8A16_ERR_UNSUPPORTED, "gemv: K must be a multiple of 16 (got %d)", K);
    W8A16_REQUIRE(aligned16(x) && aligned16(w), FP8W8A16_ERR_INVALID, "gemv: x and w must be 16-byte aligned");
    if (M == 0 || N == 0) return 0;
    const int Kb = (K + 127) / 128;
    const int row_groups = (N + kRows - 1) / kRows;
    const int k_chunk = gemv_pick_chunk(N, K);
    const int splits = (K + k_chunk - 1) / k_chunk;
    float* partial = nullptr;
    unsigned int* tickets = nullptr;
    if (splits > 1) {
        const size_t need = gemv_workspace_bytes(M, N, K);
        W8A16_REQUIRE(workspace != nullptr && workspace_bytes >= need, FP8W8A16_ERR_WORKSPACE,
                      "gemv: workspace too small (%zu < %zu bytes)", workspace_bytes, need);
        tickets = reinterpret_cast<unsigned int*>(workspace);
        partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kTicketBytes);
    }
    const int64_t units = (int64_t)row_groups * splits;
    for (int m0 = 0; m0 < M; m0 += 4) {  // more than 4 tokens: the weight is streamed once per 4 tokens
        const int mc = (M - m0) < 4 ? (M - m0) : 4;
        int64_t ctas = (units + kWarps - 1) / kWarps;
        const int64_t resident = (int64_t)sm_count() * resident_ctas_per_sm(mc);
        if (ctas > resident) ctas = resident;   // persistent: the warps stride over the units
        const unsigned grid = (unsigned)ctas;
        const __half* xm = x + (int64_t)m0 * K;
        __half* om = out + (int64_t)m0 * N;
        cudaError_t le = cudaSuccess;
        switch (mc) {
            case 1: le = launch_pdl(k_gemv<1>, dim3(grid), dim3(kThreads), 0, st, xm, w, scales, scale_dtype, om, partial, tickets, N, K, block_h, Kb, k_chunk, splits, row_groups); break;
            case 2: le = launch_pdl(k_gemv<2>, dim3(grid), dim3(kThreads), 0, st, xm, w, scales, scale_dtype, om, partial, tickets, N, K, block_h, Kb, k_chunk, splits, row_groups); break;
            case 3: le = launch_pdl(k_gemv<3>, dim3(grid), dim3(kThreads), 0, st, xm, w, scales, scale_dtype, om, partial, tickets, N, K, block_h, Kb, k_chunk, splits, row_groups); break;
            default: le = launch_pdl(k_gemv<4>, dim3(grid), dim3(kThreads), 0, st, xm, w, scales, scale_dtype, om, partial, tickets, N, K, block_h, Kb, k_chunk, splits, row_groups); break;
        }
        int rc = finish_launch(le, "gemv");
        if (rc) return rc;
    }
    return 0;
}

}  // namespace w8a16
