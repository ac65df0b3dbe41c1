// W8A16 GEMM for prefill batches on CTA PAIRS: tcgen05.mma.cta_group::2 with in-SM dequantisation.
//
//   C[m, n] = sum_k A[m, k] * RN16(cvt(W[n, k]) * S16[n / bh, k / 128])        (fp32 accumulate)
//
// Same orientation as the single-CTA kernel (gemm_tc.cu): weight rows are the MMA M dimension (tensor-memory lanes), tokens
// are the MMA N dimension.  Here a thread-block cluster of two CTAs on the two SMs of a TPC shares one 256-row x 256-token
// output tile: each CTA streams, converts and holds in ITS tensor memory 128 of the 256 weight rows, and stages in ITS shared
// memory 128 of the 256 tokens' activations; one thread of the pair's first CTA issues M = 256, N = 256 MMAs that read the A
// operand from both CTAs' tensor memory and the B operand from both CTAs' shared memory, and leave each CTA the accumulator
// rows of its own weight rows.  Against the single-CTA 128 x 256 tile this halves the activation bytes every SM has to
// stage and read per FLOP - the single-CTA tile is bound by shared-memory bandwidth, not by the tensor pipe - and that in
// turn makes room for 128-element K blocks (four stages), whose raw-tile reads are free of bank conflicts.
//
// Per CTA (320 threads):
//   warp 0      TMA producer: raw FP8 tile [128 rows x 128] and FP16 activation tile [128 tokens x 128] per K block
//   warp 1      first CTA: MMA issuer.  second CTA: relay - tells the issuer when this CTA's activation tile has landed
//   warps 2-9   convert raw -> FP16 x scale -> tensor memory (A operand), then the epilogue of the tile
// Hand-offs (mbarriers; "first" = in the first CTA's shared memory, arrived on remotely by the second CTA):
//   full_w / empty_w   local: weight tile landed / converted
//   full_x             local: activation tile landed;  peer_x (first): the second CTA's has
//   full_a (first)     one arrival per converting warp of BOTH CTAs: the operand stage is complete in both tensor memories
//   empty (both)       tcgen05.commit multicast to both CTAs: the MMAs that read operand stage s and activation stage s are done
//   acc_full (both)    commit multicast: the tile's accumulators are complete;  acc_empty (first): both epilogues have drained them
// Every wait is bounded; a wait that runs out sets a bit of the device status word, and every thread still reaches the
// teardown (cluster barrier, tensor-memory release).  No TMA multicast is used.
//
// Replaces, for batches above 128 tokens, the reference's WMMA prefill kernel (src/fp8_w8a16_sm70/fp8_dequant.cu:1933-2112)
// and TurboMind's dense GEMM (third_party/turbomind_gemm_sm70/binding/awq_sm70_gemm.cu:1068-1213).
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "gemm_tc.h"
#include "tc_ptx.cuh"

namespace w8a16 {

__device__ int g_tc2_status = 0;   // sticky error bits of this kernel's bounded waits

namespace {

constexpr int kThreads2 = 320;
constexpr int kBT = 256;              // tokens per pair tile (128 staged by each CTA)
constexpr int kBK = 128;              // K block
constexpr int kNS = 4;                // stages: raw ring, activation ring and operand ring share the index
constexpr int kRawBytes = 128 * kBK;              // 16 KiB
constexpr int kXBytes = 128 * kBK * 2;            // 32 KiB: two 64-element slabs of [128 tokens x 64]
constexpr int kACols = kBK / 2;                   // 64 tensor-memory columns per operand stage
constexpr int kAccCols = kBT;                     // 256 fp32 accumulator columns
constexpr int kTmemCols = 512;                    // 256 + 4 * 64
constexpr int kNumBars = 6 * kNS + 2;
constexpr int kSmem2 = 1024 + kNS * (kRawBytes + kXBytes) + kNumBars * 8 + 64;
constexpr unsigned long long kTimeout2 = kTimeoutNs;

// Bounded wait.  CTA-scope acquire, also for the barriers the other CTA of the pair arrives on: what is handed over
// through them lives in tensor memory or was written by the async proxy, and is ordered by the tcgen05 fences around the
// arrive and the wait (cluster-scope acquire polls cost a memory barrier each: measured, they were the top stall reason).
__device__ __forceinline__ bool wait2(uint32_t bar, uint32_t parity, volatile int* dead, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3Fu) == 0u) {
            if (*dead) return false;
            if (globaltimer_ns() - t0 > kTimeout2) {
                *dead = 1;
                atomicOr(&g_tc2_status, code);
                return false;
            }
        }
    }
    return true;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
k_gemm_tc2(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const TcParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t dyn_base = smem_u32(smem_dyn);
    const uint32_t s_raw = (dyn_base + 1023u) & ~1023u;
    const uint32_t s_x = s_raw + kNS * kRawBytes;
    const uint32_t s_bar = s_x + kNS * kXBytes;
    const uint32_t bar_full_w = s_bar, bar_empty_w = s_bar + 8 * kNS, bar_full_x = s_bar + 16 * kNS, bar_peer_x = s_bar + 24 * kNS,
                   bar_full_a = s_bar + 32 * kNS, bar_empty = s_bar + 40 * kNS, bar_acc_full = s_bar + 48 * kNS,
                   bar_acc_empty = bar_acc_full + 8;
    uint8_t* tail = smem_dyn + (s_bar - dyn_base) + kNumBars * 8;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tail);
    volatile int* s_dead = reinterpret_cast<volatile int*>(tail + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kNS; ++i) {
            mbar_init(bar_full_w + 8 * i, 1);
            mbar_init(bar_empty_w + 8 * i, 8);      // one arrival per converting warp
            mbar_init(bar_full_x + 8 * i, 1);
            mbar_init(bar_peer_x + 8 * i, 1);
            mbar_init(bar_full_a + 8 * i, 16);      // the converting warps of both CTAs
            mbar_init(bar_empty + 8 * i, 1);        // one multicast commit
        }
        mbar_init(bar_acc_full, 1);
        mbar_init(bar_acc_empty, 16);
        *s_dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // both CTAs of the pair, the same warp: the allocation is made in both tensor memories
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // both CTAs' barriers exist before either arrives on the other's
    cluster_sync_all();
    const uint32_t tmem_base = *s_tmem;
    const uint32_t tmem_a0 = tmem_base + kAccCols;

    const int total_kb = (p.K + kBK - 1) / kBK;
    const int n_sp = (p.N + 255) / 256;                 // 256-row slab pairs
    const int n_tt = (p.M + kBT - 1) / kBT;
    const int total_tiles = n_sp * n_tt;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    asm volatile("griddepcontrol.wait;" ::: "memory");

    // addresses of the first CTA's barriers as seen from this CTA
    const uint32_t first_full_a = cluster_map(bar_full_a, 0u), first_peer_x = cluster_map(bar_peer_x, 0u),
                   first_acc_empty = cluster_map(bar_acc_empty, 0u);

    if (warp == 0) {
        // ================= TMA producer (both CTAs) =================
        if (lane == 0) {
            uint32_t n = 0;
            bool ok = true;
            for (int t = pair; t < total_tiles && ok; t += n_pairs) {
                const int sp = t / n_tt, tt = t - sp * n_tt;
                const int w_row = sp * 256 + (int)rank * 128, x_row = tt * kBT + (int)rank * 128;
                for (int kb = 0; kb < total_kb; ++kb, ++n) {
                    const uint32_t s = n & (kNS - 1), ph = (n / kNS) & 1u;
                    ok = wait2(bar_empty_w + 8 * s, ph ^ 1u, s_dead, 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(bar_full_w + 8 * s, kRawBytes);
                    tma_load_2d(s_raw + s * kRawBytes, &map_w, bar_full_w + 8 * s, kb * kBK, w_row);
                    ok = wait2(bar_empty + 8 * s, ph ^ 1u, s_dead, 2);
                    if (!ok) break;
                    mbar_arrive_expect_tx(bar_full_x + 8 * s, kXBytes);
                    tma_load_2d(s_x + s * kXBytes, &map_x, bar_full_x + 8 * s, kb * kBK, x_row);
                    tma_load_2d(s_x + s * kXBytes + 128 * 128, &map_x, bar_full_x + 8 * s, kb * kBK + 64, x_row);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && !leader) {
            // ================= relay (second CTA): this CTA's activation tile has landed =================
            uint32_t n = 0;
            bool ok = true;
            for (int t = pair; t < total_tiles && ok; t += n_pairs)
                for (int kb = 0; kb < total_kb; ++kb, ++n) {
                    const uint32_t s = n & (kNS - 1), ph = (n / kNS) & 1u;
                    ok = wait2(bar_full_x + 8 * s, ph, s_dead, 4);
                    if (!ok) break;
                    mbar_arrive_peer(first_peer_x + 8 * s);
                }
        } else if (lane == 0) {
            // ================= MMA issuer (first CTA) =================
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(kBT >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);   // D fp32, A/B FP16 K-major, M = 256, N = 256
            uint32_t n = 0, tile_i = 0;
            bool ok = true;
            for (int t = pair; t < total_tiles && ok; t += n_pairs, ++tile_i) {
                // the accumulators of the previous tile must have been drained by both CTAs' epilogues
                if (tile_i > 0) ok = wait2(bar_acc_empty, (tile_i - 1) & 1u, s_dead, 8);
                for (int kb = 0; kb < total_kb && ok; ++kb, ++n) {
                    const uint32_t s = n & (kNS - 1), ph = (n / kNS) & 1u;
                    ok = wait2(bar_full_a + 8 * s, ph, s_dead, 16) && wait2(bar_full_x + 8 * s, ph, s_dead, 32) &&
                         wait2(bar_peer_x + 8 * s, ph, s_dead, 64);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_col = tmem_a0 + s * kACols;
                    const uint64_t db0 = make_desc_sw128(s_x + s * kXBytes);
#pragma unroll
                    for (int step = 0; step < 8; ++step) {
                        const int sl = step >> 2, kk = step & 3;
                        const uint64_t db = db0 + (uint64_t)((sl * (128 * 128) + kk * 32) >> 4);
                        umma2_f16_ts(tmem_base, a_col + step * 8, db, idesc, (kb > 0 || step > 0) ? 1u : 0u);
                    }
                    umma2_commit_pair(bar_empty + 8 * s);            // operand + activation stage free, in both CTAs
                }
                if (ok) umma2_commit_pair(bar_acc_full);              // the tile's accumulators are complete, in both CTAs
            }
        }
    } else {
        // ================= converting warps, then the tile's epilogue (both CTAs) =================
        const int q4 = warp & 3;
        const int r = q4 * 32 + lane;            // weight row inside this CTA's 128-row slab == tensor-memory lane
        const int hk = (warp - 2) >> 2;          // half of the stage's K range / of the epilogue's token columns
        const uint32_t r7 = (uint32_t)(r & 7);
        const uint32_t t_lane = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const uint32_t t_lane_a = t_lane + kAccCols;
        uint32_t n = 0, tile_i = 0;
        bool ok = true;
        for (int t = pair; t < total_tiles; t += n_pairs, ++tile_i) {
            const int sp = t / n_tt, tt = t - sp * n_tt;
            const int n0 = sp * 256 + (int)rank * 128;
            const int nrow = min(n0 + r, p.N - 1);
            const int64_t srow = (int64_t)(nrow / p.block_h) * p.Kb;
            __half s_cur = load_scale_h(p.scales, srow, p.scale_dtype);
            for (int kb = 0; kb < total_kb && ok; ++kb, ++n) {
                const uint32_t s = n & (kNS - 1), ph = (n / kNS) & 1u;
                const __half2 sc = __halves2half2(s_cur, s_cur);
                s_cur = load_scale_h(p.scales, srow + min(kb + 1, total_kb - 1), p.scale_dtype);   // next block's scale travels meanwhile
                ok = wait2(bar_full_w + 8 * s, ph, s_dead, 128) && wait2(bar_empty + 8 * s, ph ^ 1u, s_dead, 256);
                if (!ok) break;
                tc_fence_after();
                const uint32_t raw_row = s_raw + s * kRawBytes + r * kBK;
                const uint32_t a_dst = t_lane_a + s * kACols;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t chunk = (uint32_t)(hk * 4 + c);
                    const uint4 q = lds128(raw_row + ((chunk ^ r7) << 4));
                    uint32_t hw[8];
                    e4m3x4_scaled_hw(q.x, sc, hw[0], hw[1]);
                    e4m3x4_scaled_hw(q.y, sc, hw[2], hw[3]);
                    e4m3x4_scaled_hw(q.z, sc, hw[4], hw[5]);
                    e4m3x4_scaled_hw(q.w, sc, hw[6], hw[7]);
                    tmem_st8(a_dst + chunk * 8, hw);
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_peer(first_full_a + 8 * s);   // this warp's part of the stage is in tensor memory
                    mbar_arrive(bar_empty_w + 8 * s);            // and its reads of the raw tile are done
                }
            }
            // ---- epilogue of the tile: this CTA's 128 accumulator rows x 256 tokens ----
            if (ok) ok = wait2(bar_acc_full, tile_i & 1u, s_dead, 512);
            ok = __all_sync(0xFFFFFFFFu, ok) != 0;
            if (ok) {
                tc_fence_after();
                const int nn = n0 + r;
                const int tok0 = tt * kBT;
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 32) {       // 32 token columns per tensor-memory load
                    const int col = hk * 128 + c0;
                    float g[32];
                    tmem_ld32(t_lane + col, g);
                    if (nn < p.N) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int tok = tok0 + col + j;
                            if (tok < p.M) {
                                float v = g[j];
                                const int64_t off = (int64_t)tok * p.ldo + nn;
                                if (p.residual != nullptr) v += __half2float(p.residual[off]);
                                p.out[off] = __float2half_rn(v);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_peer(first_acc_empty);    // (also after a timed-out wait: the issuer must not be left waiting)
            if (!ok) break;
        }
    }

    // ---- teardown: both CTAs are done with both tensor memories before either releases them ----
    if (*s_dead) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}

}  // namespace

// FP8W8A16_TC2=0 keeps batches above 128 tokens on the single-CTA 128 x 256 tile.
bool tc2_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("FP8W8A16_TC2");
        v = (e && atoi(e) == 0) ? 0 : 1;
    }
    return v == 1;
}

int tc2_launch(const TcLaunch& L, cudaStream_t st) {
    static bool attr_set[64] = {};
    int dev = 0;
    W8A16_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        W8A16_CUDA(cudaFuncSetAttribute(k_gemm_tc2, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2));
        W8A16_CUDA(cudaFuncSetAttribute(k_gemm_tc2, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        attr_set[dev] = true;
    }
    CUtensorMap map_w, map_x;
    int rc = tc_encode_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, L.w, (uint64_t)L.w_total_rows, (uint64_t)L.p.K, 128, kBK, CU_TENSOR_MAP_SWIZZLE_128B, true);
    if (rc) return rc;
    rc = tc_encode_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, L.x, (uint64_t)L.p.M, (uint64_t)L.p.K, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B, false);
    if (rc) return rc;
    const int64_t tiles = (int64_t)((L.p.N + 255) / 256) * ((L.p.M + kBT - 1) / kBT);
    int64_t pairs = sm_count() / 2;
    if (tiles < pairs) pairs = tiles;
    if (pairs < 1) pairs = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(kThreads2);
    cfg.dynamicSmemBytes = kSmem2;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return finish_launch(cudaLaunchKernelEx(&cfg, k_gemm_tc2, map_w, map_x, L.p), "gemm_tc2");
}

int tc2_read_status(int* out, int reset) {
    int v = 0;
    W8A16_CUDA(cudaMemcpyFromSymbol(&v, g_tc2_status, sizeof(int)));
    if (reset && v != 0) {
        const int zero = 0;
        W8A16_CUDA(cudaMemcpyToSymbol(g_tc2_status, &zero, sizeof(int)));
    }
    *out = v;
    return 0;
}

}  // namespace w8a16
