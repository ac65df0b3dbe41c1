// W8A16 GEMM on the 5th-generation tensor cores (tcgen05) with in-SM dequantisation.
//
//   C[m, n] = sum_k A[m, k] * RN16(cvt(W[n, k]) * S16[n / bh, k / 128])        (fp32 accumulate)
//
// Orientation ("swap-AB"): the 128 weight rows of a slab are the MMA M dimension (TMEM lanes),
// the tokens are the MMA N dimension (TMEM columns, BT = 16..256), so the FP8 weight is streamed
// from HBM exactly once per token tile and a decode batch of 1..64 tokens costs one narrow MMA.
//
// Per CTA (320 threads, one work unit = slab x token tile x K range):
//   warp 0      TMA producer: raw FP8 weight tile [128 x BK bytes] and FP16 activation tile
//               [BT x BK] into shared-memory rings (hardware swizzle, zero fill out of bounds).
//   warps 2-9   dequant: raw tile -> registers -> RN16(cvt * scale) -> FP16 operand tile in the
//               canonical K-major 128-byte-swizzled UMMA layout; later the epilogue.
//   warp 1      allocates TMEM and issues tcgen05.mma.kind::f16 (A = dequantised weights,
//               B = activations, D = fp32 accumulators in TMEM), releasing stages with
//               tcgen05.commit.
// Epilogue: tcgen05.ld -> FP16 store (optionally x per-row route weight, or SiLU(gate) * up when
// the CTA carries the paired gate / up slabs of a fused MoE w13).  With split-K the partial tiles
// go to an fp32 workspace and the last CTA to arrive (ticket counter) adds them in fixed order.
// Grouped (MoE) mode: token tiles are runs of rows of one expert in an expert-sorted activation
// matrix; tiles past the device-built table exit at once, so no host synchronisation is needed.
//
// Every mbarrier wait is bounded: after ~2 s the kernel records a code in a device status word,
// every role leaves its loop, TMEM is freed and the kernel returns.
//
// Replaces the reference's prefill GEMM fp8_w8a16_gemm_wmma_kernel + a2 tail
// (src/fp8_w8a16_sm70/fp8_dequant.cu:1933-2112, 337-415), its skinny-M CUDA-core kernels a1/a3
// (:260-316, :535-594), the grouped MoE kernels (:429-508, :1091-1258, :1770-1835) and the vendored
// TurboMind dense / grouped GEMM (third_party/turbomind_gemm_sm70/binding/awq_sm70_gemm.cu:1068-1213,
// :2327-2474).  The B-operand value RN16(cvt * s16) is the same as the reference's WMMA B tile
// (fp8_dequant.cu:2029-2031) and TurboMind's __hmul dequant (kernels/gemm/transform.h:151-156).
#include <cuda.h>

#include "common.cuh"
#include "gemm_tc.h"

namespace w8a16 {

__device__ int g_tc_status = 0;  // sticky error bits set by bounded waits (0 = healthy)

namespace {

constexpr int kThreadsTc = 320;
constexpr int kDequantThreads = 256;
constexpr unsigned long long kTimeoutNs = 2000000000ull;

// ---- PTX wrappers -----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// Bounded wait.  Returns false when the CTA has been declared dead (by this or another thread).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* dead, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3Fu) == 0u) {
            if (*dead) return false;
            if (globaltimer_ns() - t0 > kTimeoutNs) {
                *dead = 1;
                atomicOr(&g_tc_status, code);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t holder_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]^T, kind::f16, issued by one thread.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 bytes apart,
// 8-row groups 1024 bytes apart (tile base 1024-byte aligned; K advances by adding bytes to the
// start address inside the swizzle atom).
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                            // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024u >> 4) << 32;                 // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                            // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                            // layout type: SWIZZLE_128B
    return d;
}

// Instruction descriptor, kind::f16: D fp32, A and B FP16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t make_idesc_f16(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// ---- compile-time configuration ------------------------------------------------------------------
template <int BT, int BK, bool PAIRED>
struct TcCfg {
    static constexpr int kWT = PAIRED ? 2 : 1;                 // weight tiles per stage (gate + up)
    static constexpr int kSlabs = BK / 64;                     // 64-element (128-byte) K slabs per stage
    static constexpr int kRawBytes = 128 * BK * kWT;           // FP8 tile(s)
    static constexpr int kXBytes = BT * BK * 2;                // FP16 activation tile
    static constexpr int kABytes = 128 * BK * 2 * kWT;         // dequantised FP16 tile(s)
    static constexpr int kNA = (kABytes <= 16384) ? 3 : 2;     // dequantised-operand stages
    static constexpr int kBudget = 225 * 1024 - 2048;          // dynamic shared memory we allow ourselves
    static constexpr int kNSraw = (kBudget - kNA * kABytes) / (kRawBytes + kXBytes);
    static constexpr int kNS = kNSraw > 8 ? 8 : kNSraw;        // TMA ring stages
    static constexpr int kAccCols = BT * kWT;
    static constexpr int kTmemCols = kAccCols <= 32 ? 32 : kAccCols <= 64 ? 64 : kAccCols <= 128 ? 128 : kAccCols <= 256 ? 256 : 512;
    static constexpr int kNumBars = 4 * kNS + 2 * kNA + 1;
    static constexpr int kSmemBytes = 1024 + kNS * (kRawBytes + kXBytes) + kNA * kABytes + kNumBars * 8 + 64;
    static_assert(kNS >= 2, "not enough shared memory for a 2-stage TMA ring");
    static_assert(kAccCols <= 512, "accumulators exceed TMEM");
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

// One output element.  `row` is the row of the activation matrix (expert-sorted row in grouped
// mode), `n` the output feature.  Rounding points follow the reference's grouped path
// (src/fp8_w8a16_sm70/vllm_serve.py:1953-1990): GEMM output -> FP16, SiLU on FP16, product FP16,
// route weight as FP16.
template <bool PAIRED>
__device__ __forceinline__ void store_out(const TcParams& p, int row, int n, float g, float u) {
    __half r;
    if (PAIRED) {
        const __half g16 = __float2half_rn(g), u16 = __float2half_rn(u);
        const __half a16 = __float2half_rn(silu_f(__half2float(g16)));
        r = __float2half_rn(__half2float(a16) * __half2float(u16));
    } else {
        r = __float2half_rn(g);
        if (p.row_weight != nullptr) {
            const __half w16 = __float2half_rn(p.row_weight[row]);
            r = __float2half_rn(__half2float(r) * __half2float(w16));
        }
    }
    p.out[(int64_t)row * p.ldo + n] = r;
}

// ---- the kernel --------------------------------------------------------------------------------
template <int BT, int BK, bool PAIRED>
__global__ void __launch_bounds__(kThreadsTc, 1)
k_gemm_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const TcParams p) {
    using C = TcCfg<BT, BK, PAIRED>;
    constexpr int kNS = C::kNS, kNA = C::kNA;

    // ---- work unit ----
    const int slab = blockIdx.x, tile_t = blockIdx.y, split = blockIdx.z;
    int expert = 0, row_begin, rows_valid;
    if (p.expert_offsets != nullptr) {
        const int n_tiles = p.tile_offsets[p.num_experts];
        if (tile_t >= n_tiles) return;  // padding tile of the upper-bound grid
        int lo = 0, hi = p.num_experts;  // largest e with tile_offsets[e] <= tile_t
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (p.tile_offsets[mid] <= tile_t) lo = mid; else hi = mid;
        }
        expert = lo;
        row_begin = p.expert_offsets[expert] + (tile_t - p.tile_offsets[expert]) * BT;
        rows_valid = min(BT, p.expert_offsets[expert + 1] - row_begin);
    } else {
        row_begin = tile_t * BT;
        rows_valid = min(BT, p.M - row_begin);
    }
    const int n0 = slab * 128;
    const int total_kb = (p.K + BK - 1) / BK;
    const int kb_begin = split * p.kblocks_per_split;
    const int nkb = min(total_kb, kb_begin + p.kblocks_per_split) - kb_begin;

    // ---- shared memory carve-up (1024-byte aligned tiles) ----
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t dyn_base = smem_u32(smem_dyn);
    const uint32_t s_base = (dyn_base + 1023u) & ~1023u;
    const uint32_t s_raw = s_base;
    const uint32_t s_x = s_raw + kNS * C::kRawBytes;
    const uint32_t s_a = s_x + kNS * C::kXBytes;
    const uint32_t s_bar = s_a + kNA * C::kABytes;
    const uint32_t bar_full_raw = s_bar, bar_empty_raw = s_bar + 8 * kNS, bar_full_x = s_bar + 16 * kNS,
                   bar_empty_x = s_bar + 24 * kNS, bar_full_a = s_bar + 32 * kNS, bar_empty_a = bar_full_a + 8 * kNA,
                   bar_acc = bar_empty_a + 8 * kNA;
    uint8_t* gen_tail = smem_dyn + (s_bar - dyn_base) + C::kNumBars * 8;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(gen_tail);
    volatile int* s_dead = reinterpret_cast<volatile int*>(gen_tail + 4);
    volatile int* s_ticket = reinterpret_cast<volatile int*>(gen_tail + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kNS; ++i) {
            mbar_init(bar_full_raw + 8 * i, 1);
            mbar_init(bar_empty_raw + 8 * i, kDequantThreads);
            mbar_init(bar_full_x + 8 * i, 1);
            mbar_init(bar_empty_x + 8 * i, 1);
        }
        for (int i = 0; i < kNA; ++i) {
            mbar_init(bar_full_a + 8 * i, kDequantThreads);
            mbar_init(bar_empty_a + 8 * i, 1);
        }
        mbar_init(bar_acc, 1);
        *s_dead = 0;
        *s_ticket = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(s_tmem), C::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            const int w_row = expert * p.w_rows_per_expert + n0;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % kNS;
                const uint32_t ph = (uint32_t)(i / kNS) & 1u;
                if (!mbar_wait(bar_empty_raw + 8 * s, ph ^ 1u, s_dead, 1)) break;
                if (!mbar_wait(bar_empty_x + 8 * s, ph ^ 1u, s_dead, 2)) break;
                const int k0 = (kb_begin + i) * BK;
                mbar_arrive_expect_tx(bar_full_raw + 8 * s, C::kRawBytes);
                tma_load_2d(s_raw + s * C::kRawBytes, &map_w, bar_full_raw + 8 * s, k0, w_row);
                if (PAIRED) tma_load_2d(s_raw + s * C::kRawBytes + 128 * BK, &map_w, bar_full_raw + 8 * s, k0, w_row + p.pair_offset);
                mbar_arrive_expect_tx(bar_full_x + 8 * s, C::kXBytes);
#pragma unroll
                for (int sl = 0; sl < C::kSlabs; ++sl)
                    tma_load_2d(s_x + s * C::kXBytes + sl * (BT * 128), &map_x, bar_full_x + 8 * s, k0 + sl * 64, row_begin);
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16(BT);
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                const int sa = i % kNA, sx = i % kNS;
                ok = mbar_wait(bar_full_a + 8 * sa, (uint32_t)(i / kNA) & 1u, s_dead, 4) &&
                     mbar_wait(bar_full_x + 8 * sx, (uint32_t)(i / kNS) & 1u, s_dead, 8);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_st = s_a + sa * C::kABytes, x_st = s_x + sx * C::kXBytes;
#pragma unroll
                for (int sl = 0; sl < C::kSlabs; ++sl) {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint32_t acc = (i > 0 || sl > 0 || kk > 0) ? 1u : 0u;
                        const uint64_t db = make_desc_sw128(x_st + sl * (BT * 128) + kk * 32);
                        umma_f16(tmem_base, make_desc_sw128(a_st + sl * 16384 + kk * 32), db, idesc, acc);
                        if (PAIRED)
                            umma_f16(tmem_base + BT, make_desc_sw128(a_st + (C::kSlabs + sl) * 16384 + kk * 32), db, idesc, acc);
                    }
                }
                umma_commit(bar_empty_a + 8 * sa);
                umma_commit(bar_empty_x + 8 * sx);
            }
            if (ok) umma_commit(bar_acc);
        }
    } else {
        // ================= dequant warps, then epilogue =================
        const int td = threadIdx.x - 64;
        const int r = td & 127;   // weight row inside the slab == TMEM lane
        const int hk = td >> 7;   // which half of the K range of the stage
        constexpr int kCPT = BK / 32;  // 16-byte chunks per thread per weight tile
        // scale-grid rows for this thread's weight row(s); clamped so tail rows stay in bounds
        int64_t srow[C::kWT];
#pragma unroll
        for (int wt = 0; wt < C::kWT; ++wt) {
            int n = n0 + r + wt * p.pair_offset;
            n = min(n, p.w_rows_per_expert - 1);
            srow[wt] = (int64_t)expert * p.scale_expert_stride + (int64_t)(n / p.block_h) * p.Kb;
        }
        const uint32_t r7 = (uint32_t)(r & 7);
        const uint32_t a_row_off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
        bool ok = true;
        for (int i = 0; i < nkb; ++i) {
            const int s = i % kNS, sa = i % kNA;
            const int k0 = (kb_begin + i) * BK;
            __half2 s256[C::kWT];
#pragma unroll
            for (int wt = 0; wt < C::kWT; ++wt) s256[wt] = scale_times_256(load_scale_h(p.scales, srow[wt] + (k0 >> 7), p.scale_dtype));
            ok = mbar_wait(bar_full_raw + 8 * s, (uint32_t)(i / kNS) & 1u, s_dead, 16) &&
                 mbar_wait(bar_empty_a + 8 * sa, ((uint32_t)(i / kNA) & 1u) ^ 1u, s_dead, 32);
            if (!ok) break;
#pragma unroll
            for (int wt = 0; wt < C::kWT; ++wt) {
                const uint32_t raw_row = s_raw + s * C::kRawBytes + wt * (128 * BK) + r * BK;
                const uint32_t a_tile = s_a + sa * C::kABytes + wt * (C::kSlabs * 16384) + a_row_off;
#pragma unroll
                for (int c = 0; c < kCPT; ++c) {
                    const uint32_t chunk = (uint32_t)(hk * kCPT + c);
                    const uint32_t phys = (BK == 128) ? (chunk ^ r7) : (chunk ^ ((uint32_t)(r >> 1) & 3u));
                    const uint4 q = lds128(raw_row + phys * 16);
                    __half2 h[8];
                    e4m3x4_scaled(q.x, s256[wt], h[0], h[1]);
                    e4m3x4_scaled(q.y, s256[wt], h[2], h[3]);
                    e4m3x4_scaled(q.z, s256[wt], h[4], h[5]);
                    e4m3x4_scaled(q.w, s256[wt], h[6], h[7]);
                    const uint32_t* hw = reinterpret_cast<const uint32_t*>(h);
                    const uint32_t j = chunk * 2;  // 16-byte FP16 chunk index along K within the stage
                    const uint32_t dst = a_tile + (j >> 3) * 16384;
                    sts128(dst + (((j & 7u) ^ r7) << 4), hw[0], hw[1], hw[2], hw[3]);
                    sts128(dst + ((((j + 1) & 7u) ^ r7) << 4), hw[4], hw[5], hw[6], hw[7]);
                }
            }
            fence_async_smem();
            mbar_arrive(bar_full_a + 8 * sa);
            mbar_arrive(bar_empty_raw + 8 * s);
        }

        // ---- epilogue ----
        if (ok) ok = mbar_wait(bar_acc, 0u, s_dead, 64);
        ok = __all_sync(0xFFFFFFFFu, ok) != 0;  // tcgen05.ld is warp-collective: keep the warp together
        const int64_t tile_linear = (int64_t)tile_t * gridDim.x + slab;
        if (ok) {
            tc_fence_after();
            const int q4 = warp & 3;              // TMEM lane quarter this warp may read
            const int ch = (warp - 2) >> 2;       // column half
            const int n_local = q4 * 32 + lane;
            const int n = n0 + n_local;
            const uint32_t t_lane = tmem_base + ((uint32_t)(q4 * 32) << 16);
            constexpr int kColsPerWarp = BT / 2;
            float* part = p.partial + ((tile_linear * p.splits + split) * C::kWT) * (int64_t)(BT * 128);
#pragma unroll 1
            for (int c0 = 0; c0 < kColsPerWarp; c0 += 8) {
                const int col = ch * kColsPerWarp + c0;
                float g[8], u[8];
                tmem_ld8(t_lane + col, g);
                if (PAIRED) tmem_ld8(t_lane + BT + col, u);
                if (p.splits == 1) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (col + j < rows_valid && n < p.N) store_out<PAIRED>(p, row_begin + col + j, n, g[j], PAIRED ? u[j] : 0.f);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        __stcg(&part[(col + j) * 128 + n_local], g[j]);
                        if (PAIRED) __stcg(&part[(BT + col + j) * 128 + n_local], u[j]);
                    }
                }
            }
        }
        tc_fence_before();
        if (p.splits > 1) {
            // All 256 epilogue threads take both barriers whatever happened above, so that a
            // timed-out wait in one thread cannot strand the others.
            __threadfence();
            epi_bar_sync();
            const bool alive = (*s_dead == 0);
            if (alive && td == 0) *s_ticket = (int)atomicAdd(&p.tickets[tile_linear], 1u);
            epi_bar_sync();
            if (alive && *s_ticket == p.splits - 1) {
                __threadfence();
                const float* tile_part = p.partial + (tile_linear * p.splits * C::kWT) * (int64_t)(BT * 128);
                for (int idx = td; idx < BT * 128; idx += kDequantThreads) {
                    const int ml = idx >> 7, nl = idx & 127;
                    if (ml < rows_valid && n0 + nl < p.N) {
                        float g = 0.f, u = 0.f;
                        for (int sp = 0; sp < p.splits; ++sp) {
                            const float* ps = tile_part + (int64_t)sp * C::kWT * (BT * 128);
                            g += __ldcg(&ps[idx]);
                            if (PAIRED) u += __ldcg(&ps[BT * 128 + idx]);
                        }
                        store_out<PAIRED>(p, row_begin + ml, n0 + nl, g, u);
                    }
                }
                if (td == 0) p.tickets[tile_linear] = 0u;  // leave the counter clean for the next launch
            }
        }
    }

    // ---- teardown: every thread arrives here, also after a timed-out wait ----
    if (*s_dead) {
        // let copies and MMAs that are still in flight land before shared memory and TMEM go away
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes` elements, box [box_rows, box_cols].
int encode_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows, uint64_t cols,
              uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = get_encode_fn();
    W8A16_REQUIRE(fn != nullptr, FP8W8A16_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t gdim[2] = {cols, rows};
    const cuuint64_t gstride[1] = {cols * (uint64_t)elem_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    W8A16_REQUIRE(r == CUDA_SUCCESS, FP8W8A16_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d) rows=%llu cols=%llu box=%ux%u",
                  (int)r, (unsigned long long)rows, (unsigned long long)cols, box_rows, box_cols);
    return 0;
}

template <int BT, int BK, bool PAIRED>
int launch_cfg(const TcLaunch& L, cudaStream_t st) {
    using C = TcCfg<BT, BK, PAIRED>;
    static bool attr_set[64] = {};
    int dev = 0;
    W8A16_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        W8A16_CUDA(cudaFuncSetAttribute(k_gemm_tc<BT, BK, PAIRED>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        attr_set[dev] = true;
    }
    CUtensorMap map_w, map_x;
    int rc = encode_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, L.w, (uint64_t)L.w_total_rows, (uint64_t)L.p.K, 128, BK,
                       BK == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    rc = encode_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, L.x, (uint64_t)L.p.M, (uint64_t)L.p.K, BT, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    const int n_slabs = (L.p.N + 127) / 128;
    const dim3 grid(n_slabs, L.token_tiles, L.p.splits);
    k_gemm_tc<BT, BK, PAIRED><<<grid, kThreadsTc, C::kSmemBytes, st>>>(map_w, map_x, L.p);
    return check_launch("gemm_tc");
}

}  // namespace

int tc_block_k(int bt, bool paired) { return (paired || bt >= 128) ? 64 : 128; }

int tc_pick_bt(int rows) {
    if (rows <= 16) return 16;
    if (rows <= 32) return 32;
    if (rows <= 64) return 64;
    if (rows <= 128) return 128;
    return 256;
}

int tc_launch(const TcLaunch& L, int bt, bool paired, cudaStream_t st) {
#define W8A16_TC_CASE(BT_, BK_, P_) return launch_cfg<BT_, BK_, P_>(L, st)
    if (!paired) {
        switch (bt) {
            case 16: W8A16_TC_CASE(16, 128, false);
            case 32: W8A16_TC_CASE(32, 128, false);
            case 64: W8A16_TC_CASE(64, 128, false);
            case 128: W8A16_TC_CASE(128, 64, false);
            case 256: W8A16_TC_CASE(256, 64, false);
        }
    } else {
        switch (bt) {
            case 16: W8A16_TC_CASE(16, 64, true);
            case 32: W8A16_TC_CASE(32, 64, true);
            case 64: W8A16_TC_CASE(64, 64, true);
            case 128: W8A16_TC_CASE(128, 64, true);
            case 256: W8A16_TC_CASE(256, 64, true);
        }
    }
#undef W8A16_TC_CASE
    return fail(FP8W8A16_ERR_UNSUPPORTED, "gemm_tc: unsupported token tile %d", bt);
}

int tc_read_status(int* out, int reset) {
    int v = 0;
    W8A16_CUDA(cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)));
    if (reset && v != 0) {
        const int zero = 0;
        W8A16_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)));
    }
    *out = v;
    return 0;
}

}  // namespace w8a16
