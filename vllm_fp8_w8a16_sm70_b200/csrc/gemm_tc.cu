// W8A16 GEMM on the 5th-generation tensor cores (tcgen05) with in-SM dequantisation.
//
//   C[m, n] = sum_k A[m, k] * RN16(cvt(W[n, k]) * S16[n / bh, k / 128])        (fp32 accumulate)
//
// Orientation ("swap-AB"): the 128 weight rows of a slab are the MMA M dimension (TMEM lanes),
// the tokens are the MMA N dimension (TMEM columns, BT = 16..256), so the FP8 weight is streamed
// from HBM exactly once per token tile and a decode batch of 1..64 tokens costs one narrow MMA.
//
// Per CTA (320 threads; work = runs of K blocks of 128-row slab x token tile output tiles):
//   warp 0      TMA producer: raw FP8 weight tile [128 x BK bytes] and FP16 activation tile
//               [BT x BK] into shared-memory rings (hardware swizzle, zero fill out of bounds).
//   warps 2-9   dequant: raw tile -> registers (cvt.rn.f16x2.e4m3x2) -> RN16(cvt * scale) -> FP16 operand tile in the
//               canonical K-major 128-byte-swizzled UMMA layout; later the epilogue.
//   warp 1      allocates TMEM and issues tcgen05.mma.kind::f16 (A = dequantised weights,
//               B = activations, D = fp32 accumulators in TMEM), releasing stages with
//               tcgen05.commit.
// Epilogue: tcgen05.ld -> FP16 store (optionally x per-row route weight, or SiLU(gate) * up when
// the CTA carries the paired gate / up slabs of a fused MoE w13).  The launch is persistent and
// splits the (tile x K block) work evenly over the CTAs (stream-K): a tile shared by several CTAs
// goes through fp32 partial tiles in a workspace and the last CTA to arrive (ticket counter) adds
// them in fixed order, so results do not depend on scheduling.
// Grouped (MoE) mode: token tiles are runs of rows of one expert in an expert-sorted activation
// matrix; the tile count is read from the device-built table, so no host synchronisation is needed.
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

#include <stdlib.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "gemm_tc.h"
#include "tc_ptx.cuh"

namespace w8a16 {

__device__ int g_tc_status = 0;  // sticky error bits set by bounded waits (0 = healthy)


namespace {

constexpr int kThreadsTc = 352;   // warp 0 TMA, warp 1 MMA, warps 2-9 dequant + epilogue, warp 10 second MMA issuer
constexpr int kDequantThreads = 256;
// Bounded wait.  Returns false when the CTA has been declared dead (by this or another thread).  `dead` points at
// the CTA's flag words: [0] dead, [kReadyWord] "the kernel this launch depends on has finished".  Converting and MMA
// warps start before that (see the dependency wait in the kernel): what they then wait for cannot happen until the
// previous kernel is done, however long that takes, so the clock of the bound only runs once the flag is up.
constexpr int kReadyWord = 3;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* dead, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait_suspend(bar, parity, 2000u)) {
        if ((++spins & 0x3Fu) == 0u) {
            if (*dead) return false;
            if (dead[kReadyWord] == 0) {
                t0 = globaltimer_ns();
            } else if (globaltimer_ns() - t0 > kTimeoutNs) {
                *dead = 1;
                atomicOr(&g_tc_status, code);
                return false;
            }
        }
    }
    return true;
}

// Packets of the fused all-reduce: 16 bytes = two 8-byte halves {2 x FP16, epoch}; 8-byte accesses are single-copy
// atomic, so a half whose epoch matches carries the data that was stored with it.
__device__ __forceinline__ void st_packet(uint2* dst, uint32_t d0, uint32_t d1, uint32_t epoch) {
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(d0), "r"(epoch), "r"(d1), "r"(epoch) : "memory");
}
__device__ __forceinline__ uint4 ld_packet(const uint2* src) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
    return v;
}

// ---- compile-time configuration ------------------------------------------------------------------
// TMEM columns of one CTA: kAccBufs accumulator buffers of kAccCols fp32 columns (BT per weight
// tile; two buffers where they fit, so the epilogue of one segment overlaps the MMAs of the next),
// then kNA stages of the dequantised FP16 A operand (BK / 2 columns per weight tile: two K elements
// per 32-bit cell).
template <int BT, int BK, bool PAIRED>
struct TcCfg {
    static constexpr int kWT = PAIRED ? 2 : 1;                 // weight tiles per stage (gate + up)
    static constexpr int kSlabs = BK / 64;                     // 64-element (128-byte) K slabs of the activation tile
    static constexpr int kRawBytes = 128 * BK * kWT;           // FP8 tile(s)
    static constexpr int kXBytes = BT * BK * 2;                // FP16 activation tile
    static constexpr int kACols = (BK / 2) * kWT;              // TMEM columns of one dequantised stage
    // One thread needs ~60-70 ns per tcgen05 instruction it issues (measured in this kernel), far longer than a narrow
    // MMA runs, and a K block costs an issuer its MMAs plus two commits and two barrier waits.  For small token tiles
    // TWO warps issue, each into its own TMEM accumulator columns; the epilogue adds the accumulators that were written
    // in the segment, in fixed order.  Stage-owner form (kAltBlocks): each issuer OWNS the operand stages of its parity
    // (stage index & 1) and takes exactly the K blocks that land in them - half the blocks each, so half the commits
    // and waits, and two blocks' MMA chains in flight at once.  Because a stage is consumed by one issuer only, an issuer
    // can never mistake an older fill of a stage for the one it waits for (a stage is not refilled before its owner has
    // released it), however far the two issuers drift apart.
    // (A single issuer at 64 tokens would leave room for a second accumulator buffer; measured 5-12 % slower.)
    static constexpr int kIssuers = (BT * kWT <= 128 && BT <= 64) ? 2 : 1;
    static constexpr int kAccCols = BT * kWT * kIssuers;       // one accumulator buffer
    // Small token tiles are sized so that TWO CTAs share an SM (half of shared memory and of TMEM
    // each): one CTA's prologue / epilogue hides behind the other's main loop, 16 warps dequantise.
    static constexpr int kCtasPerSm = (BT * kWT <= 64) ? 2 : 1;
    static constexpr int kTmemBudget = 512 / kCtasPerSm;
    // The eight converting warps are two GROUPS of four (a warp reaches only the TMEM lanes of its quarter, warp % 4).  In the
    // small-tile configurations a group takes whole K blocks in turn (even / odd blocks of the CTA) instead of half of every
    // block's K range: a block's conversion is a chain of waits (tile landed -> shared-memory loads -> conversions ->
    // tensor-memory stores -> their completion -> arrivals), and with two blocks in that chain at once a CTA gets through its
    // first and last blocks sooner (measured on B200: 2 % on every decode shape; no gain, or a loss, for 128-token tiles,
    // which keep the split of every block).
    static constexpr bool kInterleave = kCtasPerSm == 2;
    static constexpr int kStageArrivals = kInterleave ? kDequantThreads / 2 : kDequantThreads;   // converting threads that fill one stage
    static constexpr int kAccBufs = (2 * kAccCols + 2 * kACols <= kTmemBudget) ? 2 : 1;
    static constexpr int kNAraw = (kTmemBudget - kAccBufs * kAccCols) / kACols;
    static constexpr int kNA = kNAraw > 4 ? 4 : kNAraw;        // dequantised-operand stages (TMEM)
    // Two issuers share the work in one of two ways.  With three or more operand stages each issuer OWNS the stages of
    // its parity and takes the K blocks that land in them (see below); with only two stages that would leave each issuer a
    // single stage and stall the converting warps, so both issuers work on every K block, half of its K steps each
    // (measured on B200: stage ownership is 2-4 % faster at 16 tokens, 4-5 % slower at 64).
    static constexpr bool kAltBlocks = kIssuers == 2 && kNA >= 3;
    static constexpr int kUsedCols = kAccBufs * kAccCols + kNA * kACols;
    // K blocks of the NEXT segment that are converted before the previous segment's epilogue runs
    static constexpr int kDefer = kAccBufs == 2 ? kNA : 0;
    static constexpr int kTmemCols = kUsedCols <= 32 ? 32 : kUsedCols <= 64 ? 64 : kUsedCols <= 128 ? 128 : kUsedCols <= 256 ? 256 : 512;
    // grouped mode keeps the route table's two offset arrays (up to 256 experts + 1 each) in shared memory
    static constexpr int kTabExperts = 256;
    static constexpr int kTabBytes = 2 * (kTabExperts + 1) * 4 + 8;
    // Dynamic shared memory we allow ourselves: an SM has 228 KiB, 1 KiB of which every resident CTA reserves, and one CTA may
    // take 227 KiB at most; what the rings may use is that minus the alignment slack, the barriers and the small tables.
    static constexpr int kLimit = (kCtasPerSm == 2 ? 113 : 226) * 1024;
    static constexpr int kBudget = kLimit - 1024 - 64 - 512 - kTabBytes;
    static constexpr int kNSraw = kBudget / (kRawBytes + kXBytes);
    static constexpr int kNS = kNSraw > 8 ? 8 : kNSraw;        // TMA ring stages
    static constexpr int kNumBars = 4 * kNS + 2 * kNA + 2;
    static constexpr int kSmemBytes = 1024 + kNS * (kRawBytes + kXBytes) + kNumBars * 8 + 64 + kTabBytes;
    static_assert(kNS >= 2, "not enough shared memory for a 2-stage TMA ring");
    static_assert(kNumBars * 8 <= 512 && kSmemBytes <= kLimit, "shared-memory budget");
    static_assert(kNA >= 2, "not enough TMEM for two dequantised stages");
    static_assert(kTmemCols * kCtasPerSm <= 512, "co-resident CTAs exceed TMEM");
    // cluster split-K parks the fp32 partial tile in the (by then idle) raw-tile ring
    static constexpr bool kClusterOk = kWT * BT * 128 * 4 <= kNS * kRawBytes;
};

// Which issuers (bit i = issuer i) own at least one of the `nkb` K blocks of a segment whose first block lands in operand
// stage `st0` of a ring of NA stages (owner of a stage = its index & 1).
template <int NA>
__device__ __forceinline__ uint32_t owners_mask(int st0, int nkb) {
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < NA; ++j)
        if (j < nkb) m |= 1u << (((st0 + j) % NA) & 1);
    return m;
}

// ring position: stage index and the parity of the current pass over the ring
struct Ring {
    int stage = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance(int n) {
        if (++stage == n) {
            stage = 0;
            phase ^= 1u;
        }
    }
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_erf_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

// One output element.  `row` is the row of the activation matrix (expert-sorted row in grouped
// mode), `n` the output feature.  Rounding points follow the reference's grouped path
// (src/fp8_w8a16_sm70/vllm_serve.py:1953-1990): GEMM output -> FP16, SiLU on FP16, product FP16,
// route weight as FP16.
// Dense mode with a residual (the decoder's residual stream, added where the row-parallel projection's output is
// produced): out = RN16(acc + residual) - fp32 sum, one rounding.  In the fused all-reduce build this function only
// writes this rank's partial to the staging buffer; the residual is added after the cross-rank sum (ar_exchange).
template <bool PAIRED, bool AR = false>
__device__ __forceinline__ void store_out(const TcParams& p, __half* out, int row, int n, float g, float u) {
    __half r;
    if (PAIRED) {
        const __half g16 = __float2half_rn(g), u16 = __float2half_rn(u);
        const float gf = __half2float(g16);
        const __half a16 = __float2half_rn(p.activation == 2 ? gelu_erf_f(gf) : silu_f(gf));
        r = __float2half_rn(__half2float(a16) * __half2float(u16));
    } else {
        if (!AR && p.residual != nullptr) g += __half2float(p.residual[(int64_t)row * p.ldo + n]);
        r = __float2half_rn(g);
        if (p.row_weight != nullptr) {
            const __half w16 = __float2half_rn(p.row_weight[row]);
            r = __float2half_rn(__half2float(r) * __half2float(w16));
        }
    }
    out[(int64_t)row * p.ldo + n] = r;
}

// ---- work decomposition ------------------------------------------------------------------------------
// The launch is persistent.  The work is made of (output tile, K block) units; a CTA walks a few SEGMENTS, each a run
// of K blocks of one output tile, in one of three schedules chosen on the host from the shape alone:
//   cluster   one thread-block cluster per tile, rank in cluster = K range (synchronous split-K)
//   tiles     whole tiles only, dealt round-robin: tile = cta + i * grid
//   stream-K  all units, tile-major, are cut into `grid` balanced contiguous ranges (sizes differ by at most one unit).  A
//             tile whose K range is covered by one CTA is stored directly; otherwise every contributor writes its fp32
//             partial tile to its own slot of the workspace and the last one to arrive (ticket counter) adds the slots in
//             ascending CTA order.
struct Seg {
    int tile, slab, expert, row_begin, rows_valid, kb0, nkb;
    int first_c, n_contrib;
    int tkey;   // stream-K: the tile's index (its ticket and the key of its partial slots); -1 otherwise
    int a_stage0;   // operand-ring stage of the segment's first K block (set by the converting warps; see owners_mask)
};

struct Sched {
    int n_tt;
    int q, r;                   // stream-K: total units = q * grid + r; the first r CTAs own q + 1 units, the others q
    int u_begin, u_end;
    // first unit of CTA c's range, and the CTA that owns unit u (32-bit arithmetic only)
    __device__ __forceinline__ int begin_of(int c) const { return c * q + min(c, r); }
    __device__ __forceinline__ int owner_of(int u) const {
        const int big = r * (q + 1);
        return u < big ? u / (q + 1) : r + (u - big) / q;    // (q >= 1 whenever the second branch is reached)
    }
};

__device__ __forceinline__ void make_sched(const TcParams& p, int total_kb, int n_tt, int n_slabs, Sched& sc) {
    const int cta = blockIdx.x, G = gridDim.x;
    const int total_tiles = n_tt * n_slabs;
    sc.n_tt = n_tt;
    sc.q = sc.r = 0;
    if (p.cluster_size > 1) {
        // synchronous split-K: cluster = tile, rank in cluster = K range (every rank gets at least one block)
        const int S = p.cluster_size;
        const int tile = cta / S, rnk = cta - tile * S;
        const int per = (total_kb + S - 1) / S;
        const int b = min(total_kb, rnk * per), e = min(total_kb, b + per);
        sc.u_begin = tile < total_tiles ? tile * total_kb + b : 0;
        sc.u_end = tile < total_tiles ? tile * total_kb + e : 0;
    } else if (p.no_split) {
        const int per_cta = (total_tiles + G - 1) / G;
        const int mine = cta < total_tiles ? (total_tiles - cta + G - 1) / G : 0;
        sc.u_begin = cta * per_cta * total_kb;
        sc.u_end = sc.u_begin + mine * total_kb;
    } else {
        const int units = total_tiles * total_kb;
        sc.q = units / G;
        sc.r = units - sc.q * G;
        sc.u_begin = sc.begin_of(cta);
        sc.u_end = sc.begin_of(cta + 1);
    }
}

template <int BT>
__device__ __forceinline__ void get_seg(const TcParams& p, bool grouped, const int* tile_off, const int* exp_off, int u, int total_kb,
                                        int n_slabs, const Sched& sc, Seg& s) {
    s.first_c = 0;
    s.n_contrib = 1;
    s.tkey = -1;
    s.a_stage0 = 0;
    if (p.cluster_size > 1) {
        const int v = u / total_kb;
        s.kb0 = u - v * total_kb;
        s.nkb = sc.u_end - u;
        s.tile = v;
    } else if (p.no_split) {
        // whole tiles, dealt round-robin: at any moment the CTAs work on `grid` consecutive tiles (token tiles fastest),
        // so a weight slab is in flight for all its token tiles at once and is read from HBM once
        const int v = u / total_kb;
        const int per_cta = (sc.n_tt * n_slabs + (int)gridDim.x - 1) / (int)gridDim.x;
        const int c = v / per_cta;
        s.kb0 = 0;
        s.nkb = total_kb;
        s.tile = (v - c * per_cta) * (int)gridDim.x + c;
    } else {
        const int v = u / total_kb;
        s.kb0 = u - v * total_kb;
        s.nkb = min(total_kb - s.kb0, sc.u_end - u);
        s.tkey = v;
        s.tile = v;
        s.first_c = sc.owner_of(v * total_kb);
        s.n_contrib = sc.owner_of((v + 1) * total_kb - 1) - s.first_c + 1;
    }
    s.slab = s.tile / sc.n_tt;             // token tiles fastest: concurrently running CTAs share a weight slab
    const int tt = s.tile - s.slab * sc.n_tt;
    s.expert = 0;
    if (grouped) {
        int lo = 0, hi = p.num_experts;  // largest e with tile_offsets[e] <= tt
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (tile_off[mid] <= tt) lo = mid; else hi = mid;
        }
        s.expert = lo;
        s.row_begin = exp_off[lo] + (tt - tile_off[lo]) * BT;
        s.rows_valid = min(BT, exp_off[lo + 1] - s.row_begin);
    } else {
        s.row_begin = tt * BT;
        s.rows_valid = min(BT, p.M - s.row_begin);
    }
}

// Workspace slot of contributor `c` for tile `tkey`: slot 0 if the tile is the first one the CTA's range touches, slot 1
// otherwise (a range has at most two partially covered tiles: its first and its last).
__device__ __forceinline__ int partial_slot(int c, int tkey, int total_kb, const Sched& sc) {
    return (sc.begin_of(c) / total_kb == tkey) ? 2 * c : 2 * c + 1;
}

// Exchange of one region of an output tile between the ranks (see ArParams).  `stage` holds this rank's FP16
// values; every thread handles groups of four consecutive features.  Kept out of line: it runs once per tile and
// must not cost the main loop registers.
__device__ __noinline__ void ar_exchange(const ArParams& ar, const __half* stage, const __half* residual, uint32_t epoch, int N, int64_t ldo,
                                         int row_begin, int rows_valid, int n0, int lo, int hi, int td, volatile int* s_dead) {
    const int64_t box = (int64_t)(epoch & 1u) * ar.world;     // first source slot of this launch's parity
    const uint2* mine = ar.inbox[ar.rank];
    // pass 1: push this rank's values of the whole region (posted stores, nothing to wait for)
    for (int idx4 = lo + td; idx4 < hi; idx4 += kDequantThreads) {
        const int ml = idx4 >> 5, nl = (idx4 & 31) * 4;
        if (ml >= rows_valid || n0 + nl >= N) continue;
        const int64_t off = (int64_t)(row_begin + ml) * ldo + n0 + nl;
        const uint2 own = *reinterpret_cast<const uint2*>(stage + off);
        for (int r = 0; r < ar.world; ++r)
            if (r != ar.rank) st_packet(ar.inbox[r] + ((box + ar.rank) * ar.part_elems + off) / 2, own.x, own.y, epoch);
    }
    // pass 2: collect the peers' packets (the first ones cost one NVLink flight, the rest are already there)
    const unsigned long long limit = (unsigned long long)ar.timeout_ms * 1000000ull;
    bool dead = false;
    for (int idx4 = lo + td; idx4 < hi && !dead; idx4 += kDequantThreads) {
        const int ml = idx4 >> 5, nl = (idx4 & 31) * 4;
        if (ml >= rows_valid || n0 + nl >= N) continue;
        const int64_t off = (int64_t)(row_begin + ml) * ldo + n0 + nl;
        const uint2 own = *reinterpret_cast<const uint2*>(stage + off);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int r0 = 0; r0 < ar.world && !dead; r0 += 4) {        // four sources' packets in flight at a time
            uint4 v[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int r = r0 + q;
                if (r < ar.world && r != ar.rank) v[q] = ld_packet(mine + ((box + r) * ar.part_elems + off) / 2);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int r = r0 + q;
                if (r >= ar.world || dead) continue;
                uint32_t d0 = own.x, d1 = own.y;
                if (r != ar.rank) {
                    if (v[q].y != epoch || v[q].w != epoch) {
                        const uint2* src = mine + ((box + r) * ar.part_elems + off) / 2;
                        const unsigned long long t0 = globaltimer_ns();
                        uint32_t spins = 0;
                        do {
                            if ((++spins & 0x1Fu) == 0u) {
                                if (*s_dead || globaltimer_ns() - t0 > limit) {
                                    if (!*s_dead) {
                                        *s_dead = 1;
                                        atomicOr(&g_tc_status, 128);
                                    }
                                    dead = true;
                                    break;
                                }
                            }
                            v[q] = ld_packet(src);
                        } while (v[q].y != epoch || v[q].w != epoch);
                    }
                    d0 = v[q].x;
                    d1 = v[q].z;
                }
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&d0));
                const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&d1));
                acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
            }
        }
        if (dead) break;
        if (residual != nullptr) {     // the residual stream joins the cross-rank sum before the one rounding
            const uint2 rv = *reinterpret_cast<const uint2*>(residual + off);
            const float2 ra = __half22float2(*reinterpret_cast<const __half2*>(&rv.x));
            const float2 rb = __half22float2(*reinterpret_cast<const __half2*>(&rv.y));
            acc.x += ra.x; acc.y += ra.y; acc.z += rb.x; acc.w += rb.y;
        }
        const __half2 o0 = __floats2half2_rn(acc.x, acc.y), o1 = __floats2half2_rn(acc.z, acc.w);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&o0);
        o.y = *reinterpret_cast<const uint32_t*>(&o1);
        *reinterpret_cast<uint2*>(ar.out + off) = o;
    }
}

// ---- the kernel --------------------------------------------------------------------------------
template <int BT, int BK, bool PAIRED, bool AR>
__global__ void __launch_bounds__(kThreadsTc, TcCfg<BT, BK, PAIRED>::kCtasPerSm)
k_gemm_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const TcParams p,
          const ArParams ar) {
    static_assert(!(AR && PAIRED), "the fused all-reduce is a dense (row-parallel) mode");
    using C = TcCfg<BT, BK, PAIRED>;
    constexpr int kNS = C::kNS, kNA = C::kNA;

    // Programmatic dependent launch: let the next kernel of the stream start its own set-up as soon as
    // this grid's CTAs are resident; it will wait (griddepcontrol.wait) for this grid to finish before
    // it reads or writes global memory.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- shared memory carve-up (1024-byte aligned tiles) ----
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t dyn_base = smem_u32(smem_dyn);
    const uint32_t s_base = (dyn_base + 1023u) & ~1023u;
    const uint32_t s_raw = s_base;
    const uint32_t s_x = s_raw + kNS * C::kRawBytes;
    const uint32_t s_bar = s_x + kNS * C::kXBytes;
    const uint32_t bar_full_raw = s_bar, bar_empty_raw = s_bar + 8 * kNS, bar_full_x = s_bar + 16 * kNS,
                   bar_empty_x = s_bar + 24 * kNS, bar_full_a = s_bar + 32 * kNS, bar_empty_a = bar_full_a + 8 * kNA,
                   bar_acc = bar_empty_a + 8 * kNA;
    uint8_t* gen_tail = smem_dyn + (s_bar - dyn_base) + C::kNumBars * 8;
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(gen_tail);
    volatile int* s_dead = reinterpret_cast<volatile int*>(gen_tail + 4);
    volatile int* s_ticket = reinterpret_cast<volatile int*>(gen_tail + 8);
    volatile int* s_ready = s_dead + kReadyWord;          // set once the dependency wait has been passed (see mbar_wait)
    int* s_tab = reinterpret_cast<int*>(gen_tail + 64);   // [kTabExperts + 1] tile offsets, then [kTabExperts + 1] row offsets
    const int* tab_tile = p.tile_offsets;                 // route-table offsets: global, or their shared-memory copy
    const int* tab_exp = p.expert_offsets;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- this CTA's unit range ----
    // Dense problems know it from the launch parameters alone; grouped ones read the tile count from
    // the route table, which the previous kernel wrote, so they must wait for it first.
    const bool grouped = !AR && p.expert_offsets != nullptr;   // the fused all-reduce build is dense only
    const int total_kb = (p.K + BK - 1) / BK;
    const int n_slabs = (p.N + 127) / 128;
    const int cta = blockIdx.x;
    Sched sc;
    sc.u_begin = sc.u_end = 0;
    if (!grouped) make_sched(p, total_kb, p.n_token_tiles, n_slabs, sc);

    int w_preissued = 0;
    if (threadIdx.x == 0) {
        for (int i = 0; i < kNS; ++i) {
            mbar_init(bar_full_raw + 8 * i, 1);
            mbar_init(bar_empty_raw + 8 * i, C::kStageArrivals);
            mbar_init(bar_full_x + 8 * i, 1);
            mbar_init(bar_empty_x + 8 * i, C::kAltBlocks ? 1 : C::kIssuers);   // released by the issuer(s) that consumed the stage
        }
        for (int i = 0; i < kNA; ++i) {
            mbar_init(bar_full_a + 8 * i, C::kStageArrivals);
            mbar_init(bar_empty_a + 8 * i, C::kAltBlocks ? 1 : C::kIssuers);
        }
        mbar_init(bar_acc, C::kIssuers);
        mbar_init(bar_acc + 8, C::kIssuers);
        *s_dead = 0;
        *s_ready = 0;
        s_ticket[0] = 0;
        s_ticket[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // The weights are constants of the model, not results of the previous kernel: this thread (the TMA producer)
        // requests the first ring of weight tiles right here - before the CTA-wide set-up barrier, before the tensor
        // memory allocation and before the dependency wait - so that under programmatic dependent launch the HBM
        // latency of the first tiles hides behind the previous kernel's tail and this kernel's own set-up.
        if (!grouped) {
            for (int u = sc.u_begin; u < sc.u_end && w_preissued < kNS;) {
                Seg sg;
                get_seg<BT>(p, grouped, tab_tile, tab_exp, u, total_kb, n_slabs, sc, sg);
                const int w_row = sg.slab * 128;
                for (int j = 0; j < sg.nkb && w_preissued < kNS; ++j, ++w_preissued) {
                    const int st = w_preissued;  // ring is empty: stage index == unit index, no wait needed
                    mbar_arrive_expect_tx(bar_full_raw + 8 * st, C::kRawBytes);
                    tma_load_2d(s_raw + st * C::kRawBytes, &map_w, bar_full_raw + 8 * st, (sg.kb0 + j) * BK, w_row);
                    if (PAIRED) tma_load_2d(s_raw + st * C::kRawBytes + 128 * BK, &map_w, bar_full_raw + 8 * st, (sg.kb0 + j) * BK, w_row + p.pair_offset);
                }
                u += sg.nkb;
            }
        }
    }
    if (warp == 1) tmem_alloc(smem_u32(s_tmem), C::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    const uint32_t tmem_a0 = tmem_base + C::kAccBufs * C::kAccCols;  // first column of the dequantised-operand stages
    // Likewise the scales of the first segment's first two K blocks (model constants): fetched by the converting warps
    // before the dependency wait, so that their L2 / HBM latency is not the first thing on the critical path after it.
    __half pre_cur[C::kWT], pre_nx1[C::kWT];
    bool pre_ok = false;
    if (!grouped && warp >= 2 && warp <= 9 && sc.u_begin < sc.u_end) {
        Seg sg0;
        get_seg<BT>(p, grouped, tab_tile, tab_exp, sc.u_begin, total_kb, n_slabs, sc, sg0);
        const int kb_last0 = sg0.kb0 + sg0.nkb - 1;
#pragma unroll
        for (int wt = 0; wt < C::kWT; ++wt) {
            int n = sg0.slab * 128 + (warp & 3) * 32 + lane + wt * p.pair_offset;
            n = min(n, p.w_rows_per_expert - 1);
            const int64_t srow0 = (int64_t)(n / p.block_h) * p.Kb;
            pre_cur[wt] = load_scale_h(p.scales, srow0 + ((sg0.kb0 * BK) >> 7), p.scale_dtype);
            pre_nx1[wt] = load_scale_h(p.scales, srow0 + ((min(sg0.kb0 + 1, kb_last0) * BK) >> 7), p.scale_dtype);
        }
        pre_ok = true;
    }

    // Everything above read only launch parameters and model weights, so under programmatic dependent launch it may
    // have overlapped the tail of the previous kernel in the stream.  What still depends on that kernel's results:
    //   the activation tiles (TMA producer), the output / partial-tile / ticket stores (epilogue), and - grouped launches
    //   only - the route table, which fixes the schedule itself.
    // A grouped launch therefore waits here with all its threads.  A dense launch does NOT: its TMA producer waits just
    // before the first activation tile, its converting warps wait at the start of their first epilogue, and in between
    // the weight tiles that were requested above are converted into the tensor-memory operand stages while the previous
    // kernel is still finishing - when it is done, the MMAs only wait for the activation tiles.
    auto dependency_wait = [&]() {
        asm volatile("griddepcontrol.wait;" ::: "memory");
    };
    if (grouped) {
        dependency_wait();
        if (threadIdx.x == 0) *s_ready = 1;
    }
    if (grouped) {
        if (p.num_experts <= C::kTabExperts) {
            // every segment start searches these tables: keep them on chip
            for (int i = threadIdx.x; i <= p.num_experts; i += kThreadsTc) {
                s_tab[i] = p.tile_offsets[i];
                s_tab[C::kTabExperts + 1 + i] = p.expert_offsets[i];
            }
            __syncthreads();
            tab_tile = s_tab;
            tab_exp = s_tab + C::kTabExperts + 1;
        }
        make_sched(p, total_kb, tab_tile[p.num_experts], n_slabs, sc);
    }
    const int u_begin = sc.u_begin, u_end = sc.u_end;
    const bool has_work = u_begin < u_end;  // uniform for the whole CTA (and, in cluster mode, for the whole cluster)
    // Fused all-reduce: this launch's epoch (one more than the count of finished fused launches; every rank makes
    // the same sequence of launches) tags the packets; the GEMM result itself is first left in a staging buffer.
    unsigned int ar_epoch = 0;     // read after the thread's own dependency wait (the previous fused launch closes it)
    __half* out_ptr = AR ? ar.part : p.out;

    if (!has_work) {
        // nothing to do: fall through to the teardown (TMEM must still be returned)
    } else if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            if (!grouped) {
                dependency_wait();      // the activations are the previous kernel's output
                *s_ready = 1;
            }
            Ring ring;
            bool ok = true;
            int it = 0;   // K blocks handled so far; the first w_preissued of them already have their weight tile in flight
            for (int u = u_begin; u < u_end && ok;) {
                Seg sg;
                get_seg<BT>(p, grouped, tab_tile, tab_exp, u, total_kb, n_slabs, sc, sg);
                const int w_row = sg.expert * p.w_rows_per_expert + sg.slab * 128;
                for (int j = 0; j < sg.nkb; ++j, ++it) {
                    const int s = ring.stage;
                    const int k0 = (sg.kb0 + j) * BK;
                    if (it >= w_preissued) {
                        ok = mbar_wait(bar_empty_raw + 8 * s, ring.phase ^ 1u, s_dead, 1);
                        if (!ok) break;
                        mbar_arrive_expect_tx(bar_full_raw + 8 * s, C::kRawBytes);
                        tma_load_2d(s_raw + s * C::kRawBytes, &map_w, bar_full_raw + 8 * s, k0, w_row);
                        if (PAIRED) tma_load_2d(s_raw + s * C::kRawBytes + 128 * BK, &map_w, bar_full_raw + 8 * s, k0, w_row + p.pair_offset);
                    }
                    ok = mbar_wait(bar_empty_x + 8 * s, ring.phase ^ 1u, s_dead, 2);
                    if (!ok) break;
                    mbar_arrive_expect_tx(bar_full_x + 8 * s, C::kXBytes);
#pragma unroll
                    for (int sl = 0; sl < C::kSlabs; ++sl)
                        tma_load_2d(s_x + s * C::kXBytes + sl * (BT * 128), &map_x, bar_full_x + 8 * s, k0 + sl * 64, sg.row_begin);
                    ring.advance(kNS);
                }
                u += sg.nkb;
            }
        }
    } else if (warp == 1 || warp == 10) {
        // ================= MMA issuer(s) =================
        const int issuer = warp == 1 ? 0 : 1;
        if (lane == 0 && issuer < C::kIssuers) {
            constexpr uint32_t idesc = make_idesc_f16(BT);
            Ring rx, ra;
            bool ok = true;
            int si = 0;   // segment index: selects the accumulator buffer
            for (int u = u_begin; u < u_end && ok; ++si) {
                const uint32_t d_acc = tmem_base + (uint32_t)((si % C::kAccBufs) * C::kAccCols + issuer * (BT * C::kWT));
                // length of the segment that starts at u (as get_seg computes it, without the tile look-up)
                int nkb;
                if (p.cluster_size > 1) nkb = u_end - u;
                else if (!p.no_split) nkb = min(total_kb - u % total_kb, u_end - u);
                else nkb = total_kb;
                const uint32_t owners = owners_mask<kNA>(ra.stage, nkb);
                bool first = true;    // this issuer's first MMA of the segment overwrites its accumulator
                for (int j = 0; j < nkb; ++j) {
                    const bool mine = !C::kAltBlocks || C::kIssuers == 1 || (ra.stage & 1) == issuer;
                    if (mine) {   // stage-owner scheme: only the K blocks in this issuer's operand stages
                        ok = mbar_wait(bar_full_a + 8 * ra.stage, ra.phase, s_dead, 4) &&
                             mbar_wait(bar_full_x + 8 * rx.stage, rx.phase, s_dead, 8);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t a_col = tmem_a0 + ra.stage * C::kACols;
                        // one descriptor per K block; the 16-element K steps only add to its start-address field
                        const uint64_t db0 = make_desc_sw128(s_x + rx.stage * C::kXBytes);
                        constexpr int kSteps = C::kSlabs * 4;              // 16-element K steps per K block
                        constexpr int kMine = C::kAltBlocks ? kSteps : kSteps / C::kIssuers;
                        const int step0 = C::kAltBlocks ? 0 : issuer * kMine;
                        const uint32_t first_acc = first ? 0u : 1u;
                        first = false;
#pragma unroll
                        for (int t = 0; t < kMine; ++t) {
                            const int step = step0 + t;
                            const int sl = step >> 2, kk = step & 3;
                            const uint64_t db = db0 + (uint64_t)((sl * (BT * 128) + kk * 32) >> 4);
                            const uint32_t a_k = a_col + step * 8;             // 16 K elements = 8 columns
                            if (t == 0) {
                                umma_f16_ts(d_acc, a_k, db, idesc, first_acc);
                                if (PAIRED) umma_f16_ts(d_acc + BT, a_k + BK / 2, db, idesc, first_acc);
                            } else {
                                umma_f16_ts_acc(d_acc, a_k, db, idesc);
                                if (PAIRED) umma_f16_ts_acc(d_acc + BT, a_k + BK / 2, db, idesc);
                            }
                        }
                        umma_commit(bar_empty_a + 8 * ra.stage);
                        umma_commit(bar_empty_x + 8 * rx.stage);
                    }
                    ra.advance(kNA);
                    rx.advance(kNS);
                }
                // The accumulators of this segment are complete when every issuer's MMAs are: the barrier takes one arrival
                // per issuer.  An issuer that owns no block of a short segment does not arrive at all (nothing orders it
                // behind the pipeline; a free-running arrival could complete a later phase of the barrier early): the
                // issuer that does own blocks arrives twice instead.
                if (ok) {
                    if (!C::kAltBlocks || C::kIssuers == 1) {
                        umma_commit(bar_acc + 8 * (si % C::kAccBufs));
                    } else if (owners & (1u << issuer)) {
                        umma_commit(bar_acc + 8 * (si % C::kAccBufs));
                        if (owners == (1u << issuer)) umma_commit(bar_acc + 8 * (si % C::kAccBufs));
                    }
                }
                u += nkb;
            }
        }
    } else if (warp >= 2 && warp <= 9) {
        // ================= dequant warps; after each segment, the epilogue =================
        // A warp may touch only the TMEM lanes of its quarter (warp % 4), so the weight row a thread
        // converts is 32 * (warp % 4) + lane; the two warps of a quarter take alternate K blocks (small tiles) or split the
        // K range of every block (128-token tiles and up).
        const int td = threadIdx.x - 64;
        const int q4 = warp & 3;
        const int r = q4 * 32 + lane;           // weight row inside the slab == TMEM lane
        const int hk = (warp - 2) >> 2;         // this warp's group: its K blocks (or its half of every block's K range), and its half of the epilogue's columns
        constexpr int kCPT = C::kInterleave ? BK / 16 : BK / 32;   // 16-byte chunks per thread per weight tile
        const uint32_t r7 = (uint32_t)(r & 7);
        const int n_local = r;
        const uint32_t t_lane = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const uint32_t t_lane_a = t_lane + C::kAccBufs * C::kAccCols;
        constexpr int kColsPerWarp = BT / 2;
        constexpr int kTileFloats = C::kWT * BT * 128;

        Ring rr, ra;   // raw-tile ring (shared memory) and dequantised-operand ring (TMEM)
        bool ok = true;
        int blk = 0;   // K blocks seen so far (all segments): even ones belong to group 0, odd ones to group 1

        // Fused all-reduce of one finished region of an output tile (16-byte groups [lo, hi) of the BT x 128 tile).
        // Called by all 256 threads.  This rank's FP16 values of the region are already in its staging buffer (written
        // by this CTA): after a barrier every thread takes four consecutive features, pushes them to every peer's
        // inbox, then polls - bounded - its own inbox for the peers' packets of the same four features, adds all
        // contributions in ascending rank order and stores the sum.  The inbox is double-buffered by launch parity: a
        // peer can be at most one launch ahead, because finishing a launch needs this rank's packets of that launch.
        auto ar_finish = [&](const Seg& sg, int lo, int hi, int dead_in) -> int {
            if (!AR) return dead_in;
            epi_bar_sync();
            int dead = dead_in | *s_dead;
            const int n0 = sg.slab * 128;
            if (!dead) ar_exchange(ar, out_ptr, p.residual, ar_epoch, p.N, p.ldo, sg.row_begin, sg.rows_valid, n0, lo, hi, td, s_dead);
            // one verdict for the whole CTA, published by one thread between two barriers taken by all
            epi_bar_sync();
            if (td == 0) s_ticket[1] = *s_dead;
            epi_bar_sync();
            return dead_in | s_ticket[1];
        };

        // Epilogue of one finished segment: TMEM -> registers -> FP16 output, or fp32 partial tile + ticket
        // + (for the last contributor) the fixed-order reduction.  Returns the CTA-wide "dead" flag that
        // thread 0 publishes; every one of the 256 threads calls it once per segment and takes both
        // barriers inside, whatever its own `ok` says, so a timed-out wait can never strand the others.
        auto epilogue = [&](const Seg& sg, int si) -> int {
            if (!grouped) dependency_wait();   // (returns at once after the first time) output, partial tiles and tickets may be in use until now
            if (AR) ar_epoch = *reinterpret_cast<volatile unsigned int*>(ar.ctrl) + 1u;
            const int n0 = sg.slab * 128;
            const uint32_t t_acc = t_lane + (uint32_t)((si % C::kAccBufs) * C::kAccCols);
            if (ok) ok = mbar_wait(bar_acc + 8 * (si % C::kAccBufs), (uint32_t)(si / C::kAccBufs) & 1u, s_dead, 64);
            ok = __all_sync(0xFFFFFFFFu, ok) != 0;  // tcgen05.ld is warp-collective: keep the warp together
            const bool clustered = p.cluster_size > 1;
            const bool direct = !clustered && (sg.n_contrib == 1);
            if (ok) {
                tc_fence_after();
                const int n = n0 + n_local;
                // partial tile: a workspace slot (stream-K), or this CTA's idle raw-tile ring (cluster split-K)
                float* part = clustered ? reinterpret_cast<float*>(smem_dyn + (s_raw - dyn_base))
                                        : p.partial + (int64_t)partial_slot(cta, sg.tkey, total_kb, sc) * kTileFloats;
#pragma unroll 1
                for (int c0 = 0; c0 < kColsPerWarp; c0 += 8) {
                    const int col = hk * kColsPerWarp + c0;
                    float g[8], uu[8];
                    // which issuers' accumulators hold this segment (both, in the scheme where both work on every block)
                    const uint32_t owners = (C::kIssuers == 2 && C::kAltBlocks) ? owners_mask<kNA>(sg.a_stage0, sg.nkb) : (C::kIssuers == 2 ? 3u : 1u);
                    if (owners & 1u) {
                        tmem_ld8(t_acc + col, g);
                        if (PAIRED) tmem_ld8(t_acc + BT + col, uu);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) g[j] = uu[j] = 0.f;
                    }
                    if (owners & 2u) {   // the second issuer's share, added in fixed order
                        float g2[8], u2[8];
                        tmem_ld8(t_acc + BT * C::kWT + col, g2);
                        if (PAIRED) tmem_ld8(t_acc + BT * C::kWT + BT + col, u2);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            g[j] += g2[j];
                            if (PAIRED) uu[j] += u2[j];
                        }
                    }
                    if (direct) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (col + j < sg.rows_valid && n < p.N)
                                store_out<PAIRED, AR>(p, out_ptr, sg.row_begin + col + j, n, g[j], PAIRED ? uu[j] : 0.f);
                    } else if (clustered) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            part[(col + j) * 128 + n_local] = g[j];
                            if (PAIRED) part[(BT + col + j) * 128 + n_local] = uu[j];
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            __stcg(&part[(col + j) * 128 + n_local], g[j]);
                            if (PAIRED) __stcg(&part[(BT + col + j) * 128 + n_local], uu[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            // Hand-off.  All 256 threads take both barriers in every segment, whatever happened above,
            // and act only on values that thread 0 publishes between them, so that a timed-out wait
            // somewhere in the CTA can never strand part of it at a barrier.  Memory ordering: the
            // partial stores of all threads are ordered before the first barrier (CTA scope); thread 0's
            // fence + ticket increment publishes them device-wide (release, cumulative), and its fence
            // after the increment makes the other contributors' partials visible to every thread that
            // passes the second barrier (acquire).
            epi_bar_sync();
            if (td == 0) {
                const int dead = *s_dead;
                int tk = -1;
                if (!direct && !clustered && !dead) {
                    __threadfence();
                    tk = (int)atomicAdd(&p.tickets[sg.tile], 1u);
                    __threadfence();
                }
                s_ticket[0] = tk;
                s_ticket[1] = dead;
            }
            epi_bar_sync();
            const int ticket = s_ticket[0];
            const int dead_now = s_ticket[1];
            if (!direct && !clustered && ticket == sg.n_contrib - 1) {
                // Last contributor: add the partial tiles in ascending CTA order (deterministic).  Four
                // consecutive output features per thread and step; the slots are read eight at a time with
                // independent 16-byte loads so that one L2 round trip covers eight contributors.
                for (int idx4 = td; idx4 < BT * 32; idx4 += kDequantThreads) {
                    const int ml = idx4 >> 5, nl = (idx4 & 31) * 4;
                    if (ml >= sg.rows_valid || n0 + nl >= p.N) continue;
                    float4 g = make_float4(0.f, 0.f, 0.f, 0.f), uu = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int c0 = 0; c0 < sg.n_contrib; c0 += 8) {
                        float4 a[8], b[8];
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            const int cc = sg.first_c + min(c0 + t, sg.n_contrib - 1);   // clamped: extra loads are ignored below
                            const float4* ps = reinterpret_cast<const float4*>(
                                p.partial + (int64_t)partial_slot(cc, sg.tkey, total_kb, sc) * kTileFloats);
                            a[t] = __ldcg(&ps[idx4]);
                            if (PAIRED) b[t] = __ldcg(&ps[BT * 32 + idx4]);
                        }
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            if (c0 + t < sg.n_contrib) {
                                g.x += a[t].x; g.y += a[t].y; g.z += a[t].z; g.w += a[t].w;
                                if (PAIRED) { uu.x += b[t].x; uu.y += b[t].y; uu.z += b[t].z; uu.w += b[t].w; }
                            }
                        }
                    }
                    const int row = sg.row_begin + ml, n = n0 + nl;
                    store_out<PAIRED, AR>(p, out_ptr, row, n, g.x, uu.x);
                    if (n + 1 < p.N) store_out<PAIRED, AR>(p, out_ptr, row, n + 1, g.y, uu.y);
                    if (n + 2 < p.N) store_out<PAIRED, AR>(p, out_ptr, row, n + 2, g.z, uu.z);
                    if (n + 3 < p.N) store_out<PAIRED, AR>(p, out_ptr, row, n + 3, g.w, uu.w);
                }
                if (td == 0) p.tickets[sg.tile] = 0u;  // leave the counter clean for the next launch
                if (AR) return ar_finish(sg, 0, BT * 32, dead_now);
            }
            if (AR && direct) return ar_finish(sg, 0, BT * 32, dead_now);
            return dead_now;
        };

        Seg pend;          // finished segment whose epilogue is deferred (double-buffered accumulators)
        int pend_i = -1;
        int si = 0;
        int stop = 0;
        for (int u = u_begin; u < u_end; ++si) {
            Seg sg;
            get_seg<BT>(p, grouped, tab_tile, tab_exp, u, total_kb, n_slabs, sc, sg);
            sg.a_stage0 = ra.stage;
            u += sg.nkb;
            const int n0 = sg.slab * 128;
            // scale-grid rows for this thread's weight row(s); clamped so tail rows stay in bounds
            int64_t srow[C::kWT];
#pragma unroll
            for (int wt = 0; wt < C::kWT; ++wt) {
                int n = n0 + r + wt * p.pair_offset;
                n = min(n, p.w_rows_per_expert - 1);
                srow[wt] = (int64_t)sg.expert * p.scale_expert_stride + (int64_t)(n / p.block_h) * p.Kb;
            }
            // software-pipelined scale fetch: the values for K blocks j + 1 and j + 2 are in flight while
            // block j is converted (an L2 round trip is longer than one K block)
            const int kb_last = sg.kb0 + sg.nkb - 1;
            __half s_cur[C::kWT], s_nx1[C::kWT];
#pragma unroll
            for (int wt = 0; wt < C::kWT; ++wt) {
                if (pre_ok) {   // fetched before the dependency wait (first segment) or during the previous segment
                    s_cur[wt] = pre_cur[wt];
                    s_nx1[wt] = pre_nx1[wt];
                } else {
                    s_cur[wt] = load_scale_h(p.scales, srow[wt] + ((sg.kb0 * BK) >> 7), p.scale_dtype);
                    s_nx1[wt] = load_scale_h(p.scales, srow[wt] + ((min(sg.kb0 + 1, kb_last) * BK) >> 7), p.scale_dtype);
                }
            }
            pre_ok = false;
            if (!AR && u < u_end) {   // (not in the fused all-reduce build: it has no registers to spare and few segments per CTA)
                // the first scales of the NEXT segment travel while this one is converted: with short segments (a few
                // K blocks per tile, as in the MoE down projection) their latency would otherwise open every tile
                Seg nx;
                get_seg<BT>(p, grouped, tab_tile, tab_exp, u, total_kb, n_slabs, sc, nx);
                const int kb_last_n = nx.kb0 + nx.nkb - 1;
#pragma unroll
                for (int wt = 0; wt < C::kWT; ++wt) {
                    int n = nx.slab * 128 + r + wt * p.pair_offset;
                    n = min(n, p.w_rows_per_expert - 1);
                    const int64_t srow_n = (int64_t)nx.expert * p.scale_expert_stride + (int64_t)(n / p.block_h) * p.Kb;
                    pre_cur[wt] = load_scale_h(p.scales, srow_n + ((nx.kb0 * BK) >> 7), p.scale_dtype);
                    pre_nx1[wt] = load_scale_h(p.scales, srow_n + ((min(nx.kb0 + 1, kb_last_n) * BK) >> 7), p.scale_dtype);
                }
                pre_ok = true;
            }
            for (int j = 0; j < sg.nkb && ok; ++j) {
                const int s = rr.stage, sa = ra.stage;
                __half2 sc[C::kWT];
                __half s_nx2[C::kWT];
#pragma unroll
                for (int wt = 0; wt < C::kWT; ++wt) {
                    sc[wt] = __halves2half2(s_cur[wt], s_cur[wt]);
                    s_nx2[wt] = load_scale_h(p.scales, srow[wt] + ((min(sg.kb0 + j + 2, kb_last) * BK) >> 7), p.scale_dtype);
                    s_cur[wt] = s_nx1[wt];
                    s_nx1[wt] = s_nx2[wt];
                }
                // interleaved groups: this K block belongs to the group whose turn it is (blocks counted over the whole CTA)
                const bool mine = !C::kInterleave || (blk & 1) == hk;
                ++blk;
                if (mine) {
                    ok = mbar_wait(bar_full_raw + 8 * s, rr.phase, s_dead, 16);
                    ok = ok && mbar_wait(bar_empty_a + 8 * sa, ra.phase ^ 1u, s_dead, 32);
                    if (!ok) break;
                    tc_fence_after();   // the MMAs that last read this TMEM stage are complete (empty_a): order our stores after them
#pragma unroll
                    for (int wt = 0; wt < C::kWT; ++wt) {
                        const uint32_t raw_row = s_raw + s * C::kRawBytes + wt * (128 * BK) + r * BK;
                        const uint32_t a_dst = t_lane_a + sa * C::kACols + wt * (BK / 2);
#pragma unroll
                        for (int c = 0; c < kCPT; ++c) {
                            const uint32_t chunk = (uint32_t)((C::kInterleave ? 0 : hk * kCPT) + c);
                            const uint32_t phys = (BK == 128) ? (chunk ^ r7) : (chunk ^ ((uint32_t)(r >> 1) & 3u));
                            const uint4 q = lds128(raw_row + phys * 16);
                            uint32_t hw[8];
                            e4m3x4_scaled_hw(q.x, sc[wt], hw[0], hw[1]);
                            e4m3x4_scaled_hw(q.y, sc[wt], hw[2], hw[3]);
                            e4m3x4_scaled_hw(q.z, sc[wt], hw[4], hw[5]);
                            e4m3x4_scaled_hw(q.w, sc[wt], hw[6], hw[7]);
                            tmem_st8(a_dst + chunk * 8, hw);   // 16 K elements = 8 columns
                        }
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(bar_full_a + 8 * sa);
                    mbar_arrive(bar_empty_raw + 8 * s);
                }
                rr.advance(kNS);
                ra.advance(kNA);
                if (C::kDefer > 0 && pend_i >= 0 && j + 1 == min(C::kDefer, sg.nkb)) {
                    // the MMA warp now has work queued for this segment: drain the previous one meanwhile
                    stop = epilogue(pend, pend_i);
                    pend_i = -1;
                    if (stop) break;
                }
            }


            if (stop) break;
            if (pend_i >= 0) {   // only reached when a wait timed out inside the loop above
                stop = epilogue(pend, pend_i);
                pend_i = -1;
                if (stop) break;
            }
            if (C::kDefer > 0) {
                pend = sg;
                pend_i = si;
            } else {
                stop = epilogue(sg, si);
                if (stop) break;
            }
        }
        if (!stop && pend_i >= 0) stop = epilogue(pend, pend_i);
        if (p.cluster_size > 1) {
            // every CTA of the cluster has parked its fp32 partial tile in its own shared memory
            cluster_sync_all();
            if (!stop) {
                Seg last_sg;   // the one segment of this CTA
                get_seg<BT>(p, grouped, tab_tile, tab_exp, u_begin, total_kb, n_slabs, sc, last_sg);
                const int S = p.cluster_size;
                uint32_t rnk;
                asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rnk));
                const int n0 = last_sg.slab * 128;
                const int chunk = (BT * 32 + S - 1) / S;             // 16-byte groups of the tile reduced by each rank
                const int lo = (int)rnk * chunk, hi = min(BT * 32, lo + chunk);
                const uint32_t local_part = s_raw;
                // all ranks' slices are requested at once (one distributed-shared-memory round trip), then added in
                // ascending rank = ascending K order: deterministic
                for (int idx4 = lo + td; idx4 < hi; idx4 += kDequantThreads) {
                    const int ml = idx4 >> 5, nl = (idx4 & 31) * 4;
                    if (ml >= last_sg.rows_valid || n0 + nl >= p.N) continue;
                    float4 g = make_float4(0.f, 0.f, 0.f, 0.f), uu = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int wt = 0; wt < C::kWT; ++wt) {
                        constexpr int kBatch = AR ? 4 : 8;   // the fused all-reduce build has fewer registers to spare
                        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int t0 = 0; t0 < 8; t0 += kBatch) {
                            float4 a[kBatch];
#pragma unroll
                            for (int t = 0; t < kBatch; ++t)
                                if (t0 + t < S) a[t] = ld_cluster_f4(cluster_map(local_part, (uint32_t)(t0 + t)) + (uint32_t)(wt * BT * 32 + idx4) * 16u);
#pragma unroll
                            for (int t = 0; t < kBatch; ++t)
                                if (t0 + t < S) { acc.x += a[t].x; acc.y += a[t].y; acc.z += a[t].z; acc.w += a[t].w; }
                        }
                        if (wt == 0) g = acc; else uu = acc;
                    }
                    const int row = last_sg.row_begin + ml, n = n0 + nl;
                    store_out<PAIRED, AR>(p, out_ptr, row, n, g.x, uu.x);
                    if (n + 1 < p.N) store_out<PAIRED, AR>(p, out_ptr, row, n + 1, g.y, uu.y);
                    if (n + 2 < p.N) store_out<PAIRED, AR>(p, out_ptr, row, n + 2, g.z, uu.z);
                    if (n + 3 < p.N) store_out<PAIRED, AR>(p, out_ptr, row, n + 3, g.w, uu.w);
                }
            }
            // this CTA has read what it needs from its peers; nobody may leave (and free its shared memory) before
            // every peer has said the same - the matching wait is taken in the teardown
            cluster_arrive();
            if (AR) {
                Seg last_sg;
                get_seg<BT>(p, grouped, tab_tile, tab_exp, u_begin, total_kb, n_slabs, sc, last_sg);
                uint32_t rnk;
                asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rnk));
                const int chunk = (BT * 32 + p.cluster_size - 1) / p.cluster_size;
                const int lo = (int)rnk * chunk, hi = min(BT * 32, lo + chunk);
                if (lo < hi) stop = ar_finish(last_sg, lo, hi, stop);
            }
        }
    }

    if (p.cluster_size > 1) {
        if (!(has_work && warp >= 2 && warp <= 9)) {
            cluster_sync_all();   // the dequant warps of a working CTA take the first barrier and the second arrive in their branch
            cluster_arrive();
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
    // cluster split-K: nobody may leave (and free the shared memory its peers read their slices from) before every peer
    // has said it is done reading; taken last, so that the wait overlaps the tensor-memory release above
    if (p.cluster_size > 1) cluster_wait();
    if (AR && threadIdx.x == 0) {
        // the last CTA of the grid to get here closes the launch: the epoch every CTA read above is now finished
        dependency_wait();     // (a CTA without work has not waited yet)
        ar_epoch = *reinterpret_cast<volatile unsigned int*>(ar.ctrl) + 1u;
        __threadfence();
        const unsigned int prev = atomicAdd(&ar.ctrl[1], 1u);
        if (prev == gridDim.x - 1) {
            ar.ctrl[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned int*>(ar.ctrl) = ar_epoch;
        }
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

// 2-D row-major tensor [rows, cols] of `elem_bytes` elements, box [box_rows, box_cols].  Encoded descriptors are
// cached per (address, shape, box).  Weights keep their address for the life of a model: their descriptors live in a
// map that only grows with the number of distinct weights.  Activation addresses come from the caller's allocator and
// may be new on every eager call: their descriptors go through a small direct-mapped table (a colliding entry is
// simply overwritten), so a stream of fresh addresses costs one driver call each and never evicts anything else.
struct MapKey {
    const void* base;
    uint64_t rows, cols;
    uint32_t box_rows, box_cols;
    int dt, swz;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows && box_cols == o.box_cols &&
               dt == o.dt && swz == o.swz;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.base) * 0x9E3779B97F4A7C15ull;
        h ^= (k.rows * 0xC2B2AE3D27D4EB4Full) ^ (k.cols << 17) ^ ((size_t)k.box_rows << 40) ^ ((size_t)k.box_cols << 50) ^
             ((size_t)k.dt << 3) ^ (size_t)k.swz;
        return h;
    }
};

constexpr size_t kActMapSlots = 1024;

int encode_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows, uint64_t cols,
              uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz, bool is_weight) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> weights;
    struct Slot {
        bool used;
        MapKey key;
        CUtensorMap map;
    };
    static Slot* acts = new Slot[kActMapSlots]();
    const MapKey key{base, rows, cols, box_rows, box_cols, (int)dt, (int)swz};
    const size_t slot = MapKeyHash()(key) % kActMapSlots;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (is_weight) {
            auto it = weights.find(key);
            if (it != weights.end()) {
                *map = it->second;
                return 0;
            }
        } else if (acts[slot].used && acts[slot].key == key) {
            *map = acts[slot].map;
            return 0;
        }
    }
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
    {
        std::lock_guard<std::mutex> lock(mu);
        if (is_weight) {
            if (weights.size() >= (1u << 16)) weights.clear();   // far more distinct weights than any model has: start over
            weights.emplace(key, *map);
        } else {
            acts[slot].used = true;
            acts[slot].key = key;
            acts[slot].map = *map;
        }
    }
    return 0;
}

template <int BT, int BK, bool PAIRED, bool AR>
int launch_cfg(const TcLaunch& L, cudaStream_t st) {
    using C = TcCfg<BT, BK, PAIRED>;
    static bool attr_set[64] = {};
    int dev = 0;
    W8A16_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        W8A16_CUDA(cudaFuncSetAttribute(k_gemm_tc<BT, BK, PAIRED, AR>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        W8A16_CUDA(cudaFuncSetAttribute(k_gemm_tc<BT, BK, PAIRED, AR>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        attr_set[dev] = true;
    }
    CUtensorMap map_w, map_x;
    int rc = encode_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, L.w, (uint64_t)L.w_total_rows, (uint64_t)L.p.K, 128, BK,
                       BK == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, true);
    if (rc) return rc;
    rc = encode_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, L.x, (uint64_t)L.p.M, (uint64_t)L.p.K, BT, 64, CU_TENSOR_MAP_SWIZZLE_128B, false);
    if (rc) return rc;
    int64_t g = (int64_t)sm_count() * C::kCtasPerSm;
    if (L.max_units < g) g = L.max_units;
    if (g < 1) g = 1;
    const bool clustered = L.p.cluster_size > 1;
    if (clustered) {
        W8A16_REQUIRE(C::kClusterOk, FP8W8A16_ERR_UNSUPPORTED, "gemm_tc: cluster split-K does not fit this configuration");
        g = L.cluster_tiles * L.p.cluster_size;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)g);
    cfg.blockDim = dim3(kThreadsTc);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // overlap our set-up with the previous kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = clustered ? (unsigned)L.p.cluster_size : 1u;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = clustered ? 2 : 1;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, k_gemm_tc<BT, BK, PAIRED, AR>, map_w, map_x, L.p, L.ar);
    if (le != cudaSuccess) return fail(FP8W8A16_ERR_CUDA, "gemm_tc launch failed: %s", cudaGetErrorString(le));
    return check_launch("gemm_tc");
}

// How many clusters of `cs` CTAs of this configuration the device can hold at once (cached per device).
template <int BT, int BK, bool PAIRED>
int max_active_clusters(int cs) {
    using C = TcCfg<BT, BK, PAIRED>;
    static int cached[64][9] = {};   // 0 = not asked yet, -1 = query failed / none fit
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev >= 64 || cs < 2 || cs > 8 || !C::kClusterOk) return 0;
    if (cached[dev][cs] == 0) {
        cudaFuncSetAttribute(k_gemm_tc<BT, BK, PAIRED, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        cudaFuncSetAttribute(k_gemm_tc<BT, BK, PAIRED, false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(cs * 64));
        cfg.blockDim = dim3(kThreadsTc);
        cfg.dynamicSmemBytes = C::kSmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)cs;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, k_gemm_tc<BT, BK, PAIRED, false>, &cfg);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            n = 0;
        }
        // The query answers for one CTA per SM with this kernel's shared-memory size; launches place
        // kCtasPerSm (timing a 40-tile problem: 6-CTA clusters run in one wave, 7-CTA clusters in two).
        n *= C::kCtasPerSm;
        cached[dev][cs] = n > 0 ? n : -1;
    }
    return cached[dev][cs] > 0 ? cached[dev][cs] : 0;
}

int max_active_clusters_for(int bt, bool paired, int cs) {
    if (!paired) {
        switch (bt) {
            case 16: return max_active_clusters<16, 128, false>(cs);
            case 32: return max_active_clusters<32, 128, false>(cs);
            case 64: return max_active_clusters<64, 128, false>(cs);
            default: return 0;
        }
    }
    switch (bt) {
        case 16: return max_active_clusters<16, 64, true>(cs);
        case 32: return max_active_clusters<32, 64, true>(cs);
        case 64: return max_active_clusters<64, 64, true>(cs);
        default: return 0;
    }
}

}  // namespace

int tc_encode_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows, uint64_t cols,
                 uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz, bool is_weight) {
    return encode_2d(map, dt, elem_bytes, base, rows, cols, box_rows, box_cols, swz, is_weight);
}

int tc_block_k(int bt, bool paired) { return (!paired && bt <= 64) ? 128 : 64; }

int tc_ctas_per_sm(int bt, bool paired) { return (bt * (paired ? 2 : 1) <= 64) ? 2 : 1; }

int tc_grid(int bt, bool paired) { return sm_count() * tc_ctas_per_sm(bt, paired); }

size_t tc_workspace_bytes(int bt, bool paired) {
    const size_t tile_floats = (size_t)(paired ? 2 : 1) * bt * 128;
    return kTicketBytes + (size_t)tc_grid(bt, paired) * 2 * tile_floats * sizeof(float);
}

size_t tc_max_tiles_with_tickets() { return kTicketBytes / sizeof(unsigned int); }

// Cluster split-K is used when the output tiles alone cannot fill the machine: `tiles` tiles, each shared by
// the returned number of CTAs (2..8, 0 = do not use it).  Every CTA of a cluster gets at least one K block.
// Only sizes whose clusters are ALL resident at once are considered (the occupancy query accounts for how
// clusters pack into the GPCs): a second wave of clusters costs far more than the fix-up it replaces.
int tc_cluster_size(int64_t tiles, int total_kb, int bt, bool paired) {
    const int max_s = 8;    // portable cluster size limit
    if (tiles <= 0 || bt > 64) return 0;
    const int64_t capacity = tc_grid(bt, paired);
    int64_t s = capacity / tiles;
    if (s > max_s) s = max_s;
    if (s > total_kb) s = total_kb;
    for (; s >= 2; --s) {
        if (max_active_clusters_for(bt, paired, (int)s) < tiles) continue;
        const int per = (total_kb + (int)s - 1) / (int)s;
        const int eff = (total_kb + per - 1) / per;   // every rank must own at least one K block
        if (eff == (int)s) return eff;
        if (eff >= 2 && max_active_clusters_for(bt, paired, eff) >= tiles) return eff;
    }
    return 0;
}

int tc_pick_bt(int rows) {
    if (rows <= 16) return 16;
    if (rows <= 32) return 32;
    if (rows <= 64) return 64;
    if (rows <= 128) return 128;
    return 256;
}

int tc_launch(const TcLaunch& L, int bt, bool paired, cudaStream_t st) {
    // dense batches above 128 tokens: the CTA-pair kernel (gemm_tc2.cu)
    if (bt == 256 && !paired && L.ar.world <= 1 && L.p.expert_offsets == nullptr && tc2_enabled()) return tc2_launch(L, st);
#define W8A16_TC_CASE(BT_, BK_, P_) return launch_cfg<BT_, BK_, P_, false>(L, st)
#define W8A16_TC_CASE_AR(BT_, BK_) return launch_cfg<BT_, BK_, false, true>(L, st)
    if (L.ar.world > 1) {
        W8A16_REQUIRE(!paired, FP8W8A16_ERR_UNSUPPORTED, "gemm_tc: the fused all-reduce is a dense mode");
        switch (bt) {
            case 16: W8A16_TC_CASE_AR(16, 128);
            case 32: W8A16_TC_CASE_AR(32, 128);
            case 64: W8A16_TC_CASE_AR(64, 128);
            case 128: W8A16_TC_CASE_AR(128, 64);
            case 256: W8A16_TC_CASE_AR(256, 64);
        }
    } else if (!paired) {
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
        }
    }
#undef W8A16_TC_CASE_AR
#undef W8A16_TC_CASE
    return fail(FP8W8A16_ERR_UNSUPPORTED, "gemm_tc: unsupported token tile %d", bt);
}


int tc_read_status(int* out, int reset) {
    int v = 0, v2 = 0;
    W8A16_CUDA(cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)));
    if (reset && v != 0) {
        const int zero = 0;
        W8A16_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)));
    }
    const int rc = tc2_read_status(&v2, reset);
    if (rc) return rc;
    *out = v | (v2 ? (v2 | 0x400) : 0);     // bit 0x400: the wait that ran out was in the CTA-pair kernel
    return 0;
}

}  // namespace w8a16
