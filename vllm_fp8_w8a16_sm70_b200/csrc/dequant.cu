// Standalone FP8 (E4M3) -> FP16 dequantisation kernels: the bit-exact "dequantised weight"
// every GEMM result is judged against.  Pure HBM streaming (1 byte in, 2 bytes out per element):
// each thread moves 16 weight bytes with one 16-byte load and two 16-byte stores.
#include "common.cuh"

namespace w8a16 {

namespace {

constexpr int kThreads = 256;

// out[i] = cvt(in[i])                        (reference: fp8_dequant.cu:83-90)
// out[i] = cvt(in[i]) * s[i / group]         (reference: fp8_dequant.cu:94-106)
template <bool kScaled>
__global__ void __launch_bounds__(kThreads) k_flat(const uint8_t* __restrict__ in, const __half* __restrict__ scales,
                                                   __half* __restrict__ out, int64_t n, int64_t group) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n) return;
    __half v = __ushort_as_half(e4m3_to_fp16_bits(in[i]));
    if (kScaled) {
        const uint8_t b = in[i];
        if ((b & 0x7Fu) != 0x7Fu) v = __hmul(v, scales[i / group]);
    }
    out[i] = v;
}

// out[i,j] = RN16(cvt(W[i,j]) * S16[i/bh, j/bw])   (reference: fp8_dequant.cu:113-127)
// Vector path: K % 16 == 0, block_w % 16 == 0, 16-byte aligned pointers.  One thread per
// 16-byte chunk of a row; a warp covers 512 contiguous bytes of one row.
__global__ void __launch_bounds__(kThreads) k_block_vec(const uint8_t* __restrict__ w, const void* __restrict__ scales,
                                                         int scale_dtype, __half* __restrict__ out, int N, int K,
                                                         int block_h, int block_w, int Kb) {
    const int chunks_per_row = K >> 4;
    const int64_t total = (int64_t)N * chunks_per_row;
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < total; c += (int64_t)gridDim.x * kThreads) {
        const int i = (int)(c / chunks_per_row);
        const int j = (int)(c - (int64_t)i * chunks_per_row) << 4;
        const uint4 q = __ldcs(reinterpret_cast<const uint4*>(w + (int64_t)i * K + j));
        const __half s = load_scale_h(scales, (int64_t)(i / block_h) * Kb + (j / block_w), scale_dtype);
        const __half2 s2 = __halves2half2(s, s);
        const __half2 c256 = __halves2half2(__ushort_as_half((uint16_t)0x5C00), __ushort_as_half((uint16_t)0x5C00));
        const uint32_t words[4] = {q.x, q.y, q.z, q.w};
        uint32_t r[8];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            // two multiplies, exactly the reference's sequence: (mag<<7 as half) * 256, then * s
            uint32_t m01, g01, m23, g23;
            e4m3x2_split(words[t], 0x1404u, m01, g01);
            e4m3x2_split(words[t], 0x3424u, m23, g23);
            __half2 h01 = __hmul2(__hmul2(*reinterpret_cast<__half2*>(&m01), c256), s2);
            __half2 h23 = __hmul2(__hmul2(*reinterpret_cast<__half2*>(&m23), c256), s2);
            // sign is OR-ed after the multiply by |.|: the scale's own sign must still apply
            uint32_t r01 = *reinterpret_cast<uint32_t*>(&h01) ^ g01;
            uint32_t r23 = *reinterpret_cast<uint32_t*>(&h23) ^ g23;
            const uint32_t wv = words[t];
            const uint32_t z = (~wv) & 0x7F7F7F7Fu;
            if (((z - 0x01010101u) & ~z & 0x80808080u) != 0u) {  // some byte has magnitude 0x7F (NaN)
                if ((wv & 0x0000007Fu) == 0x0000007Fu) r01 = (r01 & 0xFFFF0000u) | ((wv & 0x00000080u) << 8) | 0x00007F80u;
                if ((wv & 0x00007F00u) == 0x00007F00u) r01 = (r01 & 0x0000FFFFu) | ((wv & 0x00008000u) << 16) | 0x7F800000u;
                if ((wv & 0x007F0000u) == 0x007F0000u) r23 = (r23 & 0xFFFF0000u) | ((wv & 0x00800000u) >> 8) | 0x00007F80u;
                if ((wv & 0x7F000000u) == 0x7F000000u) r23 = (r23 & 0x0000FFFFu) | (wv & 0x80000000u) | 0x7F800000u;
            }
            r[2 * t] = r01;
            r[2 * t + 1] = r23;
        }
        uint4* o = reinterpret_cast<uint4*>(out + (int64_t)i * K + j);
        __stcs(o, make_uint4(r[0], r[1], r[2], r[3]));
        __stcs(o + 1, make_uint4(r[4], r[5], r[6], r[7]));
    }
}

// Scalar path for any N, K, block shape and alignment.
__global__ void __launch_bounds__(kThreads) k_block_scalar(const uint8_t* __restrict__ w, const void* __restrict__ scales,
                                                            int scale_dtype, __half* __restrict__ out, int N, int K,
                                                            int block_h, int block_w, int Kb) {
    const int64_t total = (int64_t)N * K;
    for (int64_t idx = (int64_t)blockIdx.x * kThreads + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * kThreads) {
        const int i = (int)(idx / K);
        const int j = (int)(idx - (int64_t)i * K);
        const uint8_t b = w[idx];
        __half v = __ushort_as_half(e4m3_to_fp16_bits(b));
        if ((b & 0x7Fu) != 0x7Fu) v = __hmul(v, load_scale_h(scales, (int64_t)(i / block_h) * Kb + (j / block_w), scale_dtype));
        out[idx] = v;
    }
}

}  // namespace

int launch_e4m3_to_fp16(const uint8_t* in, __half* out, int64_t n, cudaStream_t st) {
    if (n == 0) return 0;
    const int64_t blocks = (n + kThreads - 1) / kThreads;
    W8A16_REQUIRE(blocks < (1ll << 31), FP8W8A16_ERR_INVALID, "e4m3_to_fp16: n=%lld too large", (long long)n);
    k_flat<false><<<(unsigned)blocks, kThreads, 0, st>>>(in, nullptr, out, n, 1);
    return check_launch("e4m3_to_fp16");
}

int launch_e4m3_to_fp16_scaled(const uint8_t* in, const __half* scales, __half* out, int64_t n, int64_t group,
                               cudaStream_t st) {
    if (n == 0) return 0;
    const int64_t blocks = (n + kThreads - 1) / kThreads;
    W8A16_REQUIRE(blocks < (1ll << 31), FP8W8A16_ERR_INVALID, "e4m3_to_fp16_scaled: n=%lld too large", (long long)n);
    k_flat<true><<<(unsigned)blocks, kThreads, 0, st>>>(in, scales, out, n, group);
    return check_launch("e4m3_to_fp16_scaled");
}

int launch_dequant_block(const uint8_t* w, const void* scales, int scale_dtype, __half* out, int N, int K, int block_h,
                         int block_w, cudaStream_t st) {
    if (N == 0 || K == 0) return 0;
    const int Kb = (K + block_w - 1) / block_w;
    const bool vec = (K % 16 == 0) && (block_w % 16 == 0) && aligned16(w) && aligned16(out);
    const int64_t work = vec ? (int64_t)N * (K >> 4) : (int64_t)N * K;
    int64_t blocks = (work + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)sm_count() * 64;  // grid-stride beyond 64 CTAs per SM
    if (blocks > cap) blocks = cap;
    if (vec)
        k_block_vec<<<(unsigned)blocks, kThreads, 0, st>>>(w, scales, scale_dtype, out, N, K, block_h, block_w, Kb);
    else
        k_block_scalar<<<(unsigned)blocks, kThreads, 0, st>>>(w, scales, scale_dtype, out, N, K, block_h, block_w, Kb);
    return check_launch("dequant_block_scaled");
}

}  // namespace w8a16
