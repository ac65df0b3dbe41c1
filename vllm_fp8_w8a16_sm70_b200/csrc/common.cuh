// Shared device helpers and host-side error plumbing for the sm_100a FP8 W8A16 engine.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/fp8w8a16_b200.h"

namespace w8a16 {

// ---------------------------------------------------------------------------------------------
// Host-side error reporting: every C-ABI entry point returns 0 on success or a negative
// FP8W8A16_ERR_* code, and leaves a message retrievable with fp8w8a16_last_error().
// ---------------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

#define W8A16_REQUIRE(cond, code, ...)                    \
    do {                                                  \
        if (!(cond)) return ::w8a16::fail((code), __VA_ARGS__); \
    } while (0)

#define W8A16_CUDA(call)                                                                     \
    do {                                                                                     \
        cudaError_t _e = (call);                                                             \
        if (_e != cudaSuccess)                                                               \
            return ::w8a16::fail(FP8W8A16_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(_e)); \
    } while (0)

// Kernels launched by this library in this process (reported by fp8w8a16_launch_count).
void count_launch();
void count_variant(int variant);   // FP8W8A16_VARIANT_* call counters (host side)

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(FP8W8A16_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
    count_launch();
    return 0;
}

// Outcome of a launch call: the launch API's own return code first (an invalid configuration is reported there),
// then the sticky last-error check that also counts the launch.
inline int finish_launch(cudaError_t le, const char* what) {
    if (le != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(FP8W8A16_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(le));
    }
    return check_launch(what);
}

// Programmatic dependent launch.  Device side: pdl_trigger() lets the next kernel of the stream begin
// launching while this one still runs; pdl_wait() blocks until every kernel this one depends on has
// finished and its writes are visible, and must precede the first access to memory they produce.
// Host side: launch_pdl() launches with the attribute that allows that overlap; a kernel that never
// triggers simply behaves like an ordinary launch.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device).
int sm_count();

// Every kernel that needs cross-CTA hand-off (split-K tickets) takes its counters from the first
// kTicketBytes of the caller's workspace.  The owner zeroes them once; kernels leave them at zero.
constexpr size_t kTicketBytes = 65536;

// ---------------------------------------------------------------------------------------------
// E4M3-FN -> FP16.
// The contract (reference: src/fp8_w8a16_sm70/fp8_dequant.cu:44-50) is: magnitude bits shifted
// to FP16 position, one FP16 multiply by 2^8 (exact), NaN byte (magnitude 0x7F) -> 0x7F80, sign
// OR-ed in.  Every finite E4M3 value is exactly representable in FP16, so any exact conversion
// gives the same bits; only the NaN payload is a convention.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint16_t e4m3_to_fp16_bits(uint8_t b) {
    const uint16_t sign = (uint16_t)(b & 0x80u) << 8;
    const uint16_t mag = (uint16_t)(b & 0x7Fu);
    const __half h = __hmul(__ushort_as_half((uint16_t)(mag << 7)), __ushort_as_half((uint16_t)0x5C00));  // * 256
    const uint16_t val = (mag == 0x7Fu) ? (uint16_t)0x7F80u : __half_as_ushort(h);
    return (uint16_t)(sign | val);
}

// Two bytes of a 32-bit word -> packed half2 of UNSCALED-by-2^8 magnitudes plus the sign word.
// `sel` is the prmt selector that puts byte i in the high byte of halfword 0 and byte j in the
// high byte of halfword 1 (0x1404 for bytes 0,1; 0x3424 for bytes 2,3).  The caller multiplies
// by (256 * scale) with one hmul2 and ORs the sign back in with one lop3.
__device__ __forceinline__ void e4m3x2_split(uint32_t w, uint32_t sel, uint32_t& mag_bits, uint32_t& sign_bits) {
    const uint32_t x = __byte_perm(w, 0u, sel);  // halfword = byte << 8
    mag_bits = (x >> 1) & 0x3F803F80u;           // (byte & 0x7F) << 7 per halfword
    sign_bits = x & 0x80008000u;
}

// Four E4M3 bytes (one 32-bit word, byte 0 = lowest k) -> four FP16 values, each multiplied by
// the FP16 scale `s` with ONE rounding: RN16(cvt(b) * s).  `s256` must hold (s * 256, s * 256);
// the product (mag * 2^-8) * (s * 2^8) is the same real number as cvt(b) * s, so the single
// rounding is identical to the reference's __hmul(cvt(b), s) as long as s * 256 does not overflow
// FP16 (|s| < 256; the host checks this once when weights are loaded).  The sign is applied with
// an XOR after the multiply, so a negative scale still flips it.  A NaN byte (magnitude 0x7F)
// comes out FINITE here (480 * s); e4m3x4_scaled_exact patches it where the contract needs it.
__device__ __forceinline__ void e4m3x4_scaled(uint32_t w, __half2 s256, __half2& o01, __half2& o23) {
    uint32_t m01, g01, m23, g23;
    e4m3x2_split(w, 0x1404u, m01, g01);
    e4m3x2_split(w, 0x3424u, m23, g23);
    __half2 h01 = __hmul2(*reinterpret_cast<__half2*>(&m01), s256);
    __half2 h23 = __hmul2(*reinterpret_cast<__half2*>(&m23), s256);
    uint32_t r01 = *reinterpret_cast<uint32_t*>(&h01) ^ g01;
    uint32_t r23 = *reinterpret_cast<uint32_t*>(&h23) ^ g23;
    o01 = *reinterpret_cast<__half2*>(&r01);
    o23 = *reinterpret_cast<__half2*>(&r23);
}

// Hardware path: cvt.rn.f16x2.e4m3x2 converts two bytes per instruction (exact for every finite
// value; a NaN byte becomes an FP16 NaN, payload 0x7FFF), then ONE FP16 multiply by the scale:
// RN16(cvt(b) * s), the reference's dequantised-weight value (fp8_dequant.cu:125-126).  Measured on
// B200 at 2.2x the throughput of the integer bit trick above, which is why the GEMM paths use it.
__device__ __forceinline__ void e4m3x4_cvt(uint32_t w, uint32_t& r01, uint32_t& r23) {
    asm("{\n\t.reg .b16 lo, hi;\n\t"
        "mov.b32 {lo, hi}, %2;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
        "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
        : "=r"(r01), "=r"(r23)
        : "r"(w));
}

__device__ __forceinline__ void e4m3x4_scaled_hw(uint32_t w, __half2 s, uint32_t& o01, uint32_t& o23) {
    uint32_t r01, r23;
    e4m3x4_cvt(w, r01, r23);
    const __half2 h01 = __hmul2(*reinterpret_cast<__half2*>(&r01), s);
    const __half2 h23 = __hmul2(*reinterpret_cast<__half2*>(&r23), s);
    o01 = *reinterpret_cast<const uint32_t*>(&h01);
    o23 = *reinterpret_cast<const uint32_t*>(&h23);
}

// acc += w.lo * x.lo + w.hi * x.hi with FP16 inputs and fp32 accumulation in one instruction each
// (fma.rn.f32.f16: the product of two halves is exact in fp32, so this equals
// fmaf(float(w), float(x), acc) without the two conversions).
__device__ __forceinline__ void fma2_f32_f16(float& acc, uint32_t w2, uint32_t x2) {
    asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\t"
        "mov.b32 {wl, wh}, %1;\n\t"
        "mov.b32 {xl, xh}, %2;\n\t"
        "fma.rn.f32.f16 %0, wl, xl, %0;\n\t"
        "fma.rn.f32.f16 %0, wh, xh, %0;\n\t}"
        : "+f"(acc)
        : "r"(w2), "r"(x2));
}

// Same, but NaN bytes come out as sign|0x7F80 exactly (the dequantised-weight contract).
__device__ __forceinline__ void e4m3x4_scaled_exact(uint32_t w, __half2 s256, __half2& o01, __half2& o23) {
    e4m3x4_scaled(w, s256, o01, o23);
    // any byte with magnitude 0x7F ?  (w & 0x7F7F7F7F) has a 0x7F byte  <=>  ((~w) & 0x7F7F7F7F) has a zero byte
    const uint32_t t = (~w) & 0x7F7F7F7Fu;
    if (((t - 0x01010101u) & ~t & 0x80808080u) != 0u) {
        uint32_t r01 = *reinterpret_cast<uint32_t*>(&o01);
        uint32_t r23 = *reinterpret_cast<uint32_t*>(&o23);
        if ((w & 0x0000007Fu) == 0x0000007Fu) r01 = (r01 & 0xFFFF0000u) | ((w & 0x00000080u) << 8) | 0x00007F80u;
        if ((w & 0x00007F00u) == 0x00007F00u) r01 = (r01 & 0x0000FFFFu) | ((w & 0x00008000u) << 16) | 0x7F800000u;
        if ((w & 0x007F0000u) == 0x007F0000u) r23 = (r23 & 0xFFFF0000u) | ((w & 0x00800000u) >> 8) | 0x00007F80u;
        if ((w & 0x7F000000u) == 0x7F000000u) r23 = (r23 & 0x0000FFFFu) | (w & 0x80000000u) | 0x7F800000u;
        o01 = *reinterpret_cast<__half2*>(&r01);
        o23 = *reinterpret_cast<__half2*>(&r23);
    }
}

// Scale grid element as FP16 (the reference rounds fp32/bf16 block scales to FP16 once at load,
// src/fp8_w8a16_sm70/vllm_serve.py:1512-1513; an fp32 grid handed to the engine is rounded the
// same way on the fly).
__device__ __forceinline__ __half load_scale_h(const void* scales, int64_t idx, int scale_dtype) {
    if (scale_dtype == FP8W8A16_SCALE_F32) return __float2half_rn(__ldg(reinterpret_cast<const float*>(scales) + idx));
    return __ldg(reinterpret_cast<const __half*>(scales) + idx);
}

__device__ __forceinline__ __half2 scale_times_256(__half s) {
    const __half s256 = __hmul(s, __ushort_as_half((uint16_t)0x5C00));
    return __halves2half2(s256, s256);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

}  // namespace w8a16
