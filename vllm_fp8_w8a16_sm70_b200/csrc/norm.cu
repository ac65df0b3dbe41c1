// Residual add + RMSNorm of the rows a row-parallel projection has just produced: the step that follows o_proj / down_proj
// in a decoder layer (vLLM's fused_add_rms_norm after the tensor-parallel reduce, mirrored by the reference's call site at
// src/fp8_w8a16_sm70/vllm_serve.py:2922-2959).  One CTA per row; launched with programmatic dependent launch, so its
// set-up overlaps the tail of the GEMM that produces x.
//   z = x + residual           (fp32 sum, rounded to FP16 once; z is also the new residual)
//   out = FP16(z * rsqrt(mean(z^2) + eps)) * weight      (the norm of the ROUNDED z, FP16 product: vLLM's kernel order)
// When the residual was already added in the GEMM epilogue (fp8w8a16_linear_residual / _allreduce_residual), pass
// residual = NULL: x is z.
#include "common.cuh"

namespace w8a16 {
namespace {

__global__ void __launch_bounds__(256)
k_add_rmsnorm(const __half* __restrict__ x, const __half* __restrict__ residual, const __half* __restrict__ weight, float eps,
              __half* __restrict__ out, __half* __restrict__ residual_out, int N) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int vecs = N >> 3;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (int64_t)row * N);
    const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + (int64_t)row * N) : nullptr;
    uint4* zr = residual_out ? reinterpret_cast<uint4*>(residual_out + (int64_t)row * N) : nullptr;
    extern __shared__ uint4 s_z[];          // the row of z, kept on chip between the two passes
    float ss = 0.f;
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
        uint4 v = __ldcg(xr + i);
        __half2* h = reinterpret_cast<__half2*>(&v);
        if (rr != nullptr) {
            const uint4 r = __ldcg(rr + i);
            const __half2* rh = reinterpret_cast<const __half2*>(&r);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float2 a = __half22float2(h[c]), b = __half22float2(rh[c]);
                h[c] = __floats2half2_rn(a.x + b.x, a.y + b.y);
            }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float2 f = __half22float2(h[c]);
            ss += f.x * f.x + f.y * f.y;
        }
        s_z[i] = v;
        if (zr != nullptr) zr[i] = v;
    }
    __shared__ float s_part[8];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += s_part[w];          // fixed order: deterministic
    const float inv = rsqrtf(tot / (float)N + eps);
    const uint4* wr = reinterpret_cast<const uint4*>(weight);
    uint4* orow = reinterpret_cast<uint4*>(out + (int64_t)row * N);
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
        uint4 v = s_z[i];
        const uint4 wv = __ldg(wr + i);
        __half2* h = reinterpret_cast<__half2*>(&v);
        const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float2 f = __half22float2(h[c]);
            h[c] = __hmul2(__floats2half2_rn(f.x * inv, f.y * inv), wh[c]);
        }
        orow[i] = v;
    }
}

}  // namespace

int launch_add_rmsnorm(const __half* x, const __half* residual, const __half* weight, float eps, __half* out, __half* residual_out,
                       int M, int N, cudaStream_t st) {
    const size_t smem = (size_t)N * sizeof(__half);
    W8A16_REQUIRE(smem <= 64 * 1024, FP8W8A16_ERR_UNSUPPORTED, "add_rmsnorm: rows of %d elements do not fit the on-chip row buffer (32768 at most)", N);
    if (smem > 40 * 1024) {      // beyond the default dynamic shared-memory limit: raise it, once per device
        static bool raised[64] = {};
        int dev = 0;
        W8A16_CUDA(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64 || !raised[dev]) {
            W8A16_CUDA(cudaFuncSetAttribute(k_add_rmsnorm, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
            if (dev >= 0 && dev < 64) raised[dev] = true;
        }
    }
    return finish_launch(launch_pdl(k_add_rmsnorm, dim3((unsigned)M), dim3(256), smem, st, x, residual, weight, eps, out, residual_out, N),
                         "add_rmsnorm");
}

}  // namespace w8a16
