// fp8w8a16_linear_noalloc: the decode GEMV for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc on the hot path: a serving worker whose
// memory pool was sized and handed out at start-up, code that runs under a no-allocation policy,
// or a plugin that is only ever given input and output buffers.  The split-K GEMV needs
// scratch (ticket counters + fp32 partial sums), so this entry point keeps that scratch in a
// fixed array inside the library image instead of taking a workspace argument.
//
// Cost and limits: the array is FP8W8A16_NOALLOC_SCRATCH_BYTES (768 KiB) and is resident on every
// GPU that loads the library, until the process exits.  Shapes whose scratch need exceeds it are
// rejected with FP8W8A16_ERR_WORKSPACE.  All calls on a device share the one array: two calls that
// overlap on the GPU (different streams, no ordering between them) race on it and give wrong
// results; calls on one stream, or otherwise ordered, are fine.
#include "common.cuh"

namespace w8a16 {

size_t gemv_workspace_bytes(int M, int N, int K);
int launch_gemv(const __half* x, const uint8_t* w, const void* scales, int scale_dtype, __half* out, int M, int N, int K,
                int block_h, int block_w, void* workspace, size_t workspace_bytes, cudaStream_t st);

namespace {

constexpr size_t kScratchBytes = FP8W8A16_NOALLOC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// Lives in the library's device image.  In HOST code this name is only a handle for the runtime's
// symbol table, never an address a kernel may be given: the device address comes from
// cudaGetSymbolAddress, once per device, with that device current.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

// Filled without a lock: two host threads that race on a device's first call both resolve and store the same
// address (the symbol has one address per device), so the race is benign.
void* g_scratch_ptr[kMaxDevices] = {};

// First call on a device: resolve the array's device address.  No allocation happens here, but
// cudaGetSymbolAddress may initialise the context / load the module, so the first call on a device
// should be made before any stream capture begins.
int scratch_for_current_device(void** out) {
    int dev = -1;
    W8A16_CUDA(cudaGetDevice(&dev));
    W8A16_REQUIRE(dev >= 0 && dev < kMaxDevices, FP8W8A16_ERR_UNSUPPORTED, "linear_noalloc: device index %d out of range", dev);
    if (g_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return fail(FP8W8A16_ERR_CUDA, "linear_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return 0;
}

}  // namespace
}  // namespace w8a16

using namespace w8a16;

extern "C" int fp8w8a16_linear_noalloc(const uint16_t* x, const uint8_t* w, const void* scales, int scale_dtype, uint16_t* out,
                                       int M, int N, int K, int block_h, int block_w, void* stream) {
    W8A16_REQUIRE(M >= 0 && N >= 0 && K >= 0, FP8W8A16_ERR_INVALID, "linear_noalloc: negative dimension M=%d N=%d K=%d", M, N, K);
    if (M == 0 || N == 0) return 0;
    W8A16_REQUIRE(x && w && scales && out, FP8W8A16_ERR_INVALID, "linear_noalloc: null pointer argument");
    W8A16_REQUIRE(block_w == 128 && block_h >= 1, FP8W8A16_ERR_UNSUPPORTED, "linear_noalloc: block %dx%d not supported", block_h, block_w);
    W8A16_REQUIRE(K > 0 && K % 16 == 0, FP8W8A16_ERR_UNSUPPORTED, "linear_noalloc: K must be a positive multiple of 16 (got %d)", K);
    W8A16_REQUIRE(scale_dtype == FP8W8A16_SCALE_F16 || scale_dtype == FP8W8A16_SCALE_F32, FP8W8A16_ERR_INVALID,
                  "linear_noalloc: unknown scale dtype %d", scale_dtype);
    const size_t need = gemv_workspace_bytes(M, N, K);
    W8A16_REQUIRE(need <= kScratchBytes, FP8W8A16_ERR_WORKSPACE,
                  "linear_noalloc: shape M=%d N=%d K=%d needs %zu bytes of scratch, the built-in array holds %zu; "
                  "use fp8w8a16_linear with a caller-provided workspace", M, N, K, need, kScratchBytes);
    void* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // The array keeps whatever the previous call (or an aborted one) left behind.  The partial sums are
    // fully overwritten before they are read; the ticket counters must start at zero, so clear them.
    W8A16_CUDA(cudaMemsetAsync(scratch, 0, kTicketBytes, st));
    rc = launch_gemv(reinterpret_cast<const __half*>(x), w, scales, scale_dtype, reinterpret_cast<__half*>(out), M, N, K,
                       block_h, block_w, scratch, kScratchBytes, st);
    if (rc == 0) count_variant(FP8W8A16_VARIANT_GEMV);
    return rc;
}
