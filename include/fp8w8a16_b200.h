/* C ABI of the B200 (sm_100a) block-scaled FP8 W8A16 linear / MoE engine.
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer unless it says "host"; `stream`
 * is a cudaStream_t passed as void* (NULL = the legacy default stream; callers inside PyTorch pass
 * torch.cuda.current_stream().cuda_stream — the reference launches on the current torch stream,
 * src/fp8_w8a16_sm70/fp8_dequant.cu:29-36, and so must every caller of this library).
 * Every function returns 0 or a negative FP8W8A16_ERR_* code; fp8w8a16_last_error() gives the
 * message of the calling thread's last failure (the reference raises through TORCH_CHECK,
 * fp8_dequant.cu:1518-1537; the Python binding turns a non-zero code into RuntimeError).
 * No function allocates device memory or synchronises with the host unless it says so.
 *
 * Layouts (the reference's; see the signatures at fp8_dequant.cu:1616-1622):
 *   x       FP16 [M, K] row-major          w   uint8 (raw E4M3-FN) [N, K] row-major, or [E, N, K]
 *   scales  [ceil(N/block_h), ceil(K/128)] (or [E, ., .]), FP16 or fp32 (rounded to FP16 on use),
 *           block_h = 128 (block scales) or 1 (per-output-channel "fake block" grid)
 *   out     FP16 [M, N] row-major, fp32 accumulation
 */
#ifndef FP8W8A16_B200_H_
#define FP8W8A16_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FP8W8A16_OK 0
#define FP8W8A16_ERR_INVALID (-1)     /* bad argument: null pointer, negative size, misalignment */
#define FP8W8A16_ERR_CUDA (-2)        /* a CUDA runtime / driver call failed */
#define FP8W8A16_ERR_UNSUPPORTED (-3) /* shape or block size outside what the kernels cover */
#define FP8W8A16_ERR_WORKSPACE (-4)   /* workspace missing or too small */
#define FP8W8A16_ERR_DEVICE (-5)      /* a kernel reported a timed-out wait in the device status word */

#define FP8W8A16_SCALE_F16 0
#define FP8W8A16_SCALE_F32 1

#define FP8W8A16_DTYPE_F32 0
#define FP8W8A16_DTYPE_F16 1
#define FP8W8A16_DTYPE_BF16 2

/* gated activation of the MoE gate/up projection (reference: _moe_activation, vllm_serve.py:1627-1636) */
#define FP8W8A16_ACT_SILU 1
#define FP8W8A16_ACT_GELU 2 /* erf form, torch.nn.functional.gelu's default */

/* fp8w8a16_linear `algo` */
#define FP8W8A16_ALGO_AUTO 0 /* by M, as the reference's _v100_fp8_gemm dispatch does (vllm_serve.py:1032-1100) */
#define FP8W8A16_ALGO_GEMV 1 /* CUDA-core split-K GEMV, any M (weights re-streamed per 4 tokens) */
#define FP8W8A16_ALGO_TC 2   /* tcgen05 tensor-core GEMM with in-SM dequant */

int fp8w8a16_version(void);
const char* fp8w8a16_last_error(void);

/* Number of kernels this library has launched in this process (a host-side counter; used by the
 * benchmark to report how many of its own kernels ran inside a timed region). */
uint64_t fp8w8a16_launch_count(void);

/* How the calls of this process were served, by kernel variant: the observability counterpart of the reference's
 * per-variant call counters (vllm_serve.py:1403-1429).  counts receives min(n, FP8W8A16_NUM_VARIANTS) host-side
 * counters, indexed by the FP8W8A16_VARIANT_* values; returns FP8W8A16_NUM_VARIANTS. */
#define FP8W8A16_VARIANT_GEMV 0            /* CUDA-core split-K GEMV (noalloc form included) */
#define FP8W8A16_VARIANT_TC_CLUSTER 1      /* tcgen05 GEMM, cluster split-K */
#define FP8W8A16_VARIANT_TC_STREAMK 2      /* tcgen05 GEMM, stream-K with ticketed fix-up */
#define FP8W8A16_VARIANT_TC_TILES 3        /* tcgen05 GEMM, whole tiles (prefill) */
#define FP8W8A16_VARIANT_GROUPED 4         /* grouped (MoE) GEMM, w2-style */
#define FP8W8A16_VARIANT_GROUPED_PAIRED 5  /* grouped gate/up GEMM with fused activation */
#define FP8W8A16_VARIANT_FUSED_ALLREDUCE 6 /* row-parallel GEMM with the all-reduce inside (also counted under its TC mode) */
#define FP8W8A16_VARIANT_DEQUANT 7         /* standalone dequant ops */
#define FP8W8A16_NUM_VARIANTS 8
int fp8w8a16_variant_counts(uint64_t* counts, int n);

/* Sticky device status word (bit set = a bounded wait inside a kernel gave up).  Synchronises the
 * device.  *status (host) receives the bits; reset != 0 clears them. */
int fp8w8a16_device_status(int* status, int reset);

/* out[i] = cvt(w[i]).  Replaces fp8_e4m3_to_fp16 (fp8_dequant.cu:129-148). */
int fp8w8a16_e4m3_to_fp16(const uint8_t* w, uint16_t* out, int64_t n, void* stream);

/* out[i] = cvt(w[i]) * scales_f16[i / group_size].  Replaces fp8_e4m3_to_fp16_scaled (fp8_dequant.cu:150-199). */
int fp8w8a16_e4m3_to_fp16_scaled(const uint8_t* w, const uint16_t* scales_f16, uint16_t* out, int64_t n,
                                 int64_t group_size, void* stream);

/* out[i,j] = RN16(cvt(w[i,j]) * S16[i/block_h, j/block_w]): the bit-exact dequantised weight.
 * Replaces fp8_e4m3_to_fp16_block_scaled (fp8_dequant.cu:3053-3087). */
int fp8w8a16_dequant_block_scaled(const uint8_t* w, const void* scales, int scale_dtype, uint16_t* out, int N, int K,
                                  int block_h, int block_w, void* stream);

/* Bytes of workspace fp8w8a16_linear may use for this shape (always >= 64 KiB: the first 64 KiB
 * hold hand-off counters that must be ZERO before the first call and are left at zero by every
 * call; the rest needs no initialisation).  One workspace serves one stream at a time. */
size_t fp8w8a16_linear_workspace_bytes(int M, int N, int K);

/* out[M,N] = x[M,K] @ dequant(w[N,K], scales)^T.  One entry point for the reference's whole dense
 * family — gemv_coalesced / gemv_coalesced_m / gemm_a1 / a2 / a3 / gemm_wmma_poc
 * (fp8_dequant.cu:2769, 1616, 2969, 2925, 2717, 2114) — and for the host dispatch that picks among
 * them (vllm_serve.py:1032-1100).  block_w must be 128, block_h 128 or 1, K a multiple of 16. */
int fp8w8a16_linear(const uint16_t* x, const uint8_t* w, const void* scales, int scale_dtype, uint16_t* out, int M,
                    int N, int K, int block_h, int block_w, int algo, void* workspace, size_t workspace_bytes,
                    void* stream);

/* Same result as fp8w8a16_linear with FP8W8A16_ALGO_GEMV, for callers that cannot allocate device
 * memory and so cannot provide a workspace (a worker whose memory was all handed out at start-up,
 * code under a no-allocation policy, a plugin that only ever receives input and output buffers).  It has no
 * counterpart in the reference, whose ops allocate inside every call.  The scratch the split-K GEMV
 * needs lives in a fixed array of FP8W8A16_NOALLOC_SCRATCH_BYTES inside the library image, resident
 * on every GPU that loads the library until the process exits; the call itself allocates nothing.
 * Shapes that need more scratch are rejected with FP8W8A16_ERR_WORKSPACE (use fp8w8a16_linear).
 * The first call on a device looks the array's address up (cudaGetSymbolAddress) and should be made
 * before any stream capture starts.  All calls on a device share the array: calls that overlap on the
 * GPU race on it; calls ordered on one stream (or by events) are safe. */
#define FP8W8A16_NOALLOC_SCRATCH_BYTES (768u << 10)
int fp8w8a16_linear_noalloc(const uint16_t* x, const uint8_t* w, const void* scales, int scale_dtype, uint16_t* out,
                            int M, int N, int K, int block_h, int block_w, void* stream);

/* Row-parallel linear with the tensor-parallel all-reduce fused into the GEMM kernel, over peer memory
 * (NVLink).  Replaces the pair the reference's call site runs per row-parallel layer - apply() on the rank's K
 * shard, then vLLM's tensor_model_parallel_all_reduce of the FP16 [M,N] result (vllm_serve.py:2922-2959) - with one
 * launch per rank: the CTA that finishes a piece of an output tile stores its FP16 values, tagged with the launch
 * number, straight into every peer's inbox, polls (bounded) its own inbox for the peers' values of the same piece
 * and adds all contributions in ascending rank order, so out is bit-identical on all ranks and the exchange of
 * early tiles overlaps the math of later ones.
 *
 * A communicator is one device allocation per rank (cudaMalloc at create time; nothing is allocated per call),
 * mapped into the peers through CUDA IPC: create on every rank, exchange the FP8W8A16_COMM_HANDLE_BYTES handles by
 * any host channel, attach every peer, then make the SAME sequence of fp8w8a16_linear_allreduce calls on all ranks
 * (one process per GPU).  fp8w8a16_comm_attach_ptr takes a peer mapping made by other means (cuMem / fabric
 * handles, symmetric-memory allocators) whose layout is another rank's fp8w8a16_comm_base .. + fp8w8a16_comm_bytes.
 * max_out_elems bounds M*N of a call (the buffer takes about (10 * world + 2) bytes per element); timeout_ms
 * (0 = 2000) bounds every wait for a peer: when it runs out the kernel gives up, out is not written for the
 * affected tiles and fp8w8a16_device_status reports bit 128.  N must be a multiple of 4.
 * Calls are CUDA-graph capturable (launches are counted on the device).
 *
 * The launch number lives on each rank's device and advances by one per fused launch; the ranks only agree while
 * they make the same launches.  After a one-sided launch (one rank raised before launching, or a wait ran out and
 * status bit 128 was reported) every later fused call would mismatch.  fp8w8a16_comm_reset puts a rank back to
 * launch number zero with an empty inbox (two device memsets enqueued on `stream`); it is a COLLECTIVE in the host's
 * hands: every rank must call it, none may have a fused launch in flight on any rank while the memsets run (device
 * synchronise + host barrier before), and none may launch again before all have finished (synchronise + barrier
 * after).  The reference has no counterpart: its all-reduce is vLLM's. */
#define FP8W8A16_COMM_HANDLE_BYTES 64
typedef struct fp8w8a16_comm fp8w8a16_comm;
int fp8w8a16_comm_create(int rank, int world, int64_t max_out_elems, unsigned int timeout_ms, fp8w8a16_comm** comm);
int fp8w8a16_comm_export(const fp8w8a16_comm* comm, void* handle);
int fp8w8a16_comm_attach(fp8w8a16_comm* comm, int peer, const void* handle);
int fp8w8a16_comm_attach_ptr(fp8w8a16_comm* comm, int peer, void* peer_base);
void* fp8w8a16_comm_base(const fp8w8a16_comm* comm);
size_t fp8w8a16_comm_bytes(const fp8w8a16_comm* comm);
int fp8w8a16_comm_reset(fp8w8a16_comm* comm, void* stream);
int fp8w8a16_comm_destroy(fp8w8a16_comm* comm);
int fp8w8a16_linear_allreduce(fp8w8a16_comm* comm, const uint16_t* x, const uint8_t* w, const void* scales,
                              int scale_dtype, uint16_t* out, int M, int N, int K, int block_h, int block_w,
                              void* workspace, size_t workspace_bytes, void* stream);

/* The two steps that follow a row-parallel projection (o_proj, down_proj) in a decoder layer, which in the reference's
 * deployment are vLLM's: the residual add and the RMSNorm of fused_add_rms_norm, run after apply() and the tensor-parallel
 * reduce (call site mirrored at vllm_serve.py:2922-2959).
 *   fp8w8a16_linear_residual / fp8w8a16_linear_allreduce_residual: as fp8w8a16_linear (tensor-core path, any M) and
 *     fp8w8a16_linear_allreduce with out = FP16(fp32 result + residual): the residual stream (FP16 [M,N]) joins in the
 *     GEMM's epilogue - in the fused form after the cross-rank sum - before the one rounding.  out may alias residual.
 *     A NULL residual in the all-reduce form gives fp8w8a16_linear_allreduce.
 *   fp8w8a16_add_rmsnorm: z = x + residual (fp32 sum, one FP16 rounding; residual may be NULL when it was already added
 *     in the epilogue above: z = x), residual_out = z (may alias residual or x; may be NULL when residual is NULL),
 *     out = FP16(z * rsqrt(mean(z^2) + eps)) * weight with weight FP16 [N] (vLLM's kernel order: the norm of the rounded z,
 *     FP16 product).  One CTA per row, N a multiple of 8, at most 32768. */
int fp8w8a16_linear_residual(const uint16_t* x, const uint8_t* w, const void* scales, int scale_dtype, const uint16_t* residual,
                             uint16_t* out, int M, int N, int K, int block_h, int block_w, void* workspace,
                             size_t workspace_bytes, void* stream);
int fp8w8a16_linear_allreduce_residual(fp8w8a16_comm* comm, const uint16_t* x, const uint8_t* w, const void* scales,
                                       int scale_dtype, const uint16_t* residual, uint16_t* out, int M, int N, int K,
                                       int block_h, int block_w, void* workspace, size_t workspace_bytes, void* stream);
int fp8w8a16_add_rmsnorm(const uint16_t* x, const uint16_t* residual, const uint16_t* weight, float eps, uint16_t* out,
                         uint16_t* residual_out, int M, int N, void* stream);

/* Router: logits [M,E] -> topk_ids int32 [M,topk] (descending, ties to the lowest expert id),
 * topk_weights fp32 [M,topk] = softmax probabilities of the picks (renormalize != 0: divided by
 * their sum).  Stands in for vLLM's fused_topk, whose output the reference's MoE apply consumes
 * (vllm_serve.py:2175). */
int fp8w8a16_moe_topk_softmax(const void* logits, int logits_dtype, int M, int E, int topk, int renormalize,
                              int32_t* topk_ids, float* topk_weights, void* stream);

/* Router gate and selection in one kernel: logits[m,e] = sum_h x[m,h] * gate_weight[e,h] in fp32 (x FP16 [M,H],
 * gate_weight [E,H] in FP8W8A16_DTYPE_F16 / _BF16 / _F32, as the model keeps its unquantised router), followed by the
 * selection of fp8w8a16_moe_topk_softmax on those logits.  The step before the reference's MoE apply: vLLM runs the
 * gate Linear and fused_topk, the hook only receives their result (vllm_serve.py:2175, 2799-2812).  The routed
 * weights are multiplied by routed_scale (1 = leave them).  shared_expert_id >= 0 appends one fixed route per token,
 * (shared_expert_id, weight 1), so that a shared expert stored as one more row of the expert stack is computed by the
 * same grouped GEMMs and "routed + shared" (vllm_serve.py:2832-2846) costs no extra pass; the output rows then hold
 * topk + 1 entries.  logits (fp32 [M,E]) may be null.  One CTA per token: meant for decode batches; E <= 512, H a
 * multiple of 8. */
int fp8w8a16_moe_router_topk(const uint16_t* x, const void* gate_weight, int gate_dtype, int M, int E, int H, int topk,
                             int renormalize, int shared_expert_id, float routed_scale, int32_t* topk_ids,
                             float* topk_weights, float* logits, void* stream);

/* Route table, built on the device without host synchronisation.  topk_ids: R routed slots, int32
 * or int64 (ids_are_i64).  expert_map: optional int32 [n_global_experts] global -> local id, -1 =
 * not on this rank (vllm_serve.py:2237-2243); ids < 0 or unmapped are dropped (they contribute
 * zero).  Outputs: counts [E], offsets [E+1] (first sorted row per expert), tile_offsets [E+1]
 * (prefix sum of ceil(count / token_tile)), sorted_route [R] (route index per sorted row, stable,
 * -1 past the valid rows), inv_pos [R] (sorted row per route, -1 = dropped).
 * Replaces the argsort / scatter_add / cumsum table of compressed_tensors_v100.py:776-784. */
int fp8w8a16_moe_align(const void* topk_ids, int ids_are_i64, int R, const int32_t* expert_map, int n_global_experts,
                       int num_local_experts, int token_tile, int32_t* counts, int32_t* offsets, int32_t* tile_offsets,
                       int32_t* sorted_route, int32_t* inv_pos, void* stream);

/* Token tile (16..128) the grouped GEMM uses for R routed rows over E experts. */
int fp8w8a16_moe_token_tile(int R, int num_local_experts);

/* Grouped expert GEMM over expert-sorted rows:
 *   paired == 0: out[r, n] = (x_sorted[r] . dequant(w[e(r), n])) * row_weight[r]      (row_weight may be NULL)
 *   paired != 0: w is a fused [E, 2N, K] gate/up weight; out[r, n] = act(gate) * up with act = SiLU (paired = 1,
 *                FP8W8A16_ACT_SILU) or GELU (paired = 2, FP8W8A16_ACT_GELU); FP16 rounding points as the reference
 * offsets / tile_offsets come from fp8w8a16_moe_align with the same token_tile.
 * Replaces fp8_w8a16_grouped_gemv_coalesced / grouped_routed_gemm_a3 / grouped_tiled_gemm
 * (fp8_dequant.cu:1512, 2813, 3166) and TurboMind's fp8_moe_gemm_sm70_out
 * (third_party/turbomind_gemm_sm70/binding/awq_sm70_gemm.cu:2327-2474). */
int fp8w8a16_moe_grouped_gemm(const uint16_t* x_sorted, const uint8_t* w, const void* scales, int scale_dtype,
                              uint16_t* out, const float* row_weight, const int32_t* offsets,
                              const int32_t* tile_offsets, int R, int num_local_experts, int N, int K, int block_h,
                              int paired, int token_tile, void* workspace, size_t workspace_bytes, void* stream);
size_t fp8w8a16_moe_grouped_gemm_workspace_bytes(int R, int num_local_experts, int N, int K, int paired,
                                                 int token_tile);

/* Whole routed MoE layer (routed-only output, as the reference's apply returns, vllm_serve.py:2175-2411):
 *   out[m] = sum_j w[m,j] * down_e( silu(gate_e x[m]) * up_e x[m] ),  e = topk_ids[m,j]
 * x FP16 [M,H]; topk_weights fp32 [M,topk]; w13 [E,2I,H], w2 [E,H,I] E4M3; scales as above with
 * block_h 128 or 1.  weight_on_input: multiply x by the route weight instead of the output
 * (apply_router_weight_on_input, vllm_serve.py:1868); activation: FP8W8A16_ACT_SILU or FP8W8A16_ACT_GELU.  Steps: align -> gather -> grouped w13 with
 * fused SiLU*mul -> grouped w2 with fused route weight -> combine; no host synchronisation. */
int fp8w8a16_moe_forward(const uint16_t* x, const void* topk_ids, int ids_are_i64, const float* topk_weights,
                         const int32_t* expert_map, int n_global_experts, const uint8_t* w13, const void* s13,
                         const uint8_t* w2, const void* s2, int scale_dtype, uint16_t* out, int M, int topk,
                         int num_local_experts, int H, int I, int block_h, int weight_on_input, int activation,
                         void* workspace, size_t workspace_bytes, void* stream);
size_t fp8w8a16_moe_workspace_bytes(int M, int topk, int num_local_experts, int H, int I);

/* Pieces of the layer, exported so each can be checked on its own. */
int fp8w8a16_moe_gather(const uint16_t* x, const int32_t* sorted_route, const float* topk_weights, int R, int topk,
                        int H, int weight_on_input, uint16_t* x_sorted, float* w_sorted, void* stream);
int fp8w8a16_moe_combine(const uint16_t* y_sorted, const int32_t* inv_pos, int M, int topk, int H, uint16_t* out,
                         void* stream);

/* Expert-parallel MoE layer with the token exchange done by this library's own kernels over peer memory (NVLink):
 * the experts are partitioned contiguously over the ranks (rank r owns experts [r * E/P, (r + 1) * E/P)), every rank
 * brings its own tokens.  The reference only tolerates expert parallelism - every rank sees every token, foreign routes
 * are dropped through expert_map and vLLM reduces afterwards (vllm_serve.py:2237-2243); this is the dispatch / combine
 * form of the same layer, and its definition of correct is the single-GPU fp8w8a16_moe_forward.
 *
 * A handle owns one device allocation per rank (cudaMalloc at create time; calls allocate nothing), mapped into the
 * peers exactly like a fp8w8a16_comm (export / attach / attach_ptr).  One call = three steps on the caller's stream:
 *   fp8w8a16_ep_dispatch  route table by destination rank, then every routed row is stored into its owner's inbox with
 *                         its local expert id, source route index and route weight, followed by a {count, call number}
 *                         header per destination
 *   fp8w8a16_ep_experts   bounded wait for every source's header, then align -> gather -> grouped gate/up GEMM with the
 *                         activation -> grouped down GEMM x route weight on the received rows, then every finished row
 *                         is stored into its source's return buffer, followed by a flag per source
 *   fp8w8a16_ep_combine   bounded wait for every owner's flag, then out[m] = sum of the token's routes, in route
 *                         order, fp32, one rounding (as fp8w8a16_moe_combine)
 * fp8w8a16_ep_moe_forward runs the three in order.  No host synchronisation, no NCCL: CUDA-graph capturable.
 * Every rank must make the same sequence of calls.  M may differ between ranks; M_max is the largest M of the call
 * over all ranks and MUST be passed identically by all of them (it fixes where each source's rows sit in the inbox);
 * M_max <= max_tokens of fp8w8a16_ep_create.  A wait that runs out (timeout_ms, 0 = 2000) is reported by
 * fp8w8a16_device_status (bit 256: a header, bit 512: a return flag): the missing source contributes nothing, or
 * the affected tokens come out as zeros; afterwards every rank must call fp8w8a16_ep_reset (a collective in the
 * host's hands, like fp8w8a16_comm_reset) before the next call.  The workspace is the caller's, at least
 * fp8w8a16_ep_workspace_bytes, its first 64 KiB zero on first use (the grouped GEMMs' counters). */
typedef struct fp8w8a16_ep fp8w8a16_ep;
int fp8w8a16_ep_create(int rank, int world, int max_tokens, int topk, int hidden, int n_global_experts,
                       unsigned int timeout_ms, fp8w8a16_ep** ep);
int fp8w8a16_ep_export(const fp8w8a16_ep* ep, void* handle);
int fp8w8a16_ep_attach(fp8w8a16_ep* ep, int peer, const void* handle);
int fp8w8a16_ep_attach_ptr(fp8w8a16_ep* ep, int peer, void* peer_base);
void* fp8w8a16_ep_base(const fp8w8a16_ep* ep);
size_t fp8w8a16_ep_bytes(const fp8w8a16_ep* ep);
int fp8w8a16_ep_reset(fp8w8a16_ep* ep, void* stream);
int fp8w8a16_ep_destroy(fp8w8a16_ep* ep);
size_t fp8w8a16_ep_workspace_bytes(const fp8w8a16_ep* ep, int M, int M_max, int num_local_experts, int I);
int fp8w8a16_ep_dispatch(fp8w8a16_ep* ep, const uint16_t* x, const void* topk_ids, int ids_are_i64,
                         const float* topk_weights, int M, int M_max, int num_local_experts, int I, void* workspace,
                         size_t workspace_bytes, void* stream);
int fp8w8a16_ep_experts(fp8w8a16_ep* ep, const uint8_t* w13, const void* s13, const uint8_t* w2, const void* s2,
                        int scale_dtype, int M, int M_max, int num_local_experts, int I, int block_h, int activation,
                        void* workspace, size_t workspace_bytes, void* stream);
int fp8w8a16_ep_combine(fp8w8a16_ep* ep, const void* topk_ids, int ids_are_i64, uint16_t* out, int M, void* stream);
int fp8w8a16_ep_moe_forward(fp8w8a16_ep* ep, const uint16_t* x, const void* topk_ids, int ids_are_i64,
                            const float* topk_weights, const uint8_t* w13, const void* s13, const uint8_t* w2,
                            const void* s2, int scale_dtype, uint16_t* out, int M, int M_max, int num_local_experts,
                            int I, int block_h, int activation, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FP8W8A16_B200_H_ */
