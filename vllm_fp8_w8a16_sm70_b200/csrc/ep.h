// Geometry of the expert-parallel exchange buffer (see ep.cu) and the kernel launchers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace w8a16 {

constexpr int kEpMaxWorld = 8;

// Every rank allocates the same layout; base[r] is rank r's buffer as seen from this rank (base[rank] is local).
//   ctrl    4 words: finished calls, and the CTAs-done counters of the send / return / combine kernels
//   hdr     [world] {count, call}: written by source s into slot s
//   rflag   [world] {0, call}:     written by expert owner q into slot q
//   meta_e / meta_j / meta_w  [world * cap]: local expert id, route index at the source, route weight of every inbox row
//   rows    [world * cap][H] FP16: inbox of dispatched rows (a call with at most cap_call rows per source packs them as
//           [world][cap_call])
//   ret     [cap][H] FP16: finished rows coming back, at the row of their route index
struct EpGeom {
    int world, rank;
    int H;
    int cap;                  // max_tokens * topk: rows one source may send to one destination, and routes of one source
    int experts_per_rank;
    unsigned int timeout_ms;
    int64_t off_ctrl, off_hdr, off_rflag, off_meta_e, off_meta_j, off_meta_w, off_rows, off_ret;
    char* base[kEpMaxWorld];
};

int launch_ep_send(const __half* x, const void* topk_ids, int ids_are_i64, const float* topk_w, const int* sorted_route,
                   const int* dest_offsets, int R, int topk, int cap_call, const EpGeom& g, cudaStream_t st);
// small batches: route table by destination, stores and headers in one launch (replaces the align kernel + launch_ep_send)
int launch_ep_send_small(const __half* x, const void* topk_ids, int ids_are_i64, const float* topk_w, const int* dest_map, int n_global,
                         int* counts, int* offsets, int* tile_offsets, int* sorted_route, int* inv_pos, int R, int topk, int cap_call,
                         const EpGeom& g, cudaStream_t st);
// header wait + route table of the received rows by local expert (+ the gather into expert order when fuse_gather is set)
int launch_ep_recv_align(int cap_call, int* counts_in, int E, int bt, int* counts, int* offsets, int* tile_offsets, int* sorted_route,
                         int* inv_pos, int fuse_gather, __half* x_sorted, float* w_sorted, const EpGeom& g, cudaStream_t st);
int launch_ep_return(const __half* y_sorted, const int* inv_pos, const int* counts_in, int cap_call, const EpGeom& g, cudaStream_t st);
int launch_ep_combine(const void* topk_ids, int ids_are_i64, int M, int topk, __half* out, const EpGeom& g, cudaStream_t st);
int ep_read_status(int* out, int reset);

}  // namespace w8a16
