// Launch parameters of the tcgen05 W8A16 GEMM (see gemm_tc.cu).
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace w8a16 {

struct TcParams {
    int M;                       // rows of the activation matrix (dense: tokens; grouped: all sorted rows)
    int N;                       // output features (paired gate/up mode: the intermediate size I)
    int K;
    // weights: [num_experts * w_rows_per_expert, K] E4M3 bytes, row-major
    int w_rows_per_expert;       // N, or 2 * I in paired mode
    int pair_offset;             // I in paired mode (up rows follow gate rows), else 0
    // scale grid per expert: [ceil(rows / block_h), Kb], fp16 or fp32
    const void* scales;
    int scale_dtype;
    int block_h;
    int Kb;
    int64_t scale_expert_stride; // elements between experts in the scale grid
    // grouped mode (null pointers = dense)
    const int* expert_offsets;   // [E + 1] first sorted row of each expert
    const int* tile_offsets;     // [E + 1] first token tile of each expert (prefix sum of ceil(count / BT))
    int num_experts;
    // output
    __half* out;                 // out[row * ldo + n]
    int64_t ldo;
    const float* row_weight;     // optional per-row multiplier (route weight), applied as FP16
    const __half* residual;      // optional (dense): FP16 [M, ldo] added to the fp32 result before the one rounding
    int activation;              // paired mode: 1 = SiLU(gate) * up, 2 = GELU(gate) * up (erf form)
    // persistent stream-K work split
    int n_token_tiles;           // dense: ceil(M / BT); grouped: read from tile_offsets[E] on the device
    int no_split;                // 1: every CTA takes whole tiles only (no partial tiles, no tickets)
    int cluster_size;            // > 1: synchronous split-K — the CTAs of a thread-block cluster share one output tile,
                                 //      each takes a K range, and they reduce through distributed shared memory
    float* partial;              // fp32 scratch: [gridDim.x][2][(1|2)][BT][128]
    unsigned int* tickets;       // one counter per output tile, zero on entry and on exit
};

// Fused all-reduce of a row-parallel GEMM over peer memory (one process per GPU, buffers mapped through CUDA IPC).
// Every rank runs the same launch.  The CTA that finishes a region of an output tile pushes its FP16 values into every
// peer's inbox as 8-byte packets {two FP16 values, launch epoch} (posted NVLink stores; the epoch in every packet is
// the arrival flag, so no fence and no separate flag is needed), then polls its OWN inbox for the peers' packets of
// the same region and adds all contributions in ascending rank order: the result is identical on every rank, and the
// exchange of early tiles overlaps the math of later ones.
constexpr int kArMaxWorld = 8;
struct ArParams {
    int world;                        // 0 = not fused
    int rank;
    unsigned int timeout_ms;          // bound of the wait for a peer's packets
    unsigned int* ctrl;               // local: [0] = number of finished fused launches (epoch), [1] = CTAs done in this launch
    __half* part;                     // local FP16 staging of this rank's own result [part_elems]
    uint2* inbox[kArMaxWorld];        // inbox[r]: rank r's inbox [2 parities][world sources][part_elems / 2] packets
    int64_t part_elems;
    __half* out;                      // reduced output [M, N] (local)
};

struct TcLaunch {
    TcParams p;
    ArParams ar;
    const uint8_t* w;
    const __half* x;
    int64_t w_total_rows;        // num_experts * w_rows_per_expert
    int64_t max_units;           // upper bound on (output tiles x K blocks): caps the grid
    int64_t cluster_tiles;       // cluster split-K: number of clusters (= output tiles, or their upper bound)
};

int tc_pick_bt(int rows);
int tc_block_k(int bt, bool paired);
int tc_ctas_per_sm(int bt, bool paired);
// CTAs the persistent launch uses on the current device, and the scratch it needs (ticket header included).
int tc_grid(int bt, bool paired);
size_t tc_workspace_bytes(int bt, bool paired);
size_t tc_max_tiles_with_tickets();
int tc_cluster_size(int64_t tiles, int total_kb, int bt, bool paired);
int tc_launch(const TcLaunch& L, int bt, bool paired, cudaStream_t st);
int tc_read_status(int* out, int reset);
// 2-D row-major tensor map [rows, cols], box [box_rows, box_cols]; cached per (address, shape, box)
int tc_encode_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows, uint64_t cols,
                 uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz, bool is_weight);
// CTA-pair kernel for dense batches above 128 tokens (gemm_tc2.cu)
bool tc2_enabled();
int tc2_launch(const TcLaunch& L, cudaStream_t st);
int tc2_read_status(int* out, int reset);

}  // namespace w8a16
