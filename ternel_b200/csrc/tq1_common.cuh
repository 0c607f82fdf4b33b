// Shared constants and helpers for the TQ1_G128 kernels (sm_100a).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ternel_b200.h"

namespace tq1 {

constexpr int kGroup = TQ1_GROUP;             // weights per block
constexpr int kBlockBytes = TQ1_BLOCK_BYTES;  // bytes per block
constexpr int kBlockWords = kBlockBytes / 4;  // 7 x 32-bit words, always 4-byte aligned
constexpr int kCodeBytes = 26;
constexpr int kFullBytes = 25;
constexpr int kMaxFull = 242;
constexpr int kMaxTail = 26;

// Workspace layout shared by every linear kernel: [control words, 256 B][partial-sum slots of the
// batch-1 kernel, 16 MiB][scratch of the batched kernel, or the hand-off words of a chain]. Slots
// carry sequence tags, so nothing in the slot region ever has to be cleared; no other kernel writes
// there, so calls of any shape and kind can share one workspace. The workspace must be zero-filled
// once before its first use.
constexpr size_t kWsStatusBytes = 256;
constexpr size_t kWsSlotRegionBytes = (size_t)16 << 20;
constexpr size_t kWsScratchOffset = kWsStatusBytes + kWsSlotRegionBytes;

// Checked build (-DTQ1_BOUNDS_CHECK -rdc=true): every global store of a kernel (and the reads of scratch that
// other CTAs write) first tests its index against the extent the launcher knows. A violation is counted in
// g_tq1_bounds {count, code of the first, its index, its limit} and the access is SKIPPED: the kernel neither
// traps nor touches memory it does not own. The reference's analogue is the SAFE build of its Metal kernels,
// which clamps row indices (src/ternel_mlx/kernels.py:23-27). tq1_debug_bounds() reads the record.
// Codes: 1x chain kernel (10 slot store, 11 slot read, 12 y, 13 hand-off store, 14 hand-off read),
// 2x row kernel, 3x gather, 4x batched kernel (40 result, 41 partial tile), 5x panels, 6x shard push.
#ifdef TQ1_BOUNDS_CHECK
extern __device__ unsigned long long g_tq1_bounds[4];
__device__ __forceinline__ bool tq1_in_bounds(long long index, long long limit, unsigned code) {
    if (index >= 0 && index < limit) return true;
    if (atomicAdd(&g_tq1_bounds[0], 1ull) == 0ull) {
        g_tq1_bounds[1] = code;
        g_tq1_bounds[2] = (unsigned long long)index;
        g_tq1_bounds[3] = (unsigned long long)limit;
    }
    return false;
}
#define TQ1_IN_BOUNDS(index, limit, code) tq1_in_bounds((long long)(index), (long long)(limit), (code))
#else
#define TQ1_IN_BOUNDS(index, limit, code) true
#endif

// Records a message for tq1_last_error() and returns `code`.
int fail(int code, const char *fmt, ...);
int cuda_fail(cudaError_t err, const char *what);

// Launchers implemented one per .cu file; all enqueue on `stream` and return a status.
int launch_validate(const uint8_t *blocks, int64_t groups, int64_t *counts, cudaStream_t stream);
int launch_embedding(const uint8_t *blocks, const int64_t *ids, void *out, bool out_f32,
                     int64_t T, int64_t V, int K, cudaStream_t stream);
int launch_gemv_rows(const uint8_t *blocks, const __half *x, void *y, bool y_f32,
                     int M, int N, int K, cudaStream_t stream);

// Device-side description of an output-row shard whose result is pushed to every rank
// (tq1_linear_f16_sharded): peer pointers are plain device addresses reachable over NVLink.
// Flags are per row tile: word t of a gathered buffer's flag array guards rows [16t, 16t + 16) and is
// stored, with release semantics, by the thread that has just written those rows to that rank.
constexpr int kMaxRanks = 8;
constexpr int kFlagRows = 16;
struct ShardDev {
    int world;                          // <= 1: not sharded, every other field is ignored
    int rank;
    __half *peer_y[kMaxRanks];          // rank p's gathered output, already advanced to this shard's first row
    unsigned *peer_flags[kMaxRanks];    // rank p's tile flags of that output, advanced to this shard's first tile
    const unsigned *epoch_base;         // optional device word added to both epochs (graph replays advance it)
    unsigned publish_epoch;             // value stored to a tile's flag once the tile has been written
    const unsigned *wait_flags;         // local tile flags of the activations this call reads (or null)
    int wait_tiles;                     // how many of them exist
    unsigned wait_epoch;
    int ld_total;                       // row length of the gathered output (elements)
    int swiglu;                         // unsharded only: rows are (gate, up) pairs, y[i] = silu(gate_i) * up_i
};

// Batch-1 GEMV as a persistent chain of links (TMA + integer tensor cores); needs K % 512 == 0, at most
// 128 K chunks and 16-byte aligned blocks. A single product is a chain of one link.
bool gemv_chain_shape_ok(int N, int K);
bool gemv_chain_supported(const uint8_t *blocks, int N, int K);
bool gemv_chain_fits(const uint8_t *blocks, int N, int K);      // also checks the current device's SM count
size_t gemv_chain_workspace_bytes(int N, int K);
// M = 2 .. gemv_loop_tokens() activation rows as M links of one launch over the same weights
bool gemv_looped_fits(const uint8_t *blocks, int M, int N, int K);
int launch_gemv_looped(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int M, int N, int K, bool swiglu,
                       void *workspace, cudaStream_t stream);
int gemv_loop_tokens();
int gemv_set_loop_tokens(int tokens);       // sweep recording only; process-global
// slot_bytes: room for partial-sum slots behind the workspace's control words
int launch_gemv_single(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int N, int K, bool swiglu,
                       void *workspace, size_t slot_bytes, cudaStream_t stream);
int launch_shard_wait(const ShardDev &shard, unsigned *status, cudaStream_t stream);
int launch_shard_push(const __half *local, int M, int n_local, const ShardDev &shard, cudaStream_t stream);
int launch_epoch_advance(unsigned *epoch_base, unsigned delta, cudaStream_t stream);

int gemv_noalloc(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int N, int K, cudaStream_t stream);
int gemv_noalloc_status(unsigned *out_host, cudaStream_t stream);

// Batched linear (M >= 2) on tcgen05 tensor cores; needs K % 512 == 0 and 16-byte aligned pointers.
bool gemm_tc_shape_ok(int M, int N, int K);
bool gemm_tc_supported(const uint8_t *blocks, const __half *x, int M, int N, int K);
size_t gemm_tc_workspace_bytes(int M, int N, int K);
int launch_gemm_tc(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int M, int N, int K,
                   void *workspace, cudaStream_t stream, bool swiglu = false);

// silu(gate) * up in FP32, the activation of a gated feed-forward block
__host__ __device__ inline float swiglu_f32(float gate, float up) { return gate / (1.0f + expf(-gate)) * up; }
void gemm_tc_plan(int M, int N, int K, int *tile, int *ctas, int *parts);
int gemm_tc_force_tile(int nt);

// Five base-3 digits of a byte packed two bits each (digit i at bits 2i..2i+1).
__host__ __device__ inline uint32_t trits_2bit(uint32_t byte) {
    uint32_t e = 0;
    for (int i = 0; i < 5; ++i) {
        e |= (byte % 3u) << (2 * i);
        byte /= 3u;
    }
    return e;
}

}  // namespace tq1
