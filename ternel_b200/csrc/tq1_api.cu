// C-ABI entry points of the linear and embedding path: argument checks and
// kernel selection. Checks mirror the reference wrappers' (_check_packed /
// _check_activations, src/ternel_mlx/kernels.py:1191-1212,1274-1284): shape and
// dtype violations are reported before anything is launched.
#include "tq1_common.cuh"

using namespace tq1;

extern "C" {

size_t tq1_linear_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || K % kGroup) return 0;
    if (M == 1 && gemv_chain_shape_ok(N, K)) return gemv_chain_workspace_bytes(N, K);
    if (gemm_tc_shape_ok(M, N, K)) return gemm_tc_workspace_bytes(M, N, K);
    return 0;
}

int tq1_linear_f16(const uint8_t *blocks, const void *x, void *y, int y_is_f32,
                   int M, int N, int K, void *workspace, size_t workspace_bytes, void *stream) {
    if (!blocks || !x || !y) return fail(TQ1_ERR_INVALID, "tq1_linear_f16: null pointer");
    if (M <= 0) return fail(TQ1_ERR_INVALID, "activations have an empty batch dimension");
    if (N <= 0 || K <= 0)
        return fail(TQ1_ERR_INVALID, "tensor dimensions must be positive, got %dx%d", N, K);
    if (K % kGroup)
        return fail(TQ1_ERR_INVALID, "%d columns is not a multiple of the 128-weight group", K);
    if (reinterpret_cast<uintptr_t>(blocks) & 3)
        return fail(TQ1_ERR_INVALID, "tq1_linear_f16: blocks must be 4-byte aligned");
    if (reinterpret_cast<uintptr_t>(x) & 15)
        return fail(TQ1_ERR_INVALID, "tq1_linear_f16: x must be 16-byte aligned");
    const size_t need = tq1_linear_workspace_bytes(M, N, K);
    if (need && (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255)))
        return fail(TQ1_ERR_WORKSPACE, "tq1_linear_f16: workspace of %zu bytes (256-byte aligned) required", need);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (M == 1 && gemv_chain_fits(blocks, N, K))
        return launch_gemv_single(blocks, static_cast<const __half *>(x), y, y_is_f32 != 0, N, K, false, workspace,
                                  kWsSlotRegionBytes, s);
    if (gemv_looped_fits(blocks, M, N, K) && need >= kWsScratchOffset)
        return launch_gemv_looped(blocks, static_cast<const __half *>(x), y, y_is_f32 != 0, M, N, K, false, workspace, s);
    if (gemm_tc_supported(blocks, static_cast<const __half *>(x), M, N, K))
        return launch_gemm_tc(blocks, static_cast<const __half *>(x), y, y_is_f32 != 0, M, N, K, workspace, s);
    return launch_gemv_rows(blocks, static_cast<const __half *>(x), y, y_is_f32 != 0, M, N, K, s);
}

int tq1_linear_swiglu_f16(const uint8_t *blocks, const void *x, void *y, int y_is_f32, int M, int N, int K,
                          void *workspace, size_t workspace_bytes, void *stream) {
    if (!blocks || !x || !y) return fail(TQ1_ERR_INVALID, "tq1_linear_swiglu_f16: null pointer");
    if (M <= 0) return fail(TQ1_ERR_INVALID, "activations have an empty batch dimension");
    if (N <= 0 || K <= 0) return fail(TQ1_ERR_INVALID, "tensor dimensions must be positive, got %dx%d", N, K);
    if (N > (1 << 30)) return fail(TQ1_ERR_INVALID, "tq1_linear_swiglu_f16: too many rows");
    const int rows = 2 * N;                 // (gate, up) pairs
    if (reinterpret_cast<uintptr_t>(x) & 15)
        return fail(TQ1_ERR_INVALID, "tq1_linear_swiglu_f16: x must be 16-byte aligned");
    const __half *xh = static_cast<const __half *>(x);
    const bool gemv = M == 1 && gemv_chain_fits(blocks, rows, K);
    if (!gemv && !gemm_tc_supported(blocks, xh, M, rows, K))
        return fail(TQ1_ERR_INVALID,
                    "tq1_linear_swiglu_f16: needs K %% 512 == 0 and 16-byte aligned blocks (got %dx%d)", rows, K);
    const size_t need = tq1_linear_workspace_bytes(M, rows, K);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255))
        return fail(TQ1_ERR_WORKSPACE, "tq1_linear_swiglu_f16: workspace of %zu bytes (256-byte aligned) required", need);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gemv) return launch_gemv_single(blocks, xh, y, y_is_f32 != 0, rows, K, true, workspace, kWsSlotRegionBytes, s);
    if (gemv_looped_fits(blocks, M, rows, K))
        return launch_gemv_looped(blocks, xh, y, y_is_f32 != 0, M, rows, K, true, workspace, s);
    return launch_gemm_tc(blocks, xh, y, y_is_f32 != 0, M, rows, K, workspace, s, true);
}

int tq1_linear_plan(int M, int N, int K, int aligned, int *kernel, int *token_tile, int *ctas, int *parts) {
    if (!kernel || !token_tile || !ctas || !parts) return fail(TQ1_ERR_INVALID, "tq1_linear_plan: null pointer");
    if (M <= 0 || N <= 0 || K <= 0 || K % kGroup) return fail(TQ1_ERR_INVALID, "tq1_linear_plan: bad shape");
    *token_tile = *ctas = *parts = 0;
    if (M <= (gemv_loop_tokens() > 1 ? gemv_loop_tokens() : 1) && aligned && gemv_chain_shape_ok(N, K)) {
        *kernel = TQ1_KERNEL_STREAM_GEMV;       // M > 1: one launch of M passes of the batch-1 kernel
    } else if (aligned && gemm_tc_shape_ok(M, N, K)) {
        *kernel = TQ1_KERNEL_TENSOR_CORE;
        gemm_tc_plan(M, N, K, token_tile, ctas, parts);
    } else {
        *kernel = TQ1_KERNEL_ROWS;
    }
    return TQ1_OK;
}

// Sweep recording only (ternel_b200/dispatch.py binds it by name): forces the tensor-core kernel's token tile
// for every later call of this process; 0 restores the rule. Process-global and not thread-safe, which is why
// it is not part of the public header.
// Sweep recording only: the largest batch that runs as passes of the batch-1 kernel (0: none).
int tq1_debug_set_loop_tokens(int tokens) {
    if (gemv_set_loop_tokens(tokens) != TQ1_OK)
        return fail(TQ1_ERR_INVALID, "tq1_debug_set_loop_tokens: %d is not in 0..8", tokens);
    return TQ1_OK;
}

int tq1_debug_force_token_tile(int token_tile) {
    if (gemm_tc_force_tile(token_tile) != TQ1_OK)
        return fail(TQ1_ERR_INVALID, "tq1_debug_force_token_tile: %d is not 0, 16, 32, 64, 128 or 256", token_tile);
    return TQ1_OK;
}

static size_t shard_local_bytes(int M, int N_local) {
    return ((size_t)M * N_local * sizeof(__half) + 255) & ~(size_t)255;
}

size_t tq1_linear_sharded_workspace_bytes(int M, int N_local, int K) {
    size_t base = tq1_linear_workspace_bytes(M, N_local, K);
    if (base < kWsScratchOffset) base = kWsScratchOffset;
    base = (base + 255) & ~(size_t)255;
    return base + shard_local_bytes(M, N_local);
}

int tq1_shard_advance_epoch(uint32_t *epoch_base, uint32_t delta, void *stream) {
    if (!epoch_base) return fail(TQ1_ERR_INVALID, "tq1_shard_advance_epoch: null pointer");
    return launch_epoch_advance(epoch_base, delta, static_cast<cudaStream_t>(stream));
}

int tq1_linear_f16_sharded(const uint8_t *blocks, const void *x, const tq1_shard *shard, int M, int N_local, int K,
                           void *workspace, size_t workspace_bytes, void *stream) {
    if (!blocks || !x || !shard) return fail(TQ1_ERR_INVALID, "tq1_linear_f16_sharded: null pointer");
    if (shard->world < 1 || shard->world > kMaxRanks || shard->rank < 0 || shard->rank >= shard->world)
        return fail(TQ1_ERR_INVALID, "tq1_linear_f16_sharded: rank %d of %d is out of range (at most %d ranks)",
                    shard->rank, shard->world, kMaxRanks);
    if (M <= 0) return fail(TQ1_ERR_INVALID, "activations have an empty batch dimension");
    if (N_local <= 0 || K <= 0 || K % kGroup)
        return fail(TQ1_ERR_INVALID, "tq1_linear_f16_sharded: bad shard shape %dx%d", N_local, K);
    if (N_local % kFlagRows)
        return fail(TQ1_ERR_INVALID, "tq1_linear_f16_sharded: a shard of %d rows is not a multiple of %d", N_local,
                    kFlagRows);
    if (shard->wait_flags && shard->wait_tiles < 0)
        return fail(TQ1_ERR_INVALID, "tq1_linear_f16_sharded: negative wait_tiles");
    if (shard->n_offset < 0 || shard->n_offset % 16 || shard->n_offset + N_local > shard->n_total)
        return fail(TQ1_ERR_INVALID, "tq1_linear_f16_sharded: rows [%d, %d) do not fit %d gathered rows "
                    "(the offset must be a multiple of 16)", shard->n_offset, shard->n_offset + N_local, shard->n_total);
    const size_t need = tq1_linear_sharded_workspace_bytes(M, N_local, K);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255))
        return fail(TQ1_ERR_WORKSPACE, "tq1_linear_f16_sharded: workspace of %zu bytes (256-byte aligned) required", need);
    ShardDev sd = {};
    sd.world = shard->world;
    sd.rank = shard->rank;
    for (int p = 0; p < shard->world; ++p) {
        if (!shard->peer_y[p] || !shard->peer_flags[p])
            return fail(TQ1_ERR_INVALID, "tq1_linear_f16_sharded: missing peer pointer for rank %d", p);
        sd.peer_y[p] = static_cast<__half *>(shard->peer_y[p]) + shard->n_offset;
        sd.peer_flags[p] = shard->peer_flags[p] + shard->n_offset / kFlagRows;
    }
    sd.epoch_base = shard->epoch_base;
    sd.publish_epoch = shard->publish_epoch;
    sd.wait_flags = shard->wait_flags;
    sd.wait_tiles = shard->wait_flags ? shard->wait_tiles : 0;
    sd.wait_epoch = shard->wait_epoch;
    sd.ld_total = shard->n_total;
    unsigned *status = static_cast<unsigned *>(workspace);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // wait for the inputs, compute the local slice, push it
    int rc = launch_shard_wait(sd, status, s);
    if (rc != TQ1_OK) return rc;
    const size_t base = need - shard_local_bytes(M, N_local);
    __half *local = reinterpret_cast<__half *>(static_cast<unsigned char *>(workspace) + base);
    rc = tq1_linear_f16(blocks, x, local, 0, M, N_local, K, workspace, base, stream);
    if (rc != TQ1_OK) return rc;
    return launch_shard_push(local, M, N_local, sd, s);
}

int tq1_gemv_f16_noalloc(const uint8_t *blocks, const void *x, void *y, int y_is_f32, int N, int K, void *stream) {
    if (!blocks || !x || !y) return fail(TQ1_ERR_INVALID, "tq1_gemv_f16_noalloc: null pointer");
    if (N <= 0 || K <= 0)
        return fail(TQ1_ERR_INVALID, "tensor dimensions must be positive, got %dx%d", N, K);
    if (K % kGroup)
        return fail(TQ1_ERR_INVALID, "%d columns is not a multiple of the 128-weight group", K);
    if (reinterpret_cast<uintptr_t>(x) & 15)
        return fail(TQ1_ERR_INVALID, "tq1_gemv_f16_noalloc: x must be 16-byte aligned");
    return gemv_noalloc(blocks, static_cast<const __half *>(x), y, y_is_f32 != 0, N, K,
                        static_cast<cudaStream_t>(stream));
}

int tq1_gemv_noalloc_status(uint32_t *status_host, void *stream) {
    if (!status_host) return fail(TQ1_ERR_INVALID, "tq1_gemv_noalloc_status: null pointer");
    return gemv_noalloc_status(status_host, static_cast<cudaStream_t>(stream));
}

int tq1_embedding_f16(const uint8_t *blocks, const int64_t *ids, void *out, int out_is_f32,
                      int64_t T, int64_t V, int K, void *stream) {
    if (!blocks || !ids || !out) return fail(TQ1_ERR_INVALID, "tq1_embedding_f16: null pointer");
    if (T <= 0) return fail(TQ1_ERR_INVALID, "indices are empty");
    if (V <= 0 || K <= 0)
        return fail(TQ1_ERR_INVALID, "tensor dimensions must be positive, got %lldx%d", (long long)V, K);
    if (K % kGroup)
        return fail(TQ1_ERR_INVALID, "%d columns is not a multiple of the 128-weight group", K);
    if (reinterpret_cast<uintptr_t>(blocks) & 3)
        return fail(TQ1_ERR_INVALID, "tq1_embedding_f16: blocks must be 4-byte aligned");
    if (reinterpret_cast<uintptr_t>(out) & 15)
        return fail(TQ1_ERR_INVALID, "tq1_embedding_f16: out must be 16-byte aligned");
    return launch_embedding(blocks, ids, out, out_is_f32 != 0, T, V, K, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
