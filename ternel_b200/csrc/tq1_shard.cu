// Row-sharded linear: every rank computes its slice of the output rows and the FP16 result is
// written directly into every rank's gathered activation buffer over NVLink peer mappings, each
// tile of 16 rows followed by a release store of that tile's flag; consumers acquire the flags of
// the tiles they read.
// There is no counterpart in the reference (it is single-device); the exchange replaces an
// all-gather after each sharded projection. For M = 1 the push is the streaming GEMV's own
// epilogue; larger batches compute into a local slice and push it with the kernel below.
#include "tq1_common.cuh"

namespace tq1 {

namespace {

constexpr unsigned kWaitLimit = 1u << 22;

__global__ void tq1_shard_wait_kernel(const ShardDev shard, unsigned *status) {
    const unsigned want = shard.wait_epoch + (shard.epoch_base ? *shard.epoch_base : 0u);
    for (int t = threadIdx.x; t < shard.wait_tiles; t += blockDim.x) {
        unsigned spins = 0;
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(shard.wait_flags + t) : "memory");
            if ((int)(v - want) >= 0) break;
            if (++spins > kWaitLimit) { atomicExch(status, 4u); break; }      // bounded: report, do not hang
        }
    }
}

// One warp per row tile: copy the tile's [M][16] values to every rank, then raise the tile's flag there.
__global__ void __launch_bounds__(256) tq1_shard_push_kernel(const __half *__restrict__ local, int M, int n_local,
                                                            const ShardDev shard) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int tiles = n_local / kFlagRows;
    const unsigned epoch = shard.publish_epoch + (shard.epoch_base ? *shard.epoch_base : 0u);
    for (int tile = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; tile < tiles; tile += warps) {
        for (int i = lane; i < M * kFlagRows; i += 32) {
            const int m = i / kFlagRows, n = tile * kFlagRows + (i - m * kFlagRows);
            const __half v = local[(size_t)m * n_local + n];
            if (!TQ1_IN_BOUNDS(n, n_local, 60u)) continue;
            for (int p = 0; p < shard.world; ++p) shard.peer_y[p][(size_t)m * shard.ld_total + n] = v;
        }
        __threadfence_system();          // every lane's stores are performed before any flag below
        __syncwarp();
        if (lane < shard.world)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(shard.peer_flags[lane] + tile), "r"(epoch)
                         : "memory");
    }
}

__global__ void tq1_epoch_advance_kernel(unsigned *epoch_base, unsigned delta) { *epoch_base += delta; }

}  // namespace

int launch_epoch_advance(unsigned *epoch_base, unsigned delta, cudaStream_t stream) {
    tq1_epoch_advance_kernel<<<1, 1, 0, stream>>>(epoch_base, delta);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "tq1_shard_advance_epoch: launch");
    return TQ1_OK;
}

int launch_shard_wait(const ShardDev &shard, unsigned *status, cudaStream_t stream) {
    if (shard.world <= 1 || !shard.wait_flags) return TQ1_OK;
    tq1_shard_wait_kernel<<<1, 256, 0, stream>>>(shard, status);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16_sharded: wait launch");
    return TQ1_OK;
}

int launch_shard_push(const __half *local, int M, int n_local, const ShardDev &shard, cudaStream_t stream) {
    int ctas = (n_local / kFlagRows + 7) / 8;          // eight warps (tiles) per CTA
    if (ctas > 296) ctas = 296;
    if (ctas < 1) ctas = 1;
    tq1_shard_push_kernel<<<ctas, 256, 0, stream>>>(local, M, n_local, shard);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16_sharded: push launch");
    return TQ1_OK;
}

}  // namespace tq1
