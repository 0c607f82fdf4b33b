// Row-sharded linear: every rank computes its slice of the output rows and the FP16 result is
// written directly into every rank's gathered activation buffer over NVLink peer mappings,
// followed by a release flag; consumers acquire the flags before they read the activations.
// There is no counterpart in the reference (it is single-device); the exchange replaces an
// all-gather after each sharded projection. For M = 1 the push is the streaming GEMV's own
// epilogue; larger batches compute into a local slice and push it with the kernel below.
#include "tq1_common.cuh"

namespace tq1 {

namespace {

constexpr unsigned kWaitLimit = 1u << 22;

__global__ void tq1_shard_wait_kernel(const ShardDev shard, unsigned *status) {
    const int t = threadIdx.x;
    if (t < shard.world) {
        const unsigned want = shard.wait_epoch + (shard.epoch_base ? *shard.epoch_base : 0u);
        unsigned spins = 0;
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(shard.wait_flags + t) : "memory");
            if ((int)(v - want) >= 0) break;
            if (++spins > kWaitLimit) { atomicExch(status, 4u); break; }      // bounded: report, do not hang
        }
    }
}

__global__ void __launch_bounds__(256) tq1_shard_push_kernel(const __half *__restrict__ local, int M, int n_local,
                                                            const ShardDev shard) {
    const long long total = (long long)M * n_local;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int m = (int)(i / n_local), n = (int)(i - (long long)m * n_local);
        const __half v = local[i];
        for (int p = 0; p < shard.world; ++p) shard.peer_y[p][(size_t)m * shard.ld_total + n] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned before = atomicAdd(shard.done_counter, 1u);
        if (before + 1u == gridDim.x) {
            atomicExch(shard.done_counter, 0u);
            __threadfence_system();
            const unsigned epoch = shard.publish_epoch + (shard.epoch_base ? *shard.epoch_base : 0u);
            for (int p = 0; p < shard.world; ++p)
                asm volatile("st.release.sys.global.u32 [%0], %1;"
                             ::"l"(shard.peer_flags[p] + shard.rank), "r"(epoch) : "memory");
        }
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
    tq1_shard_wait_kernel<<<1, 32, 0, stream>>>(shard, status);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16_sharded: wait launch");
    return TQ1_OK;
}

int launch_shard_push(const __half *local, int M, int n_local, const ShardDev &shard, cudaStream_t stream) {
    const long long total = (long long)M * n_local;
    int ctas = (int)((total + 255) / 256);
    if (ctas > 296) ctas = 296;
    if (ctas < 1) ctas = 1;
    tq1_shard_push_kernel<<<ctas, 256, 0, stream>>>(local, M, n_local, shard);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16_sharded: push launch");
    return TQ1_OK;
}

}  // namespace tq1
