// Packed-embedding row gather: out[t][k] = (c[id_t][k] - 1) * scale[id_t][k/128].
//
// Stands in for tq1_get_rows (src/ternel_mlx/kernels.py:863-901 of the reference)
// and k_get_rows_tq1_g128 (patches/prism-tq1-g128-distribution.patch:132-171).
// HBM-bound: per token it reads K/128*28 bytes and writes 2K (FP16) bytes.
//
// One warp decodes one 28-byte block into 128 outputs. The block is fetched as
// seven coalesced 32-bit words (one per lane 0..6) and redistributed with
// shuffles; each lane then produces four consecutive outputs and stores them
// with one 8-byte (FP16) or 16-byte (FP32) write, so a warp writes 256 or 512
// contiguous bytes.
#include "tq1_common.cuh"

namespace tq1 {

template <bool OUT_F32>
__global__ void __launch_bounds__(256) embedding_kernel(const uint8_t *__restrict__ blocks,
                                                        const int64_t *__restrict__ ids,
                                                        void *__restrict__ out,
                                                        int64_t V, int gpr) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t t = blockIdx.y;
    const int g = blockIdx.x * 8 + warp;
    if (g >= gpr) return;
    const int64_t id = ids[t];
    const bool in_range = id >= 0 && id < V;

    uint32_t word = 0;
    if (in_range && lane < kBlockWords) {
        const uint32_t *src = reinterpret_cast<const uint32_t *>(blocks + (id * gpr + g) * kBlockBytes);
        word = __ldg(src + lane);
    }
    const uint32_t w0 = __shfl_sync(0xffffffffu, word, 0);
    const float scale = __half2float(__ushort_as_half((unsigned short)(w0 & 0xffffu)));

    // Lane l owns outputs k = 4l .. 4l+3.
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int k = 4 * lane + i;
        const int slot = k < 125 ? k / 5 : 25;          // code byte index 0..25
        const int digit = k < 125 ? k - 5 * slot : k - 125;
        const int byte_pos = 2 + slot;                  // byte within the 28-byte block
        const uint32_t w = __shfl_sync(0xffffffffu, word, byte_pos >> 2);
        uint32_t code = (w >> (8 * (byte_pos & 3))) & 0xffu;
        const uint32_t pow3 = digit == 0 ? 1u : digit == 1 ? 3u : digit == 2 ? 9u : digit == 3 ? 27u : 81u;
        const int trit = (int)((code / pow3) % 3u);
        // A multiplication (not a select) so that 0 * Inf and 0 * NaN give NaN and
        // signed zeros come out as in the NumPy reference.
        v[i] = in_range ? (float)(trit - 1) * scale : 0.0f;
    }
    const int64_t base = (t * gpr + g) * (int64_t)kGroup + 4 * lane;
    if (OUT_F32) {
        *reinterpret_cast<float4 *>(static_cast<float *>(out) + base) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        __half2 lo = __floats2half2_rn(v[0], v[1]);
        __half2 hi = __floats2half2_rn(v[2], v[3]);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t *>(&lo);
        packed.y = *reinterpret_cast<uint32_t *>(&hi);
        *reinterpret_cast<uint2 *>(static_cast<__half *>(out) + base) = packed;
    }
}

int launch_embedding(const uint8_t *blocks, const int64_t *ids, void *out, bool out_f32,
                     int64_t T, int64_t V, int K, cudaStream_t stream) {
    const int gpr = K / kGroup;
    for (int64_t t0 = 0; t0 < T; t0 += 65535) {   // gridDim.y limit
        const int64_t n = T - t0 < 65535 ? T - t0 : 65535;
        dim3 grid((gpr + 7) / 8, (unsigned)n);
        const int64_t *id_ptr = ids + t0;
        if (out_f32) {
            embedding_kernel<true><<<grid, 256, 0, stream>>>(
                blocks, id_ptr, static_cast<float *>(out) + t0 * K, V, gpr);
        } else {
            embedding_kernel<false><<<grid, 256, 0, stream>>>(
                blocks, id_ptr, static_cast<__half *>(out) + t0 * K, V, gpr);
        }
        cudaError_t err = cudaGetLastError();
        if (err != cudaSuccess) return cuda_fail(err, "tq1_embedding_f16: launch");
    }
    return TQ1_OK;
}

}  // namespace tq1
