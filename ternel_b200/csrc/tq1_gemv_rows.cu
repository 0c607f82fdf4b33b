// Reference-order GEMV: one warp per output row, FP32 FMA on the CUDA cores.
//
// This is the simplest correct statement of the linear path and the fallback
// for shapes the streaming kernels do not take (K not a multiple of 512, odd
// row counts). It keeps the reference's arithmetic shape: a full FP32 sum per
// 128-weight group, then acc = fma(scale, group_sum, acc)
// (src/bonsai_tq1/reference.py:33-38, src/ternel_mlx/kernels.py:317-322).
//
// Eight lanes share one 28-byte block: lanes 0..6 of an octet each take one of
// its seven 32-bit words (coalesced: a warp reads 4 consecutive blocks = 112
// bytes per step), decode the code bytes through a 243-entry shared-memory
// table of 2-bit trits, and multiply with FP32 activations held in shared
// memory. Three shuffles sum the octet; the lane holding word 0 owns the scale.
#include "tq1_common.cuh"

namespace tq1 {

constexpr int kRowsThreads = 256;
constexpr int kRowsMaxBatch = 4;   // activation rows resident in shared memory per launch

__device__ __forceinline__ float dot_byte(uint32_t entry, const float *x, int n, float sum) {
#pragma unroll
    for (int i = 0; i < 5; ++i) {
        if (i < n) {
            const float w = (float)((int)((entry >> (2 * i)) & 3u) - 1);
            sum = fmaf(w, x[i], sum);   // 0 * NaN / 0 * Inf stay NaN, as in the reference
        }
    }
    return sum;
}

template <int MB, bool OUT_F32>
__global__ void __launch_bounds__(kRowsThreads) gemv_rows_kernel(const uint8_t *__restrict__ blocks,
                                                                 const __half *__restrict__ x,
                                                                 void *__restrict__ y,
                                                                 int N, int K, int ldy) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint16_t *lut = reinterpret_cast<uint16_t *>(smem_raw);          // 256 entries
    float *xs = reinterpret_cast<float *>(smem_raw + 512);           // [MB][K]

    for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = (uint16_t)trits_2bit(i);
    for (int i = threadIdx.x; i < MB * K; i += blockDim.x) xs[i] = __half2float(x[i]);
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int pos = lane & 7;          // word within the block (7 = idle lane)
    const int sub = lane >> 3;         // which of the 4 blocks of this step
    const int gpr = K / kGroup;
    const int warps = blockDim.x >> 5;

    for (int row = blockIdx.x * warps + warp; row < N; row += gridDim.x * warps) {
        const uint32_t *words = reinterpret_cast<const uint32_t *>(blocks + (int64_t)row * gpr * kBlockBytes);
        float acc[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[m] = 0.0f;

        for (int g0 = 0; g0 < gpr; g0 += 4) {
            const int g = g0 + sub;
            const bool live = g < gpr && pos < kBlockWords;
            const uint32_t w = live ? __ldg(words + g * kBlockWords + pos) : 0u;
            float sum[MB];
#pragma unroll
            for (int m = 0; m < MB; ++m) sum[m] = 0.0f;
            if (live) {
                // word 0 = [scale lo, scale hi, code 0, code 1]; word p>=1 = codes 4p-2 .. 4p+1
                const int first = pos == 0 ? 0 : 4 * pos - 2;
                const int count = pos == 0 ? 2 : 4;
                const uint32_t bytes = pos == 0 ? (w >> 16) : w;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    if (b < count) {
                        const int slot = first + b;
                        const uint32_t entry = lut[(bytes >> (8 * b)) & 0xffu];
                        const int n = slot == 25 ? 3 : 5;
#pragma unroll
                        for (int m = 0; m < MB; ++m)
                            sum[m] = dot_byte(entry, xs + m * K + g * kGroup + 5 * slot, n, sum[m]);
                    }
                }
            }
            const float scale = __half2float(__ushort_as_half((unsigned short)(w & 0xffffu)));
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                float s = sum[m];
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                if (live && pos == 0) acc[m] = fmaf(scale, s, acc[m]);
            }
        }
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            float a = acc[m];
            a += __shfl_xor_sync(0xffffffffu, a, 8);
            a += __shfl_xor_sync(0xffffffffu, a, 16);
            if (lane == 0) {
                if (!TQ1_IN_BOUNDS(row, N, 20u)) continue;
                if (OUT_F32) static_cast<float *>(y)[(int64_t)m * ldy + row] = a;
                else static_cast<__half *>(y)[(int64_t)m * ldy + row] = __float2half_rn(a);
            }
        }
    }
}

template <int MB>
static int launch_mb(const uint8_t *blocks, const __half *x, void *y, bool y_f32,
                     int N, int K, cudaStream_t stream) {
    const size_t smem = 512 + sizeof(float) * (size_t)MB * K;
    if (smem > 227 * 1024)
        return fail(TQ1_ERR_INVALID, "tq1_linear_f16: K=%d too large for the row kernel's shared memory", K);
    int ctas = (N + 7) / 8;
    if (ctas > 148 * 2) ctas = 148 * 2;
    auto kern_h = gemv_rows_kernel<MB, false>;
    auto kern_f = gemv_rows_kernel<MB, true>;
    cudaError_t err = cudaFuncSetAttribute(y_f32 ? kern_f : kern_h,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16: shared memory opt-in");
    if (y_f32) kern_f<<<ctas, kRowsThreads, smem, stream>>>(blocks, x, y, N, K, N);
    else kern_h<<<ctas, kRowsThreads, smem, stream>>>(blocks, x, y, N, K, N);
    err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16: launch");
    return TQ1_OK;
}

int launch_gemv_rows(const uint8_t *blocks, const __half *x, void *y, bool y_f32,
                     int M, int N, int K, cudaStream_t stream) {
    const size_t ysz = y_f32 ? 4 : 2;
    // Keep MB*K*4 bytes of activations within shared memory.
    int mb_max = kRowsMaxBatch;
    while (mb_max > 1 && 512 + sizeof(float) * (size_t)mb_max * K > 200 * 1024) mb_max >>= 1;
    for (int m0 = 0; m0 < M;) {
        int mb = M - m0 >= 4 && mb_max >= 4 ? 4 : M - m0 >= 2 && mb_max >= 2 ? 2 : 1;
        const __half *xm = x + (int64_t)m0 * K;
        void *ym = static_cast<char *>(y) + (size_t)m0 * N * ysz;
        int rc = mb == 4 ? launch_mb<4>(blocks, xm, ym, y_f32, N, K, stream)
               : mb == 2 ? launch_mb<2>(blocks, xm, ym, y_f32, N, K, stream)
                         : launch_mb<1>(blocks, xm, ym, y_f32, N, K, stream);
        if (rc != TQ1_OK) return rc;
        m0 += mb;
    }
    return TQ1_OK;
}

}  // namespace tq1
