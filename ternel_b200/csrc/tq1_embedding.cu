// Packed-embedding row gather: out[t][k] = (c[id_t][k] - 1) * scale[id_t][k/128].
//
// Stands in for tq1_get_rows (src/ternel_mlx/kernels.py:863-901 of the reference)
// and k_get_rows_tq1_g128 (patches/prism-tq1-g128-distribution.patch:132-171).
// HBM-bound: per token it reads K/128*28 bytes and writes 2K (FP16) bytes.
//
// Sixteen threads decode one 28-byte block into 128 outputs, eight consecutive outputs (one 16-byte
// FP16 store, or two for FP32) per thread; a warp therefore writes 512 contiguous bytes. A thread's
// eight trits start somewhere inside a code byte and span at most three: the bytes are looked up in a
// 243-entry table of five 2-bit trits (global memory, L1-resident), concatenated and shifted. Every
// output is one of three values per block, -1*s, 0*s, +1*s, computed once by multiplication (so that
// 0*Inf and 0*NaN give NaN and zeros keep the sign NumPy gives them) and then selected by the trit.
#include "tq1_common.cuh"

namespace tq1 {

namespace {

struct TritTable {
    uint16_t e[256];
};
constexpr TritTable make_trit_table() {
    TritTable t{};
    for (int v = 0; v < 243; ++v) {
        int x = v, e = 0;
        for (int i = 0; i < 5; ++i) {
            e |= (x % 3) << (2 * i);
            x /= 3;
        }
        t.e[v] = (uint16_t)e;
    }
    return t;
}
__device__ const TritTable g_trits = make_trit_table();

constexpr int kThreadsPerBlockRow = 16;       // threads per 28-byte block
constexpr int kBlocksPerCta = 8;
constexpr int kTokensPerThread = 4;

}  // namespace

template <bool OUT_F32>
__global__ void __launch_bounds__(kThreadsPerBlockRow * kBlocksPerCta)
embedding_kernel(const uint8_t *__restrict__ blocks, const int64_t *__restrict__ ids, void *__restrict__ out,
                 int64_t T, int64_t V, int gpr) {
    const int j = threadIdx.x & (kThreadsPerBlockRow - 1);      // which eight outputs of the block
    const int g = blockIdx.x * kBlocksPerCta + (threadIdx.x >> 4);
    if (g >= gpr) return;
    const int k0 = 8 * j;
    const int a = (k0 * 205) >> 10, off = k0 - 5 * a;            // k0 / 5 for k0 <= 120; first trit inside byte a
    const int64_t t0 = (int64_t)blockIdx.y * kTokensPerThread;

    // Several tokens per thread, every load of one kind issued for all of them before the next kind:
    // the dependent chain id -> code bytes -> table entries is a few microseconds long, and a thread
    // that follows it for one token only keeps too few bytes in flight to fill the memory system.
    int64_t id[kTokensPerThread];
    bool live[kTokensPerThread];
#pragma unroll
    for (int q = 0; q < kTokensPerThread; ++q) id[q] = t0 + q < T ? ids[t0 + q] : -1;
    const uint8_t *blk[kTokensPerThread];
    uint32_t sbits[kTokensPerThread], b0[kTokensPerThread], b1[kTokensPerThread], b2[kTokensPerThread];
#pragma unroll
    for (int q = 0; q < kTokensPerThread; ++q) {
        live[q] = id[q] >= 0 && id[q] < V;
        blk[q] = blocks + (size_t)((unsigned)(live[q] ? id[q] : 0) * (unsigned)gpr + (unsigned)g) * kBlockBytes;
        sbits[q] = *reinterpret_cast<const unsigned short *>(blk[q]);
        b0[q] = __ldg(blk[q] + 2 + a);
        b1[q] = __ldg(blk[q] + 3 + a);
        b2[q] = off >= 3 ? __ldg(blk[q] + 4 + a) : 0u;          // the third byte exists whenever it is needed
    }
    uint32_t sel[kTokensPerThread];                             // eight 2-bit trits, output i at bits 2i..2i+1
#pragma unroll
    for (int q = 0; q < kTokensPerThread; ++q) {
        const uint32_t stream = (uint32_t)g_trits.e[b0[q]] | ((uint32_t)g_trits.e[b1[q]] << 10) |
                                ((uint32_t)g_trits.e[b2[q]] << 20);
        sel[q] = (stream >> (2 * off)) & 0xffffu;
    }
#pragma unroll
    for (int q = 0; q < kTokensPerThread; ++q) {
        if (t0 + q >= T) break;
        const float scale = __half2float(__ushort_as_half((unsigned short)sbits[q]));
        // a row outside the table is all zeros, not 0 * scale
        const float c0 = live[q] ? -1.0f * scale : 0.0f, c1 = live[q] ? 0.0f * scale : 0.0f,
                    c2 = live[q] ? 1.0f * scale : 0.0f;
        const size_t base = ((size_t)(t0 + q) * gpr + g) * kGroup + 8 * j;
        if (!TQ1_IN_BOUNDS(base + 7, (size_t)T * gpr * kGroup, 30u)) continue;
        if (OUT_F32) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t trit = (sel[q] >> (2 * i)) & 3u;
                v[i] = trit == 0 ? c0 : trit == 1 ? c1 : c2;
            }
            float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(out) + base);
            dst[0] = make_float4(v[0], v[1], v[2], v[3]);
            dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {
            // The three candidate halves sit in an 8-byte pool; one byte permute per output pair picks two
            // of them. A trit t selects pool bytes 2t and 2t+1: selector nibbles (2t, 2t+1) = 0x10 + 0x22 * t.
            const uint32_t h0 = __half_as_ushort(__float2half_rn(c0));
            const uint32_t h1 = __half_as_ushort(__float2half_rn(c1));
            const uint32_t h2 = __half_as_ushort(__float2half_rn(c2));
            const uint32_t pool_lo = h0 | (h1 << 16), pool_hi = h2;
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t ta = (sel[q] >> (4 * i)) & 3u, tb = (sel[q] >> (4 * i + 2)) & 3u;
                const uint32_t selector = 0x1010u + ta * 0x22u + tb * 0x2200u;
                asm("prmt.b32 %0, %1, %2, %3;" : "=r"(w[i]) : "r"(pool_lo), "r"(pool_hi), "r"(selector));
            }
            *reinterpret_cast<uint4 *>(static_cast<__half *>(out) + base) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

int launch_embedding(const uint8_t *blocks, const int64_t *ids, void *out, bool out_f32,
                     int64_t T, int64_t V, int K, cudaStream_t stream) {
    const int gpr = K / kGroup;
    const int64_t per_launch = 65535LL * kTokensPerThread;          // gridDim.y limit
    for (int64_t t0 = 0; t0 < T; t0 += per_launch) {
        const int64_t n = T - t0 < per_launch ? T - t0 : per_launch;
        dim3 grid((gpr + kBlocksPerCta - 1) / kBlocksPerCta, (unsigned)((n + kTokensPerThread - 1) / kTokensPerThread));
        const int64_t *id_ptr = ids + t0;
        if (out_f32) {
            embedding_kernel<true><<<grid, kThreadsPerBlockRow * kBlocksPerCta, 0, stream>>>(
                blocks, id_ptr, static_cast<float *>(out) + t0 * K, n, V, gpr);
        } else {
            embedding_kernel<false><<<grid, kThreadsPerBlockRow * kBlocksPerCta, 0, stream>>>(
                blocks, id_ptr, static_cast<__half *>(out) + t0 * K, n, V, gpr);
        }
        cudaError_t err = cudaGetLastError();
        if (err != cudaSuccess) return cuda_fail(err, "tq1_embedding_f16: launch");
    }
    return TQ1_OK;
}

}  // namespace tq1
