// Host-side TQ1_G128 codec and the device-side load-time byte scan.
//
// pack/unpack/validate restate src/bonsai_tq1/format.py:66-122 of the reference;
// tile/untile restate src/bonsai_tq1/lut23_reorder.py:126-165 for row counts the
// tile divides (the MLX layout, src/ternel_mlx/layout.py:76-80).
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "tq1_common.cuh"

#ifdef TQ1_BOUNDS_CHECK
namespace tq1 {
__device__ unsigned long long g_tq1_bounds[4] = {0, 0, 0, 0};
}
#endif

namespace tq1 {

static thread_local char g_error[512] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t err, const char *what) {
    return fail(TQ1_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
}

static void scan_host(const uint8_t *blocks, int64_t groups, int64_t *bad_full, int64_t *bad_tail) {
    int64_t bf = 0, bt = 0;
    for (int64_t g = 0; g < groups; ++g) {
        const uint8_t *b = blocks + g * kBlockBytes;
        for (int j = 2; j < 27; ++j) bf += b[j] > kMaxFull;
        bt += b[27] > kMaxTail;
    }
    *bad_full = bf;
    *bad_tail = bt;
}

// The blocks are scanned as a flat array of 32-bit words, consecutive threads on consecutive words
// (coalesced). Word i of the array is word i % 7 of its block: word 0 holds the scale and two code
// bytes, words 1..5 four code bytes, word 6 three code bytes and the tail byte. Bytes above the limit
// are counted four at a time with a per-byte unsigned compare.
constexpr int kValidateThreads = 224;       // a multiple of 7: a thread always sees the same word of a block
__global__ void __launch_bounds__(kValidateThreads) validate_kernel(const uint32_t *__restrict__ words,
                                                       int64_t groups,
                                                       unsigned long long *__restrict__ counts) {
    unsigned bf = 0, bt = 0;
    const int64_t total = groups * kBlockWords;
    // the grid stride is a multiple of 7 words, so the word's place in its block never changes
    const int pos = threadIdx.x % kBlockWords;
    const uint32_t full_mask = pos == 0 ? 0xffff0000u : pos == 6 ? 0x00ffffffu : 0xffffffffu;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t v = __ldg(words + i);
        // 0xff in every byte that exceeds 242 (as unsigned bytes)
        const uint32_t over = __vcmpgtu4(v, 0xf2f2f2f2u);
        bf += __popc(over & full_mask) >> 3;
        if (pos == 6) bt += (v >> 24) > kMaxTail;
    }
    for (int o = 16; o > 0; o >>= 1) {
        bf += __shfl_xor_sync(0xffffffffu, bf, o);
        bt += __shfl_xor_sync(0xffffffffu, bt, o);
    }
    if ((threadIdx.x & 31) == 0) {
        if (bf) atomicAdd(&counts[0], (unsigned long long)bf);
        if (bt) atomicAdd(&counts[1], (unsigned long long)bt);
    }
}

int launch_validate(const uint8_t *blocks, int64_t groups, int64_t *counts, cudaStream_t stream) {
    cudaError_t err = cudaMemsetAsync(counts, 0, 2 * sizeof(int64_t), stream);
    if (err != cudaSuccess) return cuda_fail(err, "tq1_validate_blocks_device: memset");
    if (groups == 0) return TQ1_OK;
    int64_t ctas = (groups * kBlockWords + kValidateThreads - 1) / kValidateThreads;
    if (ctas > 148 * 8) ctas = 148 * 8;
    validate_kernel<<<(unsigned)ctas, kValidateThreads, 0, stream>>>(
        reinterpret_cast<const uint32_t *>(blocks), groups,
        reinterpret_cast<unsigned long long *>(counts));
    err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "tq1_validate_blocks_device: launch");
    return TQ1_OK;
}

}  // namespace tq1

using namespace tq1;

extern "C" {

int tq1_abi_version(void) { return 3; }

#ifdef TQ1_BOUNDS_CHECK
// {violations, code of the first, its index, its limit}; copies the record to host memory and clears it.
int tq1_debug_bounds(unsigned long long *out_host) {
    if (cudaMemcpyFromSymbol(out_host, tq1::g_tq1_bounds, sizeof(unsigned long long) * 4) != cudaSuccess) return TQ1_ERR_CUDA;
    const unsigned long long zero[4] = {0, 0, 0, 0};
    if (cudaMemcpyToSymbol(tq1::g_tq1_bounds, zero, sizeof(zero)) != cudaSuccess) return TQ1_ERR_CUDA;
    return TQ1_OK;
}
#endif

const char *tq1_last_error(void) { return g_error; }

int tq1_pack_blocks(const uint8_t *scales, const uint8_t *trits, uint8_t *blocks,
                    int64_t groups, int64_t *n_bad) {
    if (groups < 0 || (groups > 0 && (!scales || !trits || !blocks)))
        return fail(TQ1_ERR_INVALID, "tq1_pack_blocks: null pointer or negative group count");
    int64_t bad = 0;
    for (int64_t i = 0; i < groups * kGroup; ++i) bad += trits[i] > 2;
    if (n_bad) *n_bad = bad;
    if (bad) return fail(TQ1_ERR_FORMAT, "source contains %lld non-ternary code(s)", (long long)bad);
    for (int64_t g = 0; g < groups; ++g) {
        const uint8_t *c = trits + g * kGroup;
        uint8_t *b = blocks + g * kBlockBytes;
        b[0] = scales[2 * g];
        b[1] = scales[2 * g + 1];
        for (int j = 0; j < kFullBytes; ++j) {
            unsigned v = 0;
            for (int i = 4; i >= 0; --i) v = v * 3 + c[5 * j + i];
            b[2 + j] = (uint8_t)v;
        }
        b[27] = (uint8_t)(c[125] + 3u * c[126] + 9u * c[127]);
    }
    return TQ1_OK;
}

int tq1_validate_blocks(const uint8_t *blocks, int64_t groups,
                        int64_t *n_bad_full, int64_t *n_bad_tail) {
    if (groups < 0 || (groups > 0 && !blocks))
        return fail(TQ1_ERR_INVALID, "tq1_validate_blocks: null pointer or negative group count");
    int64_t bf = 0, bt = 0;
    scan_host(blocks, groups, &bf, &bt);
    if (n_bad_full) *n_bad_full = bf;
    if (n_bad_tail) *n_bad_tail = bt;
    if (bf || bt)
        return fail(TQ1_ERR_FORMAT, "invalid base-3 bytes: regular=%lld, tail=%lld",
                    (long long)bf, (long long)bt);
    return TQ1_OK;
}

int tq1_unpack_blocks(const uint8_t *blocks, uint8_t *scales, uint8_t *trits,
                      int64_t groups, int validate, int64_t *n_bad_full, int64_t *n_bad_tail) {
    if (groups < 0 || (groups > 0 && (!blocks || !scales || !trits)))
        return fail(TQ1_ERR_INVALID, "tq1_unpack_blocks: null pointer or negative group count");
    if (n_bad_full) *n_bad_full = 0;
    if (n_bad_tail) *n_bad_tail = 0;
    if (validate) {
        int rc = tq1_validate_blocks(blocks, groups, n_bad_full, n_bad_tail);
        if (rc != TQ1_OK) return rc;
    }
    uint8_t table[256][5];
    for (unsigned v = 0; v < 256; ++v) {
        unsigned r = v;
        for (int i = 0; i < 5; ++i) { table[v][i] = (uint8_t)(r % 3); r /= 3; }
    }
    for (int64_t g = 0; g < groups; ++g) {
        const uint8_t *b = blocks + g * kBlockBytes;
        uint8_t *c = trits + g * kGroup;
        scales[2 * g] = b[0];
        scales[2 * g + 1] = b[1];
        for (int j = 0; j < kFullBytes; ++j) memcpy(c + 5 * j, table[b[2 + j]], 5);
        memcpy(c + 125, table[b[27]], 3);
    }
    return TQ1_OK;
}

int tq1_dequantize_blocks(const uint8_t *blocks, float *out, int64_t groups) {
    if (groups < 0 || (groups > 0 && (!blocks || !out)))
        return fail(TQ1_ERR_INVALID, "tq1_dequantize_blocks: null pointer or negative group count");
    float sign[256][5];                       // byte -> its five weights as -1, 0, +1
    for (unsigned v = 0; v < 256; ++v) {
        unsigned r = v;
        for (int i = 0; i < 5; ++i) { sign[v][i] = (float)((int)(r % 3) - 1); r /= 3; }
    }
    for (int64_t g = 0; g < groups; ++g) {
        const uint8_t *b = blocks + g * kBlockBytes;
        const float d = __half2float(__ushort_as_half((unsigned short)(b[0] | (b[1] << 8))));
        float *y = out + g * kGroup;
        for (int j = 0; j < kFullBytes; ++j)
            for (int i = 0; i < 5; ++i) y[5 * j + i] = sign[b[2 + j]][i] * d;
        for (int i = 0; i < 3; ++i) y[125 + i] = sign[b[27]][i] * d;
    }
    return TQ1_OK;
}

int tq1_tile_blocks(const uint8_t *blocks, uint8_t *codes, uint16_t *scales,
                    int64_t rows, int64_t gpr, int64_t tile) {
    if (rows <= 0 || gpr <= 0 || tile <= 0 || !blocks || !codes || !scales)
        return fail(TQ1_ERR_INVALID, "tq1_tile_blocks: dimensions must be positive and pointers non-null");
    if (rows % tile)
        return fail(TQ1_ERR_INVALID, "tile %lld does not divide %lld rows", (long long)tile, (long long)rows);
    for (int64_t r = 0; r < rows; ++r) {
        int64_t t = r / tile, in = r % tile;
        for (int64_t g = 0; g < gpr; ++g) {
            const uint8_t *b = blocks + (r * gpr + g) * kBlockBytes;
            scales[(t * gpr + g) * tile + in] = (uint16_t)(b[0] | (b[1] << 8));
            uint8_t *dst = codes + ((t * gpr + g) * kCodeBytes) * tile + in;
            for (int s = 0; s < kCodeBytes; ++s) dst[s * tile] = b[2 + s];
        }
    }
    return TQ1_OK;
}

int tq1_untile_blocks(const uint8_t *codes, const uint16_t *scales, uint8_t *blocks,
                      int64_t rows, int64_t gpr, int64_t tile) {
    if (rows <= 0 || gpr <= 0 || tile <= 0 || !blocks || !codes || !scales)
        return fail(TQ1_ERR_INVALID, "tq1_untile_blocks: dimensions must be positive and pointers non-null");
    if (rows % tile)
        return fail(TQ1_ERR_INVALID, "tile %lld does not divide %lld rows", (long long)tile, (long long)rows);
    for (int64_t r = 0; r < rows; ++r) {
        int64_t t = r / tile, in = r % tile;
        for (int64_t g = 0; g < gpr; ++g) {
            uint8_t *b = blocks + (r * gpr + g) * kBlockBytes;
            uint16_t s = scales[(t * gpr + g) * tile + in];
            b[0] = (uint8_t)(s & 0xff);
            b[1] = (uint8_t)(s >> 8);
            const uint8_t *src = codes + ((t * gpr + g) * kCodeBytes) * tile + in;
            for (int k = 0; k < kCodeBytes; ++k) b[2 + k] = src[k * tile];
        }
    }
    return TQ1_OK;
}

int tq1_validate_blocks_device(const uint8_t *blocks_dev, int64_t groups,
                               int64_t *counts_dev, void *stream) {
    if (groups < 0 || !counts_dev || (groups > 0 && !blocks_dev))
        return fail(TQ1_ERR_INVALID, "tq1_validate_blocks_device: null pointer or negative group count");
    if (reinterpret_cast<uintptr_t>(blocks_dev) & 3)
        return fail(TQ1_ERR_INVALID, "tq1_validate_blocks_device: blocks must be 4-byte aligned");
    return launch_validate(blocks_dev, groups, counts_dev, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
