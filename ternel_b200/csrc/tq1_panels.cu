// Chunk-major panel layout of packed TQ1_G128 weights and its conversion from and to canonical blocks.
//
//     canonical  blocks[r][K/128][28]                      (src/bonsai_tq1/format.py:14-17 of the reference)
//     panels     panels[c][r][112], c = K/512 chunks, r = rows padded with zero blocks to a multiple of 16
//
// The streaming batch-1 kernel consumes 16 rows x 4 groups at a time. In the canonical layout those are
// sixteen 112-byte pieces a whole row apart; in a panel they are 1792 contiguous bytes, which one bulk copy
// moves at HBM speed. The reference also permutes the canonical blocks into a device-friendly form once
// at load (reorder_tensor_arrays, src/bonsai_tq1/lut23_reorder.py:126-165); like there, the permutation is
// lossless and the inverse restores the canonical bytes exactly.
#include "tq1_common.cuh"

namespace tq1 {

namespace {

constexpr int kPanelRowBytes = 4 * kBlockBytes;     // 112
constexpr int kPanelRowVecs = kPanelRowBytes / 16;  // 7
constexpr int kPanelRowQuantum = 16;

__host__ __device__ inline long long panel_pad_rows(long long rows) {
    return (rows + kPanelRowQuantum - 1) / kPanelRowQuantum * kPanelRowQuantum;
}

// One thread per 16-byte vector of the panel array.
template <bool TO_PANELS>
__global__ void __launch_bounds__(256) panels_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst,
                                                     long long rows, long long pad_rows, int chunks) {
    const long long total = (long long)chunks * pad_rows * kPanelRowVecs;
    const long long row_vecs = (long long)chunks * kPanelRowVecs;       // 16-byte vectors per canonical row
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long c = i / (pad_rows * kPanelRowVecs);
        const long long rem = i - c * pad_rows * kPanelRowVecs;
        const long long r = rem / kPanelRowVecs;
        const int j = (int)(rem - r * kPanelRowVecs);
        const long long canon = r * row_vecs + c * kPanelRowVecs + j;
        if (TO_PANELS) dst[i] = r < rows ? src[canon] : make_uint4(0u, 0u, 0u, 0u);
        else if (r < rows && TQ1_IN_BOUNDS(canon, rows * row_vecs, 50u)) dst[canon] = src[i];
    }
}

int check_panel_args(const void *a, const void *b, int N, int K, const char *who) {
    if (!a || !b) return fail(TQ1_ERR_INVALID, "%s: null pointer", who);
    if (N <= 0 || K <= 0 || K % 512)
        return fail(TQ1_ERR_INVALID, "%s: needs positive dimensions and K %% 512 == 0 (got %dx%d)", who, N, K);
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15)
        return fail(TQ1_ERR_INVALID, "%s: both arrays must be 16-byte aligned", who);
    return TQ1_OK;
}

template <bool TO_PANELS>
int launch_panels(const uint8_t *src, uint8_t *dst, int N, int K, cudaStream_t stream, const char *who) {
    const int chunks = K / 512;
    const long long pad = panel_pad_rows(N);
    const long long total = (long long)chunks * pad * kPanelRowVecs;
    long long ctas = (total + 255) / 256;
    if (ctas > 148 * 16) ctas = 148 * 16;
    panels_kernel<TO_PANELS><<<(unsigned)ctas, 256, 0, stream>>>(reinterpret_cast<const uint4 *>(src),
                                                               reinterpret_cast<uint4 *>(dst), N, pad, chunks);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, who);
    return TQ1_OK;
}

}  // namespace

}  // namespace tq1

using namespace tq1;

extern "C" {

size_t tq1_panel_bytes(int N, int K) {
    if (N <= 0 || K <= 0 || K % 512) return 0;
    return (size_t)(K / 512) * (size_t)panel_pad_rows(N) * kPanelRowBytes;
}

int tq1_blocks_to_panels_device(const uint8_t *blocks, uint8_t *panels, int N, int K, void *stream) {
    int rc = check_panel_args(blocks, panels, N, K, "tq1_blocks_to_panels_device");
    if (rc != TQ1_OK) return rc;
    return launch_panels<true>(blocks, panels, N, K, static_cast<cudaStream_t>(stream), "tq1_blocks_to_panels_device");
}

int tq1_panels_to_blocks_device(const uint8_t *panels, uint8_t *blocks, int N, int K, void *stream) {
    int rc = check_panel_args(panels, blocks, N, K, "tq1_panels_to_blocks_device");
    if (rc != TQ1_OK) return rc;
    return launch_panels<false>(panels, blocks, N, K, static_cast<cudaStream_t>(stream), "tq1_panels_to_blocks_device");
}

}  // extern "C"
