// Batched linear (M >= 2 activation rows) for TQ1_G128 on sm_100a: trits are decoded into
// FP16 tiles in tensor memory (weights) and shared memory (activations) that feed tcgen05.mma with
// FP32 accumulators in tensor memory.
//
// Stands in for the reference's prefill GEMM and small-batch kernels behind packed_matmul
// (src/ternel_mlx/kernels.py:409-858,1287-1357; src/ternel_mlx/modules.py:425-457). As in
// the reference's GEMM, the group scale is folded into the FP16 weight, which is exact:
// (c-1)*s is -s, 0 or +s (src/ternel_mlx/kernels.py:435-440).
//
// An output tile is 128 weight rows x NT activation rows:
//   D[n][m] = sum_k W[n][k] * x[m][k]      (A = W tile, B = x tile, both K-major FP16)
// Persistent CTAs (one per SM, two for the 16-token tiles). Every CTA first computes the same number
// of whole tiles; the leftover tiles are shared stream-K fashion: their (tile, K block) iterations,
// numbered tile-major, are cut into equal contiguous ranges, so every CTA does the same number of K
// blocks whatever the tile count. A range is a sequence of segments; a segment that covers a tile's
// whole K range is stored as the result, a partial one (only the first or last of a CTA's range) goes
// to the workspace as FP32 and a fix-up kernel adds the pieces of such a tile in ascending K order
// (deterministic).
//   warps 0-3, 4-7  decode: thread r of a group turns row r's 28-byte block into 128 FP16 values
//              and stores them with tcgen05.st into lane r of tensor memory, where the MMA reads
//              its A operand (the weights never pass through shared memory); the two groups take
//              alternate K blocks. After a segment's K loop warps 0-3 read the accumulator (TMEM
//              lane r = weight row r) and store it, then release it to the MMA warp
//   one warp   TMA: packed weight bytes (box 128 rows x 112 B = 4 groups) and activation tiles
//   one warp   allocates tensor memory and issues tcgen05.mma (one elected lane)
//   warps 8-11 (persistent kernel, 32- to 128-token tiles only) read finished accumulators and store
//              the results while the MMA warp fills a second accumulator with the next segment
//
// K order. Five trits per byte do not pair up in natural order, so inside every 128-wide
// group the K axis is permuted to a decode-friendly order (position p -> column pi(p) below)
// and the activations are permuted the same way once per call by a small pre-pass kernel;
// a dot product does not care about the order of its terms.
//   p = 4j+i   (j<25, i<4) : trit i of code byte j          (column 5j+i)
//   p = 100,101,102        : the three tail trits           (columns 125,126,127)
//   p = 103                : trit 4 of code byte 0          (column 4)
//   p = 104+q  (q<24)      : trit 4 of code byte q+1        (column 5(q+1)+4)
#include <cuda.h>
#include <stdlib.h>

#include "tq1_common.cuh"

namespace tq1 {

namespace {

constexpr int kTileW = 128;                 // weight rows per tile (UMMA M)
constexpr int kPackGroups = 4;
constexpr int kPackBytes = kTileW * kPackGroups * kBlockBytes;     // 14336
// Warp roles. Plain variant (320 threads): warps 0-3 and 4-7 decode, warp 8 TMA, warp 9 MMA, and the first
// decode group also stores the results. Variant with epilogue warps (448 threads, persistent kernel with
// 32- to 128-token tiles): warps 8-11 store the results out of a second accumulator while the MMA warp is
// already filling the other one; TMA and MMA move to warps 12 and 13.
__host__ __device__ constexpr bool gemm_epi_warps(int nt, bool persist) { return persist && nt >= 32 && nt <= 128; }
__host__ __device__ constexpr int gemm_threads(int nt, bool persist) { return gemm_epi_warps(nt, persist) ? 448 : 320; }
constexpr int kAStageCols = kGroup / 2;      // a 128-wide K block of FP16 weights = 64 tensor-memory columns
// Small activation tiles: three stages and little shared memory, so that two CTAs share an SM and
// hide each other's latencies. Large tiles: one CTA per SM with as many stages as fit.
__host__ __device__ constexpr int gemm_stages(int nt) { return nt > 128 ? 3 : nt <= 16 ? 3 : 4; }
// The decode table is replicated per lane (8-byte entries x 32 lanes, conflict-free) except for the
// 256-token tile: there the tensor cores set the pace, the lookups' bank conflicts are hidden, and
// the 60 KB saved by a single copy of the table pay for a third 64 KB activation stage.
// 256 entries (the 13 past 242 decode to zero weights): the table is indexed by the raw code byte, so a byte
// that escaped the load-time scan still reads inside the table instead of past the CTA's shared memory.
__host__ __device__ constexpr int gemm_lut_bytes(int nt) { return nt > 128 ? 2048 : 256 * 256; }
__host__ __device__ constexpr int gemm_tmem_cols(int nt) { return nt <= 16 ? 256 : 512; }
// packed-byte buffers (4 K blocks each): small activation tiles leave room for a deep prefetch queue,
// which is what hides HBM latency when the tensor work per K block is tiny
__host__ __device__ constexpr int gemm_pack_bufs(int nt) { return (nt == 32 || nt == 64) ? 6 : 2; }
constexpr uint32_t kSpinLimit = 1u << 24;

__host__ __device__ constexpr int perm_column(int p) {
    return p < 100 ? 5 * (p >> 2) + (p & 3) : p < 103 ? 125 + (p - 100) : p == 103 ? 4 : 5 * (p - 103) + 4;
}

// Decode table image: entry v = two words per lane.
//   word0: PRMT selector of (trit0, trit1) in bits 0-15, the 8-bit selector of trit4 in byte 2 and byte 3
//   word1: PRMT selector of (trit2, trit3) in bits 0-15
// An 8-bit selector picks the two bytes of one FP16 value out of the pool
// [0x00, s_lo, s_hi, s_hi ^ 0x80]: code 0 -> -s = (1,3), code 1 -> 0 = (0,0), code 2 -> +s = (1,2).
struct GemmLutImage {
    uint32_t w[256 * 64];
};
constexpr uint32_t sel8(uint32_t c) { return c == 0 ? 0x31u : c == 1 ? 0x00u : 0x21u; }
constexpr GemmLutImage make_gemm_lut() {
    GemmLutImage img{};
    for (int v = 0; v < 243; ++v) {
        uint32_t c[5] = {0, 0, 0, 0, 0};
        int t = v;
        for (int d = 0; d < 5; ++d) { c[d] = (uint32_t)(t % 3); t /= 3; }
        const uint32_t w0 = sel8(c[0]) | (sel8(c[1]) << 8) | (sel8(c[4]) << 16) | (sel8(c[4]) << 24);
        const uint32_t w1 = sel8(c[2]) | (sel8(c[3]) << 8);
        for (int l = 0; l < 32; ++l) {
            img.w[v * 64 + 2 * l] = w0;
            img.w[v * 64 + 2 * l + 1] = w1;
        }
    }
    return img;
}
__device__ __align__(128) const GemmLutImage g_gemm_lut = make_gemm_lut();
struct GemmLutSmall { uint32_t w[512]; };
constexpr GemmLutSmall make_gemm_lut_small() {
    GemmLutSmall img{};
    const GemmLutImage big = make_gemm_lut();
    for (int v = 0; v < 243; ++v) { img.w[2 * v] = big.w[v * 64]; img.w[2 * v + 1] = big.w[v * 64 + 1]; }
    return img;
}
__device__ __align__(128) const GemmLutSmall g_gemm_lut_small = make_gemm_lut_small();

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Bounded wait: returns false (after flagging *status) instead of hanging.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned *status) {
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (++spins > kSpinLimit) {
            atomicExch(status, 3u);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

// A operand in tensor memory (lane = weight row, 8 columns per K = 16 step), B in shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// 32 consecutive columns of this thread's tensor-memory lane <- 32 registers
__device__ __forceinline__ void tmem_store32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}

// Stream-K work split: the (output tile, K block) iterations, numbered tile-major, are dealt out in equal
// contiguous ranges to the CTAs. A range is a sequence of segments (tile, first K block, K blocks); only a
// CTA's first and last segment can cover part of a tile's K range.
//
// With fewer tiles than CTA slots the ranges are instead `splits` equal parts of every tile, cut at
// multiples of four K blocks (the packed-byte chunk), so that no CTA straddles two tiles or loads a
// chunk it uses only in part.
struct WorkSplit {
    int total_iters, ctas, groups, splits;      // splits == 0: equal contiguous ranges
    int quot, rem;                              // total_iters = ctas * quot + rem: the first `rem` ranges get one more
    // Stream-K mode only: every CTA first computes `whole_rounds` whole tiles (tiles cta * whole_rounds + k),
    // and only the remaining tiles, numbered from whole_tiles on, are cut into ranges (total_iters counts
    // their iterations). Whole tiles need neither a partial store nor the fix-up.
    int whole_rounds, whole_tiles;
    int tiles_total;                            // output tiles of the call (a CTA's last whole tiles may lie beyond)
    __host__ __device__ __forceinline__ int first_iter(int cta) const {
        if (cta >= ctas) return total_iters;
        if (splits == 0) return cta * quot + (cta < rem ? cta : rem);
        const int tile = cta / splits, part = cta - tile * splits;
        int kb = groups * part / splits;
        if (groups >= 4 * splits) kb &= ~3;
        return tile * groups + kb;
    }
};

struct GemmParams {
    const __half *xperm;      // permuted activations [M][K]
    void *y;                  // final output [M][N] (FP16/FP32)
    float *partials;          // [2 * CTAs][NT][128] FP32: K-partial tiles of the CTAs' first and last segments
    unsigned *status;
    int M, N, K;
    int tiles_m;              // activation tiles; output tile t covers weight tile t / tiles_m, token tile t % tiles_m
    WorkSplit work;           // which (tile, K block) iterations each CTA takes
    int y_f32;
    int swiglu;               // weight rows are (gate, up) pairs: y[m][n / 2] = silu(gate) * up, row length N / 2
};

// PERSIST = false: the CTA's range is known to be one segment (the equal-parts split), and the
// segment loops below compile to straight-line code.
// A CTA's segments in order: its whole tiles, then the pieces of its range of the shared tiles. Holds
// copies of the few numbers it needs: a reference to the kernel parameter would force the whole
// parameter block into local memory.
struct SegmentWalk {
    int groups, whole_rounds, whole_tiles, tiles_total, cta, round, it, end, pieces;
    __device__ __forceinline__ SegmentWalk(const WorkSplit work, int cta_)
        : groups(work.groups), whole_rounds(work.whole_rounds), whole_tiles(work.whole_tiles),
          tiles_total(work.tiles_total), cta(cta_), round(0),
          it(work.first_iter(cta_)), end(work.first_iter(cta_ + 1)), pieces(0) {}
    // slot: which of the CTA's two partial-tile slots a partial segment is stored to
    __device__ __forceinline__ bool next(int &tile, int &kb0, int &len, int &slot) {
        if (round < whole_rounds && cta * whole_rounds + round < tiles_total) {
            tile = cta * whole_rounds + round++;
            kb0 = 0;
            len = groups;
            slot = 0;
            return true;
        }
        if (it >= end) return false;
        const int t = it / groups;
        kb0 = it - t * groups;
        len = min(groups - kb0, end - it);
        tile = whole_tiles + t;
        slot = pieces++ == 0 ? 0 : 1;
        it += len;
        return true;
    }
};

template <int NT, bool PERSIST>
__global__ void __launch_bounds__(gemm_threads(NT, PERSIST), NT <= 16 ? 2 : 1)
tq1_gemm_tc_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                   const GemmParams prm) {
    constexpr bool kEpi = gemm_epi_warps(NT, PERSIST);
    constexpr int kTmaWarp = kEpi ? 12 : 8, kMmaWarp = kEpi ? 13 : 9;
    constexpr int kAccBufs = kEpi ? 2 : 1;
    // without epilogue warps, tiles of 64 tokens and more are stored by both decode groups, half the
    // token columns each (the store is not overlapped with anything there)
    constexpr bool kBothStore = !kEpi && NT >= 64;
    constexpr int kStagesG = gemm_stages(NT);
    constexpr int kPackBufs = gemm_pack_bufs(NT);
    constexpr int kBTileBytes = NT * kGroup * 2;
    constexpr int kTmemCols = gemm_tmem_cols(NT);    // accumulator (NT columns) + A stages
    constexpr int kAccCols = NT < 32 ? 32 : NT;
    constexpr int kAStageBase = kAccBufs * kAccCols;     // tensor-memory columns: accumulator(s), then the A stages
    static_assert(kAStageBase + kStagesG * kAStageCols <= kTmemCols, "tensor memory budget");
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // swizzled operand tiles must start on a 1024-byte boundary of the shared window
    unsigned char *smem = smem_raw + ((1024u - ((uint32_t)__cvta_generic_to_shared(smem_raw) & 1023u)) & 1023u);
    unsigned char *b_tiles = smem;                                       // kStagesG x NT*256, 1024-aligned
    unsigned char *packed = b_tiles + kStagesG * kBTileBytes;            // 2 x 14336
    unsigned char *lut = packed + kPackBufs * kPackBytes;                // 62208
    constexpr int kLutBytes = gemm_lut_bytes(NT);
    uint64_t *bars = reinterpret_cast<uint64_t *>(lut + kLutBytes);
    // barrier indices
    constexpr int FULL_A = 0, FULL_B = FULL_A + kStagesG, EMPTY = FULL_B + kStagesG, PACK_FULL = EMPTY + kStagesG,
                  PACK_EMPTY = PACK_FULL + kPackBufs, ACCUM = PACK_EMPTY + kPackBufs, ACC_FREE = ACCUM + 2,
                  LUT_BAR = ACC_FREE + 2, NUM_BARS = LUT_BAR + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + NUM_BARS);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    const int groups = prm.K / kGroup;
    // Without the persistent loop the CTA's range is one piece of one tile; it is worked out here once,
    // so that the walker and the loops around the segments compile away.
    const int only_begin = PERSIST ? 0 : prm.work.first_iter(blockIdx.x);
    const int only_end = PERSIST ? 0 : prm.work.first_iter(blockIdx.x + 1);
    auto first_segment = [&](SegmentWalk &walk, int &tile, int &kb0, int &len, int &slot) -> bool {
        if (PERSIST) return walk.next(tile, kb0, len, slot);
        tile = only_begin / groups;
        kb0 = only_begin - tile * groups;
        len = only_end - only_begin;
        slot = 0;
        return false;
    };

    if (tid == 0) {
        for (int s = 0; s < kStagesG; ++s) {
            mbar_init(bar(FULL_A + s), 128);
            mbar_init(bar(FULL_B + s), 1);
            mbar_init(bar(EMPTY + s), 1);
        }
        for (int p = 0; p < kPackBufs; ++p) {
            mbar_init(bar(PACK_FULL + p), 1);
            mbar_init(bar(PACK_EMPTY + p), 256);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(ACCUM + b), 1);
            mbar_init(bar(ACC_FREE + b), kBothStore ? 256 : 128);
        }
        mbar_init(bar(LUT_BAR), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(bar(LUT_BAR), kLutBytes);
        if (kLutBytes == 2048)
            bulk_load((uint32_t)__cvta_generic_to_shared(lut), &g_gemm_lut_small, kLutBytes, bar(LUT_BAR));
        else
            bulk_load((uint32_t)__cvta_generic_to_shared(lut), &g_gemm_lut, kLutBytes, bar(LUT_BAR));
    }
    if (warp == kMmaWarp) {        // tensor-memory allocation is a warp-wide operation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"((uint32_t)__cvta_generic_to_shared(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    bool ok = true;
    // Result of one segment out of accumulator `acc_col` (TMEM lane = weight row r of the tile, read by a
    // warp whose index modulo 4 names its 32 lanes). A segment that covers the tile's whole K range is
    // stored as the result; a partial one goes to this CTA's first- or last-segment slot as FP32 and is
    // added up by the fix-up kernel.
    auto store_segment = [&](int which, int len, int n0, int m0, uint32_t acc_col, int c_begin, int c_end) {
        const int r = (warp & 3) * 32 + lane;
        const bool whole = len == groups;
        float *slot = prm.partials + ((size_t)2 * blockIdx.x + which) * (size_t)(NT * kTileW);
        const int n = n0 + r;
        if (whole && prm.swiglu) {
            // (gate, up) row pairs: the even row of a pair stores silu(gate) * up. Kept apart from the plain
            // loop below, which is on the critical path of the large tiles.
#pragma unroll 1
            for (int c0 = c_begin; c0 < c_end; c0 += 32) {
                uint32_t v[32];
                if (NT >= 32 || c0 == 0) {
                    tmem_load32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + acc_col + (uint32_t)c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                }
#pragma unroll 4
                for (int c = 0; c < 32; ++c) {
                    const int m = m0 + c0 + c;
                    const float gate = __uint_as_float(v[c]);
                    const float up = __shfl_down_sync(0xffffffffu, gate, 1);
                    if (c0 + c < NT && m < prm.M && n + 1 < prm.N && (r & 1) == 0) {
                        const float out = swiglu_f32(gate, up);
                        const size_t o = (size_t)m * (prm.N >> 1) + (n >> 1);
                        if (!TQ1_IN_BOUNDS(o, (size_t)prm.M * (prm.N >> 1), 40u)) continue;
                        if (prm.y_f32) static_cast<float *>(prm.y)[o] = out;
                        else static_cast<__half *>(prm.y)[o] = __float2half_rn(out);
                    }
                }
            }
            return;
        }
#pragma unroll 1
        for (int c0 = c_begin; c0 < c_end; c0 += 32) {
            uint32_t v[32];
            if (NT >= 32 || c0 == 0) {
                tmem_load32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + acc_col + (uint32_t)c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            }
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const int m = m0 + c0 + c;
                if (c0 + c < NT && m < prm.M && n < prm.N) {
                    const float f = __uint_as_float(v[c]);
                    if (!TQ1_IN_BOUNDS(whole ? (size_t)m * prm.N + n : (size_t)(c0 + c) * kTileW + r,
                                       whole ? (size_t)prm.M * prm.N : (size_t)NT * kTileW, whole ? 40u : 41u))
                        continue;
                    if (!whole)
                        slot[(c0 + c) * kTileW + r] = f;
                    else if (prm.y_f32)
                        static_cast<float *>(prm.y)[(size_t)m * prm.N + n] = f;
                    else
                        static_cast<__half *>(prm.y)[(size_t)m * prm.N + n] = __float2half_rn(f);
                }
            }
        }
    };
    if (warp == kTmaWarp) {
        // ------------------------------------------------------------------ TMA producers
        // lane 1 keeps the queue of packed-byte chunks full, lane 0 feeds the activation tiles;
        // the two run independently so that the weight prefetch can run several chunks ahead
        if (lane == 1) {
            int pack_i = 0, tile, kb0, len, which;
            SegmentWalk walk(prm.work, blockIdx.x);
            bool more = first_segment(walk, tile, kb0, len, which);
            do {
                const int n0 = (tile / prm.tiles_m) * kTileW;
                const int first_chunk = kb0 / kPackGroups, last_chunk = (kb0 + len - 1) / kPackGroups;
                for (int c = first_chunk; c <= last_chunk && ok; ++c, ++pack_i) {
                    const int p = pack_i % kPackBufs;
                    ok = mbar_wait(bar(PACK_EMPTY + p), ((uint32_t)(pack_i / kPackBufs) & 1u) ^ 1u, prm.status);
                    if (!ok) break;
                    mbar_expect_tx(bar(PACK_FULL + p), kPackBytes);
                    tma_load_2d((uint32_t)__cvta_generic_to_shared(packed + p * kPackBytes), &wmap,
                                c * (kPackGroups * kBlockBytes), n0, bar(PACK_FULL + p));
                }
                if (PERSIST) more = walk.next(tile, kb0, len, which);
            } while (PERSIST && more && ok);
        } else if (lane == 0) {
            int i = 0, tile, kb0, len, which;
            SegmentWalk walk(prm.work, blockIdx.x);
            bool more = first_segment(walk, tile, kb0, len, which);
            do {
                const int m0 = (tile % prm.tiles_m) * NT;
                for (int kb = kb0; kb < kb0 + len && ok; ++kb, ++i) {
                    const int s = i % kStagesG;
                    ok = mbar_wait(bar(EMPTY + s), ((uint32_t)(i / kStagesG) & 1u) ^ 1u, prm.status);
                    if (!ok) break;
                    mbar_expect_tx(bar(FULL_B + s), kBTileBytes);
                    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(b_tiles + s * kBTileBytes);
                    tma_load_2d(dst, &xmap, kb * kGroup, m0, bar(FULL_B + s));
                    tma_load_2d(dst + NT * 128, &xmap, kb * kGroup + 64, m0, bar(FULL_B + s));
                }
                if (PERSIST) more = walk.next(tile, kb0, len, which);
            } while (PERSIST && more && ok);
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // instruction descriptor: FP32 accumulate, FP16 A and B, both K-major, M = 128, N = NT
            const uint32_t idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(kTileW >> 4) << 24);
            int i = 0, seg = 0, tile, kb0, len, which;
            SegmentWalk walk(prm.work, blockIdx.x);
            bool more = first_segment(walk, tile, kb0, len, which);
            do {
                // the accumulator's previous contents must have been read out
                const int buf = seg % kAccBufs, use = seg / kAccBufs;
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kAccCols);
                if (PERSIST && use > 0) ok = mbar_wait(bar(ACC_FREE + buf), (uint32_t)(use - 1) & 1u, prm.status);
                for (int ii = 0; ii < len && ok; ++ii, ++i) {
                    const int s = i % kStagesG;
                    const uint32_t ph = (uint32_t)(i / kStagesG) & 1u;
                    ok = mbar_wait(bar(FULL_A + s), ph, prm.status) && mbar_wait(bar(FULL_B + s), ph, prm.status);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_tmem = tmem_base + (uint32_t)(kAStageBase + s * kAStageCols);
                    const uint32_t b_addr = (uint32_t)__cvta_generic_to_shared(b_tiles + s * kBTileBytes);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {           // eight K = 16 steps; B: two 64-wide swizzle atoms
                        const uint64_t db = umma_desc(b_addr + (j >> 2) * (NT * 128) + (j & 3) * 32);
                        umma_f16_ts(d_tmem, a_tmem + 8u * j, db, idesc, (ii > 0 || j > 0) ? 1u : 0u);
                    }
                    umma_commit(bar(EMPTY + s));            // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(bar(ACCUM + buf));      // the segment's accumulator is complete
                ++seg;
                if (PERSIST) more = walk.next(tile, kb0, len, which);
            } while (PERSIST && more && ok);
        }
    } else if (kEpi && warp >= 8) {
        // ------------------------------------------------------------------ epilogue warps 8-11
        int seg = 0, tile, kb0, len, which;
        SegmentWalk walk(prm.work, blockIdx.x);
        bool more = first_segment(walk, tile, kb0, len, which);
        do {
            const int buf = seg % kAccBufs, use = seg / kAccBufs;
            ok = mbar_wait(bar(ACCUM + buf), (uint32_t)use & 1u, prm.status);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            store_segment(which, len, (tile / prm.tiles_m) * kTileW, (tile % prm.tiles_m) * NT,
                          (uint32_t)(buf * kAccCols), 0, NT);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(bar(ACC_FREE + buf));
            ++seg;
            if (PERSIST) more = walk.next(tile, kb0, len, which);
        } while (more);
    } else {
        // ------------------------------------------------------------------ decode (thread = weight row)
        // two groups of four warps take alternate K blocks, so two stages are being filled at a time
        const int group = warp < 4 ? 0 : 1;
        const int r = (warp & 3) * 32 + lane;            // 0..127 = tensor-memory lane (a warp reaches lanes 32*(warp%4)..)
        ok = mbar_wait(bar(LUT_BAR), 0, prm.status);
        const uint32_t lut_lane = (uint32_t)__cvta_generic_to_shared(lut) + (kLutBytes == 2048 ? 0u : (uint32_t)lane * 8u);
        constexpr int kLutShift = kLutBytes == 2048 ? 3 : 8;
        int pack_i = -1, i = 0, seg = 0, tile, kb0, len, which;
        SegmentWalk walk(prm.work, blockIdx.x);
        bool more = first_segment(walk, tile, kb0, len, which);
        do {
        const int n0 = (tile / prm.tiles_m) * kTileW;       // first weight row of the tile
        const int m0 = (tile % prm.tiles_m) * NT;           // first activation row
        for (int ii = 0; ii < len && ok; ++ii, ++i) {
            const int kb = kb0 + ii;
            if (ii == 0 || (kb % kPackGroups) == 0) {
                ++pack_i;
                ok = mbar_wait(bar(PACK_FULL + pack_i % kPackBufs), (uint32_t)(pack_i / kPackBufs) & 1u, prm.status);
                if (!ok) break;
            }
            const bool last_of_chunk = (kb % kPackGroups) == kPackGroups - 1 || ii == len - 1;
            if ((i & 1) != group) {                      // the other group's K block
                if (last_of_chunk) mbar_arrive(bar(PACK_EMPTY + pack_i % kPackBufs));
                continue;
            }
            const int s = i % kStagesG;
            ok = mbar_wait(bar(EMPTY + s), ((uint32_t)(i / kStagesG) & 1u) ^ 1u, prm.status);
            if (!ok) break;

            const uint32_t *blk = reinterpret_cast<const uint32_t *>(
                packed + (pack_i % kPackBufs) * kPackBytes + (r * kPackGroups + (kb % kPackGroups)) * kBlockBytes);
            uint32_t w[7];
#pragma unroll
            for (int k = 0; k < 7; ++k) w[k] = blk[k];
            const uint32_t sbits = w[0] & 0xffffu;
            const uint32_t pool = (sbits << 8) | (((sbits >> 8) ^ 0x80u) << 24);
            // table entries of the 26 code bytes
            uint32_t e0[26], e1[26];
#pragma unroll
            for (int j = 0; j < 26; ++j) {
                const int bytepos = 2 + j;
                const uint32_t byte = (w[bytepos >> 2] >> (8 * (bytepos & 3))) & 0xffu;
                const uint32_t addr = lut_lane + (byte << kLutShift);
                asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(e0[j]), "=r"(e1[j]) : "r"(addr));
            }
            // 64 registers = the row's 128 FP16 weights in decode order, written to this lane of tensor memory
            const uint32_t a_taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) +
                                     (uint32_t)(kAStageBase + s * kAStageCols);
            {
                uint32_t v[32];
#pragma unroll
                for (int m = 0; m < 8; ++m) {
                    v[4 * m] = prmt(pool, 0u, e0[2 * m]);
                    v[4 * m + 1] = prmt(pool, 0u, e1[2 * m]);
                    v[4 * m + 2] = prmt(pool, 0u, e0[2 * m + 1]);
                    v[4 * m + 3] = prmt(pool, 0u, e1[2 * m + 1]);
                }
                tmem_store32(a_taddr, v);
            }
            {
                // trit-4 pairs: selector byte 0 from entry a (its byte 2), byte 1 from entry b (its byte 3)
                auto c4pair = [&](int ja, int jb) { return prmt(pool, 0u, prmt(e0[ja], e0[jb], 0x4472)); };
                uint32_t v[32];
#pragma unroll
                for (int m = 8; m < 12; ++m) {
                    v[4 * (m - 8)] = prmt(pool, 0u, e0[2 * m]);
                    v[4 * (m - 8) + 1] = prmt(pool, 0u, e1[2 * m]);
                    v[4 * (m - 8) + 2] = prmt(pool, 0u, e0[2 * m + 1]);
                    v[4 * (m - 8) + 3] = prmt(pool, 0u, e1[2 * m + 1]);
                }
                v[16] = prmt(pool, 0u, e0[24]);
                v[17] = prmt(pool, 0u, e1[24]);
                v[18] = prmt(pool, 0u, e0[25]);
                v[19] = prmt(pool, 0u, prmt(e1[25], e0[0], 0x4470));      // (tail trit 2, trit 4 of byte 0)
#pragma unroll
                for (int q = 0; q < 12; ++q) v[20 + q] = c4pair(2 * q + 1, 2 * q + 2);
                tmem_store32(a_taddr + 32u, v);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(bar(FULL_A + s));
            if (last_of_chunk) mbar_arrive(bar(PACK_EMPTY + pack_i % kPackBufs));
        }

        if (!kEpi) {         // the decode warps also store the segment's result
            const bool storing = kBothStore || group == 0;
            if (ok && storing) ok = mbar_wait(bar(ACCUM), (uint32_t)seg & 1u, prm.status);
            if (ok && storing) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (kBothStore) store_segment(which, len, n0, m0, 0u, group * (NT / 2), (group + 1) * (NT / 2));
                else store_segment(which, len, n0, m0, 0u, 0, NT);
                // the accumulator columns may be overwritten by the next segment
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(bar(ACC_FREE));
            }
        }
        ++seg;
        if (PERSIST) more = walk.next(tile, kb0, len, which);
        } while (PERSIST && more && ok);   // segments
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                     : "memory");
    }
}

// x' = x with the K axis of every group permuted to the decode order. Half a warp moves one group of 128
// values: a 16-byte load per lane into shared memory, eight 2-byte picks at the permuted positions, a 16-byte
// store (the one-value-per-thread version took 28 us for 2048 x 5120 activations, a tenth of that call).
__global__ void __launch_bounds__(256) tq1_permute_x_kernel(const __half *__restrict__ x, __half *__restrict__ xp,
                                                            long long groups) {
    __shared__ __align__(16) unsigned short stage[16][kGroup];
    const int lane = threadIdx.x & 31, half = lane >> 4, l16 = lane & 15;
    const int slot = (threadIdx.x >> 5) * 2 + half;             // this half-warp's staging row
    int src[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) src[k] = perm_column(8 * l16 + k);
    for (long long g = (long long)blockIdx.x * 16 + slot; g < groups + slot; g += (long long)gridDim.x * 16) {
        const bool live = g < groups;                            // both halves of a warp stay in step
        if (live) *reinterpret_cast<uint4 *>(&stage[slot][8 * l16]) = *reinterpret_cast<const uint4 *>(x + g * kGroup + 8 * l16);
        __syncwarp();
        if (live) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) w[k] = (uint32_t)stage[slot][src[2 * k]] | ((uint32_t)stage[slot][src[2 * k + 1]] << 16);
            *reinterpret_cast<uint4 *>(xp + g * kGroup + 8 * l16) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        __syncwarp();
    }
}

// The same permutation, one value per thread: less latency for the few rows of a decode batch.
__global__ void tq1_permute_x_small_kernel(const __half *__restrict__ x, __half *__restrict__ xp, long long total) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int p = (int)(i & 127);
    xp[i] = x[i - p + perm_column(p)];
}

// Fix-up for output tiles whose K range was shared by several CTAs: adds their FP32 partial tiles in
// ascending K order (CTA order), so the result does not depend on timing. blockIdx.x + 1 names a boundary
// between two CTAs' ranges; the block of the first boundary inside a tile handles that tile (eight token
// columns per block in blockIdx.y, one thread per weight row). Tiles computed by one CTA were stored directly.
// kFixCols token columns per thread: many small blocks where the tiles to complete are few (the call is
// latency-bound there), sixteen columns for prefill shapes (fewer waves of blocks, more loads in flight).
#ifndef TQ1_FIX_COLS_SMALL
#define TQ1_FIX_COLS_SMALL 4
#endif
template <int kFixCols>
__global__ void __launch_bounds__(kTileW)
tq1_streamk_fixup_kernel(const float *__restrict__ partials, void *__restrict__ y, int y_f32,
                         int M, int N, int tiles_m, const WorkSplit work, int nt, int swiglu) {
    const int groups = work.groups, ctas = work.ctas;
    int c_lo, c_hi, tile, it0;
    if (work.splits > 0) {                       // every tile in equal parts: blockIdx.x names the tile
        tile = blockIdx.x;
        c_lo = tile * work.splits;
        c_hi = c_lo + work.splits - 1;
        it0 = tile * groups;
    } else {
        c_lo = blockIdx.x;                                             // the CTA before the boundary
        const int it_b = work.first_iter(c_lo + 1);
        if (it_b % groups == 0) return;                                // the boundary falls between two tiles
        tile = it_b / groups;                                          // among the shared tiles
        it0 = tile * groups;
        if (work.first_iter(c_lo) > it0) return;                       // an earlier boundary lies in this tile
        c_hi = c_lo + 1;
        while (c_hi + 1 < ctas && work.first_iter(c_hi + 1) < it0 + groups) ++c_hi;
    }
    const int r = threadIdx.x;
    const int out_tile = work.splits > 0 ? tile : work.whole_tiles + tile;
    const int n = (out_tile / tiles_m) * kTileW + r;
    const int m0 = (out_tile % tiles_m) * nt;
    const int c0 = blockIdx.y * kFixCols;
    const bool live = n < N;
    float total[kFixCols];
#pragma unroll
    for (int c = 0; c < kFixCols; ++c) total[c] = 0.0f;
    for (int cta = c_lo; cta <= c_hi; ++cta) {
        // the tile is that CTA's first segment if its range starts inside the tile, else its last one
        const int which = work.splits > 0 || work.first_iter(cta) >= it0 ? 0 : 1;
        const float *slot = partials + ((size_t)2 * cta + which) * (size_t)(nt * kTileW) + (size_t)c0 * kTileW + r;
        float v[kFixCols];
#pragma unroll
        for (int c = 0; c < kFixCols; ++c) v[c] = live && m0 + c0 + c < M ? slot[c * kTileW] : 0.0f;
#pragma unroll
        for (int c = 0; c < kFixCols; ++c) total[c] += v[c];
    }
#pragma unroll
    for (int c = 0; c < kFixCols; ++c) {
        if (swiglu) {                       // (gate, up) row pairs: the even row stores silu(gate) * up
            const float up = __shfl_down_sync(0xffffffffu, total[c], 1);
            if (live && n + 1 < N && (r & 1) == 0 && m0 + c0 + c < M) {
                const float out = swiglu_f32(total[c], up);
                const size_t o = (size_t)(m0 + c0 + c) * (N >> 1) + (n >> 1);
                if (y_f32) static_cast<float *>(y)[o] = out;
                else static_cast<__half *>(y)[o] = __float2half_rn(out);
            }
            continue;
        }
        if (live && m0 + c0 + c < M) {
            const size_t o = (size_t)(m0 + c0 + c) * N + n;
            if (y_f32) static_cast<float *>(y)[o] = total[c];
            else static_cast<__half *>(y)[o] = __float2half_rn(total[c]);
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn gemm_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Launch state is per DEVICE: the SM count differs between devices and the shared-memory opt-in is an
// attribute of a function on one device, so a process that drives several GPUs needs one record each.
constexpr int kMaxDevices = 64;
int current_device_slot() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    return dev;
}
int sm_count_cached() {
    static int sm_count[kMaxDevices] = {};
    const int dev = current_device_slot();
    if (!sm_count[dev]) {
        if (cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count[dev] <= 0)
            sm_count[dev] = 148;
    }
    return sm_count[dev];
}

// Time per K block of one CTA by token tile, fitted to the recorded sweep (also used by token_tile()).
constexpr float kSharingCostUs = 18.0f;
float block_time_us(int nt) {
    return nt <= 16 ? 0.85f : nt == 32 ? 0.5f : nt == 64 ? 0.55f : 0.8f;
}

// How the (tile, K block) iterations of a shape are dealt out for a given token tile.
WorkSplit split_work(int nt, int M, int N, int K) {
    const long long tiles = (long long)((N + kTileW - 1) / kTileW) * ((M + nt - 1) / nt);
    const long long slots = (long long)sm_count_cached() * (nt <= 16 ? 2 : 1);
    WorkSplit w;
    w.groups = K / kGroup;
    w.total_iters = (int)(tiles * w.groups);
    w.whole_rounds = w.whole_tiles = 0;
    w.tiles_total = (int)tiles;
    // With more than half as many tiles as slots, cutting every tile in two would need a second wave and one
    // part per tile leaves up to half of the SMs idle: those shapes are shared stream-K fashion as well.
    if (tiles >= slots || (nt > 16 && 2 * tiles > slots)) {
        w.splits = 0;
        w.ctas = (int)slots;
        // whole tiles first; what is left over is shared. A share of fewer than eight K blocks per CTA
        // would cost more in partial stores than it balances, so then one round of whole tiles is shared too.
        long long rounds = tiles / slots;
        long long shared = tiles - rounds * slots;
        if (rounds > 0 && shared > 0 && shared * w.groups < 8 * slots) {
            --rounds;
            shared += slots;
        }
        // Sharing the leftover tiles saves the idle part of one more round of whole tiles, (1 - shared/slots) of
        // a tile's time, and costs the partial tiles' round trip through the workspace and the fix-up launch
        // (about 18 us measured at 256-token tiles). Short tiles that nearly fill a round run as whole tiles.
        if (rounds > 0 && shared > 0 && shared < slots &&
            (float)(slots - shared) / (float)slots * (float)w.groups * block_time_us(nt) < kSharingCostUs) {
            ++rounds;
            shared = 0;
        }
        w.whole_rounds = (int)rounds;
        w.whole_tiles = (int)(rounds * slots);
        w.total_iters = (int)(shared * w.groups);
        if (shared == 0) w.ctas = (int)(tiles < rounds * slots ? (tiles + rounds - 1) / rounds : slots);
    } else {
        int splits = (int)(slots / tiles);
        const int max_splits = w.groups / 8 > 0 ? w.groups / 8 : 1;
        if (splits > max_splits) splits = max_splits;
        if (splits > 32) splits = 32;
        w.splits = splits;
        w.ctas = (int)tiles * splits;
    }
    w.quot = w.total_iters / w.ctas;
    w.rem = w.total_iters % w.ctas;
    return w;
}

// Activation rows per tile. Up to 16 rows always take the 16-row tile. Beyond that the tile with
// the smallest modelled time wins: (K blocks a CTA processes) x (time per K block of that tile) +
// (segments a CTA stores) x (time to store one), with the five pairs of constants fitted to the
// recorded sweep in ternel_b200/dispatch_sweep_b200.json (tests replay the file: the choice is within
// 10% of the best recorded tile for every case). g_forced_tile overrides the rule while a sweep is
// being recorded.
int g_forced_tile = 0;
int token_tile(int M, int N, int K) {
    if (g_forced_tile) return g_forced_tile;
    if (M <= 16) return 16;
    static const int tiles[5] = {16, 32, 64, 128, 256};
    static const float per_block_us[5] = {0.85f, 0.5f, 0.55f, 0.8f, 0.8f};
    static const float per_store_us[5] = {0.0f, 1.0f, 1.0f, 0.0f, 2.0f};
    int best = 128;
    float best_cost = 0.0f;
    for (int i = 0; i < 5; ++i) {
        const int nt = tiles[i];
        if (nt > 16 && nt >= 4 * M) continue;           // a tile mostly of padding
        const WorkSplit w = split_work(nt, M, N, K);
        const float shared = (float)w.total_iters / w.ctas;           // K blocks of shared tiles per CTA
        const float blocks = w.splits ? (float)((w.groups + w.splits - 1) / w.splits)
                                      : (float)w.whole_rounds * w.groups + shared;
        const float stores = w.splits ? 1.0f
                                      : (float)w.whole_rounds + (w.total_iters ? shared / w.groups + 1.0f : 0.0f);
        const float cost = blocks * per_block_us[i] + stores * per_store_us[i];
        if (i == 0 || cost < best_cost) { best = nt; best_cost = cost; }
    }
    return best;
}

// CTAs of a launch: every resident slot (two per SM for the 16-token tiles). With at least as many
// tiles as slots the iterations are dealt out stream-K fashion; with fewer, every tile is cut into
// equal parts of at least eight K blocks.
WorkSplit pick_work(int M, int N, int K) { return split_work(token_tile(M, N, K), M, N, K); }

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

template <int NT>
size_t gemm_smem_bytes() {
    return (size_t)gemm_stages(NT) * NT * kGroup * 2 +
           (size_t)gemm_pack_bufs(NT) * kPackBytes + gemm_lut_bytes(NT) + 512 + 1024;
}

template <int NT, bool PERSIST>
int launch_nt(const CUtensorMap &wmap, const CUtensorMap &xmap, const GemmParams &prm, dim3 grid, cudaStream_t stream) {
    auto kern = tq1_gemm_tc_kernel<NT, PERSIST>;
    static bool attr_set[kMaxDevices] = {};
    const size_t smem = gemm_smem_bytes<NT>();
    const int dev = current_device_slot();
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "tq1_linear_f16: shared memory opt-in (GEMM)");
        attr_set[dev] = true;
    }
    kern<<<grid, gemm_threads(NT, PERSIST), smem, stream>>>(wmap, xmap, prm);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16: GEMM launch");
    return TQ1_OK;
}

}  // namespace

int gemm_tc_force_tile(int nt) {
    if (nt != 0 && nt != 16 && nt != 32 && nt != 64 && nt != 128 && nt != 256) return TQ1_ERR_INVALID;
    g_forced_tile = nt;
    return TQ1_OK;
}

void gemm_tc_plan(int M, int N, int K, int *tile, int *ctas, int *parts) {
    const WorkSplit w = pick_work(M, N, K);
    *tile = token_tile(M, N, K);
    *ctas = w.ctas;
    *parts = w.splits;
}

bool gemm_tc_shape_ok(int M, int N, int K) {
    return M >= 2 && N >= 1 && K % (kPackGroups * kGroup) == 0;
}

bool gemm_tc_supported(const uint8_t *blocks, const __half *x, int M, int N, int K) {
    return gemm_tc_shape_ok(M, N, K) && (reinterpret_cast<uintptr_t>(blocks) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(x) & 15) == 0;
}

size_t gemm_tc_workspace_bytes(int M, int N, int K) {
    const size_t slots = (size_t)2 * pick_work(M, N, K).ctas * token_tile(M, N, K) * kTileW * sizeof(float);
    return kWsScratchOffset + align256((size_t)M * K * sizeof(__half)) + align256(slots);
}

int launch_gemm_tc(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int M, int N, int K,
                   void *workspace, cudaStream_t stream, bool swiglu) {
    EncodeTiledFn encode = gemm_encode_fn();
    if (!encode) return fail(TQ1_ERR_CUDA, "tq1_linear_f16: cuTensorMapEncodeTiled is unavailable");
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    unsigned *status = reinterpret_cast<unsigned *>(ws);
    __half *xperm = reinterpret_cast<__half *>(ws + kWsScratchOffset);
    float *partials = reinterpret_cast<float *>(ws + kWsScratchOffset + align256((size_t)M * K * sizeof(__half)));
    const int nt = token_tile(M, N, K);
    const WorkSplit work = pick_work(M, N, K);
    const int ctas = work.ctas;

    const long long total = (long long)M * K;
    if (total <= (1 << 19)) {
        tq1_permute_x_small_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(x, xperm, total);
    } else {
        const long long total_groups = total / kGroup;
        const long long permute_ctas = (total_groups + 15) / 16;
        tq1_permute_x_kernel<<<(unsigned)(permute_ctas < 148 * 8 ? permute_ctas : 148 * 8), 256, 0, stream>>>(
            x, xperm, total_groups);
    }
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16: activation permute launch");

    CUtensorMap wmap, xmap;
    {
        const cuuint64_t row_bytes = (cuuint64_t)(K / kGroup) * kBlockBytes;
        const cuuint64_t dims[2] = {row_bytes, (cuuint64_t)N};
        const cuuint64_t strides[1] = {row_bytes};
        const cuuint32_t box[2] = {kPackGroups * kBlockBytes, kTileW};
        const cuuint32_t estr[2] = {1, 1};
        CUresult res = encode(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(blocks), dims, strides,
                              box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (res != CUDA_SUCCESS) return fail(TQ1_ERR_CUDA, "tq1_linear_f16: weight tensor map failed (%d)", (int)res);
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)K * sizeof(__half)};
        const cuuint32_t box[2] = {64, (cuuint32_t)nt};
        const cuuint32_t estr[2] = {1, 1};
        CUresult res = encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xperm, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (res != CUDA_SUCCESS)
            return fail(TQ1_ERR_CUDA, "tq1_linear_f16: activation tensor map failed (%d)", (int)res);
    }
    GemmParams prm;
    prm.xperm = xperm;
    prm.y = y;
    prm.partials = partials;
    prm.status = status;
    prm.M = M;
    prm.N = N;
    prm.K = K;
    prm.tiles_m = (M + nt - 1) / nt;
    prm.work = work;
    prm.y_f32 = y_f32 ? 1 : 0;
    prm.swiglu = swiglu ? 1 : 0;
    dim3 grid((unsigned)ctas);
    int rc;
    if (work.splits > 0)        // one segment per CTA
        rc = nt == 16 ? launch_nt<16, false>(wmap, xmap, prm, grid, stream)
           : nt == 32 ? launch_nt<32, false>(wmap, xmap, prm, grid, stream)
           : nt == 64 ? launch_nt<64, false>(wmap, xmap, prm, grid, stream)
           : nt == 128 ? launch_nt<128, false>(wmap, xmap, prm, grid, stream)
                       : launch_nt<256, false>(wmap, xmap, prm, grid, stream);
    else
        rc = nt == 16 ? launch_nt<16, true>(wmap, xmap, prm, grid, stream)
           : nt == 32 ? launch_nt<32, true>(wmap, xmap, prm, grid, stream)
           : nt == 64 ? launch_nt<64, true>(wmap, xmap, prm, grid, stream)
           : nt == 128 ? launch_nt<128, true>(wmap, xmap, prm, grid, stream)
                       : launch_nt<256, true>(wmap, xmap, prm, grid, stream);
    if (rc != TQ1_OK) return rc;
    const bool shared_tiles = work.splits > 1 || (work.splits == 0 && work.total_iters > 0 &&
                                                  (work.rem != 0 || work.quot % work.groups != 0));
    if (ctas > 1 && shared_tiles) {
        const unsigned fix_blocks = work.splits > 0 ? (unsigned)(ctas / work.splits) : (unsigned)(ctas - 1);
        const int cols = M < nt ? M : nt;
        // sixteen columns per thread only where four would mean several waves of blocks
        if ((long long)fix_blocks * ((cols + TQ1_FIX_COLS_SMALL - 1) / TQ1_FIX_COLS_SMALL) < 148 * 16)
            tq1_streamk_fixup_kernel<TQ1_FIX_COLS_SMALL>
                <<<dim3(fix_blocks, (unsigned)((cols + TQ1_FIX_COLS_SMALL - 1) / TQ1_FIX_COLS_SMALL)), kTileW, 0, stream>>>(
                    partials, y, prm.y_f32, M, N, prm.tiles_m, work, nt, prm.swiglu);
        else
            tq1_streamk_fixup_kernel<16><<<dim3(fix_blocks, (unsigned)((cols + 15) / 16)), kTileW, 0, stream>>>(
                partials, y, prm.y_f32, M, N, prm.tiles_m, work, nt, prm.swiglu);
        err = cudaGetLastError();
        if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16: stream-K fix-up launch");
    }
    return TQ1_OK;
}

}  // namespace tq1
