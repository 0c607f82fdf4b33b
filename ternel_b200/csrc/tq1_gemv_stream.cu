// Batch-1 streaming GEMV for TQ1_G128 on sm_100a: TMA-staged code bytes, a
// lane-replicated 243-entry base-3 table in shared memory, and exact integer
// dot products on the tensor cores (mma.sync m16n8k32 u8 x s8 -> s32).
//
// Stands in for the reference's GEMV kernels (cuda/tq1_g128_gemv.cu:81-140,
// cuda/tq1_lut23_streamk.cu:113-256, src/ternel_mlx/kernels.py:244-342) behind
// the same operator; it shares none of their structure.
//
// Why integers on the tensor cores. 128 weights arrive per 28 bytes, so at HBM
// speed an SM has about 1.2 issue slots per weight; one FP32 FMA per weight
// cannot keep up. Each group's 128 FP16 activations are therefore turned, once
// per CTA, into 23-bit block fixed point (a shared power-of-two exponent per
// group, which is as exact as FP32 accumulation) and split into three signed
// byte planes. The trits (as unsigned codes 0/1/2) are the A operand, the three
// planes are B columns, and the s32 accumulators hold exact group sums:
//     sum_k (c_k - 1) x_k = 2^(E-21) * (S0 + 256 S1 + 65536 S2 - sum_k xi_k)
// followed by acc = fma(scale_g, group_sum, acc) in FP32 as in the reference
// (src/bonsai_tq1/reference.py:33-38). Groups containing NaN/Inf activations
// take an FP32 path that multiplies every weight, so non-finite values
// propagate as in the reference.
//
// Work decomposition. A unit is 16 rows x 4 groups (1792 bytes, one TMA box).
// Units are numbered chunk-major and dealt out in contiguous ranges to the
// warps of 148 persistent CTAs, so a warp keeps its B fragments (the
// activation digits of one 512-wide K chunk) in registers while it streams row
// tiles. Per-chunk partial sums go to a workspace; the warp that completes a
// row tile (an arrival counter) adds the chunks in ascending order, so results
// do not depend on timing.
//
// Lane roles inside mma.m16n8k32 (g = lane/4, q = lane%4): lane (g,q) decodes
// half a block of row g and half a block of row g+8; q>>1 picks which of the
// sub-unit's two groups, q&1 which half. B columns 0..2 carry the three digit
// planes of the first group, columns 4..6 those of the second, and a B lane
// holds zeros for k-slots that belong to the other group, which keeps the two
// groups' sums apart in one instruction.
#include <cuda.h>

#include "tq1_common.cuh"

namespace tq1 {

namespace {

constexpr int kTileRows = 16;
constexpr int kChunkGroups = 4;
constexpr int kChunkBytes = kChunkGroups * kBlockBytes;      // 112
constexpr int kUnitBytes = kTileRows * kChunkBytes;          // 1792
constexpr int kStages = 4;
constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxChunksPerCta = 3;
constexpr int kRegsPerSub = 18;                               // A/B registers per lane per sub-unit

// Shared-memory window layout (addresses relative to the CTA's shared window).
// The table sits at a 64 KiB multiple so that PRMT can build a complete lookup
// address (byte << 8 | lane << 2 | table base) in one instruction.
constexpr uint32_t kLutWindowAddr = 131072;
constexpr uint32_t kLutBytes = 243 * 256;                     // 2 variants x 32 lanes x 4 B per entry
constexpr uint32_t kWindowEnd = kLutWindowAddr + kLutBytes;
constexpr uint32_t kRingBytes = kWarps * kStages * kUnitBytes;                   // 114688
constexpr uint32_t kBtabBytes = kMaxChunksPerCta * 2 * kRegsPerSub * 32 * 4;     // 13824
constexpr uint32_t kCarveBytes = kRingBytes + kBtabBytes + 16 * kMaxChunksPerCta * kChunkGroups +
                                 8 * kWarps * kStages + 3 * 4 * kWarps;
static_assert(kCarveBytes + 1024 + 128 <= kLutWindowAddr, "buffers must end below the table's fixed address");
constexpr uint32_t kMaxWaitSpins = 1u << 22;

struct GroupInfo {
    int sum;          // sum of the group's fixed-point activations
    float pow2;       // 2^(E-21)
    int nonfinite;    // the group holds a NaN or an Inf
    int pad;
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// Ring-buffer words: volatile so the loads stay behind the mbarrier wait.
template <int OFF>
__device__ __forceinline__ uint32_t lds_off(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF) : "memory");
    return v;
}

// Decode-table lookups: the table never changes after the prologue, so the compiler may schedule these freely.
template <int OFF>
__device__ __forceinline__ uint32_t lds_lut(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// Decode one lane-stream (half a block: 14 code-byte slots) into 18 A registers.
// wa..wd are the four 32-bit words holding the slots (wa: bytes 2,3 only).
__device__ __forceinline__ void decode_stream(uint32_t wa, uint32_t wb, uint32_t wc, uint32_t wd,
                                              uint32_t lane_base, uint32_t (&r)[kRegsPerSub]) {
    const uint32_t pool = 0x03020100u;
    uint32_t e[14];
    // slot s uses table variant A (c4 in byte 2) when s is even, B (c4 in byte 3) when odd
    e[0] = lds_lut<0>(prmt(wa, lane_base, 0x7624));
    e[1] = lds_lut<128>(prmt(wa, lane_base, 0x7634));
    e[2] = lds_lut<0>(prmt(wb, lane_base, 0x7604));
    e[3] = lds_lut<128>(prmt(wb, lane_base, 0x7614));
    e[4] = lds_lut<0>(prmt(wb, lane_base, 0x7624));
    e[5] = lds_lut<128>(prmt(wb, lane_base, 0x7634));
    e[6] = lds_lut<0>(prmt(wc, lane_base, 0x7604));
    e[7] = lds_lut<128>(prmt(wc, lane_base, 0x7614));
    e[8] = lds_lut<0>(prmt(wc, lane_base, 0x7624));
    e[9] = lds_lut<128>(prmt(wc, lane_base, 0x7634));
    e[10] = lds_lut<0>(prmt(wd, lane_base, 0x7604));
    e[11] = lds_lut<128>(prmt(wd, lane_base, 0x7614));
    e[12] = lds_lut<0>(prmt(wd, lane_base, 0x7624));
    e[13] = lds_lut<128>(prmt(wd, lane_base, 0x7634));
#pragma unroll
    for (int s = 0; s < 14; ++s) r[s] = prmt(pool, 0u, e[s]);       // nibbles c0..c3 -> four u8 codes
#pragma unroll
    for (int u = 0; u < 3; ++u) {
        const uint32_t x = e[4 * u] + e[4 * u + 1];                  // bytes 2,3 = c4 of slots 4u, 4u+1
        const uint32_t y = e[4 * u + 2] + e[4 * u + 3];
        r[14 + u] = prmt(x, y, 0x7632);
    }
    r[17] = prmt(e[12] + e[13], 0u, 0x4432);
}

// FP32 fallback for one block (row-major canonical bytes in shared memory) against
// FP16 activations in global memory: multiplies every weight so that NaN and Inf
// propagate exactly as in the reference.
__device__ float block_dot_fp32(const uint8_t *blk, const __half *xg) {
    float sum = 0.0f;
    for (int j = 0; j < kCodeBytes; ++j) {
        uint32_t v = blk[2 + j];
        const int n = j == 25 ? 3 : 5;
        for (int i = 0; i < n; ++i) {
            const float w = (float)((int)(v % 3u) - 1);
            v /= 3u;
            sum = fmaf(w, __half2float(xg[5 * j + i]), sum);
        }
    }
    return sum;
}

template <bool OUT_F32>
__global__ void __launch_bounds__(kThreads, 1)
tq1_gemv_stream_kernel(const __grid_constant__ CUtensorMap wmap, const __half *__restrict__ x,
                       void *__restrict__ y, int N, int K, int tiles, int chunks,
                       int *__restrict__ counters, float *__restrict__ partials,
                       unsigned *__restrict__ status) {
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t window = (uint32_t)__cvta_generic_to_shared(smem);   // window address of smem[0]
    // carve-up: [ring | btab | ginfo | mbarriers] then the table at a fixed window address
    unsigned char *ring = smem;                                          // 1024-aligned is plenty for TMA (16 B)
    uint32_t *btab = reinterpret_cast<uint32_t *>(smem + kRingBytes);
    GroupInfo *ginfo = reinterpret_cast<GroupInfo *>(smem + kRingBytes + kBtabBytes);
    uint64_t *mbars = reinterpret_cast<uint64_t *>(smem + kRingBytes + kBtabBytes +
                                                   sizeof(GroupInfo) * kMaxChunksPerCta * kChunkGroups);
    float *red_max = reinterpret_cast<float *>(mbars + kWarps * kStages);
    int *red_sum = reinterpret_cast<int *>(red_max + kWarps);
    int *red_bad = red_sum + kWarps;
    unsigned char *lut = smem + (kLutWindowAddr - window);
    if (window + kCarveBytes > kLutWindowAddr) {      // the fixed-address table would overlap the buffers
        if (threadIdx.x == 0) atomicExch(status, 2u);
        return;
    }

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;

    // ---- unit range of this CTA and of this warp -------------------------------------------
    const long long total_units = (long long)tiles * chunks;
    const long long cta_begin = total_units * blockIdx.x / gridDim.x;
    const long long cta_end = total_units * (blockIdx.x + 1) / gridDim.x;
    const long long cta_units = cta_end - cta_begin;
    const long long u_begin = cta_begin + cta_units * warp / kWarps;
    const long long u_end = cta_begin + cta_units * (warp + 1) / kWarps;
    const int chunk_lo = cta_units > 0 ? (int)(cta_begin / tiles) : 0;
    const int chunk_hi = cta_units > 0 ? (int)((cta_end - 1) / tiles) : -1;

    // ---- prologue 1: mbarriers, the decode table ------------------------------------------------
    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init((uint32_t)__cvta_generic_to_shared(&mbars[warp * kStages + s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < 243 * 2; i += kThreads) {
        const int v = i >> 1, variant = i & 1;
        uint32_t c[5], t = v;
        for (int d = 0; d < 5; ++d) { c[d] = t % 3u; t /= 3u; }
        const uint32_t entry = c[0] | (c[1] << 4) | (c[2] << 8) | (c[3] << 12) | (c[4] << (variant ? 24 : 16));
        uint4 *dst = reinterpret_cast<uint4 *>(lut + v * 256 + variant * 128);
        const uint4 val = make_uint4(entry, entry, entry, entry);
#pragma unroll
        for (int k = 0; k < 8; ++k) dst[k] = val;
    }
    for (int i = tid; i < (int)(kBtabBytes / 4); i += kThreads) btab[i] = 0u;
    __syncthreads();

    // ---- prologue 2: activation digits for the chunks this CTA touches ---------------------------
    // one thread per activation: 512 threads = one chunk per pass
    for (int c = chunk_lo; c <= chunk_hi; ++c) {
        const int cl = c - chunk_lo;
        const int k = c * (kChunkGroups * kGroup) + tid;
        const float v = __half2float(x[k]);
        const float a = fabsf(v);
        const bool bad = !(a <= 65504.0f);                 // NaN or Inf
        float m = bad ? 0.0f : a;
        int anybad = bad;
        for (int o = 16; o > 0; o >>= 1) {
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            anybad |= __shfl_xor_sync(0xffffffffu, anybad, o);
        }
        if (lane == 0) { red_max[warp] = m; red_bad[warp] = anybad; }
        __syncthreads();
        const int gw = warp & ~3;                          // the four warps of this thread's group
        m = fmaxf(fmaxf(red_max[gw], red_max[gw + 1]), fmaxf(red_max[gw + 2], red_max[gw + 3]));
        anybad = red_bad[gw] | red_bad[gw + 1] | red_bad[gw + 2] | red_bad[gw + 3];
        // 2^E <= m < 2^(E+1); fixed point xi = round(v * 2^(21-E)), |xi| <= 2^22
        const int e_biased = m > 0.0f ? (int)(__float_as_uint(m) >> 23) : 127;
        const float up = __uint_as_float((uint32_t)(127 + 21 + 127 - e_biased) << 23);     // 2^(21-E)
        const float down = __uint_as_float((uint32_t)(e_biased - 21) << 23);               // 2^(E-21)
        const int xi = bad ? 0 : __float2int_rn(v * up);
        const int d0 = (xi << 24) >> 24;
        const int r1 = (xi - d0) >> 8;
        const int d1 = (r1 << 24) >> 24;
        const int d2 = (r1 - d1) >> 8;
        int s = xi;
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) red_sum[warp] = s;
        // scatter the three digits into the B-fragment table
        const int gi = tid >> 7;                           // group within the chunk
        const int el = tid & 127;
        const int j = el < 125 ? el / 5 : 25;
        const int i = el < 125 ? el - 5 * j : el - 125;
        const int h = j < 14 ? 0 : 1;
        const int slot = h ? j - 12 : j;
        const int reg = i < 4 ? slot : 14 + (slot >> 2);
        const int pos = i < 4 ? i : (slot & 3);
        const int sub = gi & 1, cls = gi >> 1;
        unsigned char *base = reinterpret_cast<unsigned char *>(btab) +
                              (((cl * 2 + sub) * kRegsPerSub + reg) * 32) * 4 + pos;
        const int qq = 2 * cls + h;
        base[(4 * (0 + 4 * cls) + qq) * 4] = (unsigned char)d0;
        base[(4 * (1 + 4 * cls) + qq) * 4] = (unsigned char)d1;
        base[(4 * (2 + 4 * cls) + qq) * 4] = (unsigned char)d2;
        __syncthreads();
        if (tid < kChunkGroups) {
            GroupInfo info;
            info.sum = red_sum[4 * tid] + red_sum[4 * tid + 1] + red_sum[4 * tid + 2] + red_sum[4 * tid + 3];
            const float gm = fmaxf(fmaxf(red_max[4 * tid], red_max[4 * tid + 1]),
                                   fmaxf(red_max[4 * tid + 2], red_max[4 * tid + 3]));
            const int eb = gm > 0.0f ? (int)(__float_as_uint(gm) >> 23) : 127;
            info.pow2 = __uint_as_float((uint32_t)(eb - 21) << 23);
            info.nonfinite = red_bad[4 * tid] | red_bad[4 * tid + 1] | red_bad[4 * tid + 2] | red_bad[4 * tid + 3];
            info.pad = 0;
            ginfo[cl * kChunkGroups + tid] = info;
        }
        (void)down;
        __syncthreads();
    }

    if (u_begin >= u_end) return;

    // ---- per-warp streaming loop ---------------------------------------------------------------------
    const int g = lane >> 2, q = lane & 3;
    const int cls = q >> 1, h = q & 1;
    const uint32_t lane_base = kLutWindowAddr + (uint32_t)lane * 4u;
    const uint32_t ring_warp = window + (uint32_t)(warp * kStages * kUnitBytes);
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&mbars[warp * kStages]);
    const int n_units = (int)(u_end - u_begin);

    auto issue = [&](int i) {       // lane 0 only
        const long long u = u_begin + i;
        const int c = (int)(u / tiles), t = (int)(u % tiles);
        const int s = i % kStages;
        mbar_expect_tx(bar0 + 8u * s, kUnitBytes);
        tma_load_2d(ring_warp + (uint32_t)(s * kUnitBytes), &wmap, c * kChunkBytes, t * kTileRows, bar0 + 8u * s);
    };
    if (lane == 0)
        for (int i = 0; i < kStages - 1 && i < n_units; ++i) issue(i);

    uint32_t breg[2][kRegsPerSub];
    int gsum[2];
    float gpow[2];
    int gbad[2];
    int cur_chunk = -1;

    for (int i = 0; i < n_units; ++i) {
        const long long u = u_begin + i;
        const int c = (int)(u / tiles), t = (int)(u % tiles);
        if (c != cur_chunk) {       // (re)load the B fragments of this K chunk
            cur_chunk = c;
            const int cl = c - chunk_lo;
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
                for (int r = 0; r < kRegsPerSub; ++r)
                    breg[sub][r] = btab[((cl * 2 + sub) * kRegsPerSub + r) * 32 + lane];
                const GroupInfo info = ginfo[cl * kChunkGroups + sub + 2 * cls];
                gsum[sub] = info.sum;
                gpow[sub] = info.pow2;
                gbad[sub] = info.nonfinite;
            }
        }
        const int s = i % kStages;
        const uint32_t parity = (uint32_t)(i / kStages) & 1u;
        uint32_t spins = 0;
        while (!mbar_try_wait(bar0 + 8u * s, parity)) {
            if (++spins > kMaxWaitSpins) {          // never hang: flag the failure and leave
                if (lane == 0) atomicExch(status, 1u);
                return;
            }
        }
        const uint32_t tile_addr = ring_warp + (uint32_t)(s * kUnitBytes);
        float acc1 = 0.0f, acc2 = 0.0f;             // rows g and g+8, this lane's two groups
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
            const int group = sub + 2 * cls;
            const uint32_t a1 = tile_addr + (uint32_t)(((g * kChunkGroups + group) * kBlockWords + 3 * h) * 4);
            const uint32_t a2 = a1 + 8u * kChunkBytes;
            const uint32_t w1a = lds_off<0>(a1), w1b = lds_off<4>(a1), w1c = lds_off<8>(a1), w1d = lds_off<12>(a1);
            const uint32_t w2a = lds_off<0>(a2), w2b = lds_off<4>(a2), w2c = lds_off<8>(a2), w2d = lds_off<12>(a2);
            uint32_t r1[kRegsPerSub], r2[kRegsPerSub];
            decode_stream(w1a, w1b, w1c, w1d, lane_base, r1);
            decode_stream(w2a, w2b, w2c, w2d, lane_base, r2);
            int acc[4] = {0, 0, 0, 0};
#pragma unroll
            for (int k = 0; k < kRegsPerSub / 2; ++k)
                mma_u8s8(acc, r1[2 * k], r2[2 * k], r1[2 * k + 1], r2[2 * k + 1], breg[sub][2 * k], breg[sub][2 * k + 1]);
            // columns: lane q=0 holds planes 0,1 of the first group, q=1 plane 2; q=2/3 the second group
            const int hi1 = __shfl_down_sync(0xffffffffu, acc[0], 1);
            const int hi2 = __shfl_down_sync(0xffffffffu, acc[2], 1);
            if (h == 0) {
                const int s1 = acc[0] + acc[1] * 256 + hi1 * 65536 - gsum[sub];
                const int s2 = acc[2] + acc[3] * 256 + hi2 * 65536 - gsum[sub];
                float dot1 = (float)s1 * gpow[sub];
                float dot2 = (float)s2 * gpow[sub];
                if (gbad[sub]) {
                    const unsigned char *tile = ring + (warp * kStages + s) * kUnitBytes;
                    const __half *xg = x + ((size_t)c * kChunkGroups + group) * kGroup;
                    dot1 = block_dot_fp32(tile + (g * kChunkGroups + group) * kBlockBytes, xg);
                    dot2 = block_dot_fp32(tile + ((g + 8) * kChunkGroups + group) * kBlockBytes, xg);
                }
                const float sc1 = __half2float(__ushort_as_half((unsigned short)(w1a & 0xffffu)));
                const float sc2 = __half2float(__ushort_as_half((unsigned short)(w2a & 0xffffu)));
                acc1 = fmaf(sc1, dot1, acc1);
                acc2 = fmaf(sc2, dot2, acc2);
            }
        }
        // the stage is fully consumed (its words are in registers): refill it
        __syncwarp();
        if (lane == 0 && i + kStages - 1 < n_units) issue(i + kStages - 1);

        // quad: lanes q=0 (groups 0,1) and q=2 (groups 2,3) -> chunk partial in lane q=0
        acc1 += __shfl_down_sync(0xffffffffu, acc1, 2);
        acc2 += __shfl_down_sync(0xffffffffu, acc2, 2);
        const int row0 = t * kTileRows;
        float *mine = partials + (size_t)c * tiles * kTileRows + row0;
        if (q == 0) {
            __stcg(mine + g, acc1);
            __stcg(mine + g + 8, acc2);
        }
        __threadfence();
        __syncwarp();
        int prev = 0;
        if (lane == 0) prev = atomicAdd(&counters[t], 1);
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev == chunks - 1) {       // this warp completed the row tile: fixed-order reduction
            __threadfence();
            if (lane < kTileRows) {
                const int row = row0 + lane;
                float total = 0.0f;
                for (int cc = 0; cc < chunks; ++cc)
                    total += __ldcg(partials + (size_t)cc * tiles * kTileRows + row);
                if (row < N) {
                    if (OUT_F32) static_cast<float *>(y)[row] = total;
                    else static_cast<__half *>(y)[row] = __float2half_rn(total);
                }
            }
            if (lane == 0) counters[t] = 0;     // ready for the next call
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

// Workspace layout: [status word, 256 B][arrival counters, fixed 64 KiB][per-chunk partial sums].
// The counter region has a fixed size so that calls of different shapes sharing one
// workspace never see another shape's partial sums where they expect zeroed counters.
constexpr size_t kHeaderBytes = 256;
constexpr int kMaxTiles = 16384;
constexpr size_t kCounterBytes = (size_t)kMaxTiles * sizeof(int);

}  // namespace

bool gemv_stream_shape_ok(int N, int K) {
    return N >= 1 && (N + kTileRows - 1) / kTileRows <= kMaxTiles && K % (kChunkGroups * kGroup) == 0 &&
           K / (kChunkGroups * kGroup) <= 256;
}

bool gemv_stream_supported(const uint8_t *blocks, int N, int K) {
    return gemv_stream_shape_ok(N, K) && (reinterpret_cast<uintptr_t>(blocks) & 15) == 0;
}

size_t gemv_stream_workspace_bytes(int N, int K) {
    const size_t tiles = (N + kTileRows - 1) / kTileRows;
    const size_t chunks = K / (kChunkGroups * kGroup);
    return kHeaderBytes + kCounterBytes + chunks * tiles * kTileRows * sizeof(float);
}

int launch_gemv_stream(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int N, int K,
                       void *workspace, cudaStream_t stream) {
    EncodeTiledFn encode = encode_fn();
    if (!encode) return fail(TQ1_ERR_CUDA, "tq1_linear_f16: cuTensorMapEncodeTiled is unavailable");
    const int tiles = (N + kTileRows - 1) / kTileRows;
    const int chunks = K / (kChunkGroups * kGroup);
    const cuuint64_t row_bytes = (cuuint64_t)(K / kGroup) * kBlockBytes;
    CUtensorMap map;
    const cuuint64_t dims[2] = {row_bytes, (cuuint64_t)N};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {kChunkBytes, kTileRows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult res = encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(blocks), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(TQ1_ERR_CUDA, "tq1_linear_f16: cuTensorMapEncodeTiled failed (%d)", (int)res);

    unsigned char *ws = static_cast<unsigned char *>(workspace);
    unsigned *status = reinterpret_cast<unsigned *>(ws);
    int *counters = reinterpret_cast<int *>(ws + kHeaderBytes);
    float *partials = reinterpret_cast<float *>(ws + kHeaderBytes + kCounterBytes);

    static int sm_count = 0;
    static size_t smem_bytes = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    // dynamic shared memory must reach the end of the table whatever the window base is (<= 1 KiB reserved)
    smem_bytes = kWindowEnd;
    auto kh = tq1_gemv_stream_kernel<false>;
    auto kf = tq1_gemv_stream_kernel<true>;
    static bool attr_set = false;     // one process drives one GPU
    if (!attr_set) {
        cudaError_t e1 = cudaFuncSetAttribute(kh, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
        cudaError_t e2 = cudaFuncSetAttribute(kf, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
        if (e1 != cudaSuccess || e2 != cudaSuccess)
            return cuda_fail(e1 != cudaSuccess ? e1 : e2, "tq1_linear_f16: shared memory opt-in");
        attr_set = true;
    }
    const long long units = (long long)tiles * chunks;
    int grid = sm_count;
    if (units < grid) grid = (int)units;
    if (y_f32)
        kf<<<grid, kThreads, smem_bytes, stream>>>(map, x, y, N, K, tiles, chunks, counters, partials, status);
    else
        kh<<<grid, kThreads, smem_bytes, stream>>>(map, x, y, N, K, tiles, chunks, counters, partials, status);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16: launch");
    return TQ1_OK;
}

}  // namespace tq1
