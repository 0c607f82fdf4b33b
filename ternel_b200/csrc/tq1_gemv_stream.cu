// Batch-1 streaming GEMV for TQ1_G128 on sm_100a: TMA-staged code bytes, a
// lane-replicated 243-entry base-3 table in shared memory, and exact integer
// dot products on the tensor cores (mma.sync m16n8k32 u8 x s8 -> s32).
//
// Stands in for the reference's GEMV kernels (cuda/tq1_g128_gemv.cu:81-140,
// cuda/tq1_lut23_streamk.cu:113-256, src/ternel_mlx/kernels.py:244-342) behind
// the same operator; it shares none of their structure.
//
// Why integers on the tensor cores. 128 weights arrive per 28 bytes, so at HBM speed an SM
// has about 1.2 issue slots per weight; one FP32 FMA per weight cannot keep up. Each group's
// 128 FP16 activations are therefore turned, once per CTA, into 23-bit block fixed point xi (a
// shared power-of-two exponent per group, which is as exact as FP32 accumulation). A table
// lookup turns a code byte b into four signed weights w0..w3 that are used directly as an A
// register; the fifth trit never has to be extracted, because
//     b = sum_i 3^i (w_i + 1)   =>   81 * sum_{i<5} w_i x_i
//                                  = sum_{i<4} w_i (81 x_i - 3^i x_4) + (b - 121) x_4
// so the raw weight words themselves (four code bytes each) serve as unsigned A registers
// against x_4, and the other activations enter as 81 x_i - 3^i x_4. Those 30-bit integers are
// split into four signed byte planes (B columns); the s32 accumulators give 81 * (group sum)
// modulo 2^32, a multiplication by 81^-1 (mod 2^32) recovers the exact integer group sum, and
// then acc = fma(scale_g, 2^(E-21) * sum, acc) in FP32 as in the reference
// (src/bonsai_tq1/reference.py:33-38). Groups containing NaN/Inf activations take an FP32
// path that multiplies every weight, so non-finite values propagate as in the reference.
//
// Work decomposition. A unit is 16 rows x 4 groups (1792 bytes, one TMA box).
// Units are numbered chunk-major and dealt out in contiguous ranges to the
// warps of 148 persistent CTAs, so a warp keeps its B fragments (the
// activation digits of one 512-wide K chunk) in registers while it streams row
// tiles. Per-chunk partial sums go to workspace slots of eight bytes, the value
// and a "present" flag written by one 64-bit store; a fixed owner per row tile
// polls the slots, adds the chunks in ascending order (so results do not depend
// on timing) and clears them for the next call.
//
// Lane roles inside mma.m16n8k32 (g = lane/4, q = lane%4): lane (g,q) decodes
// half a block of row g and half a block of row g+8; q>>1 picks which of the
// sub-unit's two groups, q&1 which half. B columns 0..3 carry the four digit
// planes of the first group, columns 4..7 those of the second, and a B lane
// holds zeros for k-slots that belong to the other group, which keeps the two
// groups' sums apart in one instruction.
#include <cuda.h>
#include <stdlib.h>

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
constexpr uint32_t kMbarBytes = 8 * (kWarps * kStages + 2);                        // per-warp stages + table barrier
constexpr uint32_t kRedBytes = 3 * 4 * kWarps * kMaxChunksPerCta;                  // group max / sum / non-finite flags
constexpr uint32_t kXiBytes = 0;
constexpr uint32_t kHighBytes = kBtabBytes + kXiBytes + kMbarBytes + kRedBytes;    // region above the table
static_assert(kRingBytes + 1024 + 128 <= kLutWindowAddr, "the ring must end below the table's fixed address");
static_assert(kWindowEnd + kHighBytes <= 227 * 1024, "shared memory budget");
constexpr uint32_t kMaxWaitSpins = 1u << 22;

// Optional phase timers (build with -DTQ1_PHASE_TIMERS): the last warp of every CTA records
// %globaltimer at each phase boundary; tq1_debug_read_phases() copies them out.
#ifdef TQ1_PHASE_TIMERS
constexpr int kPhases = 10;
__device__ unsigned long long g_phase_log[256 * kPhases];
__device__ __forceinline__ void phase_mark(int idx) {
    if ((threadIdx.x & 31) == 0 && (threadIdx.x >> 5) == kWarps - 1 && blockIdx.x < 256) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_phase_log[blockIdx.x * kPhases + idx] = t;
    }
}
#define PHASE(i) phase_mark(i)
#else
#define PHASE(i)
#endif

// The decode table as it sits in shared memory, built at compile time: entry v (a code byte)
// holds the weights (trit - 1) of trits 0..3 as four signed bytes, i.e. a ready A register.
// Entries are 256 bytes apart (so one PRMT can build the address from a code byte) and
// replicated for the 32 lanes, so lane i always reads bank i. A CTA fetches the image with one
// bulk copy.
struct LutImage {
    uint32_t w[243 * 64];
};
constexpr LutImage make_lut_image() {
    LutImage img{};
    for (int v = 0; v < 243; ++v) {
        uint32_t entry = 0;
        int t = v;
        for (int d = 0; d < 4; ++d) {
            entry |= (uint32_t)((t % 3 - 1) & 0xff) << (8 * d);
            t /= 3;
        }
        for (int l = 0; l < 32; ++l) img.w[v * 64 + l] = entry;
    }
    return img;
}
__device__ __align__(128) const LutImage g_lut_image = make_lut_image();
static_assert(sizeof(LutImage) == kLutBytes, "table image size");

// byte permute with the selector as an immediate (no register has to hold it)
template <uint32_t SEL>
__device__ __forceinline__ uint32_t prmt_imm(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "n"(SEL));
    return d;
}

// Ring-buffer words. Not volatile: the address depends on the value returned by the barrier wait,
// which keeps the loads behind it while leaving the compiler free to interleave the two sub-units.
template <int OFF>
__device__ __forceinline__ uint32_t lds_off(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}

// Decode-table lookups: the table never changes after the prologue, so the compiler may schedule these freely.
template <int OFF>
__device__ __forceinline__ uint32_t lds_lut(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
    return v;
}

// D = A * B + C with B signed bytes and A signed (SIGNED_A) or unsigned bytes; ZERO_C starts a chain.
template <bool SIGNED_A, bool ZERO_C>
__device__ __forceinline__ void mma_bytes(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    if (ZERO_C) {
        if (SIGNED_A)
            asm(
                "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
        else
            asm(
                "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    } else {
        if (SIGNED_A)
            asm(
                "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
        else
            asm(
                "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
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
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// One lane-stream (half a block: 14 code-byte slots in four words, wa holding slots 0,1 in its
// upper half) becomes 18 A registers: 14 table entries (weights of trits 0..3 of each slot) and
// the four raw words (the code bytes themselves, paired with the fifth trit's activation).
__device__ __forceinline__ void decode_stream(uint32_t wa, uint32_t wb, uint32_t wc, uint32_t wd,
                                              uint32_t lane_base, uint32_t (&r)[kRegsPerSub]) {
    r[0] = lds_lut<0>(prmt_imm<0x7624>(wa, lane_base));
    r[1] = lds_lut<0>(prmt_imm<0x7634>(wa, lane_base));
    r[2] = lds_lut<0>(prmt_imm<0x7604>(wb, lane_base));
    r[3] = lds_lut<0>(prmt_imm<0x7614>(wb, lane_base));
    r[4] = lds_lut<0>(prmt_imm<0x7624>(wb, lane_base));
    r[5] = lds_lut<0>(prmt_imm<0x7634>(wb, lane_base));
    r[6] = lds_lut<0>(prmt_imm<0x7604>(wc, lane_base));
    r[7] = lds_lut<0>(prmt_imm<0x7614>(wc, lane_base));
    r[8] = lds_lut<0>(prmt_imm<0x7624>(wc, lane_base));
    r[9] = lds_lut<0>(prmt_imm<0x7634>(wc, lane_base));
    r[10] = lds_lut<0>(prmt_imm<0x7604>(wd, lane_base));
    r[11] = lds_lut<0>(prmt_imm<0x7614>(wd, lane_base));
    r[12] = lds_lut<0>(prmt_imm<0x7624>(wd, lane_base));
    r[13] = lds_lut<0>(prmt_imm<0x7634>(wd, lane_base));
    r[14] = wa;
    r[15] = wb;
    r[16] = wc;
    r[17] = wd;
}

// Partial-sum slots: {FP32 value, flag} in one 64-bit word. A 64-bit store is a single access, so a
// reader that finds the flag set also has the value; no fence and no second round trip is needed.
constexpr unsigned long long kSlotPresent = 1ull << 32;
__device__ __forceinline__ void slot_publish(unsigned long long *p, float v) {
    const unsigned long long w = kSlotPresent | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long slot_read(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ void slot_clear(unsigned long long *p) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(0ull) : "memory");
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
                       unsigned long long *__restrict__ slots, unsigned *__restrict__ status,
                       const ShardDev shard) {
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t window = (uint32_t)__cvta_generic_to_shared(smem);   // window address of smem[0]
    // carve-up: the ring below the table's fixed window address, everything else above the table
    unsigned char *ring = smem;
    unsigned char *high = smem + (kWindowEnd - window);
    uint32_t *btab = reinterpret_cast<uint32_t *>(high);
    uint64_t *mbars = reinterpret_cast<uint64_t *>(high + kBtabBytes + kXiBytes);
    float *red_max = reinterpret_cast<float *>(high + kBtabBytes + kXiBytes + kMbarBytes);     // [chunk][warp]
    int *red_sum = reinterpret_cast<int *>(red_max + kMaxChunksPerCta * kWarps);
    int *red_bad = red_sum + kMaxChunksPerCta * kWarps;
    if (window + kRingBytes > kLutWindowAddr) {      // the fixed-address table would overlap the ring
        if (threadIdx.x == 0) atomicExch(status, 2u);
        return;
    }

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;

    PHASE(0);
    if (tid == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
    // ---- unit range of this CTA and of this warp (units are numbered chunk-major) ----------------
    const int total_units = tiles * chunks;
    // total_units <= 16384 * 256 and gridDim.x <= a few hundred, so the products fit 32 bits
    const int cta_begin = (int)((unsigned)total_units * blockIdx.x / gridDim.x);
    const int cta_end = (int)((unsigned)total_units * (blockIdx.x + 1) / gridDim.x);
    const int cta_units = cta_end - cta_begin;
    const int u_begin = cta_begin + ((cta_units * warp) >> 4);
    const int u_end = cta_begin + ((cta_units * (warp + 1)) >> 4);
    const int n_units = u_end - u_begin;
    const int chunk_lo = cta_units > 0 ? cta_begin / tiles : 0;
    const int chunk_hi = cta_units > 0 ? (cta_end - 1) / tiles : -1;
    const int c_first = u_begin / tiles;
    const int t_first = u_begin - c_first * tiles;

    // ---- barriers and the decode table first (nothing here depends on the previous kernel) ---------
    const uint32_t ring_warp = window + (uint32_t)(warp * kStages * kUnitBytes);
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&mbars[warp * kStages]);
    const uint32_t lut_bar = (uint32_t)__cvta_generic_to_shared(&mbars[kWarps * kStages]);
    int issue_c = c_first, issue_t = t_first, issued = 0;      // next unit to request (lane 0 only)
    auto issue_next = [&]() {
        const int s = issued % kStages;
        mbar_expect_tx(bar0 + 8u * s, kUnitBytes);
        tma_load_2d(ring_warp + (uint32_t)(s * kUnitBytes), &wmap, issue_c * kChunkBytes, issue_t * kTileRows,
                    bar0 + 8u * s);
        ++issued;
        if (++issue_t == tiles) { issue_t = 0; ++issue_c; }
    };
    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + 8u * s, 1);
        if (warp == 0) mbar_init(lut_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (warp == 0) {
            mbar_expect_tx(lut_bar, kLutBytes);
            bulk_load(kLutWindowAddr, &g_lut_image, kLutBytes, lut_bar);
        }
    }
    // A shard of a row-sharded projection will wait for other ranks' flags below: request its weight
    // tiles first, so that they travel while it waits (weights depend on nothing).
    if (shard.world > 1 && lane == 0)
        while (issued < kStages - 1 && issued < n_units) issue_next();
    // Let the next kernel in the stream start its own prologue as SMs free up, then wait until
    // everything before this kernel has finished before touching activations or the workspace.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (shard.world > 1 && shard.wait_flags != nullptr) {
        // Row-sharded input: the tiles of activations this CTA reads (32 per chunk) must have landed
        // in local memory from whichever rank computed them.
        const int cl = tid >> 5;
        const int tile = (chunk_lo + cl) * (kChunkGroups * kGroup / kFlagRows) + lane;
        if (cl < kMaxChunksPerCta && chunk_lo + cl <= chunk_hi && tile < shard.wait_tiles) {
            const unsigned want = shard.wait_epoch + (shard.epoch_base ? *shard.epoch_base : 0u);
            uint32_t spins = 0;
            for (;;) {
                unsigned v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(shard.wait_flags + tile) : "memory");
                if ((int)(v - want) >= 0) break;
                if (++spins > kMaxWaitSpins) { atomicExch(status, 4u); break; }   // never hang
            }
        }
        __syncthreads();
    }
    PHASE(1);

    // activations of the (at most three) chunks this CTA touches: one thread per activation, which
    // also fetches the activation of the fifth trit of its code byte (needed for 81 x_i - 3^i x_4)
    const int gi = tid >> 7;                           // group within the chunk
    const int el = tid & 127;
    const int bj = el < 125 ? el / 5 : 25;             // code byte
    const int bi = el < 125 ? el - 5 * bj : el - 125;  // trit within the byte
    const bool is_fifth = el < 125 && bi == 4;         // pairs with the raw code byte
    const int fifth = el < 125 ? gi * kGroup + 5 * bj + 4 : tid;
    float xv[kMaxChunksPerCta], x4v[kMaxChunksPerCta];
#pragma unroll
    for (int cl = 0; cl < kMaxChunksPerCta; ++cl) {
        const bool live = chunk_lo + cl <= chunk_hi;
        const __half *xc = x + (size_t)(chunk_lo + cl) * (kChunkGroups * kGroup);
        xv[cl] = live ? __half2float(__ldg(xc + tid)) : 0.0f;
        x4v[cl] = live ? __half2float(__ldg(xc + fifth)) : 0.0f;
    }
    // The activation loads are in flight: now start this warp's weight tiles. (Issued the other way
    // round, or before the wait above, the few activation bytes queue behind megabytes of weight
    // traffic and arrive 1-2 us late.)
    // One tile per warp for now, so that every warp's first tile is near the head of the queue.
    if (lane == 0 && issued < n_units) issue_next();
    for (int i = tid; i < (int)(kBtabBytes / 16); i += kThreads)
        reinterpret_cast<uint4 *>(btab)[i] = make_uint4(0u, 0u, 0u, 0u);

    // ---- activation digits: group maximum, fixed point, four signed byte planes ---------------------
    bool bad[kMaxChunksPerCta];
    const int n_chunks_cta = chunk_hi - chunk_lo + 1;
#pragma unroll
    for (int cl = 0; cl < kMaxChunksPerCta; ++cl) {
        if (cl >= n_chunks_cta) break;
        const float a = fabsf(xv[cl]);
        bad[cl] = !(a <= 65504.0f);                        // NaN or Inf
        float m = bad[cl] ? 0.0f : a;
        int anybad = bad[cl];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            anybad |= __shfl_xor_sync(0xffffffffu, anybad, o);
        }
        if (lane == 0) { red_max[cl * kWarps + warp] = m; red_bad[cl * kWarps + warp] = anybad; }
    }
    __syncthreads();
    PHASE(2);
    // every warp's first tile is on its way: now queue the rest of the ring behind them
    if (lane == 0)
        while (issued < kStages - 1 && issued < n_units) issue_next();
    {
        const int hh = bj < 14 ? 0 : 1;                    // which half-block lane decodes it
        const int slot = hh ? bj - 12 : bj;
        // trits 0..3 sit in the table-entry register of their slot; a fifth trit pairs with the raw word
        const int reg = !is_fifth ? slot : slot < 2 ? 14 : 15 + ((slot - 2) >> 2);
        const int pos = !is_fifth ? bi : slot < 2 ? slot + 2 : ((slot - 2) & 3);
        const int sub = gi & 1, cg = gi >> 1;
        const int owner = 4 * (4 * cg) + 2 * cg + hh;      // B lane of digit plane 0; plane p is 4p lanes on
        const int pow3 = bi == 0 ? 1 : bi == 1 ? 3 : bi == 2 ? 9 : 27;
        const int gw = warp & ~3;                          // the four warps of this thread's group
#pragma unroll
        for (int cl = 0; cl < kMaxChunksPerCta; ++cl) {
            if (cl >= n_chunks_cta) break;
            const float *rm = red_max + cl * kWarps + gw;
            const float m = fmaxf(fmaxf(rm[0], rm[1]), fmaxf(rm[2], rm[3]));
            // 2^E <= m < 2^(E+1); fixed point xi = round(v * 2^(21-E)), |xi| <= 2^22
            const int e_biased = m > 0.0f ? (int)(__float_as_uint(m) >> 23) : 127;
            const float up = __uint_as_float((uint32_t)(275 - e_biased) << 23);            // 2^(21-E)
            const int xi = bad[cl] ? 0 : __float2int_rn(xv[cl] * up);
            int s = is_fifth ? 121 * xi : 0;                   // 121 * sum of the fifth-trit activations
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) red_sum[cl * kWarps + warp] = s;
            // value paired with this k-slot: x_4 for the raw byte, 81 x_i - 3^i x_4 for trit i < 4
            int v = xi;
            if (!is_fifth) {
                const float a4 = fabsf(x4v[cl]);
                const int x4 = (el < 125 && a4 <= 65504.0f) ? __float2int_rn(x4v[cl] * up) : 0;
                v = 81 * xi - pow3 * x4;
            }
            const int d0 = (v << 24) >> 24;
            const int r1 = (v - d0) >> 8;
            const int d1 = (r1 << 24) >> 24;
            const int r2 = (r1 - d1) >> 8;
            const int d2 = (r2 << 24) >> 24;
            const int d3 = (r2 - d2) >> 8;
            unsigned char *base = reinterpret_cast<unsigned char *>(btab) +
                                  ((((cl * 2 + sub) * kRegsPerSub + reg) * 32 + owner) * 4) + pos;
            base[0] = (unsigned char)d0;
            base[16] = (unsigned char)d1;
            base[32] = (unsigned char)d2;
            base[48] = (unsigned char)d3;
        }
    }
    __syncthreads();
    PHASE(3);
    if (n_units <= 0) return;

    // the decode table must have landed
    {
        uint32_t spins = 0;
        while (!mbar_try_wait(lut_bar, 0)) {
            if (++spins > kMaxWaitSpins) {
                if (lane == 0) atomicExch(status, 1u);
                return;
            }
        }
    }

    // ---- per-warp streaming loop ---------------------------------------------------------------------
    const int g = lane >> 2, q = lane & 3;
    const int cls = q >> 1, h = q & 1;
    const uint32_t lane_base = kLutWindowAddr + (uint32_t)lane * 4u;

    uint32_t breg[2][kRegsPerSub];
    int gsum[2];
    float gpow[2];
    int gbad[2];
    int cur_chunk = -1;
    int c = c_first, t = t_first;

    for (int i = 0; i < n_units; ++i) {
        if (c != cur_chunk) {       // (re)load the B fragments and the group constants of this K chunk
            cur_chunk = c;
            const int cl = c - chunk_lo;
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
                for (int r = 0; r < kRegsPerSub; ++r)
                    breg[sub][r] = btab[((cl * 2 + sub) * kRegsPerSub + r) * 32 + lane];
                const int w4 = cl * kWarps + 4 * (sub + 2 * cls);          // the group's four warps
                gsum[sub] = red_sum[w4] + red_sum[w4 + 1] + red_sum[w4 + 2] + red_sum[w4 + 3];
                const float gm = fmaxf(fmaxf(red_max[w4], red_max[w4 + 1]), fmaxf(red_max[w4 + 2], red_max[w4 + 3]));
                const int eb = gm > 0.0f ? (int)(__float_as_uint(gm) >> 23) : 127;
                gpow[sub] = __uint_as_float((uint32_t)(eb - 21) << 23);                    // 2^(E-21)
                gbad[sub] = red_bad[w4] | red_bad[w4 + 1] | red_bad[w4 + 2] | red_bad[w4 + 3];
            }
        }
        const int s = i % kStages;
        const uint32_t parity = (uint32_t)(i / kStages) & 1u;
        uint32_t spins = 0, arrived;
        while (!(arrived = mbar_try_wait(bar0 + 8u * s, parity))) {
            if (++spins > kMaxWaitSpins) {          // never hang: flag the failure and leave
                if (lane == 0) atomicExch(status, 1u);
                return;
            }
        }
        if (i == 0) PHASE(4);
        // (arrived >> 8) is zero, but only the hardware knows: the tile loads depend on the wait
        const uint32_t tile_addr = ring_warp + (uint32_t)(s * kUnitBytes) + (arrived >> 8);
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
            // three independent accumulator chains keep the tensor pipe's latency off the critical path;
            // register pairs 0..6 hold signed weights, pairs 7,8 the raw (unsigned) code bytes
            int accA[4], accB[4], accC[4];
            mma_bytes<true, true>(accA, r1[0], r2[0], r1[1], r2[1], breg[sub][0], breg[sub][1]);
            mma_bytes<true, true>(accB, r1[2], r2[2], r1[3], r2[3], breg[sub][2], breg[sub][3]);
            mma_bytes<true, true>(accC, r1[4], r2[4], r1[5], r2[5], breg[sub][4], breg[sub][5]);
            mma_bytes<true, false>(accA, r1[6], r2[6], r1[7], r2[7], breg[sub][6], breg[sub][7]);
            mma_bytes<true, false>(accB, r1[8], r2[8], r1[9], r2[9], breg[sub][8], breg[sub][9]);
            mma_bytes<true, false>(accC, r1[10], r2[10], r1[11], r2[11], breg[sub][10], breg[sub][11]);
            mma_bytes<true, false>(accA, r1[12], r2[12], r1[13], r2[13], breg[sub][12], breg[sub][13]);
            mma_bytes<false, false>(accB, r1[14], r2[14], r1[15], r2[15], breg[sub][14], breg[sub][15]);
            mma_bytes<false, false>(accC, r1[16], r2[16], r1[17], r2[17], breg[sub][16], breg[sub][17]);
            int acc[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[k] = accA[k] + accB[k] + accC[k];
            // columns: lane q=0 holds planes 0,1 of the first group, q=1 planes 2,3; q=2/3 the second group
            const uint32_t p2r1 = (uint32_t)__shfl_down_sync(0xffffffffu, acc[0], 1);
            const uint32_t p3r1 = (uint32_t)__shfl_down_sync(0xffffffffu, acc[1], 1);
            const uint32_t p2r2 = (uint32_t)__shfl_down_sync(0xffffffffu, acc[2], 1);
            const uint32_t p3r2 = (uint32_t)__shfl_down_sync(0xffffffffu, acc[3], 1);
            if (h == 0) {
                // 81 * (group sum) modulo 2^32, then times 81^-1 modulo 2^32: the exact integer group sum
                const uint32_t t1 = (uint32_t)acc[0] + ((uint32_t)acc[1] << 8) + (p2r1 << 16) + (p3r1 << 24) -
                                    (uint32_t)gsum[sub];
                const uint32_t t2 = (uint32_t)acc[2] + ((uint32_t)acc[3] << 8) + (p2r2 << 16) + (p3r2 << 24) -
                                    (uint32_t)gsum[sub];
                const int s1 = (int)(t1 * 0x781948b1u);
                const int s2 = (int)(t2 * 0x781948b1u);
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
        // the stage consumed one iteration ago is free: refill it
        __syncwarp();
        if (lane == 0 && issued < n_units) issue_next();

        // quad: lanes q=0 (groups 0,1) and q=2 (groups 2,3) -> chunk partial in lane q=0
        acc1 += __shfl_down_sync(0xffffffffu, acc1, 2);
        acc2 += __shfl_down_sync(0xffffffffu, acc2, 2);
        if (q == 0) {       // value and flag travel in one 64-bit store, so whoever sees the flag has the value
            unsigned long long *mine = slots + ((size_t)c * tiles + t) * kTileRows;
            slot_publish(mine + g, acc1);
            slot_publish(mine + g + 8, acc2);
        }
        if (i == 0) PHASE(5);
        if (++t == tiles) { t = 0; ++c; }
    }

    PHASE(6);
    // ---- finish row tiles ------------------------------------------------------------------------------
    // Row tile t is finished by a fixed owner, the warp that processed its chunk t % chunks, so every
    // warp finishes about one tile per `chunks` units. The owner polls the tile's slots (bounded) until
    // every chunk's value is present. All CTAs of the grid are resident (one per SM), so the wait is
    // for warps that are running. Lane (hf, r) adds chunks hf, hf+2, ... of row r in ascending order
    // and one shuffle joins the two halves: the order of additions never depends on timing.
    PHASE(7);
    {
        const int r = lane & 15, hf = lane >> 4;
        const size_t stride = (size_t)tiles * kTileRows;
        int cc = c_first, tt = t_first;
        for (int i = 0; i < n_units; ++i) {
            if (tt % chunks == cc) {                 // warp-uniform: this warp owns row tile tt
                unsigned long long *p = slots + (size_t)tt * kTileRows + r;
                float total = 0.0f;
                for (int c0 = hf; c0 < chunks; c0 += 16) {
                    unsigned long long v[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        v[k] = c0 + 2 * k < chunks ? slot_read(p + (size_t)(c0 + 2 * k) * stride) : kSlotPresent;
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        if (c0 + 2 * k < chunks) {
                            uint32_t spins = 0;
                            while ((v[k] >> 32) != 1ull) {
                                if (++spins > kMaxWaitSpins) { atomicExch(status, 5u); break; }   // never hang
                                v[k] = slot_read(p + (size_t)(c0 + 2 * k) * stride);
                            }
                            total += __uint_as_float((uint32_t)v[k]);
                            slot_clear(p + (size_t)(c0 + 2 * k) * stride);        // ready for the next call
                        }
                    }
                }
                total += __shfl_xor_sync(0xffffffffu, total, 16);
                const int row = tt * kTileRows + r;
                if (shard.world > 1) {
                    // Fused all-gather: lane p sends the tile's 16 FP16 rows (two 16-byte stores) into
                    // rank p's gathered output and then raises the tile's flag there; the release store
                    // orders that lane's own data stores before the flag, so no fence or counter is needed.
                    const uint32_t mine = (uint32_t)__half_as_ushort(__float2half_rn(total));
                    const uint32_t pair = mine | ((uint32_t)__shfl_down_sync(0xffffffffu, mine, 1) << 16);
                    uint32_t w[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) w[k] = __shfl_sync(0xffffffffu, pair, 2 * k);
                    if (lane < shard.world) {
                        uint4 *dst = reinterpret_cast<uint4 *>(shard.peer_y[lane] + (size_t)tt * kTileRows);
                        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        const unsigned epoch = shard.publish_epoch + (shard.epoch_base ? *shard.epoch_base : 0u);
                        asm volatile("st.release.sys.global.u32 [%0], %1;"
                                     ::"l"(shard.peer_flags[lane] + tt), "r"(epoch) : "memory");
                    }
                } else if (shard.swiglu) {
                    // rows come as (gate, up) pairs: the even lane of a pair stores silu(gate) * up
                    const float up = __shfl_down_sync(0xffffffffu, total, 1);
                    if (hf == 0 && (r & 1) == 0 && row + 1 < N) {
                        const float out = swiglu_f32(total, up);
                        if (OUT_F32) static_cast<float *>(y)[row >> 1] = out;
                        else static_cast<__half *>(y)[row >> 1] = __float2half_rn(out);
                    }
                } else if (hf == 0 && row < N) {
                    if (OUT_F32) static_cast<float *>(y)[row] = total;
                    else static_cast<__half *>(y)[row] = __float2half_rn(total);
                }
            }
            if (++tt == tiles) { tt = 0; ++cc; }
        }
    }
    PHASE(8);
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


}  // namespace

bool gemv_stream_shape_ok(int N, int K) {
    return N >= 1 && K % (kChunkGroups * kGroup) == 0 && K / (kChunkGroups * kGroup) <= 256;
}

bool gemv_stream_supported(const uint8_t *blocks, int N, int K) {
    return gemv_stream_shape_ok(N, K) && (reinterpret_cast<uintptr_t>(blocks) & 15) == 0;
}

namespace {
// Rows one launch may cover: its partial-sum slots (8 bytes per row and K chunk) must fit the slot region.
int rows_per_launch(int N, int K) {
    const size_t chunks = K / (kChunkGroups * kGroup);
    const size_t cap = kWsSlotRegionBytes / (chunks * sizeof(unsigned long long)) / kTileRows * kTileRows;
    if ((size_t)N <= cap) return N;
    const size_t launches = ((size_t)N + cap - 1) / cap;
    return (int)((((size_t)N + launches - 1) / launches + kTileRows - 1) / kTileRows * kTileRows);
}
}  // namespace

size_t gemv_stream_workspace_bytes(int N, int K) {
    const size_t tiles = (rows_per_launch(N, K) + kTileRows - 1) / kTileRows;
    const size_t chunks = K / (kChunkGroups * kGroup);
    return kWsStatusBytes + chunks * tiles * kTileRows * sizeof(unsigned long long);
}

static int launch_gemv_rows_block(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int N, int K,
                                  void *workspace, cudaStream_t stream, const ShardDev *shard);

// Very tall matrices (an output head of a few hundred thousand rows) run as consecutive launches over
// row ranges, which reuse the same slots: each launch leaves them cleared.
int launch_gemv_stream(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int N, int K,
                       void *workspace, cudaStream_t stream, const ShardDev *shard) {
    const int step = rows_per_launch(N, K);
    if (step < N && shard && shard->world > 1)
        return fail(TQ1_ERR_INVALID, "tq1_linear_f16_sharded: a shard of %d rows is too tall for one launch", N);
    const int yshift = shard && shard->swiglu ? 1 : 0;        // paired rows give one output per two rows
    const size_t row_bytes = (size_t)(K / kGroup) * kBlockBytes;
    for (int n0 = 0; n0 < N; n0 += step) {
        const int rows = N - n0 < step ? N - n0 : step;
        void *yb = y_f32 ? static_cast<void *>(static_cast<float *>(y) + (n0 >> yshift))
                         : static_cast<void *>(static_cast<__half *>(y) + (n0 >> yshift));
        const int rc = launch_gemv_rows_block(blocks + (size_t)n0 * row_bytes, x, y ? yb : nullptr, y_f32, rows, K,
                                              workspace, stream, shard);
        if (rc != TQ1_OK) return rc;
    }
    return TQ1_OK;
}

static int launch_gemv_rows_block(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int N, int K,
                                  void *workspace, cudaStream_t stream, const ShardDev *shard) {
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
    unsigned long long *slots = reinterpret_cast<unsigned long long *>(ws + kWsStatusBytes);

    static int sm_count = 0;
    static size_t smem_bytes = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    // dynamic shared memory must reach the end of the table whatever the window base is (<= 1 KiB reserved)
    smem_bytes = kWindowEnd + kHighBytes;
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
    // Programmatic dependent launch: the kernel's prologue (table fetch, first weight tiles) may
    // overlap the tail of whatever precedes it in the stream; it waits (griddepcontrol.wait)
    // before it reads activations or writes anything.
    static const bool use_pdl = getenv("TQ1_DISABLE_PDL") == nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    const __half *xc = x;
    ShardDev sd = {};
    if (shard) sd = *shard;
    cudaError_t err =
        y_f32 ? cudaLaunchKernelEx(&cfg, kf, map, xc, y, N, K, tiles, chunks, slots, status, sd)
              : cudaLaunchKernelEx(&cfg, kh, map, xc, y, N, K, tiles, chunks, slots, status, sd);
    if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16: launch");
    err = cudaGetLastError();
    if (err != cudaSuccess) return cuda_fail(err, "tq1_linear_f16: launch");
    return TQ1_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the batch-1 GEMV.
//
// Some hosts cannot give this library scratch memory at call time: code that runs inside a
// stream-capture region (where cudaMalloc is illegal), plugin hosts whose whole device budget
// was handed out when the model was loaded, and real-time loops that must not touch the
// allocator. For them the scratch of the streaming GEMV (status word and per-chunk
// partial-sum slots) lives in this fixed array, which every GPU that loads the library
// holds until the process exits.
constexpr size_t kNoAllocScratchBytes = 2u << 20;       // 2 MiB: N*K up to about 1.3e8 weights
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
void *g_noalloc_ptr[kMaxDevices] = {};     // device address of g_noalloc_scratch, per device
}  // namespace

int gemv_noalloc(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int N, int K, cudaStream_t stream) {
    if (!gemv_stream_supported(blocks, N, K))
        return fail(TQ1_ERR_INVALID,
                    "tq1_gemv_f16_noalloc: needs K %% 512 == 0, at most 256 K chunks and 16-byte aligned blocks "
                    "(got N=%d K=%d)", N, K);
    const size_t need = gemv_stream_workspace_bytes(N, K);
    if (need > kNoAllocScratchBytes)
        return fail(TQ1_ERR_WORKSPACE,
                    "tq1_gemv_f16_noalloc: %dx%d needs %zu bytes of scratch, the built-in array holds %zu",
                    N, K, need, (size_t)kNoAllocScratchBytes);
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return cuda_fail(err, "tq1_gemv_f16_noalloc: cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return fail(TQ1_ERR_INVALID, "tq1_gemv_f16_noalloc: device %d out of range", dev);
    if (!g_noalloc_ptr[dev]) {
        // In host code the array's name is only a handle; the kernel needs its device address.
        void *ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (err != cudaSuccess) return cuda_fail(err, "tq1_gemv_f16_noalloc: cudaGetSymbolAddress");
        g_noalloc_ptr[dev] = ptr;
    }
    unsigned char *scratch = static_cast<unsigned char *>(g_noalloc_ptr[dev]);
    // The array keeps whatever the last call left: the status word and the slots this shape uses start at zero.
    err = cudaMemsetAsync(scratch, 0, need, stream);
    if (err != cudaSuccess) return cuda_fail(err, "tq1_gemv_f16_noalloc: clearing the scratch");
    return launch_gemv_stream(blocks, x, y, y_f32, N, K, scratch, stream);
}

}  // namespace tq1

#ifdef TQ1_PHASE_TIMERS
extern "C" int tq1_debug_read_phases(unsigned long long *out, int ctas) {
    return (int)cudaMemcpyFromSymbol(out, tq1::g_phase_log, sizeof(unsigned long long) * tq1::kPhases * ctas);
}
#endif
