// Batch-1 GEMV for TQ1_G128 on sm_100a as ONE persistent launch over a chain of projections.
//
// A decoded token issues one matrix-vector product per packed linear, back to back
// (src/ternel_mlx/modules.py:425-457 of the reference: q/k/v, o, gate/up, down, layer after
// layer). Launched one by one, each product pays a launch hand-over, a cold pipeline and a
// reduction tail that together cost as much as streaming its weights. Here a whole list of
// products ("links") runs inside one grid of persistent CTAs:
//
//   * the weight tiles of the next link are already being fetched (TMA into each warp's
//     ring) while the current one drains;
//   * a link that reads the output of an earlier link waits for exactly the activations it
//     needs, element by element: an output travels as one 64-bit word {value bits, tag}
//     written by a single store, so whoever sees the tag has the value (no fence, no flag
//     array, no second round trip). The same words are pushed into every rank's memory when
//     the rows of a projection are sharded over several GPUs (plain peer stores);
//   * the table, the barriers and the CTA's bookkeeping are set up once.
//
// The arithmetic is the exact-integer scheme of the streaming GEMV: a code byte b becomes,
// through a lane-replicated 243-entry shared-memory table, four signed weights w0..w3 that
// are used directly as an A register of mma.sync.m16n8k32.s8; the fifth trit is never
// extracted because b = sum_i 3^i (w_i + 1) gives
//     81 * sum_{i<5} w_i x_i = sum_{i<4} w_i (81 x_i - 3^i x_4) + (b - 121) x_4 ,
// so the raw code words serve as unsigned A registers against x_4. Activations are block
// fixed point (23 bits below the group's maximum, as exact as FP32 accumulation) split into
// four signed byte planes; s32 accumulators give 81 * (group sum) modulo 2^32, a multiplication
// by 81^-1 (mod 2^32) recovers the integer, then acc = fma(scale_g, 2^(E-21) * sum, acc) in
// FP32 as in src/bonsai_tq1/reference.py:33-38. Groups holding NaN/Inf activations take an
// FP32 path that multiplies every weight, so non-finite values propagate as in the reference.
//
// Work decomposition per link: a unit is 16 rows x 4 groups (1792 bytes, one TMA box); units
// are numbered chunk-major (a chunk = 512 columns) and dealt out in contiguous ranges to the
// warps of the persistent CTAs, so a warp keeps the activation digits of one chunk in
// registers while it streams row tiles. A warp's chunk partial of a row goes to a 64-bit
// workspace slot {FP32 value, tag}; row tile t has a fixed owner (the warp that processed
// chunk t % chunks of it), which polls the tile's slots (bounded), adds the chunks in
// ascending order (results never depend on timing) and stores the output. Tags are
// sequence numbers that grow with every link of every call, so nothing has to be cleared.
// Two slot regions alternate between consecutive links; a per-region arrival counter keeps
// a CTA that runs ahead from overwriting slots that have not been summed yet.
//
// Shared-memory traffic sets the pace of the loop (one 128-byte wavefront per 32 code bytes
// for the table alone), so the loop spends as few load/store-pipe operations as it can:
// plane pairs are combined before they are exchanged (two shuffles per 16 rows x 2 groups
// instead of four) and slots are never cleared.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include <type_traits>
#include <vector>

#include "tq1_common.cuh"

namespace tq1 {

namespace {

constexpr int kTileRows = 16;
constexpr int kChunkGroups = 4;
constexpr int kChunkCols = kChunkGroups * kGroup;             // 512
constexpr int kChunkBytes = kChunkGroups * kBlockBytes;       // 112
constexpr int kUnitBytes = kTileRows * kChunkBytes;           // 1792
#ifndef TQ1_GEMV_WARPS
#define TQ1_GEMV_WARPS 16
#endif
#ifndef TQ1_GEMV_STAGES
#define TQ1_GEMV_STAGES 4
#endif
constexpr int kStages = TQ1_GEMV_STAGES;
constexpr int kWarps = TQ1_GEMV_WARPS;           // warp w < 4 * (chunks of the CTA) also prepares activation group w
constexpr int kThreads = kWarps * 32;
constexpr int kMaxChunksPerCta = 3;
constexpr int kPrepWarps = 4 * kMaxChunksPerCta;               // one warp per 128-activation group
constexpr int kRegsPerSub = 18;                                // A/B registers per lane per sub-unit
static_assert(kWarps >= kPrepWarps, "one warp per activation group of the CTA's chunks");

// Per activation group, written by the warp that prepared it: 121 * (sum of the fifth-trit activations),
// 2^(E-21) for the group's exponent E, and whether the group holds NaN/Inf.
struct alignas(16) GroupConst {
    int sum;
    float pow;
    int bad;
    int pad;
};

// Shared-memory window layout (addresses relative to the CTA's shared window). The table sits
// at a 64 KiB multiple so that PRMT can build a complete lookup address
// (byte << 8 | lane << 2 | table base) in one instruction. It holds 256 entries (the 13 past
// 242 are zero), so a byte that escaped the load-time scan still reads inside the table.
constexpr uint32_t kLutWindowAddr = 131072;
constexpr uint32_t kLutBytes = 256 * 256;                     // 256 entries x (2 x 32 lanes x 4 B)
constexpr uint32_t kWindowEnd = kLutWindowAddr + kLutBytes;   // 196608
constexpr uint32_t kRingBytes = kWarps * kStages * kUnitBytes;                     // 114688
constexpr uint32_t kBtabChunk = 2 * kRegsPerSub * 32 * 4;                          // 4608: digit planes of one chunk
constexpr uint32_t kBtabOne = kMaxChunksPerCta * kBtabChunk;                       // 13824 per buffer
constexpr uint32_t kBtabBytes = 2 * kBtabOne;                                      // two links in flight
constexpr uint32_t kMbarBytes = 8 * (kWarps * kStages + 2);
constexpr uint32_t kGconstOne = kPrepWarps * sizeof(GroupConst);
constexpr uint32_t kGconstBytes = 2 * kGconstOne;
constexpr uint32_t kXchgBytes = kPrepWarps * kGroup * 4;                           // a warp's fixed-point activations
constexpr uint32_t kPrepTabBytes = kGroup * 4;                                     // where activation e of a group goes
constexpr uint32_t kMiscBytes = 16;
constexpr uint32_t kHighBytes = kBtabBytes + kMbarBytes + kGconstBytes + kXchgBytes + kPrepTabBytes + kMiscBytes;
static_assert(kRingBytes + 1024 + 128 <= kLutWindowAddr, "the ring must end below the table's fixed address");
static_assert(kWindowEnd + kHighBytes <= 227 * 1024, "shared memory budget");
constexpr uint32_t kMaxWaitSpins = 1u << 21;

// Control words at the start of the workspace.
constexpr int kCtlStatus = 0;      // non-zero: a bounded wait ran out (1 tile, 4 hand-off word, 5 slot, 6 region);
                                   // 7: results are good, but the tag base has passed kTagRefresh
constexpr unsigned kTagRefresh = 0xF0000000u;
constexpr int kCtlExit = 1;        // CTAs that have left the current launch
constexpr int kCtlEpoch = 2;       // links executed by all earlier launches on this workspace (tag base)
constexpr int kCtlArrive = 3;      // [2] CTAs that are done with the slots of the links of each region

// Optional phase timers (build with -DTQ1_PHASE_TIMERS): lane 0 of every warp of the first CTAs accumulates
// clock cycles per phase of a link; tq1_debug_read_phases() copies them out.
#ifdef TQ1_PHASE_TIMERS
constexpr int kPhases = 8;
__device__ long long g_phase_acc[64 * kWarps * kPhases];
#define PHASE_DECL long long ph_t = clock64(), ph_acc[kPhases] = {0, 0, 0, 0, 0, 0, 0, 0};
#define PHASE(i) { const long long now_ = clock64(); ph_acc[i] += now_ - ph_t; ph_t = now_; }
#define PHASE_DUMP if (lane == 0 && blockIdx.x < 64) { for (int i_ = 0; i_ < kPhases; ++i_) g_phase_acc[(blockIdx.x * kWarps + warp) * kPhases + i_] = ph_acc[i_]; }
#else
#define PHASE_DECL
#define PHASE(i)
#define PHASE_DUMP
#endif

constexpr unsigned kFlagOutF32 = 1u;
constexpr unsigned kFlagSwiglu = 2u;
constexpr unsigned kFlagPanels = 4u;           // weights in chunk-major panels: a unit is 1792 contiguous bytes
constexpr unsigned kFlagPartialOut = 8u;       // the output is one rank's partial sum over its K shard: hand-off words carry FP32
constexpr unsigned kFlagSrcF32 = 16u;          // the words this link reads carry FP32 partial sums (bits 8..11: how many to add)
constexpr int kFlagSrcPartsShift = 8;

// One link as the kernel sees it.
struct alignas(128) ChainLinkDev {
    CUtensorMap wmap;                           // [rows][row bytes] of this link's canonical blocks; with kFlagPanels its
                                                // first bytes hold a PanelRef instead
    const __half *x;                            // FP16 activations written before the launch, or null
    const unsigned long long *xin;              // hand-off words of the producing link (first element read), or null
    void *y;                                    // FP16/FP32 output, or null
    unsigned long long *xout[kMaxRanks];        // per rank: hand-off words of this link's output, at this rank's first
                                                // output element (null: nobody reads this link inside the chain)
    int N, src_stride, chunks;                  // src_stride: words from one rank's partial vector to the next rank's
    int units_q, units_r;                       // tiles * chunks = grid * units_q + units_r: CTA b takes units_q (+1 if b < units_r)
    int src_tag;                                // tag offset of the producing link
    int tag;                                    // tag offset of this link
    int world;                                  // ranks the output is pushed to
    unsigned flags;
    float out_scale;
};
static_assert(sizeof(ChainLinkDev) == 256, "link descriptor size");
// Panel layout: [K / 512 chunks][rows padded to 16][112 bytes]; row r of chunk c starts at (c * pad_rows + r) * 112.
struct PanelRef {
    const unsigned char *base;                  // first row of this link inside chunk 0's panel
    int pad_rows;                               // rows of a whole panel
};

constexpr int kInlineLinks = 8;
struct ChainParams {
    const ChainLinkDev *table;                  // device table, or null: the links are inl[]
    unsigned *ctl;
    unsigned long long *slots;
    unsigned long long region_slots;            // slots per region
    int n_links;
    int n_regions;                              // 1 (single link only) or 2
    unsigned tag_advance;                       // how far this launch moves the tag base
    int pad;
    ChainLinkDev inl[kInlineLinks];
};

struct LutImage {
    uint32_t w[256 * 64];
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
__device__ __align__(128) const LutImage g_chain_lut = make_lut_image();
static_assert(sizeof(LutImage) == kLutBytes, "table image size");

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
__device__ __forceinline__ uint32_t lds_lut(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

template <bool SIGNED_A, bool ZERO_C>
__device__ __forceinline__ void mma_bytes(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    if (ZERO_C) {
        if (SIGNED_A)
            asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
        else
            asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    } else {
        if (SIGNED_A)
            asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
        else
            asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
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
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 2000;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {      // one look, no suspension
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Called by all 32 lanes with warp-uniform arguments: one elected lane arms the barrier and starts the copy.
__device__ __forceinline__ void elected_bulk_load(uint32_t dst, const void *src, uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "@p mbarrier.arrive.expect_tx.shared::cta.b64 _, [%2], %3;\n\t"
        "@p cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %3, [%2];\n\t}"
        ::"r"(dst), "l"(src), "r"(bar), "n"(kUnitBytes) : "memory");
}
__device__ __forceinline__ void elected_tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "@p mbarrier.arrive.expect_tx.shared::cta.b64 _, [%4], %5;\n\t"
        "@p cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n\t}"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar), "n"(kUnitBytes) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// One lane-stream (half a block: 14 code-byte slots in four words, wa holding slots 0,1 in its
// upper half) becomes 18 A registers: 14 table entries (weights of trits 0..3 of each slot) and
// the four raw words (the code bytes themselves, paired with the fifth trit's activation).
__device__ __forceinline__ void decode_stream(uint32_t wa, uint32_t wb, uint32_t wc, uint32_t wd,
                                              uint32_t lane_base, uint32_t (&r)[kRegsPerSub]) {
    r[0] = lds_lut(prmt_imm<0x7624>(wa, lane_base));
    r[1] = lds_lut(prmt_imm<0x7634>(wa, lane_base));
    r[2] = lds_lut(prmt_imm<0x7604>(wb, lane_base));
    r[3] = lds_lut(prmt_imm<0x7614>(wb, lane_base));
    r[4] = lds_lut(prmt_imm<0x7624>(wb, lane_base));
    r[5] = lds_lut(prmt_imm<0x7634>(wb, lane_base));
    r[6] = lds_lut(prmt_imm<0x7604>(wc, lane_base));
    r[7] = lds_lut(prmt_imm<0x7614>(wc, lane_base));
    r[8] = lds_lut(prmt_imm<0x7624>(wc, lane_base));
    r[9] = lds_lut(prmt_imm<0x7634>(wc, lane_base));
    r[10] = lds_lut(prmt_imm<0x7604>(wd, lane_base));
    r[11] = lds_lut(prmt_imm<0x7614>(wd, lane_base));
    r[12] = lds_lut(prmt_imm<0x7624>(wd, lane_base));
    r[13] = lds_lut(prmt_imm<0x7634>(wd, lane_base));
    r[14] = wa;
    r[15] = wb;
    r[16] = wc;
    r[17] = wd;
}

// 64-bit words {payload, tag}: a 64-bit store is a single access, so a reader that finds the tag
// also has the payload.
__device__ __forceinline__ void word_publish(unsigned long long *p, uint32_t payload, uint32_t tag) {
    const unsigned long long w = ((unsigned long long)tag << 32) | payload;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void slot_publish(unsigned long long *p, float v, uint32_t tag) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long slot_read(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
// Hand-off words may have been written by another GPU into this GPU's memory.
__device__ __forceinline__ unsigned long long word_read(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ unsigned ctl_read(const unsigned *p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Value carried by a hand-off word (the tag has been checked): an FP16 output, or one rank's FP32 partial sum.
__device__ __forceinline__ float word_value(unsigned long long w, bool f32) {
    return f32 ? __uint_as_float((uint32_t)w) : __half2float(__ushort_as_half((unsigned short)(w & 0xffffu)));
}
// A sum of partial sums becomes the activation the next link reads by one rounding to FP16.
__device__ __forceinline__ float round_to_half(float v) { return __half2float(__float2half_rn(v)); }

// Activation `idx` of a link, whichever form it arrives in (the hand-off words have been waited for).
__device__ float link_x(const ChainLinkDev &L, size_t idx) {
    if (L.x) return __half2float(L.x[idx]);
    const bool f32 = (L.flags & kFlagSrcF32) != 0;
    const int parts = max(1, (int)((L.flags >> kFlagSrcPartsShift) & 15u));
    float sum = 0.0f;
    for (int r = 0; r < parts; ++r) sum += word_value(word_read(L.xin + (size_t)r * L.src_stride + idx), f32);
    return f32 ? round_to_half(sum) : sum;
}
// FP32 fallback for one block (row-major canonical bytes in shared memory): multiplies every
// weight so that NaN and Inf propagate exactly as in the reference.
__device__ float block_dot_fp32(const uint8_t *blk, const ChainLinkDev &L, size_t x0) {
    float sum = 0.0f;
    for (int j = 0; j < kCodeBytes; ++j) {
        uint32_t v = blk[2 + j];
        const int n = j == 25 ? 3 : 5;
        for (int i = 0; i < n; ++i) {
            const float w = (float)((int)(v % 3u) - 1);
            v /= 3u;
            sum = fmaf(w, link_x(L, x0 + 5 * j + i), sum);
        }
    }
    return sum;
}

// Units of a link that one warp of one CTA processes (units are numbered chunk-major).
struct WarpRange {
    int u_begin, n_units, c_first, t_first;
    int chunk_lo, chunk_hi;                 // chunks the CTA touches (chunk_hi < chunk_lo: none)
};
// u / tiles for 0 <= u < 2^22 and 1 <= tiles <= 2^16 without an integer division: the float quotient is off
// by at most one, which the remainder corrects.
__device__ __forceinline__ int div_tiles(int u, int tiles, float inv_tiles) {
    int q = (int)((float)u * inv_tiles);
    const int r = u - q * tiles;
    q += r >= tiles ? 1 : 0;
    q -= r < 0 ? 1 : 0;
    return q;
}
__device__ __forceinline__ WarpRange warp_range(int tiles, int units_q, int units_r, int warp) {
    WarpRange r;
    const int b = (int)blockIdx.x;
    const int cta_begin = b * units_q + min(b, units_r);
    const int cta_units = units_q + (b < units_r ? 1 : 0);
    r.u_begin = cta_begin + (cta_units * warp) / kWarps;
    const int u_end = cta_begin + (cta_units * (warp + 1)) / kWarps;
    r.n_units = u_end - r.u_begin;
    // one division for the CTA; a CTA spans at most kMaxChunksPerCta chunks, so the rest is comparisons
    r.chunk_lo = div_tiles(cta_begin, tiles, __frcp_rn((float)tiles));
    const int base = r.chunk_lo * tiles;
    int last = cta_begin + cta_units - 1 - base, hi = r.chunk_lo;
    int first = r.u_begin - base, cf = r.chunk_lo;
#pragma unroll
    for (int k = 1; k < kMaxChunksPerCta; ++k) {
        if (last >= tiles) { last -= tiles; ++hi; }
        if (first >= tiles) { first -= tiles; ++cf; }
    }
    r.chunk_hi = cta_units > 0 ? hi : r.chunk_lo - 1;
    r.c_first = cf;
    r.t_first = first;
    return r;
}

// ALL_PANELS: every link's weights are chunk-major panels, so the 2-D TMA path is compiled out.
template <bool ALL_PANELS>
__global__ void __launch_bounds__(kThreads, 1) tq1_gemv_chain_kernel(const __grid_constant__ ChainParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t window = (uint32_t)__cvta_generic_to_shared(smem);
    unsigned char *ring = smem;
    unsigned char *high = smem + (kWindowEnd - window);
    uint32_t *btab_all = reinterpret_cast<uint32_t *>(high);
    uint64_t *mbars = reinterpret_cast<uint64_t *>(high + kBtabBytes);
    GroupConst *gconst_all = reinterpret_cast<GroupConst *>(high + kBtabBytes + kMbarBytes);      // [buffer][group]
    int *xchg = reinterpret_cast<int *>(high + kBtabBytes + kMbarBytes + kGconstBytes) + (threadIdx.x >> 5) * kGroup;
    uint32_t *preptab = reinterpret_cast<uint32_t *>(high + kBtabBytes + kMbarBytes + kGconstBytes + kXchgBytes);
    volatile int *region_ok = reinterpret_cast<volatile int *>(high + kBtabBytes + kMbarBytes + kGconstBytes +
                                                               kXchgBytes + kPrepTabBytes);
    unsigned *ctl = P.ctl;
    if (window + kRingBytes > kLutWindowAddr) {      // the fixed-address table would overlap the ring
        if (threadIdx.x == 0) atomicExch(ctl + kCtlStatus, 2u);
        return;
    }

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int n_links = P.n_links;
    const ChainLinkDev *links = P.table ? P.table : P.inl;

    // ---- barriers, decode table, empty digit planes: nothing here depends on earlier kernels --------
    const uint32_t ring_warp = window + (uint32_t)(warp * kStages * kUnitBytes);
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&mbars[warp * kStages]);
    const uint32_t lut_bar = (uint32_t)__cvta_generic_to_shared(&mbars[kWarps * kStages]);
    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(bar0 + 8u * s, 1);
        if (warp == 0) mbar_init(lut_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (warp == 0) {
            mbar_expect_tx(lut_bar, kLutBytes);
            bulk_load(kLutWindowAddr, &g_chain_lut, kLutBytes, lut_bar);
        }
    }
    // k-slots of the other group of a sub-unit stay zero for the whole launch; the live bytes are
    // rewritten for every link
    for (int i = tid; i < (int)(kBtabBytes / 16); i += kThreads)
        reinterpret_cast<uint4 *>(btab_all)[i] = make_uint4(0u, 0u, 0u, 0u);

    // ---- producer cursor: the next unit this warp requests, possibly of a later link ------------------
    int issued = 0, consumed = 0;               // units requested / finished by this warp since the launch began
    uint32_t cstage = 0, cparity = 0;           // ring stage of the next unit to consume, and its barrier's phase
    int iss_link = 0, iss_left, iss_t, iss_tiles;
    int iss_x, iss_y;                           // canonical layout: TMA coordinates of the next unit
    const CUtensorMap *iss_map;
    const unsigned char *iss_src;               // panels: the next unit's 1792 bytes (null: canonical layout)
    size_t iss_wrap;                            // panels: extra bytes from a chunk's last tile to the next chunk's first
    auto cursor_load = [&]() {
        const ChainLinkDev &L = links[iss_link];
        const int l_tiles = (L.N + kTileRows - 1) / kTileRows;
        const WarpRange r = warp_range(l_tiles, L.units_q, L.units_r, warp);
        iss_left = r.n_units; iss_t = r.t_first; iss_tiles = l_tiles;
        iss_x = r.c_first * kChunkBytes; iss_y = r.t_first * kTileRows;
        iss_map = &L.wmap;
        iss_src = nullptr;
        if (ALL_PANELS || (L.flags & kFlagPanels)) {
            const PanelRef *ref = reinterpret_cast<const PanelRef *>(&L.wmap);
            const size_t stride = (size_t)ref->pad_rows * kChunkBytes;
            iss_src = ref->base + (size_t)r.c_first * stride + (size_t)r.t_first * kUnitBytes;
            iss_wrap = stride - (size_t)l_tiles * kUnitBytes;
        }
    };
    cursor_load();
    // Called by all 32 lanes (the cursor is warp-uniform); false when the chain has no unit left for this warp.
    auto issue_one = [&]() -> bool {
        while (iss_left == 0) {
            if (iss_link + 1 >= n_links) return false;
            ++iss_link;
            cursor_load();
        }
        const uint32_t s = (uint32_t)issued % kStages;
        if (ALL_PANELS || iss_src) {      // one contiguous bulk copy: measured 6.8 TB/s against 3.7 TB/s for the strided 112-byte rows
            elected_bulk_load(ring_warp + s * kUnitBytes, iss_src, bar0 + 8u * s);
            iss_src += kUnitBytes;
        } else {
            elected_tma_load_2d(ring_warp + s * kUnitBytes, iss_map, iss_x, iss_y, bar0 + 8u * s);
            iss_y += kTileRows;
        }
        ++issued;
        --iss_left;
        if (++iss_t == iss_tiles) {
            iss_t = 0; iss_y = 0; iss_x += kChunkBytes;
            if (ALL_PANELS || iss_src) iss_src += iss_wrap;
        }
        return true;
    };
    if (!ALL_PANELS && tid == 0 && !iss_src) asm volatile("prefetch.tensormap [%0];" ::"l"(iss_map) : "memory");

    // Let the next kernel in the stream start its own prologue as SMs free up, then wait until
    // everything before this kernel has finished before touching activations or the workspace.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const unsigned tag_base = ctl_read(ctl + kCtlEpoch);

    const int g = lane >> 2, q = lane & 3;
    const int cls = q >> 1, h = q & 1;
    const uint32_t lane_base = kLutWindowAddr + (uint32_t)lane * 4u;
    // byte offset of this lane's first half-block inside a tile (sub-unit 0, row g)
    const uint32_t lane_tile_off = (uint32_t)(((g * kChunkGroups + 2 * cls) * kBlockWords + 3 * h) * 4);

    // Where activation e of a group goes. Trits 0..3 of code byte j sit in the table-entry register of the
    // byte's slot; a fifth trit pairs with the raw word. Entry: byte offset of digit 0 inside a group's planes
    // (bits 0..15), index of the byte's fifth-trit activation (16..23, 255: the tail byte has none) and 3^i
    // (24..31, 0 for a fifth trit).
    if (tid < kGroup) {
        const int el = tid;
        const int bj = el < 125 ? el / 5 : 25;             // code byte
        const int bi = el < 125 ? el - 5 * bj : el - 125;  // trit within the byte
        const bool is_fifth = el < 125 && bi == 4;
        const int hh = bj < 14 ? 0 : 1;                    // which half-block lane decodes the byte
        const int slot = hh ? bj - 12 : bj;
        const int reg = !is_fifth ? slot : slot < 2 ? 14 : 15 + ((slot - 2) >> 2);
        const int pos = !is_fifth ? bi : slot < 2 ? slot + 2 : ((slot - 2) & 3);
        const uint32_t off = (uint32_t)((reg * 32 + hh) * 4 + pos);
        const uint32_t fifth = el < 125 ? (uint32_t)(5 * bj + 4) : 255u;
        const uint32_t pow3 = is_fifth ? 0u : bi == 0 ? 1u : bi == 1 ? 3u : bi == 2 ? 9u : 27u;
        preptab[el] = off | (fifth << 16) | (pow3 << 24);
    }
    if (tid == 0) *region_ok = 0;
    // planes of group gi of a chunk: sub-unit gi & 1, B lanes 18 * (gi >> 1) + {0, 1} (+ 4 per digit plane)
    const uint32_t warp_plane_off = (uint32_t)(((warp & 1) * kRegsPerSub * 32 + 18 * ((warp >> 1) & 1)) * 4);

    bool dead = false;                                 // a bounded wait ran out: stop waiting, finish quickly
    __syncthreads();                                   // barriers initialised, planes zeroed, table written
    PHASE_DECL

    for (int p = 0; p < n_links; ++p) {
        const ChainLinkDev &L = links[p];
        const int N = L.N, tiles = (L.N + kTileRows - 1) / kTileRows, chunks = L.chunks;
        const __half *xh = L.x;
        const unsigned long long *xin = L.xin;
        const unsigned flags = L.flags;
        const WarpRange R = warp_range(tiles, L.units_q, L.units_r, warp);
        const int n_units = R.n_units, chunk_lo = R.chunk_lo, chunk_hi = R.chunk_hi;
        const int buf = p & 1;
        uint32_t *btab = btab_all + buf * (kBtabOne / 4);
        GroupConst *gconst = gconst_all + buf * kPrepWarps;
        const unsigned tag = tag_base + (unsigned)L.tag + 1u;
        // Read the region's arrival counter now (checked after the barrier below): its round trip then
        // overlaps the wait for the activations.
        unsigned arrived_early = 0u;
        if (tid == 0 && p >= 2 && P.n_regions > 1) arrived_early = ctl_read(ctl + kCtlArrive + (p & 1));

        // ---- activation digits: warp w prepares group w & 3 of the CTA's chunk w >> 2, four activations per
        // lane: group maximum, fixed point, four signed byte planes. All reductions stay inside the warp. ------
        if (warp < 4 * (chunk_hi - chunk_lo + 1)) {
            const int cl = warp >> 2;
            const size_t x0 = (size_t)(chunk_lo + cl) * kChunkCols + (size_t)(warp & 3) * kGroup + lane;
            float xv[4];
            if (xin == nullptr) {
#pragma unroll
                for (int k = 0; k < 4; ++k) xv[k] = __half2float(xh[x0 + 32 * k]);
                // The activation loads are in flight: now top up this warp's weight tiles (issued the other
                // way round the few activation bytes queue behind megabytes of weight traffic).
                while (issued - consumed < kStages - 1 && issue_one()) {}
            } else {
                // Output of an earlier link: keep the weight pipeline full, then wait (bounded) for exactly the
                // words this lane needs.
                while (issued - consumed < kStages - 1 && issue_one()) {}
                const unsigned want = tag_base + (unsigned)L.src_tag + 1u;
                const bool src_f32 = (flags & kFlagSrcF32) != 0;
                const int parts = max(1, (int)((flags >> kFlagSrcPartsShift) & 15u));
                const size_t part_stride = (size_t)L.src_stride;
#pragma unroll
                for (int k = 0; k < 4; ++k) xv[k] = 0.0f;
                // one pass per rank that contributed a partial sum (a single pass for an ordinary source); the
                // partial sums are added in rank order, so the result does not depend on arrival order
                if (parts == 2) {
                    // two ranks' partial sums: all eight words of the lane are in flight together
                    const unsigned long long *src0 = xin + x0, *src1 = xin + part_stride + x0;
                    unsigned long long wa[4], wb[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const bool in = TQ1_IN_BOUNDS(x0 + 32 * k, (size_t)chunks * kChunkCols, 14u);
                        wa[k] = in ? word_read(src0 + 32 * k) : ((unsigned long long)want << 32);
                        wb[k] = in ? word_read(src1 + 32 * k) : ((unsigned long long)want << 32);
                    }
                    for (uint32_t spins = 0; !dead; ++spins) {
                        bool missing = false;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if ((unsigned)(wa[k] >> 32) != want) { wa[k] = word_read(src0 + 32 * k); missing = true; }
                            if ((unsigned)(wb[k] >> 32) != want) { wb[k] = word_read(src1 + 32 * k); missing = true; }
                        }
                        if (!missing) break;
                        if (spins > kMaxWaitSpins) { atomicExch(ctl + kCtlStatus, 4u); dead = true; }
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) xv[k] = (0.0f + word_value(wa[k], src_f32)) + word_value(wb[k], src_f32);
                } else
                for (int r = 0; r < parts; ++r) {
                    const unsigned long long *src = xin + (size_t)r * part_stride + x0;
                    unsigned long long wv[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        wv[k] = TQ1_IN_BOUNDS(x0 + 32 * k, (size_t)chunks * kChunkCols, 14u)
                                    ? word_read(src + 32 * k) : ((unsigned long long)want << 32);
                    // words that have not arrived are read again together: one round trip after the last of
                    // them lands, however many were late
                    for (uint32_t spins = 0; !dead; ++spins) {
                        bool missing = false;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if ((unsigned)(wv[k] >> 32) != want) {
                                wv[k] = word_read(src + 32 * k);
                                missing = true;
                            }
                        }
                        if (!missing) break;
                        if (spins > kMaxWaitSpins) { atomicExch(ctl + kCtlStatus, 4u); dead = true; }
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) xv[k] += word_value(wv[k], src_f32);
                }
                if (src_f32) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) xv[k] = round_to_half(xv[k]);
                }
            }
            PHASE(0)
            // non-negative floats order like their bit patterns: one redux instruction for the group maximum
            unsigned mbits = 0u;
            bool bad[4], anybad = false;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float a = fabsf(xv[k]);
                bad[k] = !(a <= 65504.0f);                         // NaN or Inf
                anybad = anybad || bad[k];
                mbits = max(mbits, bad[k] ? 0u : __float_as_uint(a));
            }
            mbits = __reduce_max_sync(0xffffffffu, mbits);
            const int group_bad = __any_sync(0xffffffffu, anybad);
            // 2^E <= m < 2^(E+1); fixed point xi = round(v * 2^(21-E)), |xi| <= 2^22
            const int e_biased = mbits != 0u ? (int)(mbits >> 23) : 127;
            const float up = __uint_as_float((uint32_t)(275 - e_biased) << 23);                // 2^(21-E)
            int xi[4], s5 = 0;
            uint32_t ent[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                xi[k] = bad[k] ? 0 : __float2int_rn(xv[k] * up);
                xchg[lane + 32 * k] = xi[k];                       // a code byte's first four trits need its fifth
                ent[k] = preptab[lane + 32 * k];
                s5 += (ent[k] >> 24) == 0u ? 121 * xi[k] : 0;      // 121 * sum of the fifth-trit activations
            }
            s5 = __reduce_add_sync(0xffffffffu, s5);
            if (lane == 0) {
                GroupConst gc;
                gc.sum = s5;
                gc.pow = __uint_as_float((uint32_t)(e_biased - 21) << 23);                     // 2^(E-21)
                gc.bad = group_bad;
                gc.pad = 0;
                gconst[warp] = gc;
            }
            __syncwarp();
            unsigned char *planes = reinterpret_cast<unsigned char *>(btab) + cl * kBtabChunk + warp_plane_off;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                // value paired with this k-slot: x_4 for the raw byte, 81 x_i - 3^i x_4 for trit i < 4
                const uint32_t fifth = (ent[k] >> 16) & 0xffu;
                const int x4 = fifth != 255u ? xchg[fifth] : 0;
                const int pw = (int)(ent[k] >> 24);
                const int v = pw ? 81 * xi[k] - pw * x4 : xi[k];
                // four signed byte digits: the bytes of v + 0x80808080 are the digits plus 128
                const uint32_t d = ((uint32_t)v + 0x80808080u) ^ 0x80808080u;
                unsigned char *base = planes + (ent[k] & 0xffffu);
                base[0] = (unsigned char)d;
                base[16] = (unsigned char)(d >> 8);
                base[32] = (unsigned char)(d >> 16);
                base[48] = (unsigned char)(d >> 24);
            }
        } else {
            while (issued - consumed < kStages - 1 && issue_one()) {}
            PHASE(0)
        }
        PHASE(4)
        __syncthreads();
        PHASE(5)
        // Every warp of this CTA has left link p-1, so the CTA is done with that link's slots; and
        // before anybody publishes into the region link p shares with link p-2, every CTA must be
        // done with link p-2's slots.
        if (tid == 0) {
            if (p >= 1) atomicAdd(ctl + kCtlArrive + ((p - 1) & 1), 1u);
            if (p >= 2 && P.n_regions > 1) {
                const unsigned need = gridDim.x * (unsigned)(p >> 1);
                uint32_t spins = 0;
                while (arrived_early < need && ctl_read(ctl + kCtlArrive + (p & 1)) < need) {
                    if (++spins > kMaxWaitSpins) { atomicExch(ctl + kCtlStatus, 6u); break; }
                }
            }
            *region_ok = p + 1;
        }
        PHASE(6)

        PHASE(1)
        if (p == 0) {                                   // the decode table must have landed
            uint32_t spins = 0;
            while (!mbar_try_wait(lut_bar, 0)) {
                if (++spins > kMaxWaitSpins) { if (lane == 0) atomicExch(ctl + kCtlStatus, 1u); dead = true; break; }
            }
        }

        // ---- per-warp streaming loop -------------------------------------------------------------------
        unsigned long long *slots = P.slots + (P.n_regions > 1 ? (size_t)(p & 1) * P.region_slots : 0);
        uint32_t breg[2][kRegsPerSub];
        int gsum[2];
        float gpow[2];
        int gbad[2];
        int c = R.c_first, t = R.t_first;
        // slot of row g of the current unit: units are numbered chunk-major, so it advances by 16 per unit
        unsigned long long *mine = slots + (size_t)R.u_begin * kTileRows + g;
        bool region_checked = !(p >= 2 && P.n_regions > 1);
        auto slow_wait = [&](uint32_t bar, uint32_t parity) -> uint32_t {     // the tile was not there at the first look
            uint32_t arrived = 0, spins = 0;
            while (!dead && !(arrived = mbar_try_wait(bar, parity))) {
                if (++spins > kMaxWaitSpins) {          // never hang: flag the failure and stop waiting
                    if (lane == 0) atomicExch(ctl + kCtlStatus, 1u);
                    dead = true;
                }
            }
            return arrived;
        };

        for (int left = n_units; left > 0;) {
            // ---- (re)load the B fragments and the group constants of this K chunk ----------------------
            const int cl = c - chunk_lo;
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
                for (int r = 0; r < kRegsPerSub; ++r)
                    breg[sub][r] = btab[((cl * 2 + sub) * kRegsPerSub + r) * 32 + lane];
                const GroupConst gc = gconst[cl * 4 + sub + 2 * cls];
                gsum[sub] = gc.sum;
                gpow[sub] = gc.pow;
                gbad[sub] = gc.bad;
            }
            const bool chunk_bad = __any_sync(0xffffffffu, (gbad[0] | gbad[1]) != 0);
            if (!region_checked) {      // thread 0 has seen every CTA leave the link that used these slots last
                region_checked = true;
                uint32_t spins = 0;
                while (*region_ok < p + 1 && !dead) {
                    if (++spins > kMaxWaitSpins) { if (lane == 0) atomicExch(ctl + kCtlStatus, 6u); dead = true; }
                }
            }
            const int seg = min(left, tiles - t);       // units of this chunk
            left -= seg;
            // One unit. BAD: some group of the chunk holds NaN/Inf activations and takes the FP32 path (rare; kept out
            // of the common loop so that it costs the common loop neither branches nor registers).
            auto unit = [&](auto bad_tag) {
                constexpr bool BAD = decltype(bad_tag)::value;
                const uint32_t bar = bar0 + 8u * cstage;
                uint32_t arrived = mbar_test_wait(bar, cparity);
                if (!arrived) arrived = slow_wait(bar, cparity);
                // (arrived >> 8) is zero, but only the hardware knows: the tile loads depend on the wait
                const uint32_t a1 = ring_warp + cstage * kUnitBytes + (arrived >> 8) + lane_tile_off;
                float acc1 = 0.0f, acc2 = 0.0f;             // rows g and g+8, this lane's two groups
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                    constexpr int kRow8 = 8 * kChunkBytes;
                    const uint32_t w1a = sub ? lds_off<28>(a1) : lds_off<0>(a1);
                    const uint32_t w1b = sub ? lds_off<32>(a1) : lds_off<4>(a1);
                    const uint32_t w1c = sub ? lds_off<36>(a1) : lds_off<8>(a1);
                    const uint32_t w1d = sub ? lds_off<40>(a1) : lds_off<12>(a1);
                    const uint32_t w2a = sub ? lds_off<kRow8 + 28>(a1) : lds_off<kRow8 + 0>(a1);
                    const uint32_t w2b = sub ? lds_off<kRow8 + 32>(a1) : lds_off<kRow8 + 4>(a1);
                    const uint32_t w2c = sub ? lds_off<kRow8 + 36>(a1) : lds_off<kRow8 + 8>(a1);
                    const uint32_t w2d = sub ? lds_off<kRow8 + 40>(a1) : lds_off<kRow8 + 12>(a1);
                    uint32_t r1[kRegsPerSub], r2[kRegsPerSub];
                    decode_stream(w1a, w1b, w1c, w1d, lane_base, r1);
                    decode_stream(w2a, w2b, w2c, w2d, lane_base, r2);
                    // One accumulator chain (splitting it in two or three measured the same and costs registers and
                    // additions); register pairs 0..6 hold signed weights, pairs 7,8 the raw (unsigned) code bytes.
                    int acc[4];
                    mma_bytes<true, true>(acc, r1[0], r2[0], r1[1], r2[1], breg[sub][0], breg[sub][1]);
                    mma_bytes<true, false>(acc, r1[2], r2[2], r1[3], r2[3], breg[sub][2], breg[sub][3]);
                    mma_bytes<true, false>(acc, r1[4], r2[4], r1[5], r2[5], breg[sub][4], breg[sub][5]);
                    mma_bytes<true, false>(acc, r1[6], r2[6], r1[7], r2[7], breg[sub][6], breg[sub][7]);
                    mma_bytes<true, false>(acc, r1[8], r2[8], r1[9], r2[9], breg[sub][8], breg[sub][9]);
                    mma_bytes<true, false>(acc, r1[10], r2[10], r1[11], r2[11], breg[sub][10], breg[sub][11]);
                    mma_bytes<true, false>(acc, r1[12], r2[12], r1[13], r2[13], breg[sub][12], breg[sub][13]);
                    mma_bytes<false, false>(acc, r1[14], r2[14], r1[15], r2[15], breg[sub][14], breg[sub][15]);
                    mma_bytes<false, false>(acc, r1[16], r2[16], r1[17], r2[17], breg[sub][16], breg[sub][17]);
                    // columns: lane q=0 holds planes 0,1 of the first group, q=1 planes 2,3; q=2/3 the second group.
                    // Combine each lane's plane pair first, then one shuffle per row brings the upper pair over.
                    const uint32_t pair1 = (uint32_t)acc[0] + ((uint32_t)acc[1] << 8);
                    const uint32_t pair2 = (uint32_t)acc[2] + ((uint32_t)acc[3] << 8);
                    const uint32_t hi1 = __shfl_down_sync(0xffffffffu, pair1, 1);
                    const uint32_t hi2 = __shfl_down_sync(0xffffffffu, pair2, 1);
                    // Every lane does the arithmetic (no branch); only the even lanes of a quad hold meaningful
                    // values, and only theirs are used below.
                    // 81 * (group sum) modulo 2^32, then times 81^-1 modulo 2^32: the exact integer group sum
                    const int s1 = (int)((pair1 + (hi1 << 16) - (uint32_t)gsum[sub]) * 0x781948b1u);
                    const int s2 = (int)((pair2 + (hi2 << 16) - (uint32_t)gsum[sub]) * 0x781948b1u);
                    float dot1 = (float)s1 * gpow[sub];
                    float dot2 = (float)s2 * gpow[sub];
                    if (BAD) {
                        if (h == 0 && gbad[sub]) {
                            const int group = sub + 2 * cls;
                            const unsigned char *tile = ring + (warp * kStages + cstage) * kUnitBytes;
                            const size_t x0 = ((size_t)c * kChunkGroups + group) * kGroup;
                            dot1 = block_dot_fp32(tile + (g * kChunkGroups + group) * kBlockBytes, L, x0);
                            dot2 = block_dot_fp32(tile + ((g + 8) * kChunkGroups + group) * kBlockBytes, L, x0);
                        }
                    }
                    const float sc1 = __half2float(__ushort_as_half((unsigned short)(w1a & 0xffffu)));
                    const float sc2 = __half2float(__ushort_as_half((unsigned short)(w2a & 0xffffu)));
                    acc1 = fmaf(sc1, dot1, acc1);
                    acc2 = fmaf(sc2, dot2, acc2);
                }
                // the stage consumed one iteration ago is free: refill it
                ++consumed;
                if (++cstage == kStages) { cstage = 0; cparity ^= 1u; }
                __syncwarp();
                if (issued - consumed < kStages - 1) issue_one();

                // quad: lanes q=0 (groups 0,1) and q=2 (groups 2,3) -> chunk partial in lane q=0
                acc1 += __shfl_down_sync(0xffffffffu, acc1, 2);
                acc2 += __shfl_down_sync(0xffffffffu, acc2, 2);
                if (q == 0 && TQ1_IN_BOUNDS((mine - slots) + 8, P.region_slots, 10u)) {
                    // value and tag travel in one 64-bit store, so whoever sees the tag has the value
                    slot_publish(mine, acc1, tag);
                    slot_publish(mine + 8, acc2, tag);
                }
                mine += kTileRows;
            };
            if (!chunk_bad) {
                for (int i = 0; i < seg; ++i) unit(std::false_type{});
            } else {
                for (int i = 0; i < seg; ++i) unit(std::true_type{});
            }
            t = 0;
            ++c;
        }

        PHASE(2)
        // ---- finish row tiles ----------------------------------------------------------------------------
        // Row tile t is finished by a fixed owner, the warp that processed its chunk t % chunks. The
        // owner polls the tile's slots (bounded) until every chunk's value carries this link's tag. All
        // CTAs of the grid are resident (one per SM), so the wait is for warps that are running. Lane
        // (hf, r) adds chunks hf, hf+2, ... of row r in ascending order and one shuffle joins the two
        // halves: the order of additions never depends on timing.
        {
            const int r = lane & 15, hf = lane >> 4;
            const size_t stride = (size_t)tiles * kTileRows;
            const bool swiglu = (flags & kFlagSwiglu) != 0;
            const bool out_f32 = (flags & kFlagOutF32) != 0;
            const float out_scale = L.out_scale;
            void *y = L.y;
            const int world = L.world;
            // The tiles of chunk cc that this warp owns are those with t % chunks == cc: walk them directly.
            int cc = R.c_first, t0 = R.t_first, tm0 = R.t_first % chunks;
            for (int left = n_units; left > 0;) {
                const int seg = min(left, tiles - t0);
                left -= seg;
                int first = cc - tm0;
                if (first < 0) first += chunks;
                for (int tt = t0 + first; tt < t0 + seg; tt += chunks) {
                    if (!TQ1_IN_BOUNDS((size_t)tt * kTileRows + 15 + (size_t)(chunks - 1) * stride, P.region_slots, 11u)) continue;   // warp-uniform
                    // warp-uniform: this warp owns row tile tt
                    const unsigned long long *ps = slots + (size_t)tt * kTileRows + r;
                    float total = 0.0f;
                    // BATCH slots per lane are in flight together; links with more than 16 chunks take the wide form
                    // (one round trip for K up to 18432 columns), the others the short one (fewer instructions)
                    auto gather = [&](auto batch_tag) {
                        constexpr int BATCH = decltype(batch_tag)::value;
                        for (int c0 = hf; c0 < chunks; c0 += 2 * BATCH) {
                            unsigned long long v[BATCH];
#pragma unroll
                            for (int k = 0; k < BATCH; ++k)
                                v[k] = c0 + 2 * k < chunks ? slot_read(ps + (size_t)(c0 + 2 * k) * stride)
                                                           : ((unsigned long long)tag << 32);
                            // partial sums that have not arrived are read again together (one round trip after the
                            // last of them lands); absent chunks were given the tag above
                            for (uint32_t spins = 0; !dead; ++spins) {
                                bool missing = false;
#pragma unroll
                                for (int k = 0; k < BATCH; ++k) {
                                    if ((unsigned)(v[k] >> 32) != tag) {
                                        v[k] = slot_read(ps + (size_t)(c0 + 2 * k) * stride);
                                        missing = true;
                                    }
                                }
                                if (!missing) break;
                                if (spins > kMaxWaitSpins) { atomicExch(ctl + kCtlStatus, 5u); dead = true; }
                            }
#pragma unroll
                            for (int k = 0; k < BATCH; ++k)
                                if (c0 + 2 * k < chunks) total += __uint_as_float((uint32_t)v[k]);
                        }
                    };
                    if (chunks > 16) gather(std::integral_constant<int, 18>{});
                    else gather(std::integral_constant<int, 8>{});
                    total += __shfl_xor_sync(0xffffffffu, total, 16);
                    int row = tt * kTileRows + r;
                    bool writer = hf == 0 && row < N;
                    if (swiglu) {
                        // rows come as (gate, up) pairs: the even lane of a pair holds silu(gate) * up
                        const float up = __shfl_down_sync(0xffffffffu, total, 1);
                        total = swiglu_f32(total, up);
                        writer = writer && (r & 1) == 0 && row + 1 < N;
                        row >>= 1;
                    }
                    total *= out_scale;
                    if (writer && TQ1_IN_BOUNDS(row, swiglu ? N >> 1 : N, 12u)) {
                        const __half hv = __float2half_rn(total);
                        if (y) {
                            if (out_f32) static_cast<float *>(y)[row] = total;
                            else static_cast<__half *>(y)[row] = hv;
                        }
                        // hand-off: the rounded FP16 value and this link's tag in one word, to every rank
                        // (a partial sum over this rank's K shard travels as FP32: the reader adds the ranks' words)
                        const uint32_t payload = (flags & kFlagPartialOut) ? __float_as_uint(total)
                                                                           : (uint32_t)__half_as_ushort(hv);
                        for (int pr = 0; pr < world; ++pr)
                            word_publish(L.xout[pr] + row, payload, tag);
                    }
                }
                t0 = 0;
                tm0 = 0;
                ++cc;
            }
        }
        PHASE(3)
    }
    PHASE_DUMP

    // ---- leave: the last CTA resets the launch-scoped counters and moves the tag base on ----------------
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(ctl + kCtlExit, 1u);
        if (prev == gridDim.x - 1) {
            ctl[kCtlExit] = 0u;
            ctl[kCtlArrive] = 0u;
            ctl[kCtlArrive + 1] = 0u;
            ctl[kCtlEpoch] = tag_base + P.tag_advance;
            // Tags are 32-bit: long before they could wrap onto values that old slots still carry, ask the
            // caller (through the status word) to zero the workspace between two launches.
            if (tag_base + P.tag_advance >= kTagRefresh) atomicCAS(ctl + kCtlStatus, 0u, 7u);
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

// Per-device launch state: the shared-memory opt-in is an attribute of the function on ONE device.
constexpr int kMaxDevices = 64;
struct DeviceState {
    int sm_count;
    bool attr_set;
};
DeviceState g_dev[kMaxDevices] = {};

int device_state(DeviceState **out) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return cuda_fail(err, "tq1 chain: cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) return fail(TQ1_ERR_INVALID, "tq1 chain: device %d out of range", dev);
    DeviceState &st = g_dev[dev];
    if (!st.attr_set) {
        int sms = 0;
        err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (err != cudaSuccess || sms <= 0) return cuda_fail(err, "tq1 chain: SM count");
        err = cudaFuncSetAttribute(tq1_gemv_chain_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)(kWindowEnd + kHighBytes));
        if (err == cudaSuccess)
            err = cudaFuncSetAttribute(tq1_gemv_chain_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(kWindowEnd + kHighBytes));
        if (err != cudaSuccess) return cuda_fail(err, "tq1 chain: shared memory opt-in");
        st.sm_count = sms;
        st.attr_set = true;
    }
    *out = &st;
    return TQ1_OK;
}

// A CTA keeps the digit planes of at most kMaxChunksPerCta chunks: check that no CTA of a grid of
// `grid` CTAs spans more.
bool span_ok(int tiles, int chunks, int grid) {
    const int total = tiles * chunks, q = total / grid, r = total % grid;
    for (int b = 0; b < grid; ++b) {
        const int begin = b * q + (b < r ? b : r);
        const int end = begin + q + (b < r ? 1 : 0);
        if (end > begin && (end - 1) / tiles - begin / tiles + 1 > kMaxChunksPerCta) return false;
    }
    return true;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Host side: turning caller-level links into kernel descriptors.

bool gemv_chain_shape_ok(int N, int K) {
    return N >= 1 && K >= kChunkCols && K % kChunkCols == 0 && K / kChunkCols <= 128;
}

bool gemv_chain_supported(const uint8_t *blocks, int N, int K) {
    return gemv_chain_shape_ok(N, K) && (reinterpret_cast<uintptr_t>(blocks) & 15) == 0;
}

namespace {

constexpr size_t kRegionSlotsTwo = kWsSlotRegionBytes / 2 / sizeof(unsigned long long);    // 1 Mi slots per region

// Rows of one device link: its partial-sum slots (one per row and K chunk) must fit one region.
int rows_per_link(int N, int K, size_t region_slots) {
    const size_t chunks = K / kChunkCols;
    const size_t cap = region_slots / chunks / kTileRows * kTileRows;
    if ((size_t)N <= cap) return N;
    const size_t parts = ((size_t)N + cap - 1) / cap;
    return (int)((((size_t)N + parts - 1) / parts + kTileRows - 1) / kTileRows * kTileRows);
}

int encode_link_map(CUtensorMap *map, const uint8_t *blocks, int N, int K) {
    EncodeTiledFn encode = encode_fn();
    if (!encode) return fail(TQ1_ERR_CUDA, "tq1 chain: cuTensorMapEncodeTiled is unavailable");
    const cuuint64_t row_bytes = (cuuint64_t)(K / kGroup) * kBlockBytes;
    const cuuint64_t dims[2] = {row_bytes, (cuuint64_t)N};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {kChunkBytes, kTileRows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult res = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(blocks), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(TQ1_ERR_CUDA, "tq1 chain: cuTensorMapEncodeTiled failed (%d)", (int)res);
    return TQ1_OK;
}

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// Output elements of a caller-level link on one rank, and gathered over the ranks.
int link_out_local(const tq1_chain_link &l) { return l.swiglu ? l.N / 2 : l.N; }

}  // namespace

size_t gemv_chain_handoff_bytes(const tq1_chain_link *links, int n_links, int world) {
    size_t total = 0;
    for (int i = 0; i < n_links; ++i)
        total += align256((size_t)link_out_local(links[i]) * (size_t)(world < 1 ? 1 : world) * sizeof(unsigned long long));
    return total;
}

int gemv_chain_device_links(const tq1_chain_link *links, int n_links, size_t region_slots) {
    int total = 0;
    for (int i = 0; i < n_links; ++i) {
        if (links[i].K <= 0 || links[i].K % kChunkCols) return -1;
        const int step = rows_per_link(links[i].N, links[i].K, region_slots);
        total += (links[i].N + step - 1) / step;
    }
    return total;
}

// Fills `out` (host memory, gemv_chain_device_links() entries). handoff[r] is rank r's hand-off area
// (the local one for rank == r); each caller-level link owns a 256-byte aligned range of it that holds
// the gathered output, one 64-bit word per element.
int gemv_chain_describe(const tq1_chain_link *links, int n_links, int rank, int world,
                        unsigned long long *const *handoff, size_t region_slots, int grid,
                        std::vector<ChainLinkDev> &out) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
        return fail(TQ1_ERR_INVALID, "tq1 chain: rank %d of %d is out of range (at most %d ranks)", rank, world, kMaxRanks);
    std::vector<size_t> offset(n_links);          // in words
    std::vector<bool> consumed(n_links, false);
    size_t cursor = 0;
    for (int i = 0; i < n_links; ++i) {
        offset[i] = cursor;
        cursor += align256((size_t)link_out_local(links[i]) * world * sizeof(unsigned long long)) / sizeof(unsigned long long);
        if (!links[i].x) {
            if (links[i].source < 0 || links[i].source >= i)
                return fail(TQ1_ERR_INVALID, "tq1 chain: link %d reads link %d, which does not precede it", i, links[i].source);
            consumed[links[i].source] = true;
        }
    }
    out.clear();
    for (int i = 0; i < n_links; ++i) {
        const tq1_chain_link &l = links[i];
        if (!l.blocks) return fail(TQ1_ERR_INVALID, "tq1 chain: link %d has no weights", i);
        if (l.layout != TQ1_LAYOUT_BLOCKS && l.layout != TQ1_LAYOUT_PANELS)
            return fail(TQ1_ERR_INVALID, "tq1 chain: link %d has an unknown weight layout %d", i, l.layout);
        if (!gemv_chain_supported(l.blocks, l.N, l.K))
            return fail(TQ1_ERR_INVALID,
                        "tq1 chain: link %d (%dx%d) needs K %% 512 == 0, at most 128 K chunks and 16-byte aligned blocks",
                        i, l.N, l.K);
        if (l.swiglu && (l.N % 2))
            return fail(TQ1_ERR_INVALID, "tq1 chain: link %d: %d rows cannot be (gate, up) pairs", i, l.N);
        if (world > 1 && (l.N % kTileRows))
            return fail(TQ1_ERR_INVALID, "tq1 chain: link %d: a shard of %d rows is not a multiple of %d", i, l.N, kTileRows);
        if (l.partial && l.swiglu)
            return fail(TQ1_ERR_INVALID, "tq1 chain: link %d: a partial sum cannot take the gated activation", i);
        const unsigned long long *xin = nullptr;
        unsigned src_flags = 0u;
        int src_stride = 0;
        if (!l.x) {
            const tq1_chain_link &s = links[l.source];
            // an ordinary source is the concatenation of the ranks' rows; a partial one is a sum of `world` vectors
            const long long have = (long long)link_out_local(s) * (s.partial ? 1 : world);
            if (l.source_offset < 0 || (long long)l.source_offset + l.K > have)
                return fail(TQ1_ERR_INVALID, "tq1 chain: link %d reads elements [%d, %d) of link %d, which has %lld",
                            i, l.source_offset, l.source_offset + l.K, l.source, have);
            if (!handoff || !handoff[rank]) return fail(TQ1_ERR_INVALID, "tq1 chain: no hand-off area");
            xin = handoff[rank] + offset[l.source] + l.source_offset;
            if (s.partial) {
                src_flags = kFlagSrcF32 | ((unsigned)world << kFlagSrcPartsShift);
                src_stride = link_out_local(s);
            }
        }
        const int step = rows_per_link(l.N, l.K, region_slots);
        if (step < l.N && l.swiglu && (step % 2))
            return fail(TQ1_ERR_INVALID, "tq1 chain: link %d cannot be split into row ranges", i);
        const size_t row_bytes = (size_t)(l.K / kGroup) * kBlockBytes;
        const int out_local = link_out_local(l);
        for (int n0 = 0; n0 < l.N; n0 += step) {
            const int rows = l.N - n0 < step ? l.N - n0 : step;
            ChainLinkDev d;
            memset(&d, 0, sizeof(d));
            if (l.layout == TQ1_LAYOUT_PANELS) {
                PanelRef ref;
                ref.base = l.blocks + (size_t)n0 * kChunkBytes;
                ref.pad_rows = (l.N + kTileRows - 1) / kTileRows * kTileRows;
                memcpy(&d.wmap, &ref, sizeof(ref));
            } else {
                int rc = encode_link_map(&d.wmap, l.blocks + (size_t)n0 * row_bytes, rows, l.K);
                if (rc != TQ1_OK) return rc;
            }
            d.x = static_cast<const __half *>(l.x);
            d.xin = xin;
            const int out0 = l.swiglu ? n0 / 2 : n0;
            if (l.y)
                d.y = l.y_is_f32 ? static_cast<void *>(static_cast<float *>(l.y) + out0)
                                 : static_cast<void *>(static_cast<__half *>(l.y) + out0);
            d.N = rows;
            const int d_tiles = (rows + kTileRows - 1) / kTileRows;
            d.src_stride = src_stride;
            d.chunks = l.K / kChunkCols;
            d.units_q = d_tiles * d.chunks / grid;
            d.units_r = d_tiles * d.chunks % grid;
            if (!span_ok(d_tiles, d.chunks, grid))
                return fail(TQ1_ERR_INVALID, "tq1 chain: link %d (%dx%d) spreads a CTA over more than %d K chunks",
                            i, l.N, l.K, kMaxChunksPerCta);
            d.src_tag = l.x ? 0 : l.source;
            d.tag = i;
            d.flags = (l.y_is_f32 ? kFlagOutF32 : 0u) | (l.swiglu ? kFlagSwiglu : 0u) |
                      (l.layout == TQ1_LAYOUT_PANELS ? kFlagPanels : 0u) | (l.partial ? kFlagPartialOut : 0u) | src_flags;
            d.out_scale = l.out_scale == 0.0f ? 1.0f : l.out_scale;
            d.world = 0;
            if (consumed[i] || world > 1) {
                if (!handoff) return fail(TQ1_ERR_INVALID, "tq1 chain: no hand-off area");
                d.world = world;
                for (int pr = 0; pr < world; ++pr) {
                    if (!handoff[pr]) return fail(TQ1_ERR_INVALID, "tq1 chain: no hand-off area for rank %d", pr);
                    d.xout[pr] = handoff[pr] + offset[i] + (size_t)rank * out_local + out0;
                }
            }
            out.push_back(d);
        }
    }
    return TQ1_OK;
}

// True when every link's weights are chunk-major panels (the kernel variant without the 2-D TMA path).
bool all_panels(const ChainLinkDev *links, int n) {
    for (int i = 0; i < n; ++i)
        if (!(links[i].flags & kFlagPanels)) return false;
    return n > 0;
}

int gemv_chain_launch(const ChainLinkDev *table_dev, const ChainLinkDev *inline_links, int n_dev_links,
                      bool panels_only, unsigned tag_advance, void *workspace, size_t region_slots, int n_regions,
                      cudaStream_t stream) {
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc != TQ1_OK) return rc;
    ChainParams params;
    memset(&params, 0, sizeof(params));
    params.table = table_dev;
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    params.ctl = reinterpret_cast<unsigned *>(ws);
    params.slots = reinterpret_cast<unsigned long long *>(ws + kWsStatusBytes);
    params.region_slots = region_slots;
    params.n_links = n_dev_links;
    params.n_regions = n_regions;
    params.tag_advance = tag_advance;
    if (!table_dev) {
        if (n_dev_links > kInlineLinks)
            return fail(TQ1_ERR_INVALID, "tq1 chain: %d links do not fit a launch without a plan (at most %d)",
                        n_dev_links, kInlineLinks);
        memcpy(params.inl, inline_links, sizeof(ChainLinkDev) * n_dev_links);
    }
    static const bool use_pdl = getenv("TQ1_DISABLE_PDL") == nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)st->sm_count);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kWindowEnd + kHighBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    cudaError_t err = panels_only ? cudaLaunchKernelEx(&cfg, tq1_gemv_chain_kernel<true>, params)
                                  : cudaLaunchKernelEx(&cfg, tq1_gemv_chain_kernel<false>, params);
    if (err != cudaSuccess) return cuda_fail(err, "tq1 chain: launch");
    return TQ1_OK;
}

int gemv_chain_grid(int *grid) {
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc != TQ1_OK) return rc;
    *grid = st->sm_count;
    return TQ1_OK;
}

size_t gemv_chain_region_slots() { return kRegionSlotsTwo; }
size_t gemv_chain_link_bytes() { return sizeof(ChainLinkDev); }

// One product through the chain kernel (a chain of one link per row range).
int launch_gemv_single(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int N, int K, bool swiglu,
                       void *workspace, size_t slot_bytes, cudaStream_t stream) {
    int grid = 0;
    int rc = gemv_chain_grid(&grid);
    if (rc != TQ1_OK) return rc;
    // single links never run ahead of one another inside a launch, so one region holds all the slots
    const size_t region_slots = slot_bytes / sizeof(unsigned long long);
    tq1_chain_link l;
    memset(&l, 0, sizeof(l));
    l.blocks = blocks; l.N = N; l.K = K; l.x = x; l.y = y; l.y_is_f32 = y_f32; l.swiglu = swiglu; l.out_scale = 1.0f;
    std::vector<ChainLinkDev> dev;
    rc = gemv_chain_describe(&l, 1, 0, 1, nullptr, region_slots, grid, dev);
    if (rc != TQ1_OK) return rc;
    for (size_t i = 0; i < dev.size(); ++i) {          // row ranges of a very tall matrix: one launch each
        dev[i].tag = 0;
        rc = gemv_chain_launch(nullptr, &dev[i], 1, all_panels(&dev[i], 1), 1u, workspace, region_slots, 1, stream);
        if (rc != TQ1_OK) return rc;
    }
    return TQ1_OK;
}


// A few activation rows through the batch-1 kernel: one launch of M independent links over the same weights
// (the second and later passes read them from L2). Faster than the batched kernel while M passes cost less
// than its decode-to-tensor-memory pipeline; the crossover is recorded by the dispatch sweep.
int launch_gemv_looped(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int M, int N, int K, bool swiglu,
                       void *workspace, cudaStream_t stream) {
    int grid = 0;
    int rc = gemv_chain_grid(&grid);
    if (rc != TQ1_OK) return rc;
    if (M < 1 || M > kInlineLinks) return fail(TQ1_ERR_INVALID, "tq1 chain: %d activation rows do not fit one launch", M);
    tq1_chain_link links[kInlineLinks];
    memset(links, 0, sizeof(links));
    const size_t out_row = (size_t)(swiglu ? N / 2 : N) * (y_f32 ? sizeof(float) : sizeof(__half));
    for (int m = 0; m < M; ++m) {
        links[m].blocks = blocks; links[m].N = N; links[m].K = K;
        links[m].x = x + (size_t)m * K;
        links[m].y = static_cast<unsigned char *>(y) + (size_t)m * out_row;
        links[m].y_is_f32 = y_f32; links[m].swiglu = swiglu; links[m].out_scale = 1.0f;
    }
    std::vector<ChainLinkDev> dev;
    rc = gemv_chain_describe(links, M, 0, 1, nullptr, kRegionSlotsTwo, grid, dev);
    if (rc != TQ1_OK) return rc;
    if ((int)dev.size() != M) return fail(TQ1_ERR_INVALID, "tq1 chain: matrix too tall for the looped path");
    return gemv_chain_launch(nullptr, dev.data(), M, all_panels(dev.data(), M), (unsigned)M, workspace,
                             kRegionSlotsTwo, 2, stream);
}

// Largest M that tq1_linear_f16 sends through launch_gemv_looped (0 or 1: none).
static int g_loop_tokens = 2;
int gemv_loop_tokens() { return g_loop_tokens; }
int gemv_set_loop_tokens(int tokens) {
    if (tokens < 0 || tokens > kInlineLinks) return TQ1_ERR_INVALID;
    g_loop_tokens = tokens;
    return TQ1_OK;
}
// The looped path takes the shape when one link holds the whole matrix in one slot region of the two.
bool gemv_looped_fits(const uint8_t *blocks, int M, int N, int K) {
    if (M < 2 || M > g_loop_tokens || !gemv_chain_supported(blocks, N, K)) return false;
    int grid = 0;
    if (gemv_chain_grid(&grid) != TQ1_OK) return false;
    if (rows_per_link(N, K, kRegionSlotsTwo) != N) return false;
    return span_ok((N + kTileRows - 1) / kTileRows, K / kChunkCols, grid);
}

// Whether the chain kernel takes one product of this shape on the current device.
bool gemv_chain_fits(const uint8_t *blocks, int N, int K) {
    if (!gemv_chain_supported(blocks, N, K)) return false;
    int grid = 0;
    if (gemv_chain_grid(&grid) != TQ1_OK) return false;
    const int rows = rows_per_link(N, K, kWsSlotRegionBytes / sizeof(unsigned long long));
    return span_ok((rows + kTileRows - 1) / kTileRows, K / kChunkCols, grid);
}

size_t gemv_chain_workspace_bytes(int N, int K) {
    const size_t rows = rows_per_link(N, K, kWsSlotRegionBytes / sizeof(unsigned long long));
    const size_t tiles = (rows + kTileRows - 1) / kTileRows;
    return kWsStatusBytes + (size_t)(K / kChunkCols) * tiles * kTileRows * sizeof(unsigned long long);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the batch-1 GEMV.
//
// Some hosts cannot give this library scratch memory at call time: code that runs inside a
// stream-capture region (where cudaMalloc is illegal), plugin hosts whose whole device budget
// was handed out when the model was loaded, and real-time loops that must not touch the
// allocator. For them the scratch of the GEMV (control words and per-chunk partial-sum slots)
// lives in this fixed array, which every GPU that loads the library holds until the process
// exits.
constexpr size_t kNoAllocScratchBytes = 2u << 20;       // 2 MiB: N*K up to about 1.3e8 weights
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

namespace {
void *g_noalloc_ptr[kMaxDevices] = {};     // device address of g_noalloc_scratch, per device

int noalloc_scratch(void **out, const char *who) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return cuda_fail(err, who);
    if (dev < 0 || dev >= kMaxDevices) return fail(TQ1_ERR_INVALID, "%s: device %d out of range", who, dev);
    if (!g_noalloc_ptr[dev]) {
        // In host code the array's name is only a handle; the kernel needs its device address. The
        // array starts zero-filled (static storage) and the kernel never needs it cleared again.
        void *ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (err != cudaSuccess) return cuda_fail(err, who);
        g_noalloc_ptr[dev] = ptr;
    }
    *out = g_noalloc_ptr[dev];
    return TQ1_OK;
}
}  // namespace

int gemv_noalloc(const uint8_t *blocks, const __half *x, void *y, bool y_f32, int N, int K, cudaStream_t stream) {
    if (!gemv_chain_supported(blocks, N, K))
        return fail(TQ1_ERR_INVALID,
                    "tq1_gemv_f16_noalloc: needs K %% 512 == 0, at most 128 K chunks and 16-byte aligned blocks "
                    "(got N=%d K=%d)", N, K);
    const size_t slot_bytes = kNoAllocScratchBytes - kWsStatusBytes;
    const size_t need = (size_t)(K / kChunkCols) * ((N + kTileRows - 1) / kTileRows) * kTileRows * sizeof(unsigned long long);
    if (need > slot_bytes)
        return fail(TQ1_ERR_WORKSPACE,
                    "tq1_gemv_f16_noalloc: %dx%d needs %zu bytes of scratch, the built-in array holds %zu",
                    N, K, need + kWsStatusBytes, (size_t)kNoAllocScratchBytes);
    void *scratch = nullptr;
    int rc = noalloc_scratch(&scratch, "tq1_gemv_f16_noalloc");
    if (rc != TQ1_OK) return rc;
    return launch_gemv_single(blocks, x, y, y_f32, N, K, false, scratch, slot_bytes, stream);
}

int gemv_noalloc_status(unsigned *out_host, cudaStream_t stream) {
    void *scratch = nullptr;
    int rc = noalloc_scratch(&scratch, "tq1_gemv_noalloc_status");
    if (rc != TQ1_OK) return rc;
    cudaError_t err = cudaMemcpyAsync(out_host, scratch, sizeof(unsigned), cudaMemcpyDeviceToHost, stream);
    if (err != cudaSuccess) return cuda_fail(err, "tq1_gemv_noalloc_status");
    return TQ1_OK;
}

}  // namespace tq1

#ifdef TQ1_PHASE_TIMERS
extern "C" int tq1_debug_read_phases(long long *out, int count) {
    return (int)cudaMemcpyFromSymbol(out, tq1::g_phase_acc, sizeof(long long) * count);
}
#endif

// ---------------------------------------------------------------------------------------------
// C ABI of the chain (declared in include/ternel_b200.h).

using namespace tq1;

struct tq1_chain_plan {
    std::vector<ChainLinkDev> host;     // what was uploaded (kept so the upload's source outlives the copy)
    const ChainLinkDev *table_dev;
    void *workspace;
    int n_dev_links;
    int n_links;
};

extern "C" {

size_t tq1_chain_handoff_bytes(const tq1_chain_link *links, int n_links, int world) {
    if (!links || n_links <= 0) return 0;
    return gemv_chain_handoff_bytes(links, n_links, world);
}

size_t tq1_chain_workspace_bytes(const tq1_chain_link *links, int n_links, int world) {
    if (!links || n_links <= 0) return 0;
    // control words, two slot regions, and (single GPU) the hand-off words behind them
    return kWsScratchOffset + (world <= 1 ? gemv_chain_handoff_bytes(links, n_links, 1) : 0);
}

size_t tq1_chain_table_bytes(const tq1_chain_link *links, int n_links) {
    if (!links || n_links <= 0) return 0;
    const int n = gemv_chain_device_links(links, n_links, gemv_chain_region_slots());
    return n <= 0 ? 0 : (size_t)n * sizeof(ChainLinkDev);
}

static int chain_describe_checked(const tq1_chain_link *links, int n_links, const tq1_chain_peers *peers,
                                  void *workspace, size_t workspace_bytes, std::vector<ChainLinkDev> &dev) {
    if (!links || n_links <= 0) return fail(TQ1_ERR_INVALID, "tq1 chain: no links");
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255))
        return fail(TQ1_ERR_WORKSPACE, "tq1 chain: a 256-byte aligned workspace is required");
    const int world = peers ? peers->world : 1;
    const int rank = peers ? peers->rank : 0;
    const size_t need = tq1_chain_workspace_bytes(links, n_links, world);
    if (workspace_bytes < need)
        return fail(TQ1_ERR_WORKSPACE, "tq1 chain: workspace of %zu bytes required, got %zu", need, workspace_bytes);
    unsigned long long *areas[kMaxRanks] = {};
    if (peers) {
        if (world < 1 || world > kMaxRanks) return fail(TQ1_ERR_INVALID, "tq1 chain: world size %d", world);
        for (int r = 0; r < world; ++r) {
            if (!peers->handoff[r] || (reinterpret_cast<uintptr_t>(peers->handoff[r]) & 255))
                return fail(TQ1_ERR_INVALID, "tq1 chain: hand-off area of rank %d missing or not 256-byte aligned", r);
            areas[r] = static_cast<unsigned long long *>(peers->handoff[r]);
        }
    } else {
        areas[0] = reinterpret_cast<unsigned long long *>(static_cast<unsigned char *>(workspace) + kWsScratchOffset);
    }
    int grid = 0;
    int rc = gemv_chain_grid(&grid);
    if (rc != TQ1_OK) return rc;
    return gemv_chain_describe(links, n_links, rank, world, areas, gemv_chain_region_slots(), grid, dev);
}

int tq1_chain_plan_create(const tq1_chain_link *links, int n_links, const tq1_chain_peers *peers,
                          void *workspace, size_t workspace_bytes, void *table, size_t table_bytes,
                          void *stream, tq1_chain_plan **out) {
    if (!out) return fail(TQ1_ERR_INVALID, "tq1_chain_plan_create: null pointer");
    *out = nullptr;
    tq1_chain_plan *plan = new (std::nothrow) tq1_chain_plan();
    if (!plan) return fail(TQ1_ERR_INVALID, "tq1_chain_plan_create: out of host memory");
    int rc = chain_describe_checked(links, n_links, peers, workspace, workspace_bytes, plan->host);
    if (rc != TQ1_OK) { delete plan; return rc; }
    const size_t bytes = plan->host.size() * sizeof(ChainLinkDev);
    if (!table || table_bytes < bytes || (reinterpret_cast<uintptr_t>(table) & 127)) {
        delete plan;
        return fail(TQ1_ERR_WORKSPACE, "tq1_chain_plan_create: a 128-byte aligned device table of %zu bytes is required", bytes);
    }
    cudaError_t err = cudaMemcpyAsync(table, plan->host.data(), bytes, cudaMemcpyHostToDevice,
                                      static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) { delete plan; return cuda_fail(err, "tq1_chain_plan_create: table upload"); }
    plan->table_dev = static_cast<const ChainLinkDev *>(table);
    plan->workspace = workspace;
    plan->n_dev_links = (int)plan->host.size();
    plan->n_links = n_links;
    *out = plan;
    return TQ1_OK;
}

int tq1_chain_plan_run(const tq1_chain_plan *plan, void *stream) {
    if (!plan) return fail(TQ1_ERR_INVALID, "tq1_chain_plan_run: null plan");
    return gemv_chain_launch(plan->table_dev, nullptr, plan->n_dev_links,
                             all_panels(plan->host.data(), (int)plan->host.size()), (unsigned)plan->n_links, plan->workspace,
                             gemv_chain_region_slots(), 2, static_cast<cudaStream_t>(stream));
}

void tq1_chain_plan_destroy(tq1_chain_plan *plan) { delete plan; }

int tq1_linear_chain_f16(const tq1_chain_link *links, int n_links, void *workspace, size_t workspace_bytes,
                         void *stream) {
    std::vector<ChainLinkDev> dev;
    int rc = chain_describe_checked(links, n_links, nullptr, workspace, workspace_bytes, dev);
    if (rc != TQ1_OK) return rc;
    return gemv_chain_launch(nullptr, dev.data(), (int)dev.size(), all_panels(dev.data(), (int)dev.size()),
                             (unsigned)n_links, workspace,
                             gemv_chain_region_slots(), 2, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
