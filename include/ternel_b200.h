/*
 * ternel_b200 — C ABI of the B200-native packed ternary (TQ1_G128) linear and
 * embedding path. Plain pointers and sizes only; no C++ or torch types.
 *
 * Weight layout ("canonical blocks"): W[N out][K in], K % 128 == 0, stored
 * row-major as 28-byte blocks [N][K/128][28]:
 *   byte 0..1  raw little-endian FP16 scale bits
 *   byte 2+j   sum_{i<5} c[5j+i]*3^i  (j = 0..24, value <= 242)
 *   byte 27    c[125] + 3 c[126] + 9 c[127]       (value <= 26)
 * c in {0,1,2}; logical weight = (c - 1) * scale.
 *
 * Each entry point cites the interface of the reference project
 * (inductiveML/ternel, paths relative to its root) that it stands in for.
 *
 * Conventions: every function returns TQ1_OK (0) or a negative TQ1_ERR_* code
 * and never throws, aborts or allocates device memory. Device entry points are
 * stream-ordered and asynchronous: they enqueue work on `stream` (a
 * cudaStream_t passed as void*; NULL = the legacy default stream) and return
 * without synchronising. tq1_last_error() gives a per-thread message for the
 * last failing call.
 */
#ifndef TERNEL_B200_H
#define TERNEL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TQ1_OK 0
#define TQ1_ERR_INVALID (-1)   /* bad argument, shape, alignment or null pointer */
#define TQ1_ERR_FORMAT (-2)    /* non-ternary code or illegal base-3 byte (fail closed) */
#define TQ1_ERR_CUDA (-3)      /* a CUDA runtime call or kernel launch failed */
#define TQ1_ERR_WORKSPACE (-4) /* workspace missing, misaligned or too small */

#define TQ1_GROUP 128
#define TQ1_BLOCK_BYTES 28

/* Library ABI version (bumped when a signature changes). */
int tq1_abi_version(void);

/* Message for the last failing call on this thread ("" if none). */
const char *tq1_last_error(void);

/* ---- host-side format codec -------------------------------------------- */

/* Replaces encode_tq1_blocks (src/bonsai_tq1/format.py:66-91).
 * scales: [groups][2] raw FP16 bytes; trits: [groups][128] in {0,1,2};
 * blocks: [groups][28] out. Any trit > 2 => TQ1_ERR_FORMAT, *n_bad = count,
 * nothing written. */
int tq1_pack_blocks(const uint8_t *scales, const uint8_t *trits, uint8_t *blocks,
                    int64_t groups, int64_t *n_bad);

/* Replaces decode_tq1_blocks (src/bonsai_tq1/format.py:94-122). With
 * validate != 0 any byte > 242 in slots 0..24 or > 26 in the tail slot gives
 * TQ1_ERR_FORMAT with the two counts, nothing written. */
int tq1_unpack_blocks(const uint8_t *blocks, uint8_t *scales, uint8_t *trits,
                      int64_t groups, int validate, int64_t *n_bad_full, int64_t *n_bad_tail);

/* Replaces dequantize_row_tq1_g128 (patches/prism-tq1-g128-distribution.patch:423-440), the host-side
 * "to_float" of the type: out[g * 128 + j] = (trit - 1) * scale_g as FP32, for `groups` consecutive
 * blocks in host memory (a row, or any whole number of rows). Bytes are decoded as they are (validate at
 * load). The device-side equivalent with row selection is tq1_embedding_f16. */
int tq1_dequantize_blocks(const uint8_t *blocks, float *out, int64_t groups);

/* The load-time scan of validate_packed_codes (src/ternel_mlx/packing.py:29-48)
 * and ggml_validate_row_data's TQ1 case (patches/prism-tq1-g128-distribution.patch:449-468),
 * over canonical blocks in host memory. */
int tq1_validate_blocks(const uint8_t *blocks, int64_t groups,
                        int64_t *n_bad_full, int64_t *n_bad_tail);

/* Canonical [rows][groups][28] <-> the reference's code-position-major tiles
 * codes u8[tiles][groups][26][tile], scales u16[tiles][groups][tile]
 * (reorder_tensor_arrays / restore_tensor_arrays, src/bonsai_tq1/lut23_reorder.py:126-165;
 * pack_blocks / unpack_blocks, src/ternel_mlx/packing.py:51-82). Host memory.
 * rows % tile must be 0 (the MLX layout never pads: src/ternel_mlx/layout.py:76-80). */
int tq1_tile_blocks(const uint8_t *blocks, uint8_t *codes, uint16_t *scales,
                    int64_t rows, int64_t groups_per_row, int64_t tile);
int tq1_untile_blocks(const uint8_t *codes, const uint16_t *scales, uint8_t *blocks,
                      int64_t rows, int64_t groups_per_row, int64_t tile);

/* ---- device entry points ------------------------------------------------ */

/* Same scan as tq1_validate_blocks over blocks in device memory; counts_dev is
 * a device int64[2] {n_bad_full, n_bad_tail} that the call zeroes first. */
int tq1_validate_blocks_device(const uint8_t *blocks_dev, int64_t groups,
                               int64_t *counts_dev, void *stream);

/* Scratch the linear entry point needs for this shape (0 when none). The
 * caller owns the buffer, as the caller of launch_tq1_lut23_smem_streamk owns
 * its workspace (cuda/tq1_lut23_streamk.cu:320-367, lut23_workspace_bytes). */
size_t tq1_linear_workspace_bytes(int M, int N, int K);

/* y[m][n] = sum_g f32(scale[n][g]) * sum_{k in g} (c[n][k]-1) * f32(x[m][k]),
 * FP32 accumulation, one narrowing at the store.
 * Replaces tq1_matmul / tq1_gemm behind packed_matmul
 * (src/ternel_mlx/kernels.py:1215-1271,1287-1357; src/ternel_mlx/modules.py:425-457)
 * and launch_tq1_g128_gemv_v1 / launch_tq1_lut23_smem_streamk
 * (cuda/tq1_g128_gemv.cu:144-193, cuda/tq1_lut23_streamk.cu:320-367).
 *   blocks    device, canonical [N][K/128][28], 4-byte aligned
 *   x         device FP16 [M][K] row-major, 16-byte aligned
 *   y         device [M][N] row-major, FP16 (y_is_f32 == 0) or FP32
 *   workspace device, >= tq1_linear_workspace_bytes(M,N,K) bytes, 256-byte
 *             aligned (may be NULL when that is 0). It must be zero-filled
 *             once before its first use; every call leaves it ready for the
 *             next one, of any shape. Calls that may overlap on the GPU
 *             (different streams) need separate workspaces. Layout: control
 *             words (256 B; word 0 becomes non-zero if a bounded wait inside
 *             a kernel ran out, words 1..4 are counters of the M == 1 kernel),
 *             then 16 MiB of partial-sum slots for M == 1 (eight bytes per row
 *             and 512-wide K chunk: the value and a sequence tag in one 64-bit
 *             word, so nothing is ever cleared), then the scratch of the
 *             M >= 2 kernels. After a non-zero status, zero-fill the workspace
 *             again. Status 7 is not a failure: the results are good, but the
 *             32-bit sequence tags have passed 0xF0000000 executed projections
 *             and the workspace must be zero-filled before they wrap.
 * The kernel is chosen from M: 1 => streaming GEMV, 2..16 => small-batch
 * split-K GEMV, larger => tiled GEMM. Illegal code bytes must have been
 * rejected at load (tq1_validate_blocks*): the kernels carry no clamp. */
int tq1_linear_f16(const uint8_t *blocks, const void *x, void *y, int y_is_f32,
                   int M, int N, int K, void *workspace, size_t workspace_bytes, void *stream);

/* Gated feed-forward input in one call: blocks holds 2N rows, gate row i at row 2i and up row i at
 * row 2i + 1 (interleave the two packed matrices once at load: rows are independent byte ranges),
 * and y[m][i] = silu(gate_i . x_m) * (up_i . x_m) with the dot products and the activation in FP32
 * and one narrowing at the store. Replaces two tq1_matmul calls plus the elementwise nn.silu(gate) * up
 * of the converted model's MLP (the reference computes those as separate graph nodes). Needs
 * K % 512 == 0 and 16-byte aligned blocks and x; workspace as for tq1_linear_f16(M, 2N, K). */
int tq1_linear_swiglu_f16(const uint8_t *blocks, const void *x, void *y, int y_is_f32, int M, int N, int K,
                          void *workspace, size_t workspace_bytes, void *stream);

/* Which kernel and which tiling tq1_linear_f16 picks for a shape (host-side, launches nothing).
 * Stands in for the reference's recorded dispatch rules select_lut23 / select_gemm
 * (src/ternel_mlx/modules.py:331-422), which its tests replay against committed sweeps
 * (tests/test_mlx_modules.py:553-1084); here the sweep is ternel_b200/dispatch_sweep_b200.json.
 *   aligned     1 if blocks and x are 16-byte aligned (the fast kernels need it)
 *   kernel      TQ1_KERNEL_*;  token_tile / ctas / parts: tensor-core kernel only (activation rows
 *               per tile, CTAs launched, equal K parts per tile or 0 for the stream-K split) */
#define TQ1_KERNEL_ROWS 0
#define TQ1_KERNEL_STREAM_GEMV 1
#define TQ1_KERNEL_TENSOR_CORE 2
int tq1_linear_plan(int M, int N, int K, int aligned, int *kernel, int *token_tile, int *ctas, int *parts);

/* ---- row-sharded linear over several GPUs -------------------------------- */

/* One rank's view of an output-row shard. Output rows are independent, so rank r owns rows
 * [n_offset, n_offset + N_local) of a projection and the FP16 results are written straight
 * into every rank's gathered activation buffer (peer mappings over NVLink). Flags are per tile
 * of 16 rows: after a tile has been written to a rank, word (row / 16) of that rank's flag array
 * for the buffer is set to the publish epoch with a release store. A consumer waits until the
 * flags of the tiles it reads have reached its wait epoch. The reference has no multi-device
 * path (its CUDA branch states "currently supports one CUDA device",
 * patches/prism-tq1-g128-distribution.patch:373). */
typedef struct tq1_shard {
    int rank, world;            /* world <= 8 */
    int n_offset;               /* first gathered row of this shard, a multiple of 16 */
    int n_total;                /* rows of the gathered output */
    void *peer_y[8];            /* device pointers: rank p's gathered output, FP16 [M][n_total] */
    uint32_t *peer_flags[8];    /* device pointers: rank p's tile flags of that output, n_total / 16 words */
    const uint32_t *epoch_base; /* optional device word added to both epochs below (NULL: 0); lets a
                                   captured CUDA graph publish fresh epochs on every replay */
    uint32_t publish_epoch;     /* stored to a tile's flag on every rank once the tile is there */
    const uint32_t *wait_flags; /* local tile flags of the buffer x lives in (NULL: do not wait); flag t
                                   guards x[..][16t .. 16t+15] */
    uint32_t wait_epoch;        /* wait until the flags have reached this value */
    int wait_tiles;             /* number of words behind wait_flags; M == 1 waits only for the tiles a
                                   CTA reads, M >= 2 for all of them */
} tq1_shard;

size_t tq1_linear_sharded_workspace_bytes(int M, int N_local, int K);

/* *epoch_base += delta on the stream (one per decode step, before its first sharded call). */
int tq1_shard_advance_epoch(uint32_t *epoch_base, uint32_t delta, void *stream);

/* blocks: this rank's rows [N_local][K/128][28] (N_local a multiple of 16); x: the whole FP16
 * activations [M][K] in local memory. Waits are bounded: if a flag never arrives the status word
 * at the start of the workspace becomes 4 and the call completes with whatever was there.
 * Reuse of a gathered buffer: the flags order a reader after its writers, nothing orders a later
 * writer after an earlier reader. A gathered buffer (and its flags) may therefore be written again
 * only after every rank has finished the call that reads it, for instance by alternating two buffers
 * per output size, or by a buffer per projection as the chain's hand-off areas do. */
int tq1_linear_f16_sharded(const uint8_t *blocks, const void *x, const tq1_shard *shard,
                           int M, int N_local, int K, void *workspace, size_t workspace_bytes, void *stream);

/* Batch-1 linear for callers that cannot supply scratch memory. No counterpart in the
 * reference: it exists for hosts that must not allocate at call time -- code running inside a
 * stream-capture region (cudaMalloc is illegal there), plugin hosts whose device budget was
 * fixed when the model was loaded, real-time loops that stay away from the allocator.
 * Same arithmetic and result as tq1_linear_f16 with M == 1, but the scratch (control words
 * and per-chunk partial-sum slots) lives in a 2 MiB array built into the library,
 * which every GPU that loads the library holds until the process exits.
 *   - Limits: K % 512 == 0, blocks 16-byte aligned, and N*K/64 + 256 bytes of scratch must
 *     fit in 2 MiB (N*K up to about 1.3e8 weights, e.g. 5120 x 17408); larger shapes are
 *     rejected with TQ1_ERR_WORKSPACE and a message, nothing is launched.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) with that device current; make that first call outside any
 *     stream capture.
 *   - Every call on a device shares the one array, which keeps what the last call left: the
 *     partial sums carry sequence tags, so nothing has to start at zero except the array's
 *     initial state, but calls that may overlap on the GPU (different streams) race with
 *     each other; keep them on one stream or order them with events.
 *   - Calls no cudaMalloc, cudaFree or allocating library routine.
 *   - A bounded wait that ran out inside the kernel leaves a non-zero status word in the
 *     array (and a wrong y); it stays until the process exits. tq1_gemv_noalloc_status
 *     copies it to host memory on `stream` (4 bytes, no allocation). */
int tq1_gemv_f16_noalloc(const uint8_t *blocks, const void *x, void *y, int y_is_f32,
                         int N, int K, void *stream);
int tq1_gemv_noalloc_status(uint32_t *status_host, void *stream);

/* ---- streaming layout for batch-1 decoding ---------------------------------- */

/* Chunk-major panels: the same 28-byte blocks, permuted once at load so that the 16 rows x 4 groups a
 * warp consumes at a time are 1792 CONTIGUOUS bytes:
 *     panels[c][r][112]   c = K/512 column chunks, r = rows padded with zero blocks to a multiple of 16,
 *                         112 bytes = the four blocks of row r in columns [512c, 512c + 512)
 * On B200 a fetch of sixteen 112-byte row pieces 1120+ bytes apart (canonical layout) sustains 3.7 TB/s,
 * a contiguous 1792-byte copy 6.8 TB/s. The reference likewise permutes the canonical blocks into a
 * kernel-friendly device form at load (reorder_tensor_arrays, src/bonsai_tq1/lut23_reorder.py:126-165;
 * pack_blocks, src/ternel_mlx/packing.py:51-82); the permutation is lossless and
 * tq1_panels_to_blocks_device restores the canonical bytes exactly. Needs K % 512 == 0 and 16-byte
 * aligned pointers. Chain links accept either form (tq1_chain_link.layout). */
#define TQ1_LAYOUT_BLOCKS 0
#define TQ1_LAYOUT_PANELS 1
size_t tq1_panel_bytes(int N, int K);
int tq1_blocks_to_panels_device(const uint8_t *blocks, uint8_t *panels, int N, int K, void *stream);
int tq1_panels_to_blocks_device(const uint8_t *panels, uint8_t *blocks, int N, int K, void *stream);

/* ---- a chain of batch-1 products in one launch ----------------------------- */

/* A decoded token runs one matrix-vector product per packed linear, back to back: the
 * reference's converted model calls packed_matmul for q/k/v, o, gate/up and down of every
 * layer (src/ternel_mlx/modules.py:425-457,460-495), one kernel launch each. A chain runs a
 * list of such products ("links") inside one persistent kernel: the next link's weights are
 * already streaming while the current one finishes, and a link that reads an earlier link's
 * output waits, element by element, for exactly the activations it needs. The arithmetic of
 * every link is that of tq1_linear_f16 with M == 1 (bit-identical results).
 *
 * Link i computes  out = f(W_i x_i) * out_scale  with f the identity or, with swiglu != 0,
 * silu(gate) * up over (gate, up) row pairs as in tq1_linear_swiglu_f16; `out` has N (or N/2)
 * elements, is rounded to FP16 for any later link that reads it, and is stored to y (FP16 or
 * FP32) when y is not NULL. */
typedef struct tq1_chain_link {
    const uint8_t *blocks; /* device, canonical [N][K/128][28] (or panels, see layout), 16-byte aligned; this rank's rows */
    int N, K;              /* K % 512 == 0, K <= 65536 */
    const void *x;         /* device FP16 [K], complete before the launch; NULL: read link `source` */
    int source;            /* with x == NULL: index of an EARLIER link whose output is this link's input */
    int source_offset;     /* first element of that output to read (e.g. the q part of a fused q|k|v) */
    void *y;               /* device output of this rank's rows, or NULL */
    int y_is_f32;
    int swiglu;            /* rows are (gate, up) pairs: N/2 outputs */
    float out_scale;       /* multiplies every output; 0 is taken as 1 */
    int layout;            /* TQ1_LAYOUT_BLOCKS: `blocks` is canonical; TQ1_LAYOUT_PANELS: it is the panel form below */
    int partial;           /* sharded chains only, see below: this rank holds a COLUMN range of the matrix, all N rows */
} tq1_chain_link;

/* Row-sharded chains: every rank runs the same list over its own rows of every matrix (rank r owns
 * output elements [r * n_out, (r + 1) * n_out) of each link) and each finished output is written,
 * as a 64-bit word {FP16 bits, sequence tag}, straight into the hand-off area of EVERY rank (plain
 * peer stores over NVLink, no multicast); readers poll their own memory. handoff[r] is rank r's
 * area (tq1_chain_handoff_bytes, zero-filled once, 256-byte aligned, mapped into this process).
 * Every rank must issue the same sequence of chain calls on its area, and start a call within the
 * bounded wait of its peers (2^21 polls, some tenths of a second): a link that waits longer for another
 * rank's words gives up with status 4. The reference has no multi-device path
 * (patches/prism-tq1-g128-distribution.patch:373).
 *
 * A link may instead be sharded by COLUMNS (partial != 0): rank r holds columns [r * K, (r + 1) * K) of
 * all N rows (`blocks`: that column range, canonical [N][K/128][28] or K/512 consecutive panels of the
 * full matrix) and reads the matching K activations, for instance exactly the output rows this rank
 * produced for a row-sharded link before it (source_offset = rank * n_out), so that hand-over needs no
 * other GPU. Its output is the rank's partial sum (y, if given, receives the partial, after out_scale);
 * the ranks' partial sums travel as FP32 words, and a link that reads a partial link receives their sum,
 * added in rank order and rounded once to FP16 (source_offset then indexes the N summed outputs). Two
 * row-sharded and two column-sharded projections per decoder layer halve the number of hand-overs that
 * cross NVLink. swiglu and partial exclude each other. */
typedef struct tq1_chain_peers {
    int rank, world;       /* world <= 8 */
    void *handoff[8];
} tq1_chain_peers;

/* Bytes of workspace a chain needs: control words, two alternating 8 MiB slot regions and, on a
 * single GPU (world <= 1), the hand-off words of the links behind them. Zero-fill once. A chain
 * workspace may also serve tq1_linear_f16 calls with M == 1, but not M >= 2 calls (their scratch
 * would overwrite hand-off words). */
size_t tq1_chain_workspace_bytes(const tq1_chain_link *links, int n_links, int world);
size_t tq1_chain_handoff_bytes(const tq1_chain_link *links, int n_links, int world);

/* Up to 8 links, described on the spot (single GPU). */
int tq1_linear_chain_f16(const tq1_chain_link *links, int n_links, void *workspace, size_t workspace_bytes,
                         void *stream);

/* Longer chains (a whole decode step) are described once: the link table lives in caller-owned
 * device memory (tq1_chain_table_bytes, 128-byte aligned; uploaded on `stream`), the returned
 * handle is a small host object. tq1_chain_plan_run enqueues one launch; the plan keeps the
 * pointers it was created with (weights, x, y, workspace, hand-off areas). */
typedef struct tq1_chain_plan tq1_chain_plan;
size_t tq1_chain_table_bytes(const tq1_chain_link *links, int n_links);
int tq1_chain_plan_create(const tq1_chain_link *links, int n_links, const tq1_chain_peers *peers,
                          void *workspace, size_t workspace_bytes, void *table, size_t table_bytes,
                          void *stream, tq1_chain_plan **out);
int tq1_chain_plan_run(const tq1_chain_plan *plan, void *stream);
void tq1_chain_plan_destroy(tq1_chain_plan *plan);

/* out[t][k] = (c[id_t][k]-1) * scale[id_t][k/128], exact; an id outside [0,V)
 * gives a zero row. Replaces tq1_get_rows (src/ternel_mlx/kernels.py:1360-1398,
 * 863-901) and k_get_rows_tq1_g128 (patches/prism-tq1-g128-distribution.patch:132-171).
 *   ids  device int64[T];  out device [T][K], FP16 or FP32 (out_is_f32) */
int tq1_embedding_f16(const uint8_t *blocks, const int64_t *ids, void *out, int out_is_f32,
                      int64_t T, int64_t V, int K, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* TERNEL_B200_H */
