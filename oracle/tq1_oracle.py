"""CPU oracle for the packed ternary (TQ1_G128) linear and embedding path.

TEST INFRASTRUCTURE ONLY. Nothing in the shipped package imports this module;
it exists so the CUDA kernels can be checked against an independent NumPy
restatement of the reference algorithm. Only the test-suite, the smoke check
and the CPU-baseline leg of the benchmark may import it.

Parity status: PINNED. Every function below is checked (tests/test_oracle_golden.py)
against fixtures produced by importing the unmodified reference in place
(tests/golden/make_golden.py) and against the reference's own constructive
known-answer designs (tests/test_format.py:46-113,146-158 of the reference).

Block layout (src/bonsai_tq1/format.py:14-28,66-122 of the reference):
    byte 0..1   raw little-endian FP16 scale bits
    byte 2+j    sum_{i<5} c[5j+i] * 3**i     j = 0..24   (value <= 242)
    byte 27     c[125] + 3 c[126] + 9 c[127]              (value <= 26)
with c in {0,1,2} and the logical weight (c - 1) * scale.
"""

from __future__ import annotations

import numpy as np

GROUP = 128            # weights per block
BLOCK_BYTES = 28       # bytes per block
CODE_BYTES = 26        # code bytes per block (25 full + 1 tail)
FULL_BYTES = 25
MAX_FULL = 242         # 3**5 - 1
MAX_TAIL = 26          # 3**3 - 1
PREFERRED_TILE = 256   # src/ternel_mlx/layout.py:41-51

_POW5 = np.array([1, 3, 9, 27, 81], dtype=np.uint16)
_POW3 = np.array([1, 3, 9], dtype=np.uint16)


class FormatError(ValueError):
    """Same role as bonsai_tq1.format.FormatError (format.py:33)."""


# --------------------------------------------------------------------------
# codec — format.py:66-122
# --------------------------------------------------------------------------

def encode_blocks(scales, codes) -> np.ndarray:
    """(G,2) raw scale bytes + (G,128) trits in {0,1,2} -> (G,28) blocks.

    Follows encode_tq1_blocks (format.py:66-91): rejects any code > 2 with the
    count in the message.
    """
    s = np.asarray(scales, dtype=np.uint8)
    c = np.asarray(codes, dtype=np.uint8)
    if s.ndim == 1:
        s = s.reshape(-1, 2)
    if c.ndim == 1:
        c = c.reshape(-1, GROUP)
    if s.ndim != 2 or s.shape[1] != 2:
        raise FormatError(f"expected scale bytes shaped (N, 2), got {s.shape}")
    if c.ndim != 2 or c.shape[1] != GROUP:
        raise FormatError(f"expected codes shaped (N, 128), got {c.shape}")
    if s.shape[0] != c.shape[0]:
        raise FormatError("scale and code block counts differ")
    bad = int(np.count_nonzero(c > 2))
    if bad:
        raise FormatError(f"source contains {bad} non-ternary code(s)")
    g = c.shape[0]
    out = np.empty((g, BLOCK_BYTES), dtype=np.uint8)
    out[:, 0:2] = s
    full = c[:, :125].reshape(g, FULL_BYTES, 5).astype(np.uint16)
    out[:, 2:27] = (full * _POW5).sum(axis=2).astype(np.uint8)
    out[:, 27] = (c[:, 125:].astype(np.uint16) * _POW3).sum(axis=1).astype(np.uint8)
    return out


def decode_blocks(blocks, *, validate: bool = True):
    """(G,28) blocks -> ((G,2) scale bytes, (G,128) trits).

    Follows decode_tq1_blocks (format.py:94-122): with validate, counts bytes
    above 242 in the 25 full slots and above 26 in the tail slot and raises
    ``invalid base-3 bytes: regular=<n>, tail=<m>``.
    """
    b = np.asarray(blocks, dtype=np.uint8)
    if b.ndim == 1:
        if b.size % BLOCK_BYTES:
            raise FormatError("TQ1 byte length is not divisible by 28")
        b = b.reshape(-1, BLOCK_BYTES)
    if b.ndim != 2 or b.shape[1] != BLOCK_BYTES:
        raise FormatError(f"expected TQ1 blocks shaped (N, 28), got {b.shape}")
    if validate:
        n_full = int(np.count_nonzero(b[:, 2:27] > MAX_FULL))
        n_tail = int(np.count_nonzero(b[:, 27] > MAX_TAIL))
        if n_full or n_tail:
            raise FormatError(f"invalid base-3 bytes: regular={n_full}, tail={n_tail}")
    g = b.shape[0]
    trits = np.empty((g, GROUP), dtype=np.uint8)
    full = b[:, 2:27].astype(np.uint16)
    digits = np.stack([(full // p) % 3 for p in (1, 3, 9, 27, 81)], axis=2)
    trits[:, :125] = digits.reshape(g, 125)
    tail = b[:, 27].astype(np.uint16)
    for i, p in enumerate((1, 3, 9)):
        trits[:, 125 + i] = (tail // p) % 3
    return b[:, 0:2].copy(), trits


def scale_values(scale_bytes, dtype=np.float32) -> np.ndarray:
    """Raw (G,2) FP16 bytes -> float values (reference.py:9-11)."""
    return np.ascontiguousarray(scale_bytes, dtype=np.uint8).view("<f2").reshape(-1).astype(dtype)


# --------------------------------------------------------------------------
# decode-then-dot GEMV — src/bonsai_tq1/reference.py:14-39,55-65 (THE oracle)
# --------------------------------------------------------------------------

def reference_gemv(blocks, x, *, rows: int, columns: int, row_chunk: int = 256) -> np.ndarray:
    """y[n] = sum_g f32(scale[n,g]) * sum_{k in g} (c-1) * x[k], all float32.

    Same arithmetic, and the same NumPy reductions along the same contiguous
    axes, as ``_reference_gemv`` (reference.py:14-39); rows are processed in
    chunks instead of one per Python iteration. The golden test asserts the
    result is bit-identical to the reference's.
    """
    if columns % GROUP:
        raise ValueError("columns must be divisible by 128")
    gpr = columns // GROUP
    raw = np.asarray(blocks, dtype=np.uint8)
    if raw.size != rows * gpr * BLOCK_BYTES:
        raise ValueError("packed matrix byte count does not match shape")
    xv = np.asarray(x, dtype=np.float32)
    if xv.shape != (columns,):
        raise ValueError(f"expected activation shape {(columns,)}, got {xv.shape}")
    mat = raw.reshape(rows, gpr, BLOCK_BYTES)
    xg = xv.reshape(gpr, GROUP)
    y = np.zeros(rows, dtype=np.float32)
    for r0 in range(0, rows, row_chunk):
        part = mat[r0:r0 + row_chunk]
        n = part.shape[0]
        sb, trits = decode_blocks(part.reshape(-1, BLOCK_BYTES))
        w = (trits.astype(np.int8) - 1).astype(np.float32).reshape(n, gpr, GROUP)
        dots = np.empty((n, gpr), dtype=np.float32)
        for i in range(n):  # per-row product keeps the reduction identical to the reference's
            dots[i] = np.sum(w[i] * xg, axis=1, dtype=np.float32)
        sc = scale_values(sb).reshape(n, gpr)
        for i in range(n):
            y[r0 + i] = np.sum(dots[i] * sc[i], dtype=np.float32)
    return y


def reference_matmul(blocks, x, *, rows: int, columns: int) -> np.ndarray:
    """Batched form: one reference_gemv per activation row (reference.py:180-193 of ternel_mlx)."""
    xa = np.asarray(x, dtype=np.float32)
    if xa.ndim != 2 or xa.shape[1] != columns:
        raise FormatError(f"activations must be (batch, {columns}), got shape {xa.shape}")
    return np.stack([reference_gemv(blocks, row, rows=rows, columns=columns) for row in xa])


def dense_weights(blocks, *, rows: int, columns: int, dtype=np.float64) -> np.ndarray:
    """(rows, columns) dense (c-1)*scale (ternel_mlx/reference.py:155-167)."""
    gpr = columns // GROUP
    sb, trits = decode_blocks(np.asarray(blocks, dtype=np.uint8).reshape(-1, BLOCK_BYTES))
    w = trits.astype(np.int8).astype(dtype) - dtype(1)
    s = scale_values(sb, dtype).reshape(-1, 1)
    return (w * s).reshape(rows, gpr * GROUP)


def float64_matmul(blocks, x, *, rows: int, columns: int) -> np.ndarray:
    """Dense float64 product, the exactness reference (ternel_mlx/reference.py:171-177)."""
    xa = np.asarray(x)
    if xa.ndim != 2 or xa.shape[1] != columns:
        raise FormatError(f"activations must be (batch, {columns}), got shape {xa.shape}")
    return xa.astype(np.float64) @ dense_weights(blocks, rows=rows, columns=columns).T


# --------------------------------------------------------------------------
# tiled (code-position-major) layout — lut23_reorder.py:126-165, packing.py:51-82
# --------------------------------------------------------------------------

def select_tile(rows: int) -> int:
    """256 when it divides ``rows`` else ``rows`` (layout.py:41-51)."""
    if rows <= 0:
        raise FormatError(f"row count must be positive, got {rows}")
    return PREFERRED_TILE if rows % PREFERRED_TILE == 0 else rows


def tile_blocks(blocks, *, tile: int):
    """(rows, groups, 28) -> codes u8[tiles, groups, 26, tile], scales u16[tiles, groups, tile].

    Zero-pads a ragged last tile as reorder_tensor_arrays does
    (lut23_reorder.py:126-142); scales are the raw FP16 bits viewed as
    little-endian uint16 (packing.py:62-64).
    """
    src = np.asarray(blocks, dtype=np.uint8)
    if src.ndim != 3 or src.shape[2] != BLOCK_BYTES:
        raise ValueError("blocks must have shape (rows, groups, 28)")
    if tile <= 0:
        raise ValueError("tile must be positive")
    rows, groups, _ = src.shape
    tiles = -(-rows // tile)
    padded = np.zeros((tiles * tile, groups, BLOCK_BYTES), dtype=np.uint8)
    padded[:rows] = src
    per_tile = padded.reshape(tiles, tile, groups, BLOCK_BYTES)
    codes = np.ascontiguousarray(per_tile[..., 2:].transpose(0, 2, 3, 1))
    pairs = np.ascontiguousarray(per_tile[..., :2].transpose(0, 2, 1, 3))
    scales = pairs.reshape(-1).view("<u2").reshape(tiles, groups, tile)
    return codes, scales


def untile_blocks(codes, scales, rows: int, *, tile: int) -> np.ndarray:
    """Inverse of tile_blocks (restore_tensor_arrays, lut23_reorder.py:145-165)."""
    c = np.asarray(codes, dtype=np.uint8)
    s = np.ascontiguousarray(np.asarray(scales, dtype="<u2"))
    if (c.ndim != 4 or c.shape[2:] != (CODE_BYTES, tile)
            or s.shape != (c.shape[0], c.shape[1], tile)
            or not 0 < rows <= c.shape[0] * tile):
        raise ValueError("invalid reordered tensor geometry")
    tiles, groups = c.shape[0], c.shape[1]
    out = np.empty((tiles * tile, groups, BLOCK_BYTES), dtype=np.uint8)
    view = out.reshape(tiles, tile, groups, BLOCK_BYTES)
    view[..., 2:] = c.transpose(0, 3, 1, 2)
    view[..., :2] = s.reshape(-1).view(np.uint8).reshape(tiles, groups, tile, 2).transpose(0, 2, 1, 3)
    return np.ascontiguousarray(out[:rows])


def validate_tiled_codes(codes) -> None:
    """Load-time scan of tiled codes (packing.py:29-48)."""
    a = np.asarray(codes)
    if a.dtype != np.uint8:
        raise FormatError(f"codes must be uint8, got {a.dtype}")
    if a.ndim != 4:
        raise FormatError(f"codes must be 4-D (tiles, groups, slots, tile), got {a.shape}")
    n_full = int(np.count_nonzero(a[:, :, :FULL_BYTES, :] > MAX_FULL))
    n_tail = int(np.count_nonzero(a[:, :, FULL_BYTES, :] > MAX_TAIL))
    if n_full or n_tail:
        raise FormatError(
            f"packed codes contain out-of-range base-3 bytes: regular={n_full} "
            f"(max {MAX_FULL}), tail={n_tail} (max {MAX_TAIL})")


# --------------------------------------------------------------------------
# LUT23 order reference — ternel_mlx/reference.py:56-152
# --------------------------------------------------------------------------

def _digits(entries: int, position: int) -> np.ndarray:
    return ((np.arange(entries, dtype=np.int64) // 3 ** position) % 3).astype(np.float32) - 1.0


def group_tables(xg: np.ndarray):
    """L2[25,9], L3[25,27], tail[27] for one group's 128 activations (reference.py:56-86)."""
    x = np.asarray(xg, dtype=np.float32)
    if x.shape != (GROUP,):
        raise FormatError(f"expected {GROUP} activations, got shape {x.shape}")
    slot = x[:125].reshape(FULL_BYTES, 5)
    l2 = (slot[:, 0:1] * _digits(9, 0) + slot[:, 1:2] * _digits(9, 1)).astype(np.float32)
    l3 = (slot[:, 2:3] * _digits(27, 0) + slot[:, 3:4] * _digits(27, 1)
          + slot[:, 4:5] * _digits(27, 2)).astype(np.float32)
    t = x[125:]
    tail = (t[0] * _digits(27, 0) + t[1] * _digits(27, 1) + t[2] * _digits(27, 2)).astype(np.float32)
    return l2, l3, tail


def _fma32(a, b, c):
    """Correctly rounded float32 a*b+c via float64 (reference.py:89-97)."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


def lut23_matmul(blocks, x, *, rows: int, columns: int) -> np.ndarray:
    """Table-driven product in the LUT23 kernels' summation order (reference.py:117-152).

    Takes canonical blocks; the tiling only permutes rows, so the per-row
    arithmetic is unchanged.
    """
    gpr = columns // GROUP
    mat = np.asarray(blocks, dtype=np.uint8).reshape(rows, gpr, BLOCK_BYTES)
    xa = np.asarray(x, dtype=np.float32)
    if xa.ndim != 2 or xa.shape[1] != columns:
        raise FormatError(f"activations must be (batch, {columns}), got shape {xa.shape}")
    full = mat[:, :, 2:27].astype(np.uint32)          # rows, groups, 25
    hi = (full * np.uint32(57)) >> np.uint32(9)
    lo = full - np.uint32(9) * hi
    tailc = mat[:, :, 27]
    sc = scale_values(mat[:, :, 0:2].reshape(-1, 2)).reshape(rows, gpr)
    out = np.zeros((xa.shape[0], rows), dtype=np.float32)
    for m in range(xa.shape[0]):
        acc = np.zeros(rows, dtype=np.float32)
        for g in range(gpr):
            l2, l3, tail = group_tables(xa[m, g * GROUP:(g + 1) * GROUP])
            total = np.zeros(rows, dtype=np.float32)
            for s in range(FULL_BYTES):
                total += l2[s][lo[:, g, s]] + l3[s][hi[:, g, s]]
            total += tail[tailc[:, g]]
            acc = _fma32(sc[:, g], total, acc)
        out[m] = acc
    return out


# --------------------------------------------------------------------------
# embedding rows — ternel_mlx/reference.py:196-230
# --------------------------------------------------------------------------

def get_rows(blocks, ids, *, rows: int, columns: int, dtype=np.float16) -> np.ndarray:
    """out[t] = (trits(id_t) - 1) * scale in ``dtype``; ids outside [0, rows) raise."""
    idx = np.asarray(ids)
    if idx.ndim != 1:
        raise FormatError(f"indices must be 1-D, got shape {idx.shape}")
    if idx.size and (idx.min() < 0 or idx.max() >= rows):
        raise FormatError(f"indices fall outside [0, {rows})")
    gpr = columns // GROUP
    mat = np.asarray(blocks, dtype=np.uint8).reshape(rows, gpr, BLOCK_BYTES)
    sel = mat[idx.astype(np.int64)]
    sb, trits = decode_blocks(sel.reshape(-1, BLOCK_BYTES))
    dt = np.dtype(dtype)
    w = trits.astype(np.int8).astype(dt) - dt.type(1)
    s = scale_values(sb, dt).reshape(-1, 1)
    return (w * s).reshape(idx.size, columns)


# --------------------------------------------------------------------------
# synthetic inputs with the benchmark's distributions
# --------------------------------------------------------------------------

def synth_matrix(rows: int, columns: int, seed: int = 0, *, p_zero: float = 0.40):
    """Random ternary matrix packed to blocks, plus an FP16 activation vector.

    Codes {0,1,2} with P = [(1-p0)/2, p0, (1-p0)/2] (weights -1/0/+1); one scale
    per group |N(0,1)|*0.02 stored as FP16 bits; x ~ N(0,1) as FP16.
    """
    rng = np.random.default_rng(seed)
    groups = rows * columns // GROUP
    p = [(1 - p_zero) / 2, p_zero, (1 - p_zero) / 2]
    trits = rng.choice(3, size=(groups, GROUP), p=p).astype(np.uint8)
    sc = (np.abs(rng.standard_normal(groups)) * 0.02).astype(np.float16)
    blocks = encode_blocks(sc.view(np.uint8).reshape(-1, 2), trits)
    x = rng.standard_normal(columns).astype(np.float16)
    return blocks.reshape(rows, columns // GROUP, BLOCK_BYTES), x


def normalised_error(got, want) -> float:
    """max |got-want| / max |want| per activation case, worst case returned
    (kernel_gate.py:290-372 of the reference: normalised within a case)."""
    a = np.atleast_2d(np.asarray(got, dtype=np.float64))
    b = np.atleast_2d(np.asarray(want, dtype=np.float64))
    finite = np.isfinite(a) & np.isfinite(b)
    err = np.abs(np.where(finite, a, 0.0) - np.where(finite, b, 0.0))
    mag = np.abs(np.where(finite, b, 0.0)).max(axis=1)
    mag = np.where(mag > 0, mag, 1.0)
    return float((err / mag[:, None]).max())


def nonfinite_classes(values) -> np.ndarray:
    """0 finite, 1 +inf, 2 -inf, 3 nan (kernel_gate.py:277-288)."""
    v = np.asarray(values, dtype=np.float64)
    c = np.zeros(v.shape, dtype=np.uint8)
    c[np.isposinf(v)] = 1
    c[np.isneginf(v)] = 2
    c[np.isnan(v)] = 3
    return c
