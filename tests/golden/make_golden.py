"""Generate tests/golden/*.npz by running the UNMODIFIED reference in place.

Run in a container that has the reference checked out (it is not needed, and
not available, where the GPU tests run):

    python tests/golden/make_golden.py --reference /path/to/reference

The reference's NumPy modules import without Apple's ``mlx``; only
``ternel_mlx.reference`` pulls three integers from the Metal kernel module, so
``mlx`` is stubbed before that import. Every array written here is an output of
the reference's own functions on seeded inputs; nothing is computed by this
repository's code.
"""

from __future__ import annotations

import argparse
import hashlib
import sys
from pathlib import Path
from unittest.mock import MagicMock

import numpy as np

HERE = Path(__file__).resolve().parent


def _import_reference(root: Path):
    sys.path.insert(0, str(root / "src"))
    for name in ("mlx", "mlx.core", "mlx.nn", "mlx.utils"):
        sys.modules.setdefault(name, MagicMock())
    import bonsai_tq1.format as fmt
    import bonsai_tq1.reference as ref
    import bonsai_tq1.lut23_reorder as reorder
    import ternel_mlx.layout as layout
    import ternel_mlx.packing as packing
    import ternel_mlx.reference as mref
    return fmt, ref, reorder, layout, packing, mref


def _random_case(fmt, rows, columns, seed, *, dist):
    rng = np.random.default_rng(seed)
    groups = rows * columns // 128
    if dist == "bench":      # the benchmark's distribution: P(0)=0.40, scales |N|*0.02
        trits = rng.choice(3, size=(groups, 128), p=[0.30, 0.40, 0.30]).astype(np.uint8)
        scales = (np.abs(rng.standard_normal(groups)) * 0.02).astype(np.float16)
    else:                    # the reference tests' distribution: uniform trits, N(0, 0.05)
        trits = rng.integers(0, 3, size=(groups, 128), dtype=np.uint8)
        scales = rng.normal(0.0, 0.05, size=groups).astype(np.float16)
    blocks = fmt.encode_tq1_blocks(scales.view(np.uint8).reshape(-1, 2), trits)
    return trits, scales, blocks.reshape(rows, columns // 128, 28), rng


def _write_sidecars(fmt, reorder) -> None:
    """A two-tensor ``.tq1g128`` file assembled with the reference's header and manifest code the way
    its packer does, and the LUT23 container its ``reorder_sidecar`` makes from it."""
    import json

    tensors = []
    for name, rows, columns, seed in (("blk.0.ffn_down.weight", 300, 256, 21), ("blk.0.ssm_a.weight", 48, 128, 22)):
        _, _, blocks, _ = _random_case(fmt, rows, columns, seed, dist="tests")
        tensors.append((name, rows, columns, blocks))
    path = HERE / "sidecar_small.tq1g128"
    entries = []
    with path.open("wb") as handle:
        handle.write(bytes(fmt.HEADER_BYTES))
        for index, (name, rows, columns, blocks) in enumerate(tensors):
            offset = fmt.align_up(handle.tell(), fmt.ALIGNMENT)
            fmt.write_padding(handle, offset)
            data = blocks.tobytes()
            handle.write(data)
            entries.append({
                "index": index, "name": name, "shape_gguf": [columns, rows], "elements": rows * columns,
                "groups": rows * columns // 128, "source_type": "Q2_0", "source_offset": 0, "source_bytes": 0,
                "packed_offset": offset, "packed_bytes": len(data),
                "logical_weight_sha256": "11" * 32, "scale_bits_sha256": "22" * 32,
                "packed_payload_sha256": hashlib.sha256(data).hexdigest(),
            })
        manifest_offset = handle.tell()
        manifest = {"format": "TQ1_G128", "version": fmt.VERSION, "block_size": 128, "block_bytes": 28,
                    "alignment": fmt.ALIGNMENT, "mapping": {"-1": 0, "0": 1, "+1": 2},
                    "packed_payload_bytes": sum(e["packed_bytes"] for e in entries), "tensors": entries}
        raw = fmt.canonical_json_bytes(manifest)
        handle.write(raw)
        header = fmt.SidecarHeader(version=fmt.VERSION, header_bytes=fmt.HEADER_BYTES, block_size=128, block_bytes=28,
                                   alignment=fmt.ALIGNMENT, tensor_count=len(entries), source_file_bytes=4242,
                                   manifest_offset=manifest_offset, manifest_bytes=len(raw), source_sha256="ab" * 32)
        handle.seek(0)
        handle.write(header.pack())
    fmt.read_sidecar(path)                                   # the reference's own reader accepts it
    import os
    cwd = os.getcwd()
    os.chdir(HERE)              # the LUT23 manifest records the source path as given: keep it relative
    try:
        reorder.reorder_sidecar(Path(path.name), Path("sidecar_small.lut23"))
    finally:
        os.chdir(cwd)
    np.savez_compressed(HERE / "sidecar_small_blocks.npz", **{name: blocks for name, _, _, blocks in tensors})
    print("wrote sidecar_small.tq1g128, sidecar_small.lut23, sidecar_small_blocks.npz")


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", type=Path, required=True)
    parser.add_argument("--sidecars-only", action="store_true", help="write only the two sidecar fixtures")
    args = parser.parse_args()
    fmt, ref, reorder, layout, packing, mref = _import_reference(args.reference)
    _write_sidecars(fmt, reorder)
    if args.sidecars_only:
        return

    # 1. codec: every legal byte value in slot 0 and the tail, odd scale bit patterns.
    codes = np.ones((243, 128), dtype=np.uint8)
    for value in range(243):
        v = value
        for t in range(5):
            codes[value, t] = v % 3
            v //= 3
        codes[value, 125:] = [(value % 27) % 3, (value % 27) // 3 % 3, (value % 27) // 9]
    scale_words = (np.arange(243, dtype=np.uint32) * 269 + 7).astype(np.uint16)
    packed = fmt.encode_tq1_blocks(scale_words.view(np.uint8).reshape(-1, 2), codes)
    np.savez_compressed(HERE / "codec_bytes.npz", trits=codes, scale_words=scale_words, blocks=packed)

    # 2. small matmul cases through all four references + the tiled layout.
    cases = {}
    for name, rows, columns, batch, seed, dist in (
        ("r48_k640_m3", 48, 640, 3, 11, "tests"),
        ("r300_k256_m2", 300, 256, 2, 12, "tests"),
        ("r512_k384_m4", 512, 384, 4, 13, "bench"),
        ("r256_k1280_m1", 256, 1280, 1, 14, "bench"),
    ):
        trits, scales, blocks, rng = _random_case(fmt, rows, columns, seed, dist=dist)
        x = rng.standard_normal((batch, columns)).astype(np.float16)
        lay = layout.PackedTensorLayout.for_tensor(rows, columns)
        tcodes, tscales = packing.pack_blocks(blocks, layout=lay)
        xf = x.astype(np.float32)
        ids = rng.integers(0, rows, size=7).astype(np.uint32)
        cases[name] = dict(
            rows=rows, columns=columns, tile=lay.tile, blocks=blocks, x=x,
            tiled_codes=tcodes, tiled_scales=tscales,
            y_gemv=np.stack([ref.tq1_g128_reference_gemv(blocks, xf[m], rows=rows, columns=columns)
                             for m in range(batch)]),
            y_lut23=mref.lut23_matmul(tcodes, tscales, xf, layout=lay),
            y_f64=mref.oracle_matmul(tcodes, tscales, xf, layout=lay),
            y_restored=mref.restored_matmul(tcodes, tscales, xf, layout=lay),
            ids=ids,
            rows_f16=mref.get_rows_reference(tcodes, tscales, ids, layout=lay, dtype=np.dtype(np.float16)),
            rows_f32=mref.get_rows_reference(tcodes, tscales, ids, layout=lay, dtype=np.dtype(np.float32)),
        )
    flat = {f"{case}/{key}": np.asarray(value) for case, d in cases.items() for key, value in d.items()}
    np.savez_compressed(HERE / "matmul_cases.npz", **flat)

    # 3. the 4096x4096 single-matrix configuration, seed 0: keep y and hashes only.
    rows = columns = 4096
    trits, scales, blocks, rng = _random_case(fmt, rows, columns, 0, dist="bench")
    x = rng.standard_normal(columns).astype(np.float16)
    y = ref.tq1_g128_reference_gemv(blocks, x.astype(np.float32), rows=rows, columns=columns)
    np.savez_compressed(
        HERE / "single_matrix_4096.npz",
        y=y, x=x,
        blocks_sha256=np.frombuffer(hashlib.sha256(blocks.tobytes()).digest(), dtype=np.uint8),
        first_blocks=blocks[:2].copy(),
    )
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    main()
