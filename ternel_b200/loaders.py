"""Readers for the reference's on-disk forms of packed weights, ending in canonical blocks.

Three containers hold TQ1_G128 tensors in the reference project:

* the ``.tq1g128`` sidecar: a 256-byte header, canonical ``[rows][groups][28]`` blocks per tensor at
  256-byte aligned offsets, and a JSON manifest at the end (src/bonsai_tq1/format.py:149-246,
  written by src/bonsai_tq1/pack_model.py:60-150);
* the LUT23 sidecar: the same tensors in the tiled code-position-major form
  ``codes u8[tiles][groups][26][256]`` / ``scales u8[tiles][groups][256][2]`` with rows padded to
  whole tiles (src/bonsai_tq1/lut23_reorder.py:42-123,126-165,323-334);
* a safetensors file that names ``<module>.codes`` (U8) and ``<module>.scales`` (U16) per packed
  module (src/ternel_mlx/convert.py:256-273; header layout as parsed by
  src/ternel_mlx/remote_safetensors.py:110-153).

Everything here is host-side load-time code: parse, bounds-check, verify the recorded hashes,
run the fail-closed byte scan, and hand back canonical blocks (NumPy) that ``PackedLinear.load_blocks``
copies to the device once. Writers exist for the first two containers so that round trips can be
tested and small artifacts produced without the reference.
"""

from __future__ import annotations

import hashlib
import json
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from .format import BLOCK_BYTES, BLOCK_SIZE, FormatError, validate_blocks
from .layout import CODE_SLOTS, PREFERRED_TILE, PackedTensorLayout, unpack_blocks, validate_packed_codes

ALIGNMENT = 256
HEADER_BYTES = 256
TQ1_MAGIC = b"TQ1G128\0"
TQ1_VERSION = 1
LUT23_MAGIC = b"TQ1L23\0\0"
LUT23_VERSION = 1
LUT23_FORMAT = "TQ1_LUT23_CODE_POSITION_MAJOR"
_TQ1_HEADER = struct.Struct("<8sIIIIIIQQQ32s")        # magic, version, header, block size, block bytes,
                                                      # alignment, tensors, source bytes, manifest offset/bytes, hash
_LUT23_HEADER = struct.Struct("<8sIIIIIIIQQQ32s")     # magic, version, header, tile, slots, block bytes, alignment, ...


def _align(value: int) -> int:
    return (value + ALIGNMENT - 1) & -ALIGNMENT


def _canonical_json(value) -> bytes:
    return json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode("utf-8")


def _digest_hex(text: str) -> bytes:
    if len(text) != 64:
        raise FormatError("source SHA-256 must contain 64 hexadecimal characters")
    try:
        return bytes.fromhex(text)
    except ValueError as exc:
        raise FormatError("source SHA-256 is not hexadecimal") from exc


# --------------------------------------------------------------------------------------------
# .tq1g128 sidecar
# --------------------------------------------------------------------------------------------

@dataclass(frozen=True)
class SidecarHeader:
    tensor_count: int
    source_file_bytes: int
    manifest_offset: int
    manifest_bytes: int
    source_sha256: str
    version: int = TQ1_VERSION

    def pack(self) -> bytes:
        fixed = _TQ1_HEADER.pack(TQ1_MAGIC, self.version, HEADER_BYTES, BLOCK_SIZE, BLOCK_BYTES, ALIGNMENT,
                                 self.tensor_count, self.source_file_bytes, self.manifest_offset,
                                 self.manifest_bytes, _digest_hex(self.source_sha256))
        return fixed + bytes(HEADER_BYTES - len(fixed))

    @classmethod
    def unpack(cls, data: bytes) -> "SidecarHeader":
        if len(data) < HEADER_BYTES:
            raise FormatError("truncated TQ1 header")
        (magic, version, header_bytes, block_size, block_bytes, alignment, tensors, source_bytes,
         manifest_offset, manifest_bytes, digest) = _TQ1_HEADER.unpack_from(data)
        if any(data[_TQ1_HEADER.size:HEADER_BYTES]):
            raise FormatError("nonzero reserved TQ1 header bytes")
        if magic != TQ1_MAGIC:
            raise FormatError("invalid TQ1 magic")
        if version != TQ1_VERSION:
            raise FormatError(f"unsupported TQ1 version {version}")
        if (header_bytes, block_size, block_bytes, alignment) != (HEADER_BYTES, BLOCK_SIZE, BLOCK_BYTES, ALIGNMENT):
            raise FormatError("unsupported TQ1 geometry")
        return cls(tensors, source_bytes, manifest_offset, manifest_bytes, digest.hex(), version)


def read_sidecar(path) -> tuple[SidecarHeader, dict]:
    """Header and manifest of a ``.tq1g128`` file after every structural check of the reference
    reader (src/bonsai_tq1/format.py:213-246): manifest inside the file, format tag, tensor count,
    each tensor 256-byte aligned, in order, sized ``groups * 28`` and clear of the manifest."""
    path = Path(path)
    size = path.stat().st_size
    with path.open("rb") as handle:
        header = SidecarHeader.unpack(handle.read(HEADER_BYTES))
        if header.manifest_offset < HEADER_BYTES or header.manifest_offset + header.manifest_bytes > size:
            raise FormatError("manifest points outside the sidecar")
        handle.seek(header.manifest_offset)
        try:
            manifest = json.loads(handle.read(header.manifest_bytes))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise FormatError("invalid sidecar manifest") from exc
    if not isinstance(manifest, dict) or manifest.get("format") != "TQ1_G128":
        raise FormatError("unexpected sidecar manifest format")
    tensors = manifest.get("tensors")
    if not isinstance(tensors, list) or len(tensors) != header.tensor_count:
        raise FormatError("sidecar tensor count does not match manifest")
    floor = HEADER_BYTES
    for entry in tensors:
        offset, nbytes, groups = int(entry["packed_offset"]), int(entry["packed_bytes"]), int(entry["groups"])
        if offset % ALIGNMENT or offset < _align(floor) or nbytes != groups * BLOCK_BYTES:
            raise FormatError(f"invalid tensor extent for {entry.get('name', '<unknown>')}")
        if offset + nbytes > header.manifest_offset:
            raise FormatError("tensor data overlaps the manifest")
        floor = offset + nbytes
    return header, manifest


def _entry(manifest: dict, name: str) -> dict:
    for entry in manifest["tensors"]:
        if entry.get("name") == name:
            return entry
    raise FormatError(f"no tensor named {name!r} in the manifest")


def _shape_of(entry: dict) -> tuple[int, int]:
    """(rows, columns); the manifest keeps the GGUF order, innermost dimension first."""
    if "shape_gguf" in entry:
        columns, rows = (int(v) for v in entry["shape_gguf"])
    else:
        rows, columns = int(entry["rows"]), int(entry["columns"])
    if columns % BLOCK_SIZE:
        raise FormatError(f"{entry.get('name')}: {columns} columns is not a multiple of the 128-weight group")
    return rows, columns


def load_sidecar_tensor(path, manifest: dict, name: str, *, verify: bool = True) -> np.ndarray:
    """Canonical blocks ``[rows][columns/128][28]`` of one tensor of a ``.tq1g128`` file.

    With ``verify`` the payload hash recorded by the packer is checked when present and the
    fail-closed byte scan is run (illegal code bytes raise ``FormatError`` with their counts)."""
    entry = _entry(manifest, name)
    rows, columns = _shape_of(entry)
    groups = int(entry["groups"])
    if rows * (columns // BLOCK_SIZE) != groups:
        raise FormatError(f"shape/group mismatch for {name}")
    raw = np.fromfile(path, dtype=np.uint8, count=groups * BLOCK_BYTES, offset=int(entry["packed_offset"]))
    if raw.size != groups * BLOCK_BYTES:
        raise FormatError(f"truncated payload for {name}")
    if verify:
        recorded = entry.get("packed_payload_sha256")
        if recorded is not None and hashlib.sha256(raw.tobytes()).hexdigest() != recorded:
            raise FormatError(f"payload hash mismatch for {name}")
        validate_blocks(raw.reshape(-1, BLOCK_BYTES))
    return raw.reshape(rows, columns // BLOCK_SIZE, BLOCK_BYTES)


def write_sidecar(path, tensors, *, source_sha256: str = "00" * 32, source_file_bytes: int = 0) -> dict:
    """Write ``[(name, blocks[rows][groups][28]), ...]`` as a ``.tq1g128`` file the reference reader accepts.

    Returns the manifest. Blocks are scanned first: an illegal code byte never reaches the disk."""
    path = Path(path)
    entries, cursor = [], HEADER_BYTES
    payloads = []
    for index, (name, blocks) in enumerate(tensors):
        array = np.ascontiguousarray(blocks, dtype=np.uint8)
        if array.ndim != 3 or array.shape[2] != BLOCK_BYTES:
            raise FormatError(f"{name}: blocks must have shape (rows, groups, 28), got {array.shape}")
        validate_blocks(array.reshape(-1, BLOCK_BYTES))
        rows, groups_per_row, _ = array.shape
        offset = _align(cursor)
        data = array.tobytes()
        entries.append({
            "index": index, "name": str(name), "shape_gguf": [groups_per_row * BLOCK_SIZE, rows],
            "elements": rows * groups_per_row * BLOCK_SIZE, "groups": rows * groups_per_row,
            "packed_offset": offset, "packed_bytes": len(data),
            "packed_payload_sha256": hashlib.sha256(data).hexdigest(),
        })
        payloads.append((offset, data))
        cursor = offset + len(data)
    manifest = {
        "format": "TQ1_G128", "version": TQ1_VERSION, "block_size": BLOCK_SIZE, "block_bytes": BLOCK_BYTES,
        "alignment": ALIGNMENT, "mapping": {"-1": 0, "0": 1, "+1": 2},
        "packed_payload_bytes": sum(len(d) for _, d in payloads), "tensors": entries,
    }
    manifest_raw = _canonical_json(manifest)
    header = SidecarHeader(len(entries), source_file_bytes, cursor, len(manifest_raw), source_sha256)
    with path.open("wb") as handle:
        handle.write(header.pack())
        for offset, data in payloads:
            handle.write(bytes(offset - handle.tell()))
            handle.write(data)
        handle.write(manifest_raw)
    return manifest


# --------------------------------------------------------------------------------------------
# LUT23 sidecar (tiled, rows padded to whole 256-row tiles)
# --------------------------------------------------------------------------------------------

@dataclass(frozen=True)
class Lut23Header:
    tensor_count: int
    source_file_bytes: int
    manifest_offset: int
    manifest_bytes: int
    source_sha256: str

    def pack(self) -> bytes:
        fixed = _LUT23_HEADER.pack(LUT23_MAGIC, LUT23_VERSION, HEADER_BYTES, PREFERRED_TILE, CODE_SLOTS, BLOCK_BYTES,
                                   ALIGNMENT, self.tensor_count, self.source_file_bytes, self.manifest_offset,
                                   self.manifest_bytes, _digest_hex(self.source_sha256))
        return fixed + bytes(HEADER_BYTES - len(fixed))

    @classmethod
    def unpack(cls, data: bytes) -> "Lut23Header":
        if len(data) != HEADER_BYTES:
            raise FormatError("truncated LUT23 header")
        fields = _LUT23_HEADER.unpack_from(data)
        if fields[0] != LUT23_MAGIC:
            raise FormatError("invalid LUT23 magic")
        if fields[1:7] != (LUT23_VERSION, HEADER_BYTES, PREFERRED_TILE, CODE_SLOTS, BLOCK_BYTES, ALIGNMENT):
            raise FormatError("unsupported LUT23 geometry")
        if any(data[_LUT23_HEADER.size:]):
            raise FormatError("nonzero LUT23 reserved header bytes")
        return cls(fields[7], fields[8], fields[9], fields[10], fields[11].hex())


def read_lut23_sidecar(path) -> tuple[Lut23Header, dict]:
    path = Path(path)
    with path.open("rb") as handle:
        header = Lut23Header.unpack(handle.read(HEADER_BYTES))
        if header.manifest_offset + header.manifest_bytes > path.stat().st_size:
            raise FormatError("manifest outside LUT23 sidecar")
        handle.seek(header.manifest_offset)
        try:
            manifest = json.loads(handle.read(header.manifest_bytes))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise FormatError("invalid LUT23 manifest") from exc
    if not isinstance(manifest, dict) or manifest.get("format") != LUT23_FORMAT:
        raise FormatError("unexpected LUT23 manifest format")
    if len(manifest.get("tensors", [])) != header.tensor_count:
        raise FormatError("LUT23 tensor count mismatch")
    return header, manifest


def _lut23_extent(rows: int, groups_per_row: int, start: int) -> dict:
    tiles = (rows + PREFERRED_TILE - 1) // PREFERRED_TILE
    padded = tiles * PREFERRED_TILE
    codes_offset = _align(start)
    codes_bytes = padded * groups_per_row * CODE_SLOTS
    scales_offset = _align(codes_offset + codes_bytes)
    scales_bytes = padded * groups_per_row * 2
    return {"tiles": tiles, "padded_rows": padded, "codes_offset": codes_offset, "codes_bytes": codes_bytes,
            "scales_offset": scales_offset, "scales_bytes": scales_bytes, "end": scales_offset + scales_bytes}


def load_lut23_tensor(path, manifest: dict, name: str, *, verify: bool = True) -> np.ndarray:
    """Canonical blocks of one tensor of a LUT23 sidecar: the tiled arrays are read, scanned
    (every byte, padding included) and turned back into row-major blocks; padded rows are dropped."""
    entry = _entry(manifest, name)
    rows, groups = int(entry["rows"]), int(entry["groups_per_row"])
    tiles = int(entry["tiles"])
    if tiles * PREFERRED_TILE != int(entry["padded_rows"]) or not 0 < rows <= tiles * PREFERRED_TILE:
        raise FormatError(f"invalid reordered tensor geometry for {name}")
    if int(entry["codes_bytes"]) != tiles * PREFERRED_TILE * groups * CODE_SLOTS or \
            int(entry["scales_bytes"]) != tiles * PREFERRED_TILE * groups * 2:
        raise FormatError(f"invalid tensor extent for {name}")
    codes = np.fromfile(path, dtype=np.uint8, count=int(entry["codes_bytes"]), offset=int(entry["codes_offset"]))
    scales = np.fromfile(path, dtype="<u2", count=int(entry["scales_bytes"]) // 2, offset=int(entry["scales_offset"]))
    if codes.size != int(entry["codes_bytes"]) or scales.size * 2 != int(entry["scales_bytes"]):
        raise FormatError(f"truncated payload for {name}")
    codes = codes.reshape(tiles, groups, CODE_SLOTS, PREFERRED_TILE)
    scales = scales.reshape(tiles, groups, PREFERRED_TILE)
    if verify:
        validate_packed_codes(codes)
    padded = PackedTensorLayout(tiles * PREFERRED_TILE, groups * BLOCK_SIZE, PREFERRED_TILE)
    return np.ascontiguousarray(unpack_blocks(codes, scales, layout=padded)[:rows])


def write_lut23_sidecar(path, tensors, *, source_sha256: str = "00" * 32, source_file_bytes: int = 0) -> dict:
    """Write ``[(name, blocks[rows][groups][28]), ...]`` in the LUT23 container (zero-padded tiles)."""
    from .layout import pack_blocks

    path = Path(path)
    entries, cursor, payloads = [], HEADER_BYTES, []
    for index, (name, blocks) in enumerate(tensors):
        array = np.ascontiguousarray(blocks, dtype=np.uint8)
        validate_blocks(array.reshape(-1, BLOCK_BYTES))
        rows, groups_per_row, _ = array.shape
        extent = _lut23_extent(rows, groups_per_row, cursor)
        padded = np.zeros((extent["padded_rows"], groups_per_row, BLOCK_BYTES), dtype=np.uint8)
        padded[:rows] = array
        codes, scales = pack_blocks(padded, layout=PackedTensorLayout(extent["padded_rows"],
                                                                       groups_per_row * BLOCK_SIZE, PREFERRED_TILE))
        extent.update({"index": index, "name": str(name), "rows": rows, "columns": groups_per_row * BLOCK_SIZE,
                       "groups_per_row": groups_per_row})
        entries.append(extent)
        payloads.append((extent["codes_offset"], codes.tobytes()))
        payloads.append((extent["scales_offset"], scales.astype("<u2").tobytes()))
        cursor = extent["end"]
    manifest_offset = _align(cursor)
    manifest = {"format": LUT23_FORMAT, "version": LUT23_VERSION, "m_tile": PREFERRED_TILE, "code_slots": CODE_SLOTS,
                "block_size": BLOCK_SIZE, "block_bytes": BLOCK_BYTES, "alignment": ALIGNMENT,
                "packed_payload_bytes": sum(e["codes_bytes"] + e["scales_bytes"] for e in entries),
                "tensors": entries}
    manifest_raw = _canonical_json(manifest)
    header = Lut23Header(len(entries), source_file_bytes, manifest_offset, len(manifest_raw), source_sha256)
    with path.open("wb") as handle:
        handle.write(header.pack())
        for offset, data in payloads:
            handle.write(bytes(offset - handle.tell()))
            handle.write(data)
        handle.write(bytes(manifest_offset - handle.tell()))
        handle.write(manifest_raw)
    return manifest


# --------------------------------------------------------------------------------------------
# safetensors with <module>.codes / <module>.scales
# --------------------------------------------------------------------------------------------

_SAFETENSORS_DTYPES = {"U8": np.dtype("u1"), "U16": np.dtype("<u2"), "I16": np.dtype("<i2"),
                       "F16": np.dtype("<f2"), "F32": np.dtype("<f4"), "I32": np.dtype("<i4"), "I64": np.dtype("<i8")}
_MAX_SAFETENSORS_HEADER = 100 * 1024 * 1024


class SafetensorsFile:
    """The header of a safetensors file and range reads of its tensors (no dependency on a
    safetensors package: an 8-byte little-endian length, a JSON object, then raw data)."""

    def __init__(self, path) -> None:
        self.path = Path(path)
        size = self.path.stat().st_size
        with self.path.open("rb") as handle:
            prefix = handle.read(8)
            if len(prefix) != 8:
                raise FormatError(f"{self.path} is too short for a safetensors header")
            (length,) = struct.unpack("<Q", prefix)
            if length <= 0 or length > _MAX_SAFETENSORS_HEADER or 8 + length > size:
                raise FormatError(f"implausible safetensors header length {length} in {self.path}")
            try:
                header = json.loads(handle.read(length))
            except (UnicodeDecodeError, json.JSONDecodeError) as exc:
                raise FormatError(f"safetensors header of {self.path} is not valid JSON") from exc
        if not isinstance(header, dict):
            raise FormatError(f"safetensors header of {self.path} is not a JSON object")
        self.data_start = 8 + length
        self.metadata = header.pop("__metadata__", None)
        self.entries: dict[str, dict] = {}
        for name, value in header.items():
            if not isinstance(value, dict):
                raise FormatError(f"header entry {name} is not an object")
            offsets = value.get("data_offsets")
            if (not isinstance(offsets, list) or len(offsets) != 2 or not all(isinstance(v, int) for v in offsets)
                    or not 0 <= offsets[0] <= offsets[1] or self.data_start + offsets[1] > size):
                raise FormatError(f"header entry {name} has malformed data_offsets")
            self.entries[name] = value
        if not self.entries:
            raise FormatError(f"safetensors header of {self.path} declares no tensors")

    def names(self) -> list[str]:
        return sorted(self.entries)

    def read(self, name: str) -> np.ndarray:
        if name not in self.entries:
            raise FormatError(f"no tensor named {name!r} in {self.path}")
        entry = self.entries[name]
        dtype = _SAFETENSORS_DTYPES.get(entry.get("dtype"))
        if dtype is None:
            raise FormatError(f"{name}: unsupported safetensors dtype {entry.get('dtype')!r}")
        shape = tuple(int(v) for v in entry.get("shape", ()))
        begin, end = entry["data_offsets"]
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if count * dtype.itemsize != end - begin:
            raise FormatError(f"{name}: shape {shape} of {entry.get('dtype')} does not fill its {end - begin} bytes")
        return np.fromfile(self.path, dtype=dtype, count=count, offset=self.data_start + begin).reshape(shape)


def write_safetensors(path, arrays: dict[str, np.ndarray], metadata: dict | None = None) -> None:
    """A minimal writer (tests and small artifacts): U8 / U16 / F16 / F32 / I32 / I64 arrays."""
    codes = {v: k for k, v in _SAFETENSORS_DTYPES.items() if k != "I16"}
    header, cursor, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(arrays):
        array = np.ascontiguousarray(arrays[name])
        dtype = array.dtype.newbyteorder("<") if array.dtype.byteorder == ">" else array.dtype
        if np.dtype(dtype) not in codes:
            raise FormatError(f"{name}: dtype {array.dtype} cannot be written")
        data = array.astype(dtype, copy=False).tobytes()
        header[name] = {"dtype": codes[np.dtype(dtype)], "shape": list(array.shape),
                        "data_offsets": [cursor, cursor + len(data)]}
        cursor += len(data)
        blobs.append(data)
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-(8 + len(raw)) % 8)
    with Path(path).open("wb") as handle:
        handle.write(struct.pack("<Q", len(raw)))
        handle.write(raw)
        for data in blobs:
            handle.write(data)


def load_packed_pair(file: SafetensorsFile, module_path: str, layout: PackedTensorLayout) -> np.ndarray:
    """Canonical blocks from the ``<module_path>.codes`` / ``.scales`` pair of a converted checkpoint,
    with the shape checks and the byte scan of the reference loader (src/ternel_mlx/packing.py:29-82)."""
    codes = file.read(f"{module_path}.codes")
    scales = file.read(f"{module_path}.scales")
    if codes.dtype != np.uint8 or tuple(codes.shape) != layout.codes_shape:
        raise FormatError(f"{module_path}.codes: expected uint8 {layout.codes_shape}, got {codes.dtype} {codes.shape}")
    if scales.dtype.itemsize != 2 or tuple(scales.shape) != layout.scales_shape:
        raise FormatError(
            f"{module_path}.scales: expected uint16 {layout.scales_shape}, got {scales.dtype} {scales.shape}")
    validate_packed_codes(codes)
    return unpack_blocks(codes, scales.view("<u2"), layout=layout)


def load_packed_model(model, file: SafetensorsFile, *, strict: bool = True) -> dict[str, int]:
    """Fill every ``PackedLinear`` / ``PackedEmbedding`` below ``model`` from a converted checkpoint.

    Returns ``{"loaded": n, "missing": m}``; with ``strict`` a packed module without its pair raises."""
    from .modules import _PackedBase

    loaded = missing = 0
    for path, module in model.named_modules():
        if not isinstance(module, _PackedBase):
            continue
        if f"{path}.codes" not in file.entries or f"{path}.scales" not in file.entries:
            if strict:
                raise FormatError(f"checkpoint has no codes/scales pair for {path}")
            missing += 1
            continue
        module.load_blocks(load_packed_pair(file, path, module.layout), validate=False)
        module._validated = True
        loaded += 1
    return {"loaded": loaded, "missing": missing}
