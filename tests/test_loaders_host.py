"""Readers of the reference's on-disk containers against files written by the reference itself
(tests/golden/sidecar_small.*; see make_golden.py), plus round trips and the corruption cases the
reference's own reader tests cover (tests/test_format.py:199-275 of the reference)."""

import json
import struct
from pathlib import Path

import numpy as np
import pytest

from ternel_b200 import FormatError
from ternel_b200 import loaders
from ternel_b200.layout import PackedTensorLayout, pack_blocks

GOLDEN = Path(__file__).resolve().parent / "golden"
WANT = np.load(GOLDEN / "sidecar_small_blocks.npz")
NAMES = ("blk.0.ffn_down.weight", "blk.0.ssm_a.weight")


def test_reads_a_sidecar_written_by_the_reference():
    header, manifest = loaders.read_sidecar(GOLDEN / "sidecar_small.tq1g128")
    assert header.tensor_count == 2 and header.source_file_bytes == 4242 and header.source_sha256 == "ab" * 32
    assert [t["name"] for t in manifest["tensors"]] == list(NAMES)
    for name in NAMES:
        blocks = loaders.load_sidecar_tensor(GOLDEN / "sidecar_small.tq1g128", manifest, name)
        assert blocks.shape == WANT[name].shape and np.array_equal(blocks, WANT[name])
    with pytest.raises(FormatError, match="no tensor named"):
        loaders.load_sidecar_tensor(GOLDEN / "sidecar_small.tq1g128", manifest, "nope")


def test_reads_a_lut23_sidecar_written_by_the_reference():
    header, manifest = loaders.read_lut23_sidecar(GOLDEN / "sidecar_small.lut23")
    assert header.tensor_count == 2
    assert manifest["tensors"][0]["padded_rows"] == 512 and manifest["tensors"][1]["padded_rows"] == 256
    for name in NAMES:
        blocks = loaders.load_lut23_tensor(GOLDEN / "sidecar_small.lut23", manifest, name)
        assert np.array_equal(blocks, WANT[name])       # padded rows dropped, bytes identical


def test_header_bytes_match_the_reference_writer():
    raw = (GOLDEN / "sidecar_small.tq1g128").read_bytes()
    header = loaders.SidecarHeader.unpack(raw[:256])
    assert header.pack() == raw[:256]
    raw23 = (GOLDEN / "sidecar_small.lut23").read_bytes()
    assert loaders.Lut23Header.unpack(raw23[:256]).pack() == raw23[:256]


def test_own_writers_round_trip_and_lay_tensors_out_like_the_reference(tmp_path):
    tensors = [(name, WANT[name]) for name in NAMES]
    manifest = loaders.write_sidecar(tmp_path / "a.tq1g128", tensors, source_sha256="ab" * 32, source_file_bytes=4242)
    _, ref_manifest = loaders.read_sidecar(GOLDEN / "sidecar_small.tq1g128")
    for mine, theirs in zip(manifest["tensors"], ref_manifest["tensors"]):
        for key in ("name", "shape_gguf", "groups", "packed_offset", "packed_bytes", "packed_payload_sha256"):
            assert mine[key] == theirs[key]
    header, again = loaders.read_sidecar(tmp_path / "a.tq1g128")
    assert np.array_equal(loaders.load_sidecar_tensor(tmp_path / "a.tq1g128", again, NAMES[0]), WANT[NAMES[0]])

    m23 = loaders.write_lut23_sidecar(tmp_path / "a.lut23", tensors)
    _, ref23 = loaders.read_lut23_sidecar(GOLDEN / "sidecar_small.lut23")
    for mine, theirs in zip(m23["tensors"], ref23["tensors"]):
        for key in ("tiles", "padded_rows", "codes_offset", "codes_bytes", "scales_offset", "scales_bytes", "end"):
            assert mine[key] == theirs[key]
    # payload bytes identical to the reference's file up to the manifest
    end = ref23["tensors"][-1]["end"]
    assert (tmp_path / "a.lut23").read_bytes()[256:end] == (GOLDEN / "sidecar_small.lut23").read_bytes()[256:end]


def _small_sidecar() -> bytes:
    tensors = [{"name": "a", "packed_offset": 256, "packed_bytes": 56, "groups": 2},
               {"name": "b", "packed_offset": 512, "packed_bytes": 28, "groups": 1}]
    manifest = json.dumps({"format": "TQ1_G128", "tensors": tensors}, sort_keys=True, separators=(",", ":")).encode()
    header = loaders.SidecarHeader(2, 999, 540, len(manifest), "ab" * 32)
    return header.pack() + bytes(540 - 256) + manifest


@pytest.mark.parametrize(("mutation", "message"), [
    ("magic", "magic"), ("version", "version"), ("geometry", "geometry"), ("reserved", "reserved"),
    ("manifest_bounds", "outside"), ("manifest_json", "manifest"), ("manifest_format", "format"),
    ("tensor_count", "tensor count"), ("unaligned_tensor", "extent"), ("wrong_tensor_size", "extent"),
    ("overlap_manifest", "overlaps"),
])
def test_corrupt_sidecars_are_rejected(tmp_path, mutation, message):
    data = bytearray(_small_sidecar())
    header = loaders.SidecarHeader.unpack(bytes(data[:256]))
    manifest = json.loads(data[header.manifest_offset:].decode())
    if mutation == "magic":
        data[0] ^= 0xFF
    elif mutation == "version":
        struct.pack_into("<I", data, 8, 99)
    elif mutation == "geometry":
        struct.pack_into("<I", data, 16, 127)
    elif mutation == "reserved":
        data[255] = 1
    elif mutation == "manifest_bounds":
        struct.pack_into("<Q", data, 48, len(data) + 1)
    elif mutation == "manifest_json":
        data[header.manifest_offset] = 0xFF
    else:
        if mutation == "manifest_format":
            manifest["format"] = "wrong"
        elif mutation == "tensor_count":
            manifest["tensors"].pop()
        elif mutation == "unaligned_tensor":
            manifest["tensors"][1]["packed_offset"] = 511
        elif mutation == "wrong_tensor_size":
            manifest["tensors"][1]["packed_bytes"] = 27
        elif mutation == "overlap_manifest":
            manifest["tensors"][1]["packed_offset"] = 768
        raw = json.dumps(manifest, sort_keys=True, separators=(",", ":")).encode()
        del data[header.manifest_offset:]
        data.extend(raw)
        struct.pack_into("<Q", data, 48, len(raw))
    path = tmp_path / "bad.tq1g128"
    path.write_bytes(bytes(data))
    with pytest.raises(FormatError, match=message):
        loaders.read_sidecar(path)


def test_payload_hash_and_illegal_bytes_fail_closed(tmp_path):
    path = tmp_path / "a.tq1g128"
    loaders.write_sidecar(path, [(NAMES[1], WANT[NAMES[1]])])
    _, manifest = loaders.read_sidecar(path)
    data = bytearray(path.read_bytes())
    data[256 + 5] = 250                                         # an unrepresentable code byte
    path.write_bytes(bytes(data))
    with pytest.raises(FormatError, match="hash mismatch"):
        loaders.load_sidecar_tensor(path, manifest, NAMES[1])
    manifest["tensors"][0].pop("packed_payload_sha256")
    with pytest.raises(FormatError, match="regular=1"):
        loaders.load_sidecar_tensor(path, manifest, NAMES[1])
    bad = WANT[NAMES[1]].copy()
    bad[0, 0, 27] = 27
    with pytest.raises(FormatError, match="tail=1"):
        loaders.write_sidecar(tmp_path / "b.tq1g128", [("x", bad)])


def test_safetensors_pairs(tmp_path):
    arrays, layouts = {}, {}
    for module, name in (("model.layers.0.mlp.down_proj", NAMES[0]), ("model.layers.0.gate", NAMES[1])):
        blocks = WANT[name][: 256 if name == NAMES[0] else 48]
        lay = PackedTensorLayout.for_tensor(blocks.shape[0], blocks.shape[1] * 128)
        codes, scales = pack_blocks(blocks, layout=lay)
        arrays[f"{module}.codes"], arrays[f"{module}.scales"] = codes, scales
        layouts[module] = (lay, blocks)
    arrays["model.norm.weight"] = np.ones(4, dtype=np.float16)
    loaders.write_safetensors(tmp_path / "m.safetensors", arrays, metadata={"format": "pt"})
    file = loaders.SafetensorsFile(tmp_path / "m.safetensors")
    assert "model.norm.weight" in file.names() and file.metadata == {"format": "pt"}
    assert np.array_equal(file.read("model.norm.weight"), np.ones(4, dtype=np.float16))
    for module, (lay, blocks) in layouts.items():
        assert np.array_equal(loaders.load_packed_pair(file, module, lay), blocks)
    with pytest.raises(FormatError, match="expected uint8"):
        loaders.load_packed_pair(file, "model.layers.0.gate", layouts["model.layers.0.mlp.down_proj"][0])
    with pytest.raises(FormatError, match="no tensor named"):
        loaders.load_packed_pair(file, "model.layers.1.gate", layouts["model.layers.0.gate"][0])
    raw = bytearray((tmp_path / "m.safetensors").read_bytes())
    struct.pack_into("<Q", raw, 0, 1 << 40)
    (tmp_path / "bad.safetensors").write_bytes(bytes(raw))
    with pytest.raises(FormatError, match="implausible"):
        loaders.SafetensorsFile(tmp_path / "bad.safetensors")


def test_load_packed_model_fills_a_swapped_model(tmp_path):
    import torch
    from ternel_b200.packed_model import blocks_from_ternary, replace_with_packed
    from tests.test_packed_model_host import Toy

    rng = np.random.default_rng(9)
    model = Toy(vocab=256, hidden=128, ffn=256, layers=1)
    replace_with_packed(model)
    arrays, want = {}, {}
    for path, module in model.named_modules():
        if hasattr(module, "layout"):
            lay = module.layout
            blocks = blocks_from_ternary(rng.integers(-1, 2, (lay.rows, lay.columns)),
                                         np.abs(rng.standard_normal((lay.rows, lay.columns // 128))).astype(np.float16))
            arrays[f"{path}.codes"], arrays[f"{path}.scales"] = pack_blocks(blocks, layout=lay)
            want[path] = blocks
    loaders.write_safetensors(tmp_path / "model.safetensors", arrays)
    counts = loaders.load_packed_model(model, loaders.SafetensorsFile(tmp_path / "model.safetensors"))
    assert counts == {"loaded": 4, "missing": 0}
    for path, blocks in want.items():
        assert np.array_equal(model.get_submodule(path).blocks.numpy(), blocks)
    del arrays["head.codes"]
    loaders.write_safetensors(tmp_path / "partial.safetensors", arrays)
    with pytest.raises(FormatError, match="head"):
        loaders.load_packed_model(model, loaders.SafetensorsFile(tmp_path / "partial.safetensors"))
    assert torch.is_tensor(model.head.blocks)
