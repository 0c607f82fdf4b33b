"""Host side of the library: codec, layout bridge, module loading, exported symbols (no GPU)."""

import ctypes
import itertools
import re
from pathlib import Path

import numpy as np
import pytest
import torch

import ternel_b200 as tb
from ternel_b200 import _native
from ternel_b200.modules import PackedEmbedding, PackedLinear
from oracle import tq1_oracle as o
from tests.conftest import GOLDEN, ROOT


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "ternel_b200.h").read_text()
    declared = set(re.findall(r"^(?:int|void|size_t|const char \*)\s*(tq1_[a-z0-9_]+)\s*\(", header, re.M))
    assert declared, "no declarations found"
    assert declared == set(_native.SIGNATURES), declared ^ set(_native.SIGNATURES)
    handle = ctypes.CDLL(str(_native.LIB_PATH))
    for name in declared:
        assert hasattr(handle, name), name
    assert _native.lib().tq1_abi_version() >= 1


def test_every_legal_five_trit_byte_round_trips():
    codes = np.ones((243, 128), dtype=np.uint8)
    for value in range(243):
        v = value
        for t in range(5):
            codes[value, t] = v % 3
            v //= 3
    scales = np.arange(243, dtype=np.uint16).view(np.uint8).reshape(243, 2)
    packed = tb.encode_tq1_blocks(scales, codes)
    assert np.array_equal(packed[:, 2], np.arange(243, dtype=np.uint8))
    s, c = tb.decode_tq1_blocks(packed)
    assert np.array_equal(s, scales) and np.array_equal(c, codes)


@pytest.mark.parametrize("tail", range(27))
def test_every_legal_tail_byte_round_trips(tail):
    codes = np.ones((1, 128), dtype=np.uint8)
    v = tail
    for i in range(3):
        codes[0, 125 + i] = v % 3
        v //= 3
    packed = tb.encode_tq1_blocks(np.asarray([[0x34, 0x12]], dtype=np.uint8), codes)
    assert int(packed[0, 27]) == tail
    assert np.array_equal(tb.decode_tq1_blocks(packed)[1], codes)


def test_all_fp16_scale_bit_patterns_are_preserved():
    words = np.arange(1 << 16, dtype=np.uint16)
    scales = words.view(np.uint8).reshape(-1, 2)
    codes = np.ones((words.size, 128), dtype=np.uint8)
    packed = tb.encode_tq1_blocks(scales, codes)
    s, c = tb.decode_tq1_blocks(packed)
    assert s.tobytes() == scales.tobytes() and np.array_equal(c, codes)


def test_codec_matches_reference_fixture_and_oracle():
    g = np.load(GOLDEN / "codec_bytes.npz")
    scales = g["scale_words"].view(np.uint8).reshape(-1, 2)
    assert np.array_equal(tb.encode_tq1_blocks(scales, g["trits"]), g["blocks"])
    rng = np.random.default_rng(5)
    trits = rng.integers(0, 3, size=(1000, 128), dtype=np.uint8)
    sc = rng.integers(0, 256, size=(1000, 2), dtype=np.uint8)
    packed = tb.encode_tq1_blocks(sc, trits)
    assert np.array_equal(packed, o.encode_blocks(sc, trits))
    s, c = tb.decode_tq1_blocks(packed)
    assert np.array_equal(s, sc) and np.array_equal(c, trits)
    # chunking invariance
    pieces = [tb.encode_tq1_blocks(sc[i:i + 7], trits[i:i + 7]) for i in range(0, 1000, 7)]
    assert np.array_equal(np.concatenate(pieces), packed)


def test_non_ternary_and_illegal_bytes_fail_closed():
    codes = np.tile(np.asarray([0, 1, 2, 3], dtype=np.uint8), 32).reshape(1, 128)
    with pytest.raises(tb.FormatError, match="32 non-ternary"):
        tb.encode_tq1_blocks(np.zeros((1, 2), dtype=np.uint8), codes)
    packed = np.zeros((1, 28), dtype=np.uint8)
    packed[0, 2] = 243
    with pytest.raises(tb.FormatError, match="regular=1"):
        tb.decode_tq1_blocks(packed)
    assert tb.decode_tq1_blocks(packed, validate=False)[1].shape == (1, 128)
    packed[0, 2] = 0
    packed[0, 27] = 27
    with pytest.raises(tb.FormatError, match="tail=1"):
        tb.decode_tq1_blocks(packed)
    with pytest.raises(tb.FormatError, match="tail=1"):
        tb.validate_blocks(packed)
    with pytest.raises(tb.FormatError, match="divisible by 28"):
        tb.decode_tq1_blocks(np.zeros(29, dtype=np.uint8))
    with pytest.raises(tb.FormatError, match=r"\(N, 128\)"):
        tb.encode_tq1_blocks(np.zeros((1, 2), dtype=np.uint8), np.zeros((1, 127), dtype=np.uint8))


def test_empty_input_round_trips():
    packed = tb.encode_tq1_blocks(np.zeros((0, 2), dtype=np.uint8), np.zeros((0, 128), dtype=np.uint8))
    assert packed.shape == (0, 28)
    s, c = tb.decode_tq1_blocks(packed)
    assert s.shape == (0, 2) and c.shape == (0, 128)


MODEL_SHAPES = ((48, 5120), (1024, 5120), (5120, 6144), (5120, 17408), (6144, 5120), (10240, 5120),
                (12288, 5120), (17408, 5120), (248320, 5120), (5120, 5120), (4096, 4096), (151936, 5120))


@pytest.mark.parametrize(("rows", "columns"), MODEL_SHAPES)
def test_layout_accounting(rows, columns):
    layout = tb.PackedTensorLayout.for_tensor(rows, columns)
    assert layout.tile == (256 if rows % 256 == 0 else rows)
    assert layout.payload_bytes == layout.canonical_bytes == rows * columns // 128 * 28
    assert layout.bits_per_weight == 1.75
    assert layout.codes_shape == (rows // layout.tile, columns // 128, 26, layout.tile)


def test_layout_rejects_bad_geometry():
    with pytest.raises(tb.FormatError, match="multiple of the 128"):
        tb.PackedTensorLayout.for_tensor(8, 100)
    with pytest.raises(tb.FormatError, match="does not divide"):
        tb.PackedTensorLayout(rows=300, columns=256, tile=256)
    with pytest.raises(tb.FormatError, match="positive"):
        tb.select_tile(0)


def test_tiled_bridge_matches_reference(golden_cases):
    for name, c in golden_cases.items():
        layout = tb.PackedTensorLayout.for_tensor(int(c["rows"]), int(c["columns"]))
        codes, scales = tb.pack_blocks(c["blocks"], layout=layout)
        assert np.array_equal(codes, c["tiled_codes"]) and np.array_equal(scales, c["tiled_scales"]), name
        assert np.array_equal(tb.unpack_blocks(codes, scales, layout=layout), c["blocks"])
        tb.validate_packed_codes(codes)
        bad = codes.copy()
        bad[0, 0, 3, 0] = 243
        bad[0, 0, 25, 1] = 27
        with pytest.raises(tb.FormatError, match=r"regular=1 \(max 242\), tail=1 \(max 26\)"):
            tb.validate_packed_codes(bad)
        with pytest.raises(tb.FormatError, match="uint16"):
            tb.unpack_blocks(codes, scales.astype(np.int32), layout=layout)


def test_modules_check_before_launch_and_load_checkpoints(golden_cases):
    c = golden_cases["r512_k384_m4"]
    layout = tb.PackedTensorLayout.for_tensor(512, 384)
    lin = PackedLinear(layout)
    with pytest.raises(tb.FormatError, match="activation has 100 columns, weight expects 384"):
        lin(torch.zeros(2, 100, dtype=torch.float16))
    with pytest.raises(tb.FormatError, match="cannot carry a bias"):
        PackedLinear.from_linear(torch.nn.Linear(128, 8, bias=True))
    assert PackedLinear.from_linear(torch.nn.Linear(256, 48, bias=False)).layout.tile == 48
    # a CPU tensor is refused: there is no CPU path
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        lin(torch.zeros(2, 384, dtype=torch.float16))
    with pytest.raises(tb.FormatError, match="activations must be one of"):
        lin(torch.zeros(2, 384, dtype=torch.float32))

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = PackedLinear(layout)
            self.embed = PackedEmbedding(layout)

    net = Net()
    state = {
        "proj.codes": torch.from_numpy(c["tiled_codes"]),
        "proj.scales": torch.from_numpy(c["tiled_scales"].view(np.int16)),
        "embed.blocks": torch.from_numpy(c["blocks"]),
    }
    net.load_state_dict(state, strict=True)
    assert np.array_equal(net.proj.blocks.numpy(), c["blocks"])
    assert np.array_equal(net.embed.blocks.numpy(), c["blocks"])
    with pytest.raises(RuntimeError, match="Missing key"):
        net.load_state_dict({"proj.codes": state["proj.codes"], "embed.blocks": state["embed.blocks"]})
    bad = c["tiled_codes"].copy()
    bad[0, 0, 0, 0] = 255
    with pytest.raises(RuntimeError, match="out-of-range base-3 bytes"):
        net.load_state_dict({**state, "proj.codes": torch.from_numpy(bad)})
    with pytest.raises(RuntimeError, match="does not match"):
        net.load_state_dict({**state, "proj.codes": torch.from_numpy(c["tiled_codes"][:1])})
    bad_blocks = c["blocks"].copy()
    bad_blocks[3, 1, 27] = 99
    with pytest.raises(RuntimeError, match="tail=1"):
        net.load_state_dict({**state, "embed.blocks": torch.from_numpy(bad_blocks)})


def test_c_abi_argument_checks_need_no_gpu():
    lib = _native.lib()
    rc = lib.tq1_linear_f16(None, None, None, 0, 1, 8, 128, None, 0, None)
    assert rc == _native.TQ1_ERR_INVALID and "null" in _native.last_error()
    buf = np.zeros(64, dtype=np.uint8)
    p = buf.ctypes.data
    assert lib.tq1_linear_f16(p, p, p, 0, 0, 8, 128, None, 0, None) == _native.TQ1_ERR_INVALID
    assert "empty batch" in _native.last_error()
    assert lib.tq1_linear_f16(p, p, p, 0, 1, 8, 100, None, 0, None) == _native.TQ1_ERR_INVALID
    assert "multiple of the 128" in _native.last_error()
    assert lib.tq1_embedding_f16(p, p, p, 0, 0, 8, 128, None) == _native.TQ1_ERR_INVALID
    assert "indices are empty" in _native.last_error()


def test_dequantize_blocks_is_the_decoded_trits_times_the_scale():
    """The host-side to_float of the type against the oracle's decode: exact, including every byte value, negative
    and subnormal scales and signed zeros."""
    from ternel_b200.format import dequantize_blocks
    from oracle import tq1_oracle as o
    rng = np.random.default_rng(11)
    groups = 300
    trits = rng.integers(0, 3, size=(groups, 128), dtype=np.uint8)
    scales = rng.normal(0.0, 0.05, size=groups).astype(np.float16)
    scales[:4] = np.array([0.0, -0.0, 6e-8, -65504.0], dtype=np.float16)
    blocks = o.encode_blocks(scales.view(np.uint8).reshape(-1, 2), trits)
    got = dequantize_blocks(blocks)
    want = (trits.astype(np.float32) - 1.0) * scales.astype(np.float32)[:, None]
    assert got.dtype == np.float32 and got.shape == (groups, 128)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
