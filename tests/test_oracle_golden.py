"""The oracle (NumPy and C restatements) against fixtures made by the reference itself."""

import hashlib

import numpy as np
import pytest

from oracle import c_oracle, tq1_oracle as o
from tests.conftest import GOLDEN


def test_codec_matches_reference_bytes():
    g = np.load(GOLDEN / "codec_bytes.npz")
    scales = g["scale_words"].view(np.uint8).reshape(-1, 2)
    assert np.array_equal(o.encode_blocks(scales, g["trits"]), g["blocks"])
    assert np.array_equal(c_oracle.encode(scales, g["trits"]), g["blocks"])
    for decode in (o.decode_blocks, c_oracle.decode):
        s, c = decode(g["blocks"])
        assert np.array_equal(s, scales) and np.array_equal(c, g["trits"])


def test_matmul_references_bit_equal(golden_cases):
    for name, c in golden_cases.items():
        rows, cols = int(c["rows"]), int(c["columns"])
        x = c["x"].astype(np.float32)
        assert np.array_equal(o.reference_matmul(c["blocks"], x, rows=rows, columns=cols), c["y_gemv"]), name
        assert np.array_equal(o.reference_matmul(c["blocks"], x, rows=rows, columns=cols), c["y_restored"]), name
        assert np.array_equal(o.lut23_matmul(c["blocks"], x, rows=rows, columns=cols), c["y_lut23"]), name
        assert np.array_equal(o.float64_matmul(c["blocks"], x, rows=rows, columns=cols), c["y_f64"]), name
        got = c_oracle.matmul_f32(c["blocks"], x, rows=rows, columns=cols)
        assert o.normalised_error(got, c["y_f64"]) < 1e-6, name


def test_tiling_and_rows_match(golden_cases):
    for name, c in golden_cases.items():
        rows, cols, tile = int(c["rows"]), int(c["columns"]), int(c["tile"])
        assert o.select_tile(rows) == tile
        tc, ts = o.tile_blocks(c["blocks"], tile=tile)
        assert np.array_equal(tc, c["tiled_codes"]) and np.array_equal(ts, c["tiled_scales"]), name
        assert np.array_equal(o.untile_blocks(tc, ts, rows, tile=tile), c["blocks"])
        assert np.array_equal(o.get_rows(c["blocks"], c["ids"], rows=rows, columns=cols, dtype=np.float16),
                              c["rows_f16"])
        assert np.array_equal(o.get_rows(c["blocks"], c["ids"], rows=rows, columns=cols, dtype=np.float32),
                              c["rows_f32"])
        assert np.array_equal(c_oracle.get_rows_f32(c["blocks"], c["ids"], rows=rows, columns=cols),
                              c["rows_f32"])


def test_single_matrix_configuration_reproduces():
    g = np.load(GOLDEN / "single_matrix_4096.npz")
    blocks, x = o.synth_matrix(4096, 4096, seed=0)
    digest = np.frombuffer(hashlib.sha256(blocks.tobytes()).digest(), dtype=np.uint8)
    assert np.array_equal(digest, g["blocks_sha256"])
    assert np.array_equal(x, g["x"])
    assert np.array_equal(blocks[:2], g["first_blocks"])
    y = o.reference_gemv(blocks, x.astype(np.float32), rows=4096, columns=4096)
    assert np.array_equal(y, g["y"])
    yc = c_oracle.matmul_f32(blocks, x.astype(np.float32), rows=4096, columns=4096)
    assert o.normalised_error(yc, g["y"]) < 1e-5


def test_oracle_rejects_illegal_bytes():
    packed = np.zeros((1, 28), dtype=np.uint8)
    packed[0, 2] = 243
    with pytest.raises(o.FormatError, match="regular=1"):
        o.decode_blocks(packed)
    with pytest.raises(ValueError, match="regular=1"):
        c_oracle.decode(packed)
    packed[0, 2] = 0
    packed[0, 27] = 27
    with pytest.raises(o.FormatError, match="tail=1"):
        o.decode_blocks(packed)
    with pytest.raises(ValueError, match="tail=1"):
        c_oracle.decode(packed)


def test_l2_l3_split_is_division_by_nine():
    p = np.arange(243, dtype=np.uint32)
    assert np.array_equal((p * 57) >> 9, p // 9)
