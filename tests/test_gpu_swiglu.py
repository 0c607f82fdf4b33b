"""Gate and up projections with SiLU(gate) * up fused into the kernels' epilogues. Needs a B200."""

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import tq1_oracle as o
from tests.gpu_util import random_blocks, to_dev

pytestmark = pytest.mark.gpu


def _want(gate, up, x, rows, columns):
    xf = x.astype(np.float32)
    g = c_oracle.matmul_f32(gate, xf, rows=rows, columns=columns).astype(np.float64)
    u = c_oracle.matmul_f32(up, xf, rows=rows, columns=columns).astype(np.float64)
    return g / (1.0 + np.exp(-g)) * u


@pytest.mark.parametrize("batch", (1, 2, 16, 40, 200, 1100))
@pytest.mark.parametrize(("rows", "columns"), ((17408, 5120), (1000, 1536), (264, 17408)))
def test_fused_swiglu_matches_two_products(rows, columns, batch):
    from ternel_b200.ops import interleave_gate_up, tq1_matmul, tq1_swiglu
    if batch > 200 and rows > 2000:
        pytest.skip("the oracle would take minutes")
    gate, rng = random_blocks(rows, columns, seed=rows + batch, dist="tests")
    up, _ = random_blocks(rows, columns, seed=rows + batch + 1, dist="tests")
    x = (rng.standard_normal((batch, columns)) * 0.5).astype(np.float16)
    want = _want(gate, up, x, rows, columns)
    both = interleave_gate_up(to_dev(gate), to_dev(up))
    assert both.shape == (2 * rows, columns // 128, 28)
    xd = to_dev(x)
    got = tq1_swiglu(both, xd, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert got.shape == (batch, rows)
    assert o.normalised_error(got.cpu().numpy(), want) < 5e-5
    got16 = tq1_swiglu(both, xd).float().cpu().numpy()
    assert o.normalised_error(got16, want) < 2e-3
    # and against the unfused path of this library: the same dot products (up to the summation order of a
    # different K split), activation applied by torch in FP32
    g = tq1_matmul(to_dev(gate), xd, out_dtype=torch.float32)
    u = tq1_matmul(to_dev(up), xd, out_dtype=torch.float32)
    unfused = (torch.nn.functional.silu(g) * u).cpu().numpy()
    assert o.normalised_error(got.cpu().numpy(), unfused) < 5e-5
    assert np.array_equal(tq1_swiglu(both, xd, out_dtype=torch.float32).cpu().numpy(), got.cpu().numpy())


def test_swiglu_argument_checks():
    from ternel_b200 import FormatError
    from ternel_b200.ops import interleave_gate_up, tq1_swiglu
    gate, rng = random_blocks(64, 512, seed=1)
    up, _ = random_blocks(32, 512, seed=2)
    with pytest.raises(FormatError, match="differ in shape"):
        interleave_gate_up(to_dev(gate), to_dev(up))
    odd = to_dev(gate[:63])
    with pytest.raises(FormatError, match="pairs"):
        tq1_swiglu(odd, to_dev(np.zeros((1, 512), np.float16)))
    narrow, _ = random_blocks(64, 640, seed=3)          # K not a multiple of 512: no fused kernel for it
    with pytest.raises(FormatError, match="512"):
        tq1_swiglu(to_dev(narrow), to_dev(np.zeros((1, 640), np.float16)))
