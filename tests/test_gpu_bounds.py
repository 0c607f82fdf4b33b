"""Memory-safety evidence for the kernels without a sanitizer. Needs a B200.

Two instruments:

* canaries: every output and every workspace handed to the C ABI sits between two guard pages filled with a
  known byte; after the launch the guards must be untouched and the result must equal the oracle's. The cases
  are the ragged corners (one row, one group, row counts off the 16-row tile, token counts off the token tile).
* the bounds-checking build (-DTQ1_BOUNDS_CHECK): the small cases of the GPU suite run again in a child
  process against it; tests/conftest.py then asserts after every test that the violation record stayed zero.
"""

import ctypes
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import tq1_oracle as o
from tests.gpu_util import random_blocks, to_dev

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
GUARD = 4096
CANARY = 0xA5
TOL = 2e-5              # the batched kernel's pinned worst case is 1.5e-5; the batch-1 kernels stay below 1e-5


class Guarded:
    """`nbytes` of zeroed device memory between two guard pages."""

    def __init__(self, nbytes):
        self.nbytes = int(nbytes)
        padded = (self.nbytes + 255) // 256 * 256
        self.whole = torch.full((GUARD + padded + GUARD,), CANARY, dtype=torch.uint8, device="cuda")
        self.payload = self.whole[GUARD:GUARD + self.nbytes]
        self.payload.zero_()

    @property
    def ptr(self):
        return self.payload.data_ptr() if self.nbytes else None

    def view(self, dtype, shape):
        return self.payload.view(dtype).reshape(shape)

    def assert_intact(self, what):
        torch.cuda.synchronize()
        head = self.whole[:GUARD]
        tail = self.whole[GUARD + self.nbytes:]
        assert bool((head == CANARY).all()), f"{what}: bytes before the buffer were written"
        assert bool((tail == CANARY).all()), f"{what}: bytes after the buffer were written"


def native():
    from ternel_b200 import _native
    return _native


def check(rc):
    assert rc == 0, native().last_error()


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("batch,rows,columns", [
    (1, 1, 128), (1, 1, 512), (1, 7, 640), (1, 17, 512), (1, 16, 1024), (1, 100, 1536), (1, 1000, 512),
    (2, 1, 128), (3, 17, 256), (5, 100, 640), (8, 31, 512), (16, 16, 128), (17, 33, 384), (33, 129, 512),
    (64, 1, 128), (129, 200, 256),
])
def test_linear_stays_inside_its_buffers(batch, rows, columns):
    lib = native().lib()
    blocks, rng = random_blocks(rows, columns, seed=batch * 1000 + rows)
    x = rng.standard_normal((batch, columns)).astype(np.float16)
    for out_f32 in (1, 0):
        width = 4 if out_f32 else 2
        y = Guarded(batch * rows * width)
        ws = Guarded(lib.tq1_linear_workspace_bytes(batch, rows, columns))
        xd, bd = to_dev(x), to_dev(blocks)
        for _ in range(2):                  # the second call runs on the control words the first one left
            check(lib.tq1_linear_f16(bd.data_ptr(), xd.data_ptr(), y.ptr, out_f32, batch, rows, columns,
                                     ws.ptr, ws.nbytes, stream()))
        y.assert_intact(f"y {batch}x{rows}x{columns}")
        ws.assert_intact(f"workspace {batch}x{rows}x{columns}")
        got = y.view(torch.float32 if out_f32 else torch.float16, (batch, rows)).float().cpu().numpy()
        want = o.float64_matmul(blocks, x.astype(np.float32), rows=rows, columns=columns)
        err = o.normalised_error(got, want)
        assert err < (TOL if out_f32 else 1e-3), err


@pytest.mark.parametrize("batch,half_rows,columns", [(1, 1, 512), (1, 9, 512), (1, 24, 1024), (3, 9, 512), (17, 40, 1024)])
def test_swiglu_stays_inside_its_buffers(batch, half_rows, columns):
    lib = native().lib()
    blocks, rng = random_blocks(2 * half_rows, columns, seed=half_rows)
    x = rng.standard_normal((batch, columns)).astype(np.float16)
    y = Guarded(batch * half_rows * 4)
    ws = Guarded(lib.tq1_linear_workspace_bytes(batch, 2 * half_rows, columns))
    xd, bd = to_dev(x), to_dev(blocks)
    check(lib.tq1_linear_swiglu_f16(bd.data_ptr(), xd.data_ptr(), y.ptr, 1, batch, half_rows, columns,
                                    ws.ptr, ws.nbytes, stream()))
    y.assert_intact("swiglu y")
    ws.assert_intact("swiglu workspace")
    full = o.float64_matmul(blocks, x.astype(np.float32), rows=2 * half_rows, columns=columns).astype(np.float32)
    gate, up = full[:, 0::2], full[:, 1::2]
    want = gate / (1.0 + np.exp(-gate)) * up
    got = y.view(torch.float32, (batch, half_rows)).cpu().numpy()
    assert o.normalised_error(got, want) < 5e-5


@pytest.mark.parametrize("tokens,vocabulary,columns", [(1, 1, 128), (3, 5, 384), (7, 2, 5120), (257, 9, 256)])
def test_gather_stays_inside_its_buffer(tokens, vocabulary, columns):
    lib = native().lib()
    blocks, rng = random_blocks(vocabulary, columns, seed=tokens)
    ids = rng.integers(0, vocabulary, size=tokens).astype(np.int64)
    bd, idd = to_dev(blocks), to_dev(ids)
    for out_f32 in (1, 0):
        out = Guarded(tokens * columns * (4 if out_f32 else 2))
        check(lib.tq1_embedding_f16(bd.data_ptr(), idd.data_ptr(), out.ptr, out_f32,
                                    tokens, vocabulary, columns, stream()))
        out.assert_intact("gathered rows")
        got = out.view(torch.float32 if out_f32 else torch.float16, (tokens, columns)).cpu().numpy()
        want = o.get_rows(blocks, ids, rows=vocabulary, columns=columns, dtype=got.dtype)
        assert np.array_equal(got, want)


@pytest.mark.parametrize("rows,columns", [(1, 512), (17, 512), (16, 1024), (100, 1536)])
def test_panel_conversion_stays_inside_its_buffers(rows, columns):
    lib = native().lib()
    blocks, _ = random_blocks(rows, columns, seed=rows)
    bd = to_dev(blocks)
    panels = Guarded(lib.tq1_panel_bytes(rows, columns))
    check(lib.tq1_blocks_to_panels_device(bd.data_ptr(), panels.ptr, rows, columns, stream()))
    panels.assert_intact("panels")
    back = Guarded(blocks.size)
    check(lib.tq1_panels_to_blocks_device(panels.ptr, back.ptr, rows, columns, stream()))
    back.assert_intact("canonical blocks")
    assert np.array_equal(back.payload.cpu().numpy(), blocks.reshape(-1))


def test_chain_stays_inside_its_buffers():
    """Three dependent links with ragged row counts; the workspace is exactly as large as the library asks."""
    from ternel_b200 import _native
    lib = _native.lib()
    shapes = [(520, 512), (517, 512), (1, 512)]           # link i reads the first 512 values of link i-1's output
    rng = np.random.default_rng(5)
    x0 = rng.standard_normal(512).astype(np.float16)
    weights = [random_blocks(n, k, seed=40 + i)[0] for i, (n, k) in enumerate(shapes)]
    held = [to_dev(w) for w in weights]
    xd = to_dev(x0)
    outs = [Guarded(n * 4) for n, _ in shapes]
    links = (_native.ChainLink * len(shapes))()
    for i, (n, k) in enumerate(shapes):
        links[i].blocks = held[i].data_ptr()
        links[i].N, links[i].K = n, k
        links[i].x = xd.data_ptr() if i == 0 else None
        links[i].source = -1 if i == 0 else i - 1
        links[i].source_offset = 0
        links[i].y = outs[i].ptr
        links[i].y_is_f32 = 1
        links[i].swiglu = 0
        links[i].out_scale = 0.25
        links[i].layout = 0
    ws = Guarded(lib.tq1_chain_workspace_bytes(ctypes.addressof(links), len(shapes), 1))
    for _ in range(3):
        check(lib.tq1_linear_chain_f16(ctypes.addressof(links), len(shapes), ws.ptr, ws.nbytes, stream()))
    ws.assert_intact("chain workspace")
    assert int(ws.payload[:4].view(torch.int32)[0].item()) == 0, "a bounded device wait ran out"
    x = x0
    for i, (n, k) in enumerate(shapes):
        outs[i].assert_intact(f"link {i} output")
        got = outs[i].view(torch.float32, (n,)).cpu().numpy()
        want = o.float64_matmul(weights[i], x.astype(np.float32)[None, :], rows=n, columns=k)[0] * np.float32(0.25)
        assert o.normalised_error(got[None, :], want[None, :].astype(np.float32)) < 1e-5, i
        x = got.astype(np.float16)[:512]


SMALL_CASE_MODULES = [
    "tests/test_gpu_chain.py", "tests/test_gpu_linear.py", "tests/test_gpu_swiglu.py", "tests/test_gpu_embedding.py",
    "tests/test_gpu_gemv_stream.py", "tests/test_gpu_gemm.py", "tests/test_gpu_sharded.py", "tests/test_gpu_loaders.py",
]


def test_suite_is_green_on_the_bounds_checking_build():
    """The other GPU modules, and this module's canary cases, against the build whose kernels test every global
    store index; conftest asserts a zero violation record after each test."""
    from ternel_b200.build import CHECKED_LIB_PATH, build_checked
    from ternel_b200._native import LIBRARY_ENV
    if os.environ.get(LIBRARY_ENV):
        pytest.skip("already running against an overriding library")
    build_checked()
    env = dict(os.environ, **{LIBRARY_ENV: str(CHECKED_LIB_PATH)})
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider",
           *SMALL_CASE_MODULES, "tests/test_gpu_bounds.py"]
    done = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=1500)
    tail = (done.stdout + done.stderr)[-4000:]
    assert done.returncode == 0, tail
    assert " passed" in done.stdout, tail


def test_the_record_reports_what_the_checked_build_exports():
    """In the child process above (checked build) the record is readable and zero; in the product build it is absent."""
    from ternel_b200 import _native
    record = _native.bounds_record()
    if os.environ.get(_native.LIBRARY_ENV):
        assert record is not None and record[0] == 0
    else:
        assert record is None
