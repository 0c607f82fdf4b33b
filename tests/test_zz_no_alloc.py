"""The allocation-free batch-1 entry point against the regular one. Needs a B200.

`tq1_gemv_f16_noalloc` serves hosts that cannot hand the library scratch memory when they
call it (stream-capture regions, plugin hosts with a fixed device budget, real-time loops).
Its scratch is an array built into the library, so the things to check are that the result is
the same as `tq1_linear_f16`'s, that a second call right after the first (which finds the
array as the first call left it) is still right, and that shapes beyond the array's size are
refused. The file sorts last so that a failure here cannot hide another test's result.
"""

import ctypes

import numpy as np
import pytest
import torch

from oracle import tq1_oracle as o
from tests.gpu_util import random_blocks

pytestmark = pytest.mark.gpu


def _call_both(lib, blocks_dev, x_dev, rows, columns, out_f32):
    from ternel_b200 import _native
    dtype = torch.float32 if out_f32 else torch.float16
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = lib.tq1_linear_workspace_bytes(1, rows, columns)
    ws = torch.zeros(max(need, 256), dtype=torch.uint8, device="cuda")
    want = torch.full((1, rows), 7.0, dtype=dtype, device="cuda")
    rc = lib.tq1_linear_f16(blocks_dev.data_ptr(), x_dev.data_ptr(), want.data_ptr(), int(out_f32), 1, rows,
                            columns, ws.data_ptr(), ws.numel(), stream)
    assert rc == 0, _native.last_error()
    got = torch.full((1, rows), -7.0, dtype=dtype, device="cuda")
    rc = lib.tq1_gemv_f16_noalloc(blocks_dev.data_ptr(), x_dev.data_ptr(), got.data_ptr(), int(out_f32), rows,
                                  columns, stream)
    assert rc == 0, _native.last_error()
    torch.cuda.synchronize()
    return got.cpu().numpy(), want.cpu().numpy()


def test_no_alloc_entry_matches_the_regular_entry_twice_in_a_row():
    from ternel_b200 import _native
    lib = _native.lib()
    for rows, columns, out_f32 in ((1024, 5120, True), (5120, 17408, False), (300, 1536, True)):
        blocks, rng = random_blocks(rows, columns, seed=rows + columns)
        blocks_dev = torch.from_numpy(blocks).cuda()
        for call in range(2):           # the second call starts from the first call's leftovers
            x = rng.standard_normal((1, columns)).astype(np.float16)
            got, want = _call_both(lib, blocks_dev, torch.from_numpy(x).cuda(), rows, columns, out_f32)
            # same kernel, same summation order: the two entry points agree bit for bit
            assert np.array_equal(got, want), (rows, columns, call)
            assert np.isfinite(got).all() and np.abs(got).max() > 0
            # and both agree with the float64 oracle (FP32 out: the reference's 1e-5; after an FP16 store: 2e-3)
            exact = o.float64_matmul(blocks, x, rows=rows, columns=columns)
            assert o.normalised_error(got, exact) < (1e-5 if out_f32 else 2e-3), (rows, columns, call)
    # no bounded wait ran out in any of those calls: the array's status word is still zero
    status = np.full(1, 99, dtype=np.uint32)
    assert lib.tq1_gemv_noalloc_status(status.ctypes.data, None) == 0, _native.last_error()
    torch.cuda.synchronize()
    assert int(status[0]) == 0


def test_no_alloc_entry_refuses_what_does_not_fit():
    from ternel_b200 import _native
    lib = _native.lib()
    dummy = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = dummy.data_ptr()
    # 65536 x 8192 would need about 4 MiB of scratch: rejected before anything is launched
    assert lib.tq1_gemv_f16_noalloc(p, p, p, 0, 65536, 8192, None) == _native.TQ1_ERR_WORKSPACE
    assert "scratch" in _native.last_error()
    assert lib.tq1_gemv_f16_noalloc(p, p, p, 0, 64, 640, None) == _native.TQ1_ERR_INVALID
    assert "512" in _native.last_error()
    torch.cuda.synchronize()
