"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

from oracle import tq1_oracle as o

POWERS = np.array([1, 3, 9, 27, 81], dtype=np.float32)


def random_blocks(rows, columns, seed, *, dist="bench"):
    rng = np.random.default_rng(seed)
    groups = rows * columns // 128
    if dist == "bench":
        trits = rng.choice(3, size=(groups, 128), p=[0.30, 0.40, 0.30]).astype(np.uint8)
        scales = (np.abs(rng.standard_normal(groups)) * 0.02).astype(np.float16)
    elif dist == "real":     # the converted model's measured trit frequencies
        trits = rng.choice(3, size=(groups, 128), p=[0.352, 0.297, 0.351]).astype(np.uint8)
        scales = (np.abs(rng.standard_normal(groups)) * 0.02).astype(np.float16)
    else:                    # the reference tests' distribution
        trits = rng.integers(0, 3, size=(groups, 128), dtype=np.uint8)
        scales = rng.normal(0.0, 0.05, size=groups).astype(np.float16)
    blocks = o.encode_blocks(scales.view(np.uint8).reshape(-1, 2), trits)
    return blocks.reshape(rows, columns // 128, 28), rng


def to_dev(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def run_linear(blocks, x, *, out_dtype=torch.float32):
    """x: NumPy (M, K), any float dtype; it is cast to FP16 on the way in."""
    from ternel_b200.ops import tq1_matmul
    xd = to_dev(np.asarray(x).astype(np.float16))
    y = tq1_matmul(to_dev(blocks), xd, out_dtype=out_dtype)
    torch.cuda.synchronize()
    return y.float().cpu().numpy()
