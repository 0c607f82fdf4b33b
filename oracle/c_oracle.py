"""ctypes loader for oracle/libtq1_oracle.so (the C restatement; test infrastructure only)."""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB = None


def build() -> Path:
    subprocess.run(["make", "-s", "-C", str(_DIR), "libtq1_oracle.so"], check=True)
    return _DIR / "libtq1_oracle.so"


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = _DIR / "libtq1_oracle.so"
        if not path.exists():
            build()
        _LIB = ctypes.CDLL(str(path))
        _LIB.tq1o_matmul_f32.restype = ctypes.c_int
        _LIB.tq1o_get_rows_f32.restype = ctypes.c_int
        _LIB.tq1o_encode.restype = ctypes.c_int
        _LIB.tq1o_decode.restype = ctypes.c_int
        _LIB.tq1o_threads.restype = ctypes.c_int
    return _LIB


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def threads() -> int:
    return int(lib().tq1o_threads())


def matmul_f32(blocks: np.ndarray, x: np.ndarray, *, rows: int, columns: int, threads: int = 0) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    xa = np.ascontiguousarray(np.atleast_2d(x), dtype=np.float32)
    y = np.empty((xa.shape[0], rows), dtype=np.float32)
    rc = lib().tq1o_matmul_f32(_p(b), _p(xa), _p(y), ctypes.c_int(xa.shape[0]), ctypes.c_int(rows),
                               ctypes.c_int(columns), ctypes.c_int(threads))
    if rc:
        raise ValueError("tq1o_matmul_f32 rejected the shape")
    return y


def get_rows_f32(blocks: np.ndarray, ids, *, rows: int, columns: int) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    idx = np.ascontiguousarray(ids, dtype=np.int64)
    out = np.empty((idx.size, columns), dtype=np.float32)
    rc = lib().tq1o_get_rows_f32(_p(b), _p(idx), _p(out), ctypes.c_int64(idx.size),
                                 ctypes.c_int64(rows), ctypes.c_int(columns))
    if rc:
        raise ValueError("tq1o_get_rows_f32 rejected the shape")
    return out


def encode(scales: np.ndarray, trits: np.ndarray) -> np.ndarray:
    s = np.ascontiguousarray(scales, dtype=np.uint8).reshape(-1, 2)
    c = np.ascontiguousarray(trits, dtype=np.uint8).reshape(-1, 128)
    out = np.empty((c.shape[0], 28), dtype=np.uint8)
    bad = ctypes.c_int64(0)
    rc = lib().tq1o_encode(_p(s), _p(c), _p(out), ctypes.c_int64(c.shape[0]), ctypes.byref(bad))
    if rc:
        raise ValueError(f"source contains {bad.value} non-ternary code(s)")
    return out


def decode(blocks: np.ndarray, validate: bool = True):
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 28)
    s = np.empty((b.shape[0], 2), dtype=np.uint8)
    c = np.empty((b.shape[0], 128), dtype=np.uint8)
    nf, nt = ctypes.c_int64(0), ctypes.c_int64(0)
    rc = lib().tq1o_decode(_p(b), _p(s), _p(c), ctypes.c_int64(b.shape[0]), ctypes.c_int(int(validate)),
                           ctypes.byref(nf), ctypes.byref(nt))
    if rc:
        raise ValueError(f"invalid base-3 bytes: regular={nf.value}, tail={nt.value}")
    return s, c
