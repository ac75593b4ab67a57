"""Binary file formats of the GLIDE pipeline (reference ``load.cuh``).

* matrix (``.fbin`` and every stage matrix): u32 rows, u32 dim, rows*dim packed values
  (load.cuh:10-30, save :90-103);
* segment file: u32 S, u32 start[S], u32 length[S] (load.cuh:33-68, :106-117);
* id vector: u32 n, u32[n] (load.cuh:71-86, :120-127).

The reference prints a message and carries on when a file cannot be opened
(load.cuh:12-14); here that, a short file and a size mismatch raise ``IOError``.
"""
from __future__ import annotations

import os

import numpy as np


def _check_size(path: str, expected: int) -> None:
    actual = os.path.getsize(path)
    if actual < expected:
        raise IOError(f"{path}: truncated ({actual} bytes, header promises {expected})")


def load_matrix_data(path: str, dtype=np.float32) -> np.ndarray:
    with open(path, "rb") as f:
        head = np.fromfile(f, dtype=np.uint32, count=2)
        if head.size != 2:
            raise IOError(f"{path}: missing 8-byte header")
        rows, dim = int(head[0]), int(head[1])
        _check_size(path, 8 + rows * dim * np.dtype(dtype).itemsize)
        data = np.fromfile(f, dtype=dtype, count=rows * dim)
    return data.reshape(rows, dim)


def save_matrix_data(path: str, matrix: np.ndarray) -> None:
    m = np.ascontiguousarray(matrix)
    if m.ndim != 2:
        raise ValueError("matrix must be 2-D")
    if m.dtype not in (np.float32, np.uint32, np.int32, np.uint8):
        # readers take the element type from the caller, not from the file (load.cuh:10-30): writing
        # float64 or int64 under this header would be read back as twice as many 4-byte values
        raise TypeError(f"matrix files hold fp32, u32/i32 or uint8 elements, got {m.dtype}")
    with open(path, "wb") as f:
        np.array(m.shape, dtype=np.uint32).tofile(f)
        m.tofile(f)


def load_segment(path: str) -> tuple[np.ndarray, np.ndarray]:
    """Returns (segment_start, segment_length)."""
    with open(path, "rb") as f:
        head = np.fromfile(f, dtype=np.uint32, count=1)
        if head.size != 1:
            raise IOError(f"{path}: missing header")
        s = int(head[0])
        _check_size(path, 4 + 8 * s)
        start = np.fromfile(f, dtype=np.uint32, count=s)
        length = np.fromfile(f, dtype=np.uint32, count=s)
    return start, length


def save_segment(path: str, start: np.ndarray, length: np.ndarray) -> None:
    start = np.ascontiguousarray(start, dtype=np.uint32)
    length = np.ascontiguousarray(length, dtype=np.uint32)
    if start.shape != length.shape:
        raise ValueError("start and length differ in size")
    with open(path, "wb") as f:
        np.array([start.size], dtype=np.uint32).tofile(f)
        start.tofile(f)
        length.tofile(f)


def load_vector_data(path: str) -> np.ndarray:
    with open(path, "rb") as f:
        head = np.fromfile(f, dtype=np.uint32, count=1)
        if head.size != 1:
            raise IOError(f"{path}: missing header")
        n = int(head[0])
        _check_size(path, 4 + 4 * n)
        return np.fromfile(f, dtype=np.uint32, count=n)


def save_vector_data(path: str, vec: np.ndarray) -> None:
    v = np.ascontiguousarray(vec, dtype=np.uint32)
    with open(path, "wb") as f:
        np.array([v.size], dtype=np.uint32).tofile(f)
        v.tofile(f)
