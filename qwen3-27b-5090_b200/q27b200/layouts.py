"""Host-side layout helpers (numpy / torch index arithmetic only): the swizzled scale-factor layout and the
gate | up interleave, mirrors of csrc/layout.h for preparing operands and reading results on the host."""

import numpy as np


def sf_bytes(rows: int, kblocks: int) -> int:
    return ((rows + 127) // 128) * 128 * ((kblocks + 3) // 4) * 4


def sf_index(rows: int, kblocks: int) -> np.ndarray:
    """Swizzled byte offset of every (row, k-block) as an int64 [rows, kblocks] array."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    kb = np.arange(kblocks, dtype=np.int64)[None, :]
    katoms = (kblocks + 3) // 4
    return ((r // 128) * katoms + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (kb % 4)


def swizzle(sf_rowmajor: np.ndarray) -> np.ndarray:
    rows, kblocks = sf_rowmajor.shape
    out = np.zeros(sf_bytes(rows, kblocks), dtype=np.uint8)
    out[sf_index(rows, kblocks)] = sf_rowmajor
    return out


def unswizzle(buf: np.ndarray, rows: int, kblocks: int) -> np.ndarray:
    return np.asarray(buf)[sf_index(rows, kblocks)]


def glu_rows(inter: int) -> np.ndarray:
    """Interleaved row of gate rows 0..I-1 followed by up rows 0..I-1 (blocks of 64 rows, gate then up)."""
    r = np.arange(inter, dtype=np.int64)
    return np.concatenate([(r // 64) * 128 + r % 64, (r // 64) * 128 + 64 + r % 64])


def interleave_glu(rows_major):
    """[2I, ...] (gate rows then up rows) -> interleaved order; works for numpy arrays and torch tensors."""
    idx = glu_rows(rows_major.shape[0] // 2)
    if isinstance(rows_major, np.ndarray):
        out = np.empty_like(rows_major)
        out[idx] = rows_major
        return out
    import torch

    out = torch.empty_like(rows_major)
    out[torch.from_numpy(idx).to(rows_major.device)] = rows_major
    return out
