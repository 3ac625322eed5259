"""Tile schedules for the persistent GEMM.

``hilbert_schedule`` gives the visiting order the reference's persistent GEMM
test builds on the host (tests/gpu/end2end/wgmma_persis.co:156-197): walk the
Hilbert curve over the smallest power-of-two square that covers the tile grid
and keep the cells that fall inside it; ``schedule_m`` receives the curve's x,
``schedule_n`` its y.
"""
from __future__ import annotations

import numpy as np


def _hilbert_d2xy(size: int, index: int) -> tuple[int, int]:
    x = y = 0
    scale = 1
    while scale < size:
        rx = 1 & (index // 2)
        ry = 1 & (index ^ rx)
        if ry == 0:
            if rx == 1:
                x = scale - 1 - x
                y = scale - 1 - y
            x, y = y, x
        x += scale * rx
        y += scale * ry
        index //= 4
        scale *= 2
    return x, y


def hilbert_schedule(tiles_m: int, tiles_n: int) -> tuple[np.ndarray, np.ndarray]:
    """Returns (schedule_m, schedule_n), int32 arrays of length tiles_m*tiles_n."""
    if tiles_m <= 0 or tiles_n <= 0:
        return np.zeros(0, np.int32), np.zeros(0, np.int32)
    size = 1
    while size < max(tiles_m, tiles_n):
        size *= 2
    sm, sn = [], []
    for index in range(size * size):
        x, y = _hilbert_d2xy(size, index)
        if x < tiles_m and y < tiles_n:
            sm.append(x)
            sn.append(y)
    return np.asarray(sm, np.int32), np.asarray(sn, np.int32)


def row_major_schedule(tiles_m: int, tiles_n: int) -> tuple[np.ndarray, np.ndarray]:
    """Tile order of the reference's non-Hilbert persistent kernels
    (block_m = tile_id / tiles_n, block_n = tile_id % tiles_n;
    tests/gpu/end2end/wgmma_persis.co:48-49)."""
    ids = np.arange(tiles_m * tiles_n, dtype=np.int32)
    return (ids // max(tiles_n, 1)).astype(np.int32), (ids % max(tiles_n, 1)).astype(np.int32)
