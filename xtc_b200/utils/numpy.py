"""Default evaluation inputs (the reference's ``xtc/utils/numpy.py:12-19``)."""

from __future__ import annotations

from collections.abc import Sequence

import numpy as np


def np_init(shape: Sequence[int], dtype: str) -> np.ndarray:
    """An array of the given shape filled with 1..9 cycling in C order."""
    count = 1
    for dim in shape:
        count *= int(dim)
    return (np.arange(count) % 9 + 1).reshape(tuple(shape)).astype(dtype)
