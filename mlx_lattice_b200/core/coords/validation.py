"""Coordinate array checks (``native/features/coordinates/validation.cpp:8-15``)."""

from __future__ import annotations

import torch


def validate_coords(coords: torch.Tensor) -> None:
    if not isinstance(coords, torch.Tensor) or coords.ndim != 2 or coords.shape[1] != 4:
        raise ValueError('coords must have shape (N, 4).')
    if coords.dtype not in (torch.int32, torch.int64):
        raise ValueError('coords must be int32 or int64.')
