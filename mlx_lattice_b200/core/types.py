"""Small shared types (``mlx_lattice/core/types.py``)."""

from __future__ import annotations

from collections.abc import Sequence

Triple = tuple[int, int, int]


def triple(value: int | Sequence[int], *, name: str = 'value') -> Triple:
    """Normalise an int or a 3-sequence to a tuple of three ints."""
    if isinstance(value, bool):
        raise ValueError(f'{name} must be an int or a sequence of three ints.')
    if isinstance(value, int):
        return (value, value, value)
    values = tuple(int(v) for v in value)
    if len(values) != 3:
        raise ValueError(f'{name} must be an int or a sequence of three ints.')
    return (values[0], values[1], values[2])
