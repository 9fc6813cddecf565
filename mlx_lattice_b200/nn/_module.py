"""Minimal module base: named tensors with device / dtype movement.

The reference modules derive from a third-party ``Module`` class that only stores
arrays on the object; this stand-in does the same for CUDA tensors.
"""

from __future__ import annotations

import torch


class Module:
    def __contains__(self, name: str) -> bool:
        return getattr(self, name, None) is not None

    def parameters(self) -> dict[str, torch.Tensor]:
        return {k: v for k, v in vars(self).items() if isinstance(v, torch.Tensor)}

    def children(self) -> dict[str, 'Module']:
        return {k: v for k, v in vars(self).items() if isinstance(v, Module)}

    def to(self, device=None, dtype: torch.dtype | None = None) -> 'Module':
        """Move every tensor; ``dtype`` applies to floating tensors only."""
        for name, value in list(vars(self).items()):
            if isinstance(value, torch.Tensor):
                moved = value if device is None else value.to(device)
                if dtype is not None and moved.is_floating_point():
                    moved = moved.to(dtype)
                setattr(self, name, moved)
            elif isinstance(value, Module):
                value.to(device, dtype)
            elif isinstance(value, (list, tuple)):
                for item in value:
                    if isinstance(item, Module):
                        item.to(device, dtype)
        return self

    def freeze(self) -> 'Module':
        return self
