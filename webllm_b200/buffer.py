"""Tensor handles and alignment — the reference's ``src/gpu/buffer.ts:3-18``."""
from __future__ import annotations

from dataclasses import dataclass, field

ALIGN = 256


def align_to(n: int, align: int = ALIGN) -> int:
    """``alignTo`` (src/gpu/buffer.ts:6-9)."""
    return -(-n // align) * align


@dataclass
class Tensor:
    """``Tensor`` (src/gpu/buffer.ts:11-18): a slice of the activation slab. ``offset`` is in bytes,
    ``length`` in elements. ``dtype`` is ``"f32"`` (the reference's only activation type) or ``"f16"``."""
    offset: int
    length: int
    shape: list = field(default_factory=list)
    dtype: str = "f32"

    @property
    def itemsize(self) -> int:
        return 4 if self.dtype == "f32" else 2

    @property
    def nbytes(self) -> int:
        return self.length * self.itemsize
