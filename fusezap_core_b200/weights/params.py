"""What a part says about each tensor it needs: shape, role and how the random-weights writer fills it."""
from __future__ import annotations
from dataclasses import dataclass


@dataclass(frozen=True)
class ParamSpec:
    shape: tuple[int, ...]        # a size of -1 is left open: whatever the checkpoint has (the part reads it at `bind`)
    role: str = "matrix"          # "matrix": cast to the compute dtype; "vector": a tensor stored in 32-bit stays so;
                                  # "int_table": kept as int32
    init: str = "normal"          # "normal" (std 0.02), "ones", "zeros"
    group: str | None = None      # None: required. Otherwise the name of an all-or-none group of optional tensors
    ignore: bool = False          # accepted if present, never loaded (a tied model's stored output matrix)
    high: int = 0                 # "int_table" only: the random-weights writer fills every row with distinct values
                                  # drawn from range(high) (0: a table of zeros)
    open: int = 0                 # what the random-weights writer puts in place of an open size

    def filled_shape(self) -> tuple[int, ...]:
        """The shape with every open size replaced by `open` (for writers of random weights)."""
        if any(n < 0 for n in self.shape) and self.open <= 0:
            raise ValueError(f"a tensor of shape {self.shape} has an open size and no value to fill it with")
        return tuple(self.open if n < 0 else n for n in self.shape)
