"""Shape/dtype records exchanged once per pipeline edge.

The reference packs ``[dtype_index, *shape]`` into 16 float32 values
(``elf/utils.py:150-220``): at most 15 dims, sizes exact only below 2**24, and one
blocking ``.item()`` per element on decode.  Here the record is an int64 vector,
decoded with a single ``tolist()``, and it also carries whether dim 0 is the
micro-batch dim so that un-batched outputs survive.
"""

from __future__ import annotations

from typing import List, Sequence

import torch

__all__ = ["TensorMetadata", "DTYPES"]

DTYPES: List[torch.dtype] = [
    torch.float16,
    torch.bfloat16,
    torch.float32,
    torch.float64,
    torch.int16,
    torch.int32,
    torch.int64,
    torch.complex32,
    torch.complex64,
    torch.complex128,
    torch.bool,
    torch.uint8,
    torch.int8,
    torch.float8_e4m3fn,
    torch.float8_e5m2,
]


def _default_device():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


class TensorMetadata:
    """``shape`` excludes the leading micro-batch dim, as in the reference."""

    MAX_SIZE = 16

    def __init__(self, t: torch.Tensor | None = None, *, shape: Sequence[int] | None = None, dtype=None, device=None):
        if t is not None:
            shape, dtype = list(t.shape), t.dtype
        self.shape = list(shape or [])
        self.dtype = dtype or torch.float32
        self.device = device if device is not None else _default_device()

    # wire format ------------------------------------------------------------
    def to_tensor(self, device=None) -> torch.Tensor:
        if len(self.shape) + 2 > self.MAX_SIZE:
            raise ValueError(f"at most {self.MAX_SIZE - 2} dims can be described")
        rec = [DTYPES.index(self.dtype), len(self.shape), *self.shape]
        rec += [0] * (self.MAX_SIZE - len(rec))
        return torch.tensor(rec, dtype=torch.int64, device=device if device is not None else self.device)

    @staticmethod
    def from_tensor(t: torch.Tensor, device=None) -> "TensorMetadata":
        assert t.dim() == 1, "Metadata should only have one dimension"
        rec = [int(v) for v in t.tolist()]
        ndim = rec[1]
        return TensorMetadata(shape=rec[2 : 2 + ndim], dtype=DTYPES[rec[0]], device=device)

    # buffers ------------------------------------------------------------------
    def get_buffer(self, batch_size: int) -> torch.Tensor:
        return torch.empty((batch_size, *self.shape), dtype=self.dtype, device=self.device)

    def nbytes(self, batch_size: int = 1) -> int:
        n = batch_size
        for s in self.shape:
            n *= s
        return n * torch.empty(0, dtype=self.dtype).element_size()

    def __eq__(self, other) -> bool:
        return isinstance(other, TensorMetadata) and self.shape == other.shape and self.dtype == other.dtype

    def __repr__(self) -> str:
        return f"TensorMetadata({self.shape}, {self.dtype})"
