"""Small argument helpers (torchsparse/utils/utils.py:9-33)."""
from functools import lru_cache
from typing import List, Tuple, Union

import torch

__all__ = ["make_ntuple", "make_tensor", "make_divisible"]


def make_ntuple(x: Union[int, List[int], Tuple[int, ...], torch.Tensor], ndim: int) -> Tuple[int, ...]:
    """``ndim`` ints from an int (repeated), a list / tuple or a tensor (a device tensor costs a read)."""
    if type(x) is tuple and len(x) == ndim and all(type(v) is int for v in x):
        return x                                  # the common case on the hot path: already canonical
    if isinstance(x, torch.Tensor):
        x = x.reshape(-1).tolist()
    values = (int(x),) * ndim if isinstance(x, int) else tuple(int(v) for v in x)
    if len(values) != ndim:
        raise AssertionError(f"expected {ndim} values, got {values}")
    return values


@lru_cache()
def make_tensor(x: Tuple[int, ...], dtype: torch.dtype, device) -> torch.Tensor:
    """A small constant tensor; one instance per (values, dtype, device)."""
    return torch.tensor(x, dtype=dtype, device=device)


def make_divisible(x: int, divisor: int) -> int:
    """x rounded up to a multiple of divisor."""
    return -(-x // divisor) * divisor
