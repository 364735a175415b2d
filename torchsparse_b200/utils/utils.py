from functools import lru_cache
from itertools import repeat
from typing import List, Tuple, Union

import torch

__all__ = ["make_ntuple", "make_tensor", "make_divisible"]


def make_ntuple(x: Union[int, List[int], Tuple[int, ...], torch.Tensor], ndim: int) -> Tuple[int, ...]:
    """int / list / tuple / tensor -> tuple of ``ndim`` ints (torchsparse/utils/utils.py:9-21)."""
    if type(x) is tuple and len(x) == ndim and all(type(v) is int for v in x):
        return x
    if isinstance(x, int):
        x = tuple(repeat(x, ndim))
    elif isinstance(x, torch.Tensor):
        x = tuple(int(v) for v in x.view(-1).cpu().tolist())
    elif isinstance(x, (list, tuple)):
        x = tuple(int(v) for v in x)
    assert isinstance(x, tuple) and len(x) == ndim, x
    return x


@lru_cache()
def make_tensor(x: Tuple[int, ...], dtype: torch.dtype, device) -> torch.Tensor:
    return torch.tensor(x, dtype=dtype, device=device)


def make_divisible(x: int, divisor: int) -> int:
    return (x + divisor - 1) // divisor * divisor
