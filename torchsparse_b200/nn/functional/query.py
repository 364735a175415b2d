import torch

from ... import backend

__all__ = ["sphashquery"]


def sphashquery(queries: torch.Tensor, references: torch.Tensor) -> torch.Tensor:
    """Index of each query hash inside ``references`` (-1 when absent), same shape as
    ``queries`` (torchsparse/nn/functional/query.py:8-37)."""
    sizes = queries.size()
    out = backend.hash_query_cuda(queries.contiguous().view(-1), references.contiguous())
    return (out - 1).view(*sizes)
