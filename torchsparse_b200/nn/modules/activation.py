"""Activation modules that act on the feature matrix of a SparseTensor
(torchsparse/nn/modules/activation.py)."""
from torch import nn

from ..utils import fapply

__all__ = ["ReLU", "LeakyReLU", "SiLU"]


def _featurewise(dense_cls, name: str):
    """Subclass of a torch activation whose forward maps the features and keeps coordinates,
    stride and the kernel-map cache; constructor arguments are the dense module's."""

    def forward(self, input):
        return fapply(input, lambda feats: dense_cls.forward(self, feats))

    return type(name, (dense_cls,), {"forward": forward, "__doc__": f"``torch.nn.{name}`` on SparseTensor features."})


ReLU = _featurewise(nn.ReLU, "ReLU")
LeakyReLU = _featurewise(nn.LeakyReLU, "LeakyReLU")
SiLU = _featurewise(nn.SiLU, "SiLU")
