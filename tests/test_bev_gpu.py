"""GPU parity of the bird's-eye-view heads against their CPU restatement (oracle/bev_oracle.py)."""
import numpy as np
import pytest
import torch

from conftest import random_coords, rel_l2
from oracle import bev_oracle as bo

pytestmark = pytest.mark.gpu


def _tensor(rng, n, shape, batch, channels, stride=1, dtype=torch.float32):
    from torchsparse_b200 import SparseTensor

    coords = random_coords(rng, n, shape, batch) * np.array([1, stride, stride, stride], dtype=np.int32)
    feats = rng.standard_normal((coords.shape[0], channels)).astype(np.float32)
    x = SparseTensor(torch.from_numpy(feats).cuda().to(dtype), torch.from_numpy(coords).cuda(), (stride,) * 3)
    return x, coords, feats


@pytest.mark.parametrize("dim", [0, 1, 2])
def test_bev_reduction(dim):
    from torchsparse_b200 import nn as spnn

    rng = np.random.default_rng(3 + dim)
    x, coords, feats = _tensor(rng, 700, (12, 9, 7), 2, 16)
    out = spnn.ToBEVReduction(dim)(x)
    want_c, want_f = bo.bev_reduction(coords, feats, dim)
    assert np.array_equal(out.coords.cpu().numpy(), want_c)
    assert rel_l2(out.feats.float().cpu().numpy(), want_f) < 1e-5
    assert out.stride == x.stride


@pytest.mark.parametrize("dim,stride,tstride,bias", [(1, 1, 1, False), (2, 1, 2, True), (1, 2, 1, True), (0, 2, 2, False)])
def test_bev_convolution_forward_and_gradients(dim, stride, tstride, bias):
    from torchsparse_b200 import backends, nn as spnn

    rng = np.random.default_rng(11 + dim + stride)
    shape = (10, 9, 8)
    x, coords, feats = _tensor(rng, 500, shape, 2, 16, tstride)
    layer = spnn.ToBEVConvolution(16, 24, shape[dim], stride=stride, dim=dim, bias=bias).cuda()
    if bias:
        with torch.no_grad():
            layer.bias.uniform_(-0.5, 0.5)
    old = backends.allow_tf32
    backends.allow_tf32 = False
    try:
        x.feats.requires_grad_(True)
        out = layer(x)
        kernel = layer.kernel.detach().cpu().numpy()
        b = layer.bias.detach().cpu().numpy() if bias else None
        want_c, want_f, ratio = bo.bev_convolution(coords, feats, (tstride,) * 3, kernel, b, dim, stride)
        assert np.array_equal(out.coords.cpu().numpy(), want_c)
        assert tuple(out.stride) == ratio
        assert rel_l2(out.feats.detach().cpu().numpy(), want_f) < 1e-5
        # gradients against the same sum written with torch ops
        g = torch.from_numpy(rng.standard_normal(out.feats.shape).astype(np.float32)).cuda()
        out.feats.backward(g)
        k = torch.from_numpy(coords[:, dim + 1] // tstride).long().cuda()
        cell_of = {tuple(c): i for i, c in enumerate(want_c)}
        cc = coords.copy()
        cc[:, dim + 1] = 0
        if stride > 1:
            cc[:, 1:] = cc[:, 1:] // (tstride * stride) * (tstride * stride)
        inv = torch.tensor([cell_of[tuple(c)] for c in cc]).cuda()
        xf = torch.from_numpy(feats).cuda().requires_grad_(True)
        kw = layer.kernel.detach().clone().requires_grad_(True)
        ref = torch.zeros_like(out.feats).index_add(0, inv, torch.einsum("nc,nco->no", xf, kw[k]))
        ref.backward(g)
        assert rel_l2(x.feats.grad.cpu().numpy(), xf.grad.cpu().numpy()) < 1e-5
        assert rel_l2(layer.kernel.grad.cpu().numpy(), kw.grad.cpu().numpy()) < 1e-5
    finally:
        backends.allow_tf32 = old


def test_bev_convolution_fp16_many_layers_runs_on_the_conv_kernels():
    """41 height layers (more than the tensor-core kernel's 32 offsets) and fp16 features."""
    from torchsparse_b200 import nn as spnn

    rng = np.random.default_rng(5)
    x, coords, feats = _tensor(rng, 4000, (30, 41, 30), 1, 32, dtype=torch.float16)
    layer = spnn.ToBEVConvolution(32, 64, 41, dim=1).cuda().half()
    out = layer(x)
    kernel = layer.kernel.detach().float().cpu().numpy()
    want_c, want_f, _ = bo.bev_convolution(coords, x.feats.float().cpu().numpy(), (1, 1, 1), kernel, None, 1, 1)
    assert np.array_equal(out.coords.cpu().numpy(), want_c)
    assert rel_l2(out.feats.detach().float().cpu().numpy(), want_f) < 2e-3


@pytest.mark.parametrize("dim,offset,bias", [(1, (0, 0, 0), False), (2, (2, 1, 0), True)])
def test_dense_bev_convolution_and_height_compression(dim, offset, bias):
    from torchsparse_b200 import backends, nn as spnn

    rng = np.random.default_rng(17 + dim)
    shape = (11, 9, 6)
    x, coords, feats = _tensor(rng, 400, (13, 10, 6) if dim == 2 else shape, 2, 8)
    old = backends.allow_tf32
    backends.allow_tf32 = False
    try:
        layer = spnn.ToDenseBEVConvolution(8, 16, shape, offset, dim, bias).cuda()
        if bias:
            with torch.no_grad():
                layer.bias.uniform_(-0.5, 0.5)
        out = layer(x)
        b = layer.bias.detach().cpu().numpy() if bias else None
        want = bo.dense_bev_convolution(coords, feats, (1, 1, 1), layer.kernel.detach().cpu().numpy(), b, shape, offset,
                                        dim)
        assert tuple(out.shape) == want.shape
        assert rel_l2(out.detach().cpu().numpy(), want) < 1e-5
    finally:
        backends.allow_tf32 = old
    # a map two layers lower than the tensor: the voxels above it share its top layer
    low = tuple(v - 2 if a == dim else v for a, v in enumerate(shape))
    hc = spnn.ToBEVHeightCompression(8, low, offset, dim).cuda()
    x.feats.requires_grad_(True)
    got = hc(x)
    want = bo.bev_height_compression(coords, feats, (1, 1, 1), low, offset, dim)
    assert tuple(got.shape) == want.shape
    assert rel_l2(got.detach().cpu().numpy(), want) < 1e-6
    got.sum().backward()
    assert x.feats.grad is not None and bool(torch.isfinite(x.feats.grad).all())
