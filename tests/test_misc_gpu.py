"""GPU checks of smaller pieces: gradients of the point <-> voxel operators against torch autograd of the same
sums, weight-cache invalidation of the tensor-core path, the output gather's row counts, convolutions on a
second device of one process."""
import numpy as np
import pytest
import torch

from conftest import random_coords, rel_l2
from oracle import kmap_oracle as ko

pytestmark = pytest.mark.gpu


def test_voxelize_and_devoxelize_gradients():
    from torchsparse_b200.nn import functional as F

    rng = np.random.default_rng(3)
    n, nv, c = 5000, 700, 24
    idx = torch.from_numpy(rng.integers(0, nv, n).astype(np.int32)).cuda()
    counts = torch.bincount(idx.long(), minlength=nv).int()
    x = torch.from_numpy(rng.standard_normal((n, c)).astype(np.float32)).cuda().requires_grad_()
    g = torch.from_numpy(rng.standard_normal((nv, c)).astype(np.float32)).cuda()
    y = F.spvoxelize(x, idx, counts)
    y.backward(g)
    xr = x.detach().clone().requires_grad_()
    want = torch.zeros(nv, c, device="cuda").index_add(0, idx.long(), xr) / counts.clamp(min=1)[:, None]
    want.backward(g)
    assert rel_l2(y.detach().cpu().numpy(), want.detach().cpu().numpy()) < 1e-5
    assert rel_l2(x.grad.cpu().numpy(), xr.grad.cpu().numpy()) < 1e-6

    ind = rng.integers(-1, nv, (n, 8)).astype(np.int32)
    w = rng.uniform(0, 1, (n, 8)).astype(np.float32)
    w[ind < 0] = 0
    ind_t, w_t = torch.from_numpy(ind).cuda(), torch.from_numpy(w).cuda()
    v = torch.from_numpy(rng.standard_normal((nv, c)).astype(np.float32)).cuda().requires_grad_()
    gp = torch.from_numpy(rng.standard_normal((n, c)).astype(np.float32)).cuda()
    out = F.spdevoxelize(v, ind_t, w_t)
    out.backward(gp)
    vr = v.detach().clone().requires_grad_()
    want = (vr[ind_t.clamp(min=0).long()] * w_t[:, :, None]).sum(1)
    want.backward(gp)
    assert rel_l2(out.detach().cpu().numpy(), want.detach().cpu().numpy()) < 1e-5
    assert rel_l2(v.grad.cpu().numpy(), vr.grad.cpu().numpy()) < 1e-5


def test_weights_changed_in_place_reach_the_tensor_core_path():
    """Packed weight copies are rebuilt after an in-place update through torch (version counter), after
    Conv3d.reset_parameters(), and after FusedConv.invalidate() for writes the counter does not see."""
    import torchsparse_b200 as ts
    from torchsparse_b200 import nn as spnn
    from torchsparse_b200.nn import FusedConv

    rng = np.random.default_rng(5)
    coords = random_coords(rng, 3000, (24, 24, 24))
    feats = rng.standard_normal((3000, 32)).astype(np.float32)
    km = ko.build_kmap(coords, 3, 1, 1)
    conv = spnn.Conv3d(32, 64, 3).cuda().half()

    def check(layer, kernel):
        x = ts.SparseTensor(torch.from_numpy(feats).cuda().half(), torch.from_numpy(coords).cuda())
        with torch.no_grad():
            y = layer(x)
        want = ko.conv_from_map(torch.from_numpy(feats).half().float().numpy(), kernel.detach().float().cpu().numpy(),
                                km["out_in_map"], 3000)
        assert rel_l2(y.feats.float().cpu().numpy(), want) < 2e-3

    check(conv, conv.kernel)
    with torch.no_grad():
        conv.kernel.mul_(-0.5)                      # in place through torch
    check(conv, conv.kernel)
    conv.reset_parameters()
    check(conv, conv.kernel)
    fused = FusedConv(conv).cuda()
    check(fused, fused.kernel)
    fused.kernel.data.copy_(torch.randn_like(fused.kernel) * 0.05)      # invisible to the version counter
    fused.invalidate()
    check(fused, fused.kernel)


def test_padded_gather_counts_of_back_to_back_calls():
    """Two gathers queued behind a long-running kernel keep their own row counts."""
    from torchsparse_b200.sharding import PaddedGather

    pg = PaddedGather(64, 4, torch.float32, torch.device("cuda", 0))
    a, b = torch.ones(10, 4, device="cuda"), torch.full((37, 4), 2.0, device="cuda")
    torch.cuda._sleep(20_000_000)                   # ~10 ms: both calls are queued before either runs
    _, c1 = pg(a)
    c1 = c1.clone()
    buf, c2 = pg(b)
    torch.cuda.synchronize()
    assert int(c1[0]) == 10 and int(c2[0]) == 37
    assert bool((buf[0, :37] == 2.0).all())
    n_dev = torch.tensor([5], dtype=torch.int32, device="cuda")
    full = torch.full((64, 4), 3.0, device="cuda")
    buf, c3 = pg(full, n_dev)
    torch.cuda.synchronize()
    assert int(c3[0]) == 5 and bool((buf[0] == 3.0).all())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_convolution_on_a_second_device_of_one_process():
    from torchsparse_b200 import backend

    rng = np.random.default_rng(7)
    coords = random_coords(rng, 2000, (20, 20, 20))
    km = ko.build_kmap(coords, 3, 1, 1)
    f = torch.from_numpy(rng.standard_normal((2000, 96)).astype(np.float32)).half()
    w = torch.from_numpy((rng.standard_normal((27, 96, 96)) / 50).astype(np.float32)).half()
    want = ko.conv_from_map(f.float().numpy(), w.float().numpy(), km["out_in_map"], 2000)
    for dev in (0, 1):
        with torch.cuda.device(dev):
            y = backend.conv_forward_implicit_gemm_cuda(f.cuda(dev), w.cuda(dev), torch.from_numpy(km["out_in_map"]).cuda(dev),
                                                        2000, 96)
            assert rel_l2(y.float().cpu().numpy(), want) < 2e-3


@pytest.mark.parametrize("transpose", [False, True])
def test_gather_scatter_backward_entry_fills_callers_buffers(transpose):
    """`conv_backward_gather_scatter_cuda` with the reference's argument list
    (torchsparse/nn/functional/conv/func/gather_scatter.py:116): the caller's zero-filled gradient tensors are
    written in place; checked against the fp64 oracle."""
    from torchsparse_b200 import backend

    rng = np.random.default_rng(91)
    coords = random_coords(rng, 900, (12, 12, 12))
    n, cin, cout = coords.shape[0], 16, 24
    km = ko.build_kmap(coords, 2, 2, 0)
    m = km["sizes"][1]
    nbmaps, nbsizes = ko.pairs_from_map(km["out_in_map"])
    if transpose:                       # the pair list of the strided layer, used from its outputs to its inputs
        n_in, n_out, omap = m, n, ko.transpose_map(km["out_in_map"], ko.pad_rows(n))
    else:
        n_in, n_out, omap = n, m, km["out_in_map"]
    feats = rng.standard_normal((n_in, cin)).astype(np.float32)
    w = (rng.standard_normal((8, cin, cout)) * 0.2).astype(np.float32)
    gy = rng.standard_normal((n_out, cout)).astype(np.float32)
    want_dx, want_dw = ko.conv_backward_from_map(feats, w, omap, n_out, gy)

    x = torch.from_numpy(feats).cuda()
    wt = torch.from_numpy(w).cuda()
    gx, gw = torch.zeros_like(x), torch.zeros_like(wt)
    backend.conv_backward_gather_scatter_cuda(x, gx, torch.from_numpy(gy).cuda(), wt, gw,
                                              torch.from_numpy(nbmaps).cuda(), torch.from_numpy(nbsizes), transpose)
    assert rel_l2(gx.cpu().numpy(), want_dx) < 1e-5
    assert rel_l2(gw.cpu().numpy(), want_dw) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n,cg,cd,ks", [(1500, 32, 48, 3), (4000, 96, 96, 3), (3000, 64, 256, 3), (2500, 256, 128, 3),
                                        (3000, 136, 320, 2), (900, 8, 16, 3)])
def test_tensor_core_weight_gradient_vs_oracle(dtype, n, cg, cd, ks):
    """tsb_conv_wgrad_igemm (tcgen05, both operands MN-major, row range divided among CTAs, fp32 atomic adds)
    against the fp64 oracle on 16-bit-rounded operands.  Tolerance: relative L2 <= 1e-5 on the fp32 result (fp32
    accumulation of exact 16-bit products; the order of the atomic adds moves the last bits only)."""
    from torchsparse_b200 import backend

    rng = np.random.default_rng(n + cg + cd)
    coords = random_coords(rng, n, (24, 24, 24), 2)
    n = coords.shape[0]
    st, pad = (1, 1) if ks == 3 else (2, 0)
    km = ko.build_kmap(coords, ks, st, pad)
    m = km["sizes"][1]
    x = torch.from_numpy(rng.standard_normal((n, cg)).astype(np.float32)).to(dtype)
    dy = torch.from_numpy(rng.standard_normal((m, cd)).astype(np.float32)).to(dtype)
    w0 = np.zeros((ks ** 3, cg, cd), dtype=np.float32)
    _, want = ko.conv_backward_from_map(x.float().numpy(), w0, km["out_in_map"], m, dy.float().numpy())
    got = backend.conv_wgrad_implicit_gemm_cuda(x.cuda(), dy.cuda(), torch.from_numpy(km["out_in_map"]).cuda())
    assert got.dtype == torch.float32 and got.shape == want.shape
    assert rel_l2(got.cpu().numpy(), want) < 1e-5
    # the reference-named entry on the transposed map returns the [Kvol, Cout, Cin] form
    map_t = torch.from_numpy(ko.transpose_map(km["out_in_map"], ko.pad_rows(n))).cuda()
    got_t = backend.conv_backward_wgrad_implicit_gemm_cuda(dy.cuda(), x.cuda(), map_t, 32)
    assert got_t.dtype == dtype and got_t.numel() == want.size
    assert rel_l2(got_t.float().reshape(ks ** 3, cd, cg).transpose(1, 2).cpu().numpy(), want) < 4e-3


def test_to_dense_gradient_and_group_norm():
    """`to_dense` is differentiable (gather of the dense gradient, torchsparse/utils/to_dense.py:41-64) and `GroupNorm`
    normalises every batch sample on its own (torchsparse/nn/modules/norm.py:25-57)."""
    import torchsparse_b200 as ts
    from torchsparse_b200 import nn as spnn
    from torchsparse_b200.utils.to_dense import to_dense

    rng = np.random.default_rng(5)
    coords = random_coords(rng, 300, (10, 9, 8), 2)
    n, c = coords.shape[0], 12
    feats = torch.from_numpy(rng.standard_normal((n, c)).astype(np.float32)).cuda().requires_grad_()
    ct = torch.from_numpy(coords).cuda()
    dense = to_dense(feats, ct, (2, 10, 9, 8))
    g = torch.from_numpy(rng.standard_normal(tuple(dense.shape)).astype(np.float32)).cuda()
    dense.backward(g)
    idx = ct.long()
    want = g[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]]
    assert torch.equal(feats.grad, want)
    assert torch.equal(dense[idx[:, 0], idx[:, 1], idx[:, 2], idx[:, 3]], feats.detach())

    gn = spnn.GroupNorm(4, c).cuda()
    with torch.no_grad():
        gn.weight.uniform_(0.5, 1.5)
        gn.bias.uniform_(-0.5, 0.5)
    with torch.no_grad():
        y = gn(ts.SparseTensor(feats.detach(), ct)).feats
        for b in range(2):
            rows = ct[:, 0] == b
            ref = torch.nn.functional.group_norm(feats.detach()[rows].t().unsqueeze(0), 4, gn.weight, gn.bias, gn.eps)
            assert rel_l2(y[rows].cpu().numpy(), ref.squeeze(0).t().cpu().numpy()) < 1e-6
