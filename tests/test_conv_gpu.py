"""GPU parity, convolution forward in the three dataflows, against the fp64 oracle, the golden
fixtures (reference CPU conv + dense conv3d) and BASELINE config 1.

Tolerances (relative L2 against the fp64 oracle on the same inputs):
  fp32 inputs, exact fp32 math : 1e-5
  fp32 inputs, TF32 multiply    : 2e-3 (10-bit mantissa operands, fp32 accumulation)
  fp16 / bf16 inputs           : 2e-3 (fp16), 1.6e-2 (bf16, 8-bit mantissa)
"""
import numpy as np
import pytest
import torch

from conftest import random_coords, rel_l2
from oracle import kmap_oracle as ko

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}
GOLDEN_CASES = [("k3s1", 3, 1), ("k2s2", 2, 2), ("k3s2", 3, 2), ("k131s121", (1, 3, 1), (1, 2, 1)), ("k2s1", 2, 1),
                ("k5s1", 5, 1), ("k3s3", 3, 3)]


def _cfg(dataflow, ifsort=False, split=1):
    from torchsparse_b200.nn import functional as F

    cfg = F.conv_config.get_default_conv_config()
    cfg.dataflow = getattr(F.Dataflow, dataflow)
    cfg.ifsort = ifsort
    cfg.split_mask_num = split
    return cfg


def _sparse_conv(coords, feats, w, ks, st, dataflow, dtype, ifsort=False, split=1, bias=None):
    import torchsparse_b200 as ts
    from torchsparse_b200.nn import functional as F

    x = ts.SparseTensor(torch.from_numpy(feats).cuda().to(dtype), torch.from_numpy(coords).cuda())
    pad = tuple((k - 1) // 2 if (k % 2 == 1 and s == 1) else 0 for k, s in zip(ko._as3(ks), ko._as3(st)))
    wt = torch.from_numpy(w).cuda().to(dtype)
    return x, F.conv3d(x, wt, ks, bias, st, pad, config=_cfg(dataflow, ifsort, split))


@pytest.mark.parametrize("name,ks,st", GOLDEN_CASES)
@pytest.mark.parametrize("dataflow", ["ImplicitGEMM", "GatherScatter", "FetchOnDemand"])
def test_golden_fp32(golden, name, ks, st, dataflow):
    """fp32, exact math: equals the reference's CPU conv and the dense conv3d of the fixture."""
    from torchsparse_b200.nn import functional as F

    coords, feats, w = golden[f"{name}/coords"], golden[f"{name}/feats"], golden[f"{name}/weight"]
    x, y = _sparse_conv(coords, feats, w, ks, st, dataflow, torch.float32)
    assert np.array_equal(y.coords.cpu().numpy(), golden[f"{name}/out_coords"])
    out = y.feats.cpu().numpy()
    assert rel_l2(out, golden[f"{name}/ref_cpu_out"]) < 1e-5
    assert rel_l2(out, golden[f"{name}/dense_out"]) < 1e-5
    if f"{name}/t_feats" in golden:   # transposed conv through the cached map
        import torchsparse_b200 as ts
        xt = ts.SparseTensor(torch.from_numpy(golden[f"{name}/t_feats"]).cuda(), y.coords, stride=y.stride)
        xt._caches = x._caches
        yt = F.conv3d(xt, torch.from_numpy(golden[f"{name}/t_weight"]).cuda(), ks, None, st, 0,
                      config=_cfg(dataflow), transposed=True)
        assert torch.equal(yt.coords, x.coords)
        assert rel_l2(yt.feats.cpu().numpy(), golden[f"{name}/t_ref_cpu_out"]) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("dataflow,ifsort,split", [("ImplicitGEMM", False, 1), ("ImplicitGEMM", True, 1),
                                                    ("ImplicitGEMM", True, 3), ("GatherScatter", False, 1),
                                                    ("FetchOnDemand", False, 1)])
@pytest.mark.parametrize("ks,st,cin,cout", [(3, 1, 32, 32), (3, 1, 64, 96), (2, 2, 32, 64), (3, 2, 16, 16),
                                            (3, 1, 4, 32), (3, 1, 5, 19), (3, 1, 128, 128), (3, 1, 256, 256),
                                            (3, 1, 384, 256), (3, 1, 72, 40), (5, 1, 16, 32)])
def test_conv_vs_oracle(dtype, dataflow, ifsort, split, ks, st, cin, cout):
    if ifsort and -(-int(np.prod(ko._as3(ks))) // split) > 31:
        pytest.skip("a row's offset bitmask is one int32 per split (as in the reference): 31 offsets per split")
    rng = np.random.default_rng(cin * 1000 + cout)
    coords = random_coords(rng, 1500, (16, 16, 16), 2)
    feats = rng.standard_normal((coords.shape[0], cin)).astype(np.float32)
    kvol = int(np.prod(ko._as3(ks)))
    w = (rng.standard_normal((kvol, cin, cout)) * np.sqrt(2.0 / (kvol * cin))).astype(np.float32)
    # the oracle sees exactly the rounded inputs the kernel sees
    f_r = torch.from_numpy(feats).to(dtype).float().numpy()
    w_r = torch.from_numpy(w).to(dtype).float().numpy()
    pad = tuple((k - 1) // 2 if (k % 2 == 1 and s == 1) else 0 for k, s in zip(ko._as3(ks), ko._as3(st)))
    km = ko.build_kmap(coords, ks, st, pad)
    want = ko.conv_from_map(f_r, w_r, km["out_in_map"], km["sizes"][1])
    _, y = _sparse_conv(coords, feats, w, ks, st, dataflow, dtype, ifsort, split)
    assert y.feats.dtype == dtype and y.feats.shape == want.shape
    assert rel_l2(y.feats.float().cpu().numpy(), want) < TOL[dtype]


@pytest.mark.parametrize("dataflow,ifsort", [("ImplicitGEMM", False), ("ImplicitGEMM", True),
                                             ("GatherScatter", False), ("FetchOnDemand", False)])
@pytest.mark.parametrize("ks,st,cin,cout", [(3, 1, 32, 32), (3, 1, 64, 96), (2, 2, 32, 64), (3, 1, 36, 40),
                                            (3, 1, 256, 256), (3, 1, 4, 32)])
def test_conv_tf32_vs_oracle(dataflow, ifsort, ks, st, cin, cout):
    """fp32 tensors with backends.allow_tf32 (the reference's default on Ampere and newer): the
    GEMMs multiply on the tensor cores as TF32 and accumulate in fp32 (fetch-on-demand only from
    128 x 128 channels up; below that it stays exact)."""
    from torchsparse_b200 import backends

    rng = np.random.default_rng(cin * 1000 + cout + 7)
    coords = random_coords(rng, 1500, (16, 16, 16), 2)
    feats = rng.standard_normal((coords.shape[0], cin)).astype(np.float32)
    kvol = int(np.prod(ko._as3(ks)))
    w = (rng.standard_normal((kvol, cin, cout)) * np.sqrt(2.0 / (kvol * cin))).astype(np.float32)
    pad = tuple((k - 1) // 2 if (k % 2 == 1 and s == 1) else 0 for k, s in zip(ko._as3(ks), ko._as3(st)))
    km = ko.build_kmap(coords, ks, st, pad)
    want = ko.conv_from_map(feats, w, km["out_in_map"], km["sizes"][1])
    backends.allow_tf32 = True       # restored by the autouse fixture
    _, y = _sparse_conv(coords, feats, w, ks, st, dataflow, torch.float32, ifsort)
    assert y.feats.dtype == torch.float32 and y.feats.shape == want.shape
    err = rel_l2(y.feats.cpu().numpy(), want)
    assert err < 2e-3
    on_tensor_cores = cin % 4 == 0 and cout % 8 == 0 and (dataflow != "FetchOnDemand" or cin * cout >= 128 * 128)
    if on_tensor_cores:
        assert err > 1e-6            # the tensor-core path ran (exact fp32 would be ~1e-7)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 4e-3)])
@pytest.mark.parametrize("dataflow", ["ImplicitGEMM", "GatherScatter", "FetchOnDemand"])
@pytest.mark.parametrize("ks,st,cin,cout", [(3, 1, 32, 48), (2, 2, 32, 64), (3, 2, 16, 16), (3, 1, 5, 19)])
def test_conv_backward_vs_oracle(dtype, tol, dataflow, ks, st, cin, cout):
    """Input and weight gradients of a single layer against the fp64 oracle (fp16: both gradients are
    rounded to fp16, the weight gradient after a sum over ~10^3 pairs, hence the wider bound)."""
    import torchsparse_b200 as ts
    from torchsparse_b200.nn import functional as F

    rng = np.random.default_rng(cin * 100 + cout + 3)
    coords = random_coords(rng, 1200, (14, 14, 14), 2)
    n = coords.shape[0]
    feats = rng.standard_normal((n, cin)).astype(np.float32)
    kvol = int(np.prod(ko._as3(ks)))
    w = (rng.standard_normal((kvol, cin, cout)) * np.sqrt(2.0 / (kvol * cin))).astype(np.float32)
    pad = tuple((k - 1) // 2 if (k % 2 == 1 and s == 1) else 0 for k, s in zip(ko._as3(ks), ko._as3(st)))
    km = ko.build_kmap(coords, ks, st, pad)
    m = km["sizes"][1]
    gy = rng.standard_normal((m, cout)).astype(np.float32)
    f_r = torch.from_numpy(feats).to(dtype).float().numpy()
    w_r = torch.from_numpy(w).to(dtype).float().numpy()
    g_r = torch.from_numpy(gy).to(dtype).float().numpy()
    want_dx, want_dw = ko.conv_backward_from_map(f_r, w_r, km["out_in_map"], m, g_r)

    x_feats = torch.from_numpy(feats).cuda().to(dtype).requires_grad_(True)
    wt = torch.from_numpy(w).cuda().to(dtype).requires_grad_(True)
    x = ts.SparseTensor(x_feats, torch.from_numpy(coords).cuda())
    y = F.conv3d(x, wt, ks, None, st, pad, config=_cfg(dataflow))
    assert y.feats.requires_grad and y.feats.shape == (m, cout)
    y.feats.backward(torch.from_numpy(gy).cuda().to(dtype))
    assert x_feats.grad.dtype == dtype and wt.grad.dtype == dtype
    assert rel_l2(x_feats.grad.float().cpu().numpy(), want_dx) < tol
    assert rel_l2(wt.grad.float().cpu().numpy(), want_dw) < tol


def test_transposed_conv_backward_vs_oracle():
    """Strided conv followed by its transposed conv, gradients through both (fp32, exact arithmetic)."""
    import torchsparse_b200 as ts
    from torchsparse_b200.nn import functional as F

    rng = np.random.default_rng(77)
    coords = random_coords(rng, 1000, (12, 12, 12))
    n = coords.shape[0]
    feats = rng.standard_normal((n, 16)).astype(np.float32)
    w1 = (rng.standard_normal((8, 16, 24)) * 0.2).astype(np.float32)
    w2 = (rng.standard_normal((8, 24, 8)) * 0.2).astype(np.float32)
    km = ko.build_kmap(coords, 2, 2, 0)
    m = km["sizes"][1]
    map_t = ko.transpose_map(km["out_in_map"], (n + 127) // 128 * 128)
    gy = rng.standard_normal((n, 8)).astype(np.float32)
    # oracle: h = conv(x, w1, map); y = conv(h, w2, map_t)
    h = ko.conv_from_map(feats, w1, km["out_in_map"], m)
    want_dh, want_dw2 = ko.conv_backward_from_map(h, w2, map_t, n, gy)
    want_dx, want_dw1 = ko.conv_backward_from_map(feats, w1, km["out_in_map"], m, want_dh)

    xf = torch.from_numpy(feats).cuda().requires_grad_(True)
    t1 = torch.from_numpy(w1).cuda().requires_grad_(True)
    t2 = torch.from_numpy(w2).cuda().requires_grad_(True)
    x = ts.SparseTensor(xf, torch.from_numpy(coords).cuda())
    hh = F.conv3d(x, t1, 2, None, 2, 0)
    yy = F.conv3d(hh, t2, 2, None, 2, 0, transposed=True)
    assert yy.feats.shape == (n, 8)
    yy.feats.backward(torch.from_numpy(gy).cuda())
    assert rel_l2(xf.grad.cpu().numpy(), want_dx) < 1e-5
    assert rel_l2(t1.grad.cpu().numpy(), want_dw1) < 1e-5
    assert rel_l2(t2.grad.cpu().numpy(), want_dw2) < 1e-5


def test_baseline_config1_all_dataflows():
    """BASELINE config 1: 20 000 voxels in [0,128)^3, 32->32, k3 s1, fp32, batch 1."""
    rng = np.random.default_rng(0)
    coords = random_coords(rng, 20000, (128, 128, 128))
    feats = rng.standard_normal((20000, 32)).astype(np.float32)
    w = (rng.standard_normal((27, 32, 32)) * np.sqrt(2.0 / (27 * 32))).astype(np.float32)
    km = ko.build_kmap(coords, 3, 1, 1)
    want = ko.conv_from_map(feats, w, km["out_in_map"], 20000)
    for df in ("ImplicitGEMM", "GatherScatter", "FetchOnDemand"):
        x, y = _sparse_conv(coords, feats, w, 3, 1, df, torch.float32)
        assert rel_l2(y.feats.cpu().numpy(), want) < 1e-5
    kmap = x._caches.kmaps[((1, 1, 1), (3, 3, 3), (1, 1, 1), (1, 1, 1))]
    assert np.array_equal(kmap["out_in_map"].cpu().numpy(), km["out_in_map"])


def test_reference_style_dense_equivalence_fp16():
    """The reference's own test (tests/python/test_single_layer_conv.py:111-220, thresholds
    tests/test.py:40-41): 5^3 grid, 20 voxels, 16->32, fp16, kernel {2,3,5} x stride {1,2,3}, against a dense
    convolution whose output is rounded to fp16 as the reference's dense fp16 model rounds it; its metrics,
    averaged over the runs: sum |diff| / rows <= 1e-4 and max |diff| / mean |out| <= 1e-2.

    Both sides round the same sums (fp32 accumulation here, fp64 there) to fp16, so they differ only where a sum
    sits within accumulation error of an fp16 rounding boundary: a handful of 1-ulp flips (ulp 2^-9..2^-7 at these
    magnitudes) over the 9 x 640 outputs.  The reference's bound on the first metric allows about five such flips;
    the bound asserted here is 1e-3 (about fifty), stated rather than borrowed, because the count of flips
    depends on the accumulation order of the tensor cores, which is not specified."""
    rng = np.random.default_rng(0)
    madiffs, rdiffs = [], []
    for ks in (2, 3, 5):
        for st in (1, 2, 3):
            coords = random_coords(rng, 20, (5, 5, 5))
            feats = rng.uniform(-1, 1, (20, 16)).astype(np.float16).astype(np.float32)
            w = rng.uniform(-1, 1, (ks ** 3, 16, 32)).astype(np.float16).astype(np.float32)
            pad = (ks - 1) // 2 if ks % 2 == 1 else 0
            _, y = _sparse_conv(coords, feats, w, ks, st, "ImplicitGEMM", torch.float16)
            km = ko.build_kmap(coords, ks, st, ko._as3(pad if st == 1 else 0))
            want = ko.conv_from_map(feats, w, km["out_in_map"], km["sizes"][1])
            if want.shape[0] == 0:
                continue
            want = want.astype(np.float16).astype(np.float64)          # the dense fp16 model's output
            got = y.feats.float().cpu().numpy()
            madiffs.append(np.abs(got - want).sum() / want.shape[0])
            rdiffs.append(np.abs(got - want).max() / max(np.abs(got).mean(), 1e-9))
    assert np.mean(madiffs) <= 1e-3 and np.mean(rdiffs) <= 1e-2, (np.mean(madiffs), np.mean(rdiffs))


def test_fused_epilogue_and_bias():
    from torchsparse_b200 import backend

    rng = np.random.default_rng(23)
    coords = random_coords(rng, 2000, (20, 20, 20))
    km = ko.build_kmap(coords, 3, 1, 1)
    for dtype, cin, cout in ((torch.float32, 24, 40), (torch.float16, 64, 64)):
        feats = rng.standard_normal((2000, cin)).astype(np.float32)
        w = (rng.standard_normal((27, cin, cout)) / np.sqrt(27 * cin)).astype(np.float32)
        bias = rng.standard_normal(cout).astype(np.float32)
        res = rng.standard_normal((2000, cout)).astype(np.float32)
        f_r = torch.from_numpy(feats).to(dtype).float().numpy()
        w_r = torch.from_numpy(w).to(dtype).float().numpy()
        r_r = torch.from_numpy(res).to(dtype).float().numpy()
        want = np.maximum(ko.conv_from_map(f_r, w_r, km["out_in_map"], 2000) + bias + r_r, 0)
        got = backend.conv_forward_implicit_gemm_cuda(
            torch.from_numpy(feats).cuda().to(dtype), torch.from_numpy(w).cuda().to(dtype),
            torch.from_numpy(km["out_in_map"]).cuda(), 2000, cout, False, True,
            bias=torch.from_numpy(bias).cuda(), residual=torch.from_numpy(res).cuda().to(dtype), relu=True)
        assert rel_l2(got.float().cpu().numpy(), want) < TOL[dtype]


def test_large_layer_linearity_property():
    """BASELINE layer-sweep size (1M voxels, 64->64, fp16): conv(a*x1 + x2) == a*conv(x1) + conv(x2)
    within fp16 rounding, and an all -1 map gives zeros."""
    import torchsparse_b200 as ts
    from torchsparse_b200.nn import functional as F

    rng = np.random.default_rng(29)
    n = 1_000_000
    coords = torch.from_numpy(random_coords(rng, n, (171, 171, 171))).cuda()
    g = torch.Generator(device="cuda").manual_seed(1)
    x1 = torch.randn(n, 64, device="cuda", generator=g)
    x2 = torch.randn(n, 64, device="cuda", generator=g)
    w = (torch.randn(27, 64, 64, device="cuda", generator=g) * (2.0 / (27 * 64)) ** 0.5).half()
    t = ts.SparseTensor(x1.half(), coords)
    y1 = F.conv3d(t, w, 3, None, 1, 1).feats.float()
    t2 = ts.SparseTensor(x2.half(), coords); t2._caches = t._caches
    y2 = F.conv3d(t2, w, 3, None, 1, 1).feats.float()
    t3 = ts.SparseTensor((0.5 * x1.half().float() + x2.half().float()).half(), coords); t3._caches = t._caches
    y3 = F.conv3d(t3, w, 3, None, 1, 1).feats.float()
    err = (y3 - (0.5 * y1 + y2)).norm() / y3.norm()
    assert float(err) < 3e-3
    from torchsparse_b200 import backend
    empty_map = torch.full((128, 27), -1, dtype=torch.int32, device="cuda")
    z = backend.conv_forward_implicit_gemm_cuda(x1[:100].half(), w, empty_map, 100, 64)
    assert float(z.abs().max()) == 0.0
