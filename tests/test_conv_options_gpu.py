"""GPU parity of the options of the tensor-core implicit-GEMM entry point (tsb_conv_igemm_run) against the
fp64 oracle: per-tile offset masks, the row-sorted column-major map, a two-matrix input (unwritten channel
concatenation), the map-less 1x1x1 form, chained offset ranges with fp32 partial sums, a row count held in
device memory, and the launch-configuration overrides.

Tolerance: relative L2 <= 2e-3 for fp16 operands (fp32 accumulation, one rounding), as for every fp16
convolution test of this suite."""
import numpy as np
import pytest
import torch

from conftest import random_coords, rel_l2
from oracle import kmap_oracle as ko

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _case(n=5000, shape=(40, 40, 40), cin=64, cout=96, seed=0, ks=3):
    rng = np.random.default_rng(seed)
    coords = random_coords(rng, n, shape)
    feats = rng.standard_normal((n, cin)).astype(np.float32)
    kvol = ks ** 3
    w = (rng.standard_normal((kvol, cin, cout)) / np.sqrt(kvol * cin)).astype(np.float32)
    km = ko.build_kmap(coords, ks, 1, (ks - 1) // 2)
    f16 = torch.from_numpy(feats).half()
    w16 = torch.from_numpy(w).half()
    want = ko.conv_from_map(f16.float().numpy(), w16.float().numpy(), km["out_in_map"], n)
    return coords, f16.cuda(), w16.cuda(), km, want


def test_tile_mask_matches_oracle():
    from torchsparse_b200 import backend

    _, _, _, km, _ = _case(n=3000)
    m = km["out_in_map"]
    n = km["sizes"][1]
    got = backend.tile_mask_cuda(torch.from_numpy(m).cuda(), n).cpu().numpy().astype(np.uint32)
    valid = (m >= 0)
    valid[n:] = False
    tiles = (n + 127) // 128
    want = np.array([sum(1 << k for k in np.nonzero(valid[t * 128:(t + 1) * 128].any(0))[0]) for t in range(tiles)],
                    dtype=np.uint32)
    assert np.array_equal(got[:tiles], want)
    # the same masks from a column-major copy of the map
    cm = torch.from_numpy(np.ascontiguousarray(m.T)).cuda()
    got_cm = backend.tile_mask_cuda(cm, n, 1, m.shape[0]).cpu().numpy().astype(np.uint32)
    assert np.array_equal(got_cm[:tiles], want)


def test_sorted_cm_artefacts_are_a_permutation_of_the_map():
    from torchsparse_b200 import backend

    _, _, _, km, _ = _case(n=3000)
    m = km["out_in_map"]
    n = km["sizes"][1]
    sm = backend.sorted_cm_artefacts_cuda(torch.from_numpy(m).cuda(), n, max_offsets=4)
    map_cm, loc, tmask = sm.map_cm.cpu().numpy(), sm.loc.cpu().numpy(), sm.tile_mask.cpu().numpy().astype(np.uint32)
    assert sorted(loc[:n].tolist()) == list(range(n))               # the valid rows, each once
    assert np.array_equal(map_cm[:, :n], m[loc[:n]].T)               # row r of the sorted map is map row loc[r]
    assert (map_cm[:, n:] == -1).all()
    masks = ((m[:n] >= 0) * (1 << np.arange(m.shape[1]))).sum(1)
    keys = masks                                                     # the order covers every mask bit
    assert (np.diff(keys[loc[:n]]) <= 0).all()                       # descending neighbour masks
    same = keys[loc[:n]][1:] == keys[loc[:n]][:-1]
    assert (np.diff(loc[:n])[same] > 0).all()                        # stable: equal keys keep row order
    valid = map_cm >= 0
    want = np.array([sum(1 << k for k in np.nonzero(valid[:, t * 128:(t + 1) * 128].any(1))[0])
                     for t in range(m.shape[0] // 128)], dtype=np.uint32)
    assert np.array_equal(tmask, want)
    # the work-item table: every tile once, its offsets divided among ceil(count / 4) consecutive parts; the
    # items are grouped by weight class (offsets per item: >= 14, >= 7, >= 3, fewer), heaviest class first, and
    # keep the tile order inside a class
    items = sm.items.cpu().numpy()[: int(sm.n_items.item())]
    assert len(items) <= sm.n_items_max
    slot = 0
    budget = m.shape[0] // 128                          # scratch slots: one per tile of the map
    expected = []                                       # (class, tile, parts, first slot)
    for t, mask in enumerate(want):
        pc = bin(int(mask)).count("1")
        parts = wanted = max(1, -(-pc // 4))
        if parts > 1 and slot + parts > budget:        # beyond the scratch slots: the tile stays whole
            parts = 1
        per = -(-pc // parts)
        cls = 0 if per >= 14 else 1 if per >= 7 else 2 if per >= 3 else 3
        expected.append((cls, t, parts, slot))
        slot += wanted if wanted > 1 else 0             # slots are numbered as if every heavy tile were split
    pos = 0
    for cls, t, parts, slot0 in sorted(expected, key=lambda e: e[0]):      # a stable sort
        rows = items[pos: pos + parts]
        assert (rows[:, 0] == t).all()
        got_mask = 0
        for j, r in enumerate(rows):
            pm = int(r[1]) & 0xffffffff
            assert (pm or not want[t]) and (pm & got_mask) == 0 and (parts == 1 or bin(pm).count("1") <= 4)
            got_mask |= pm
            if parts > 1:
                assert int(r[2]) & 0xffff == (j | (parts << 8)) and int(r[2]) >> 16 == slot0
            else:
                assert int(r[2]) == 0
        assert got_mask == int(want[t])
        pos += parts
    assert pos == len(items)


@pytest.mark.parametrize("cin,cout", [(64, 96), (96, 96), (32, 32), (256, 128), (8, 32)])
@pytest.mark.parametrize("max_offsets", [8, 3, 27])
def test_sorted_cm_conv(cin, cout, max_offsets):
    """The sorted map with its tiles split into parts of at most max_offsets offsets (27: no tile is split)
    gives the result of the plain map; the split sums are formed in part order, so two runs agree bit for bit."""
    from torchsparse_b200 import backend

    _, f, w, km, want = _case(cin=cin, cout=cout)
    n = km["sizes"][1]
    sm = backend.sorted_cm_artefacts_cuda(torch.from_numpy(km["out_in_map"]).cuda(), n, max_offsets=max_offsets)
    y = backend.conv_forward_implicit_gemm_cuda(f, w, None, n, cout, smap=sm)
    assert rel_l2(y.float().cpu().numpy(), want) < TOL
    y2 = backend.conv_forward_implicit_gemm_cuda(f, w, None, n, cout, smap=sm)
    assert torch.equal(y, y2)
    assert int(sm.flags.abs().sum().item()) == 0          # the part counters are back at zero
    # without the item table (whole tiles): the same map through explicit arguments
    y3 = backend.conv_forward_implicit_gemm_cuda(f, w, sm.map_cm, n, cout, reorder_loc=sm.loc, tile_mask=sm.tile_mask,
                                                 map_strides=(1, sm.rows))
    assert rel_l2(y3.float().cpu().numpy(), want) < TOL


@pytest.mark.parametrize("c1,c2,cout", [(64, 32, 96), (96, 32, 96), (256, 128, 256), (8, 8, 16)])
def test_two_matrix_input_equals_concatenation(c1, c2, cout):
    from torchsparse_b200 import backend

    _, f, w, km, want = _case(cin=c1 + c2, cout=cout, n=3000)
    n = km["sizes"][1]
    m = torch.from_numpy(km["out_in_map"]).cuda()
    fa, fb = f[:, :c1].contiguous(), f[:, c1:].contiguous()
    y = backend.conv_forward_implicit_gemm_cuda(fa, w, m, n, cout, in_feats2=fb)
    assert rel_l2(y.float().cpu().numpy(), want) < TOL
    y_cat = backend.conv_forward_implicit_gemm_cuda(f, w, m, n, cout)
    assert torch.equal(y, y_cat)     # the same arithmetic on the same operands


def test_pointwise_without_a_map():
    from torchsparse_b200 import backend

    rng = np.random.default_rng(1)
    n, cin, cout = 4001, 192, 128
    f = torch.from_numpy(rng.standard_normal((n, cin)).astype(np.float32)).half()
    w = torch.from_numpy((rng.standard_normal((1, cin, cout)) / np.sqrt(cin)).astype(np.float32)).half()
    scale = torch.from_numpy(rng.uniform(0.5, 1.5, cout).astype(np.float32))
    bias = torch.from_numpy(rng.standard_normal(cout).astype(np.float32))
    res = torch.from_numpy(rng.standard_normal((n, cout)).astype(np.float32)).half()
    want = np.maximum(f.double().numpy() @ w[0].double().numpy() * scale.double().numpy() + bias.double().numpy()
                      + res.double().numpy(), 0)
    y = backend.conv_forward_implicit_gemm_cuda(f.cuda(), w.cuda(), None, n, cout, scale=scale.cuda(), bias=bias.cuda(),
                                                residual=res.cuda(), relu=True)
    assert rel_l2(y.float().cpu().numpy(), want) < TOL
    # and from two matrices
    y2 = backend.conv_forward_implicit_gemm_cuda(f[:, :128].contiguous().cuda(), w.cuda(), None, n, cout,
                                                 scale=scale.cuda(), bias=bias.cuda(), residual=res.cuda(), relu=True,
                                                 in_feats2=f[:, 128:].contiguous().cuda())
    assert torch.equal(y, y2)


def test_offset_ranges_chained_through_fp32_partial_sums():
    from torchsparse_b200 import backend

    _, f, w, km, want = _case(cin=64, cout=64, n=3000)
    n = km["sizes"][1]
    m = torch.from_numpy(km["out_in_map"]).cuda()
    acc = torch.empty((n, 64), dtype=torch.float32, device="cuda")
    bias = torch.linspace(-1, 1, 64, device="cuda")
    backend.conv_forward_implicit_gemm_cuda(f, w, m, n, 64, k_range=(0, 9), acc_out=acc)
    backend.conv_forward_implicit_gemm_cuda(f, w, m, n, 64, k_range=(9, 18), acc_in=acc, acc_out=acc)
    y = backend.conv_forward_implicit_gemm_cuda(f, w, m, n, 64, k_range=(18, 27), acc_in=acc, bias=bias)
    assert rel_l2(y.float().cpu().numpy(), want + bias.cpu().numpy()) < TOL


def test_row_count_in_device_memory():
    from torchsparse_b200 import backend

    _, f, w, km, want = _case(cin=64, cout=64, n=3000)
    n = km["sizes"][1]
    m = torch.from_numpy(km["out_in_map"]).cuda()
    rows_max = 4096                                   # upper bound the launch is sized for
    m_big = torch.full((rows_max, 27), -1, dtype=torch.int32, device="cuda")
    m_big[: m.shape[0]] = m
    out = torch.full((rows_max, 64), 7.0, dtype=torch.float16, device="cuda")
    n_dev = torch.tensor([n], dtype=torch.int32, device="cuda")
    backend.conv_forward_implicit_gemm_cuda(f, w, m_big, rows_max, 64, n_out_dev=n_dev, out=out)
    assert rel_l2(out[:n].float().cpu().numpy(), want) < TOL
    assert (out[(n + 127) // 128 * 128:] == 7.0).all()        # tiles beyond the device-side count are not touched


@pytest.mark.parametrize("cfg", [dict(cpb=2), dict(cpb=2, ctas=1), dict(n_tile=64), dict(ctas=1, stages=3),
                                 dict(n_tile=32, cpb=2, ctas=2)])
def test_launch_configuration_overrides(cfg):
    from torchsparse_b200 import backend

    _, f, w, km, want = _case(cin=96, cout=128, n=3000)
    n = km["sizes"][1]
    m = torch.from_numpy(km["out_in_map"]).cuda()
    old = dict(backend.igemm_tuning)
    try:
        backend.igemm_tuning.update(cfg)
        y = backend.conv_forward_implicit_gemm_cuda(f, w, m, n, 128)
    finally:
        backend.igemm_tuning.update(old)
    assert rel_l2(y.float().cpu().numpy(), want) < TOL


def test_split_sorted_on_tensor_cores_fp16():
    """F.set_conv_mode(2)'s configuration (row-sorted map, 3 mask splits) through F.conv3d."""
    import torchsparse_b200 as ts
    from torchsparse_b200.nn import functional as F

    coords, f, w, km, want = _case(cin=64, cout=64, n=4000)
    cfg = F.conv_config.get_default_conv_config()
    cfg.ifsort, cfg.split_mask_num = True, 3
    x = ts.SparseTensor(f, torch.from_numpy(coords).cuda())
    y = F.conv3d(x, w, 3, None, 1, 1, config=cfg)
    assert rel_l2(y.feats.float().cpu().numpy(), want) < TOL


@pytest.mark.parametrize("cin,cout,c1", [(64, 64, 0), (96, 96, 0), (8, 32, 0), (128, 96, 96), (384, 256, 256), (40, 48, 24)])
def test_copy_engine_gather_equals_cp_async_gather(cin, cout, c1):
    """The two ways the gathered operand reaches shared memory (TMA gather4 by one producer warp, 16-byte cp.async by
    eight gather warps) give the same rows: bit-identical for one feature matrix (same K order), within fp16
    rounding for a two-matrix input whose first part is not a multiple of 64 channels (the chunks are cut per
    matrix with the copy engine, so the fp32 sums are added in another order)."""
    from torchsparse_b200 import backend

    rng = np.random.default_rng(cin + cout + c1)
    coords = random_coords(rng, 3000, (20, 20, 20), 2)
    n = coords.shape[0]
    km = ko.build_kmap(coords, 3, 1, 1)
    omap = torch.from_numpy(km["out_in_map"]).cuda()
    x = torch.from_numpy(rng.standard_normal((n, cin)).astype(np.float32)).cuda().half()
    w = torch.from_numpy((rng.standard_normal((27, cin, cout)) * 0.1).astype(np.float32)).cuda().half()
    kw = {}
    feats = x
    if c1:
        feats, kw = x[:, :c1].contiguous(), {"in_feats2": x[:, c1:].contiguous()}
    outs = []
    try:
        for mode in (2, 1):
            backend.igemm_tuning["gather"] = mode
            outs.append(backend.conv_forward_implicit_gemm_cuda(feats, w, omap, n, cout, **kw))
    finally:
        backend.igemm_tuning["gather"] = 0
    want = ko.conv_from_map(x.float().cpu().numpy(), w.float().cpu().numpy(), km["out_in_map"], n)
    assert rel_l2(outs[0].float().cpu().numpy(), want) < TOL
    if c1 % 64 == 0:
        assert torch.equal(outs[0], outs[1])
    else:
        assert rel_l2(outs[0].float().cpu().numpy(), outs[1].float().cpu().numpy()) < 1e-3


@pytest.mark.parametrize("cin,cout", [(32, 48), (96, 96), (4, 16)])
def test_exact_fp32_by_three_tf32_passes(cin, cout):
    """fp32 operands with allow_tf32 = False: the three-pass TF32 split on the tensor cores and the CUDA-core kernel
    both stay within relative L2 1e-5 of the fp64 oracle (the tolerance of every exact-fp32 test of this suite),
    while a single TF32 pass does not."""
    from torchsparse_b200 import backend, backends

    rng = np.random.default_rng(cin * 7 + cout)
    coords = random_coords(rng, 4000, (30, 30, 30))
    n = coords.shape[0]
    km = ko.build_kmap(coords, 3, 1, 1)
    x = rng.standard_normal((n, cin)).astype(np.float32)
    w = (rng.standard_normal((27, cin, cout)) / np.sqrt(27 * cin)).astype(np.float32)
    want = ko.conv_from_map(x, w, km["out_in_map"], n)
    xt, wt, m = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(km["out_in_map"]).cuda()
    errs = {}
    try:
        for name, split, tf32 in (("split", True, False), ("cuda_cores", False, False), ("tf32", True, True)):
            backends.fp32_by_split_tf32 = split
            y = backend.conv_forward_implicit_gemm_cuda(xt, wt, m, n, cout, tf32)
            assert y.dtype == torch.float32
            errs[name] = rel_l2(y.cpu().numpy(), want)
    finally:
        backends.fp32_by_split_tf32 = True
    assert errs["split"] < 1e-5 and errs["cuda_cores"] < 1e-5, errs
    assert errs["tf32"] > 1e-5, errs                       # one pass rounds the operands to 10 mantissa bits
    # the fused epilogue rides on the last pass
    scale = torch.rand(cout, device="cuda") + 0.5
    bias = torch.randn(cout, device="cuda")
    y = backend.conv_forward_implicit_gemm_cuda(xt, wt, m, n, cout, False, scale=scale, bias=bias, relu=True)
    ref = np.maximum(want * scale.cpu().numpy() + bias.cpu().numpy(), 0)
    assert rel_l2(y.cpu().numpy(), ref) < 1e-5
