"""GPU parity, kernel maps: every integer artefact is compared bit for bit with the oracle."""
import numpy as np
import pytest
import torch

from conftest import random_coords, rel_l2
from oracle import kmap_oracle as ko

pytestmark = pytest.mark.gpu

CASES = [(3, 1), (2, 2), (3, 2), ((1, 3, 1), (1, 2, 1)), (2, 1), (5, 1), (3, 3), ((3, 1, 1), (2, 1, 1)), (2, 3),
         ((1, 1, 3), 1), (5, 2)]


def _pad(ks, st):
    return tuple((k - 1) // 2 if (k % 2 == 1 and s == 1) else 0 for k, s in zip(ko._as3(ks), ko._as3(st)))


def _build(coords_np, ks, st, pad, spatial_range=None, **kw):
    from torchsparse_b200.nn import functional as F

    coords = torch.from_numpy(coords_np).cuda()
    return F.build_kernel_map(coords, coords.shape[0], ks, st, pad, None, None, spatial_range, "hashmap_on_the_fly",
                              **kw)


@pytest.mark.parametrize("ks,st", CASES)
@pytest.mark.parametrize("n,shape,batch", [(20, (5, 5, 5), 1), (900, (16, 13, 11), 3), (1, (3, 3, 3), 1)])
def test_kernel_map_bit_exact(ks, st, n, shape, batch):
    rng = np.random.default_rng(hash((str(ks), str(st), n)) % 2**31)
    coords = random_coords(rng, n, shape, batch)
    pad = _pad(ks, st)
    want = ko.build_kmap(coords, ks, st, pad)
    got = _build(coords, ks, st, pad)
    assert got["sizes"] == want["sizes"]
    assert np.array_equal(got["coords"].cpu().numpy(), want["coords"])
    assert np.array_equal(got["out_in_map"].cpu().numpy(), want["out_in_map"])


def test_kernel_map_explicit_padding_and_spatial_range():
    rng = np.random.default_rng(11)
    coords = random_coords(rng, 1500, (20, 18, 8), 2)
    for ks, st, pad in [(3, 2, (1, 1, 1)), (3, 2, (0, 1, 1)), ((3, 1, 1), (2, 1, 1), (1, 0, 0)), (3, 1, (1, 1, 1))]:
        for sr in (None, (2, 20, 18, 8)):
            want = ko.build_kmap(coords, ks, st, pad, sr)
            got = _build(coords, ks, st, pad, sr)
            assert got["spatial_range"] == want["spatial_range"]
            assert np.array_equal(got["coords"].cpu().numpy(), want["coords"])
            assert np.array_equal(got["out_in_map"].cpu().numpy(), want["out_in_map"])


def test_baseline_config1_map_and_large_map_properties():
    """BASELINE config 1 (20 000 voxels in 128^3) bit-exact, then a 2M-voxel map checked through
    size-independent properties: symmetry of the odd submanifold map and map/transposed-map duality."""
    rng = np.random.default_rng(0)
    coords = random_coords(rng, 20000, (128, 128, 128))
    want = ko.build_kmap(coords, 3, 1, 1)
    got = _build(coords, 3, 1, 1)
    assert np.array_equal(got["out_in_map"].cpu().numpy(), want["out_in_map"])

    n = 2_000_000
    big = random_coords(rng, n, (215, 215, 215))  # ~20% occupancy
    g = _build(big, 3, 1, 1)
    m = g["out_in_map"][:n]
    assert bool((m[:, 13] == torch.arange(n, device="cuda", dtype=torch.int32)).all())
    # symmetry: map[map[i][k]][26-k] == i wherever map[i][k] >= 0
    for k in (0, 5, 12):
        col = m[:, k].long()
        rows = torch.nonzero(col >= 0).squeeze(1)
        assert bool((m[col[rows], 26 - k].long() == rows).all())
    from torchsparse_b200.nn.functional import convert_transposed_out_in_map
    mt = convert_transposed_out_in_map(g["out_in_map"], g["out_in_map"].shape[0])
    assert bool((mt[:n] == m.flip(1)).all())
    # strided: every input appears exactly once in a k2 s2 map, outputs sorted by ravel order
    d = _build(big, 2, 2, 0)
    dm = d["out_in_map"][: d["sizes"][1]]
    assert int((dm >= 0).sum()) <= n
    oc = d["coords"].long()
    key = ((oc[:, 0] * 1000 + oc[:, 1]) * 1000 + oc[:, 2]) * 1000 + oc[:, 3]
    assert bool((key[1:] > key[:-1]).all())
    vals = dm[dm >= 0].long()
    assert vals.unique().numel() == vals.numel()


@pytest.mark.parametrize("split", [1, 2, 3])
def test_sorted_artefacts(split):
    from torchsparse_b200 import backend

    rng = np.random.default_rng(7)
    coords = random_coords(rng, 1100, (15, 15, 15), 2)
    want = ko.build_kmap(coords, 3, 1, 1)
    m_np, n = want["out_in_map"], coords.shape[0]
    m = torch.from_numpy(m_np).cuda()
    bm = backend.derive_bitmask_from_out_in_map(m, split, n)
    bm_np = ko.derive_bitmask(m_np, split, n)
    assert np.array_equal(bm.cpu().numpy(), bm_np)
    sm, loc = backend.sort_bitmask_cuda(bm, 27)
    sm_np, loc_np = ko.sort_bitmask(bm_np)
    assert np.array_equal(sm.cpu().numpy(), sm_np)
    assert np.array_equal(loc.cpu().numpy(), loc_np)   # both sorts are stable
    ro = backend.reorder_out_in_map_cuda(m, loc)
    assert np.array_equal(ro.cpu().numpy(), ko.reorder_map(m_np, loc_np))
    for tile in (128, 64):
        red = backend.reduce_bitmask_cuda(sm, tile)
        assert np.array_equal(red.cpu().numpy(), ko.reduce_bitmask(sm_np, tile))
    with pytest.raises(RuntimeError):
        backend.reduce_bitmask_cuda(sm, 6)


@pytest.mark.parametrize("ks,st", [(3, 1), (2, 2), (3, 2)])
def test_pair_lists_scans_masks_transpose(ks, st):
    from torchsparse_b200 import backend

    rng = np.random.default_rng(13)
    coords = random_coords(rng, 1300, (17, 14, 12), 2)
    want = ko.build_kmap(coords, ks, st, _pad(ks, st))
    m_np = want["out_in_map"]
    n, mo = want["sizes"]
    m = torch.from_numpy(m_np).cuda()
    nb_np, sz_np = ko.pairs_from_map(m_np)
    a_np, qa_np = ko.scan_quantified(sz_np)
    for fod in (False, True):
        nbmaps, nbsizes, sizes_host, nbaddrs, qnbaddrs, qmapsize = backend.pairs_from_out_in_map(m, fod)
        assert sizes_host == sz_np.tolist() and qmapsize == int(qa_np[-1])
        assert np.array_equal(nbsizes.cpu().numpy(), sz_np)
        assert np.array_equal(nbaddrs.cpu().numpy(), a_np) and np.array_equal(qnbaddrs.cpu().numpy(), qa_np)
        got = nbmaps.cpu().numpy()
        assert np.array_equal(got.T if fod else got, nb_np)
    nbmaps = torch.from_numpy(nb_np).cuda()
    im, om = backend.build_mask_from_kmap(n, mo, nbmaps, torch.from_numpy(sz_np).cuda())
    im_np, om_np = ko.masks_from_pairs(n, mo, nb_np, sz_np)
    assert np.array_equal(im.cpu().numpy(), im_np) and np.array_equal(om.cpu().numpy(), om_np)
    # the reference-named scan wrapper writes into its arguments
    a = torch.zeros(len(sz_np) + 1, dtype=torch.int32, device="cuda")
    qa = torch.zeros_like(a)
    backend.exclusive_scan_quantified_wrapper(len(sz_np), torch.from_numpy(sz_np).cuda(), a, qa)
    assert np.array_equal(a.cpu().numpy(), a_np) and np.array_equal(qa.cpu().numpy(), qa_np)
    # transposed map, reference-style call with a pre-filled destination
    rows_t = ko.pad_rows(n)
    mt = torch.full((rows_t, m.shape[1]), -1, dtype=torch.int32, device="cuda")
    backend.convert_transposed_out_in_map(m, mt)
    assert np.array_equal(mt.cpu().numpy(), ko.transpose_map(m_np, rows_t))


def test_hash_table_api_and_full_table_error():
    from torchsparse_b200 import backend

    rng = np.random.default_rng(17)
    keys = torch.from_numpy(rng.choice(10**12, 5000, replace=False).astype(np.int64) + 1).cuda()
    table = backend.GPUHashTable(torch.zeros(10007, dtype=torch.int64, device="cuda"),
                                 torch.zeros(10007, dtype=torch.int32, device="cuda"))   # non power-of-two capacity
    table.insert_vals(keys)
    got = table.lookup_vals(keys)
    assert got.shape[0] == 5120 and bool((got[:5000] == torch.arange(1, 5001, device="cuda")).all())
    assert bool((got[5000:] == 0).all())
    miss = table.lookup_vals(keys[:100] + 10**13)
    assert bool((miss == 0).all())
    # a table that cannot hold the keys reports it instead of spinning forever
    small = backend.GPUHashTable(64)
    with pytest.raises(ValueError):
        small.insert_vals(keys[:200])


def test_32bit_key_table_api_and_limits():
    """The packed layout (reference: hashtable32, sparsemapping_cuda.cu:259-300, 347-426): same stored values as the
    64-bit layout, full-table and key-range errors reported instead of wrong answers."""
    from torchsparse_b200 import backend

    rng = np.random.default_rng(23)
    keys = torch.from_numpy(rng.choice(2**32 - 2, 5000, replace=False).astype(np.int64) + 1).cuda()
    table = backend.GPUHashTable32(torch.zeros(10007, dtype=torch.int64, device="cuda"))
    table.insert_vals(keys)
    got = table.lookup_vals(keys)
    assert bool((got[:5000] == torch.arange(1, 5001, device="cuda")).all()) and bool((got[5000:] == 0).all())
    absent = torch.from_numpy(np.setdiff1d(np.arange(1, 20000), keys.cpu().numpy())[:100].astype(np.int64)).cuda()
    assert bool((table.lookup_vals(absent) == 0).all())
    assert bool((table.lookup_vals(keys[:100] + 2**32) == 0).all())      # beyond the key range: never found
    with pytest.raises(ValueError):
        backend.GPUHashTable32(64).insert_vals(keys[:200])                # full
    with pytest.raises(ValueError):
        backend.GPUHashTable32(1024).insert_vals(keys[:10] + 2**32)       # key does not fit a packed slot
    # a box of 2^32 cells or more is refused by the builders before anything is launched
    coords = torch.from_numpy(random_coords(rng, 50, (8, 8, 8))).cuda()
    with pytest.raises(Exception):
        backend.build_kernel_map_subm_hashmap_int32(backend.GPUHashTable32(256), coords, (0, 0, 0, 0),
                                                    (0, 70000, 70000, 8), (3, 3, 3))
    with pytest.raises(ValueError):
        backend.build_kernel_map_subm_hashmap_int32(backend.GPUHashTable(256), coords, (0, 0, 0, 0), (0, 7, 7, 7), (3, 3, 3))


@pytest.mark.parametrize("ks,st", [(3, 1), (2, 2), (3, 2), ((1, 3, 1), (1, 2, 1)), (2, 1), (5, 1)])
def test_32bit_and_64bit_key_tables_build_the_same_maps(ks, st):
    from torchsparse_b200 import backend, backends

    rng = np.random.default_rng(29)
    coords_np = random_coords(rng, 3000, (40, 33, 17), 2)
    pad = _pad(ks, st)
    want = ko.build_kmap(coords_np, ks, st, pad)
    seen = {}
    for flag in (True, False):
        backends.hash_keys_32bit = flag
        try:
            got = _build(coords_np, ks, st, pad)
        finally:
            backends.hash_keys_32bit = True
        assert (got["hashmap_vals"] is None) == flag
        assert np.array_equal(got["coords"].cpu().numpy(), want["coords"])
        assert np.array_equal(got["out_in_map"].cpu().numpy(), want["out_in_map"])
        seen[flag] = got
    # the reference-named entry points over an explicit table
    ks3, st3 = ko._as3(ks), ko._as3(st)
    coords = torch.from_numpy(coords_np).cuda()
    cmax = tuple(int(v) for v in coords_np.max(0))
    if all(s == 1 for s in st3):
        m = backend.build_kernel_map_subm_hashmap_int32(backend.GPUHashTable32(8192), coords, (0, 0, 0, 0), cmax, ks3)[0]
        assert np.array_equal(m.cpu().numpy(), want["out_in_map"])
    else:
        cmax_out = (cmax[0],) + tuple((cmax[1 + i] + 2 * pad[i] - (ks3[i] - 1)) // st3[i] for i in range(3))
        m, oc = backend.build_kernel_map_downsample_hashmap_int32(backend.GPUHashTable32(8192), coords, (0, 0, 0, 0),
                                                                  cmax_out, ks3, st3, pad)
        assert np.array_equal(oc.cpu().numpy(), want["coords"])
        assert np.array_equal(m.cpu().numpy(), want["out_in_map"])


def test_duplicate_free_determinism():
    rng = np.random.default_rng(19)
    coords = random_coords(rng, 4000, (30, 30, 30), 2)
    a = _build(coords, 3, 2, 0)
    b = _build(coords, 3, 2, 0)
    assert torch.equal(a["out_in_map"], b["out_in_map"]) and torch.equal(a["coords"], b["coords"])


def test_empty_and_vanishing_inputs():
    """No voxels in, or a strided conv that keeps none: empty tensors, no error."""
    import torchsparse_b200 as ts
    from torchsparse_b200.nn import functional as F

    empty = torch.zeros((0, 4), dtype=torch.int32, device="cuda")
    g = F.build_kernel_map(empty, 0, 3, 1, 1, None, None, None, "hashmap_on_the_fly")
    assert g["out_in_map"].shape == (0, 27) and g["sizes"] == (0, 0)
    # one voxel at even max coordinate: k2 s2 drops it (bound (max-1)//2), as the oracle says
    one = torch.tensor([[0, 4, 4, 4]], dtype=torch.int32, device="cuda")
    x = ts.SparseTensor(torch.ones(1, 8, device="cuda"), one)
    w = torch.ones(8, 8, 16, device="cuda")
    y = F.conv3d(x, w, 2, None, 2, 0)
    assert y.coords.shape == (0, 4) and y.feats.shape == (0, 16)
    z = F.conv3d(y, torch.ones(27, 16, 16, device="cuda"), 3, None, 1, 1)
    assert z.feats.shape == (0, 16)


@pytest.mark.parametrize("ks,st,pd", [(3, 1, 1), (2, 2, 0), (3, 2, 1)])
def test_negative_coordinates(ks, st, pd):
    """set_allow_negative_coordinates(True): the key space starts at the (padding-adjusted) smallest
    coordinate instead of 0 (torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:39-43);
    maps and output coordinates bit-exact against the oracle run with the same bound rule."""
    import torchsparse_b200 as ts
    from torchsparse_b200.nn import functional as F
    from torchsparse_b200.tensor import set_allow_negative_coordinates

    rng = np.random.default_rng(5)
    coords = random_coords(rng, 3000, (24, 20, 16), 2)
    coords[:, 1:] -= np.array([11, 7, 9], dtype=np.int32)          # roughly centred on the origin
    want = ko.build_kmap(coords, ks, st, pd, allow_negative=True)
    set_allow_negative_coordinates(True)
    try:
        x = ts.SparseTensor(torch.zeros(coords.shape[0], 8, device="cuda"), torch.from_numpy(coords).cuda())
        w = torch.zeros(ks ** 3, 8, 8, device="cuda")
        y = F.conv3d(x, w, ks, None, st, pd)
        kmap = x._caches.kmaps[((1, 1, 1), (ks,) * 3, (st,) * 3, (1, 1, 1))]
    finally:
        set_allow_negative_coordinates(False)
    assert np.array_equal(y.coords.cpu().numpy(), want["coords"])
    assert np.array_equal(kmap["out_in_map"].cpu().numpy(), want["out_in_map"])
    assert (want["coords"][:, 1:] < 0).any()


@pytest.mark.parametrize("ks,st,pd", [(3, 1, 1), (2, 2, 0), (3, 2, 1), (2, 1, 0), ((1, 3, 1), (1, 2, 1), 0)])
def test_kmap_mode_hashmap(ks, st, pd):
    """kmap_mode="hashmap": spdownsample output coordinates, FNV-keyed table (GPUHashTable.insert_coords /
    lookup_coords), map bit-exact against the oracle, and the convolution on that map."""
    import torchsparse_b200 as ts
    from torchsparse_b200.nn import functional as F

    rng = np.random.default_rng(9)
    coords = random_coords(rng, 2500, (20, 18, 16), 2)
    want = ko.build_kmap_hashmap_mode(coords, ks, st, pd)
    cfg = F.conv_config.get_default_conv_config()
    cfg.kmap_mode = "hashmap"
    kvol = int(np.prod(ko._as3(ks)))
    feats = rng.standard_normal((coords.shape[0], 16)).astype(np.float32)
    w = (rng.standard_normal((kvol, 16, 24)) * 0.1).astype(np.float32)
    x = ts.SparseTensor(torch.from_numpy(feats).cuda(), torch.from_numpy(coords).cuda())
    y = F.conv3d(x, torch.from_numpy(w).cuda(), ks, None, st, pd, config=cfg)
    kmap = x._caches.kmaps[((1, 1, 1), ko._as3(ks), ko._as3(st), (1, 1, 1))]
    assert np.array_equal(y.coords.cpu().numpy(), want["coords"])
    assert np.array_equal(kmap["out_in_map"].cpu().numpy(), want["out_in_map"])
    ref = ko.conv_from_map(feats, w, want["out_in_map"], want["sizes"][1])
    assert rel_l2(y.feats.cpu().numpy(), ref) < 1e-5
    # a second convolution at the same stride reuses the table
    y2 = F.conv3d(x, torch.from_numpy(w).cuda(), ks, None, st, pd, config=cfg)
    assert torch.equal(y2.feats, y.feats)


def test_spdownsample_and_downsample_cuda():
    from torchsparse_b200.nn import functional as F

    rng = np.random.default_rng(10)
    coords = random_coords(rng, 3000, (24, 24, 12), 2)
    c = torch.from_numpy(coords).cuda()
    got = F.spdownsample(c, 2, 2, 0).cpu().numpy()
    want = np.unique(np.concatenate([coords[:, :1], coords[:, 1:] // 2], 1), axis=0)
    assert np.array_equal(got, want)
    got3 = F.spdownsample(c, 2, 3, 1).cpu().numpy()                 # stride != kernel: native enumeration
    want3 = ko.build_kmap(coords, 3, 2, 1)["coords"]
    assert np.array_equal(got3, want3)


@pytest.mark.parametrize("ks,st", [(2, 2), (3, 2)])
def test_generative_transposed_convolution(ks, st):
    """Generative transposed convolution (kmap_mode="hashmap"): generated output coordinates and the kernel map
    bit-exact against the oracle, the features against the oracle convolution, gradients flow, the kernel-map
    caches are emptied afterwards (torchsparse/nn/functional/conv/conv.py:161-203), and `generative_add` of the
    result with a tensor on other coordinates sums over the union."""
    import torchsparse_b200 as ts
    from torchsparse_b200.nn import functional as F

    rng = np.random.default_rng(21)
    coords = random_coords(rng, 1500, (12, 12, 12), 2)
    srange = (2, 32, 32, 32)
    want = ko.build_kmap_generative(coords, ks, st, 0, srange)
    cfg = F.conv_config.get_default_conv_config()
    cfg.kmap_mode = "hashmap"
    kvol = ks ** 3
    feats = rng.standard_normal((coords.shape[0], 16)).astype(np.float32)
    w = (rng.standard_normal((kvol, 16, 24)) * 0.1).astype(np.float32)
    xf = torch.from_numpy(feats).cuda().requires_grad_(True)
    wt = torch.from_numpy(w).cuda().requires_grad_(True)
    x = ts.SparseTensor(xf, torch.from_numpy(coords).cuda(), stride=(st,) * 3, spatial_range=srange)
    y = F.conv3d(x, wt, ks, None, st, 0, config=cfg, transposed=True, generative=True)
    assert y.stride == (1, 1, 1) and tuple(y.spatial_range) == tuple(want["spatial_range"])
    assert np.array_equal(y.coords.cpu().numpy(), want["coords"])
    m = want["sizes"][1]
    ref = ko.conv_from_map(feats, w, want["out_in_map"], m)
    assert rel_l2(y.feats.detach().cpu().numpy(), ref) < 1e-5
    assert x._caches.kmaps == {} and x._caches.hashmaps == {}
    gy = rng.standard_normal((m, 24)).astype(np.float32)
    y.feats.backward(torch.from_numpy(gy).cuda())
    want_dx, want_dw = ko.conv_backward_from_map(feats, w, want["out_in_map"], m, gy)
    assert rel_l2(xf.grad.cpu().numpy(), want_dx) < 1e-5 and rel_l2(wt.grad.cpu().numpy(), want_dw) < 1e-5
    # generative_add: union of coordinates, equal coordinates summed
    other_c = np.unique(np.concatenate([want["coords"][::3], random_coords(rng, 200, (20, 20, 20), 2)]), axis=0)
    other_f = rng.standard_normal((other_c.shape[0], 24)).astype(np.float32)
    z = ts.generative_add(ts.SparseTensor(y.feats.detach(), y.coords), ts.SparseTensor(torch.from_numpy(other_f).cuda(),
                                                                                      torch.from_numpy(other_c).cuda()))
    union = np.unique(np.concatenate([want["coords"], other_c]), axis=0)
    assert np.array_equal(z.coords.cpu().numpy(), union)
    dense = {tuple(c): f.copy() for c, f in zip(want["coords"].tolist(), y.feats.detach().cpu().numpy())}
    for c, f in zip(other_c.tolist(), other_f):
        dense[tuple(c)] = dense.get(tuple(c), 0) + f
    want_z = np.stack([dense[tuple(c)] for c in union.tolist()])
    assert rel_l2(z.feats.cpu().numpy(), want_z) < 1e-6
