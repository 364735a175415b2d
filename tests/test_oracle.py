"""CPU suite, part 1: the oracle itself is pinned against (a) a dense torch conv3d, the way the
reference's own test pins its kernels (tests/python/test_single_layer_conv.py:111-220), (b) the
golden fixtures generated from the reference's CPU sources and numpy code."""
import numpy as np
import pytest

from conftest import random_coords, rel_l2
from oracle import kmap_oracle as ko

CASES = [("k3s1", 3, 1), ("k2s2", 2, 2), ("k3s2", 3, 2), ("k131s121", (1, 3, 1), (1, 2, 1)), ("k2s1", 2, 1),
         ("k5s1", 5, 1), ("k3s3", 3, 3)]


def _pad(ks, st):
    return tuple((k - 1) // 2 if (k % 2 == 1 and s == 1) else 0 for k, s in zip(ko._as3(ks), ko._as3(st)))


@pytest.mark.parametrize("name,ks,st", CASES)
def test_oracle_matches_reference_cpu_conv_and_dense(golden, name, ks, st):
    coords, feats, w = golden[f"{name}/coords"], golden[f"{name}/feats"], golden[f"{name}/weight"]
    km = ko.build_kmap(coords, ks, st, _pad(ks, st))
    assert np.array_equal(km["coords"], golden[f"{name}/out_coords"])
    y = ko.conv_from_map(feats, w, km["out_in_map"], km["sizes"][1])
    assert rel_l2(y, golden[f"{name}/ref_cpu_out"]) < 1e-6      # the reference's own CPU conv
    assert rel_l2(y, golden[f"{name}/dense_out"]) < 1e-6        # dense conv3d (pins the kernel map)
    nbmaps, nbsizes = ko.pairs_from_map(km["out_in_map"])
    y2 = ko.conv_from_pairs(feats, w, nbmaps, nbsizes, km["sizes"][1])
    assert np.allclose(y, y2, atol=1e-12)
    if f"{name}/t_feats" in golden:
        mt = ko.transpose_map(km["out_in_map"], ko.pad_rows(coords.shape[0]))
        yt = ko.conv_from_map(golden[f"{name}/t_feats"], golden[f"{name}/t_weight"], mt, coords.shape[0])
        assert rel_l2(yt, golden[f"{name}/t_ref_cpu_out"]) < 1e-6


@pytest.mark.parametrize("name,ks,st", CASES)
def test_kernel_digit_order_matches_reference_offsets(golden, name, ks, st):
    ks3 = ko._as3(ks)
    digits = ko.kernel_digits(ks3)
    centred = digits - np.array([(k - 1) // 2 if k % 2 else k // 2 - 1 for k in ks3])
    # get_kernel_offsets enumerates arange(-k//2+1, k//2+1): same order, possibly shifted by a constant
    ref = golden[f"{name}/offsets"]
    assert np.array_equal(ref - ref[0], centred - centred[0])


def test_oracle_quantize_matches_reference_numpy(golden):
    for tag, vs in (("q05", 0.05), ("q37", (0.3, 0.7, 0.25)), ("q64", 0.1)):
        c, i, inv = ko.sparse_quantize(golden[f"{tag}/points"], vs, return_index=True, return_inverse=True)
        assert np.array_equal(c, golden[f"{tag}/coords"])
        assert np.array_equal(i, golden[f"{tag}/index"])
        assert np.array_equal(inv, golden[f"{tag}/inverse"])


def test_oracle_pointops_match_reference_cpu(golden):
    hc = golden["hash/coords"]
    assert np.array_equal(ko.fnv_hash(hc, fold60=True), golden["hash/ref_cpu_fold60"])
    assert np.array_equal(ko.count(golden["pts/idx"], 90), golden["pts/counts"])
    v = ko.voxelize(golden["pts/feats"], golden["pts/idx_nonneg"], golden["pts/counts"])
    assert rel_l2(v, golden["pts/voxelized"]) < 1e-6
    d = ko.devoxelize(golden["devox/vox_feats"], golden["devox/indices"], golden["devox/weights"])
    assert rel_l2(d, golden["devox/out"]) < 1e-6


def test_transpose_bitmask_reorder_reduce_roundtrip():
    rng = np.random.default_rng(3)
    coords = random_coords(rng, 700, (14, 12, 9), batch=2)
    km = ko.build_kmap(coords, 3, 1, 1)
    m = km["out_in_map"]
    n = coords.shape[0]
    # submanifold odd maps are symmetric: transposing twice is the identity, and map_t[i][k] == map[i][K-1-k]
    mt = ko.transpose_map(m, m.shape[0])
    assert np.array_equal(ko.transpose_map(mt, m.shape[0]), m)
    assert np.array_equal(mt[:n], m[:n, ::-1])
    for split in (1, 2, 3):
        bm = ko.derive_bitmask(m, split, n)
        assert (bm[:, n:] == -1).all()
        sm, loc = ko.sort_bitmask(bm)
        assert (np.diff(sm.astype(np.int64), axis=1) <= 0).all()
        for s in range(split):
            assert np.array_equal(np.sort(loc[s]), np.arange(m.shape[0]))
        ro = ko.reorder_map(m, loc)
        red = ko.reduce_bitmask(sm, 128)
        split_len = (27 + split - 1) // split
        for t in range(red.shape[1]):
            for c in range(27):
                s, bit = c // split_len, c % split_len
                has = (ro[t * 128:(t + 1) * 128, c] >= 0).any()
                if has:
                    assert (red[s, t] >> bit) & 1


def test_pairs_scans_masks():
    rng = np.random.default_rng(5)
    coords = random_coords(rng, 500, (10, 10, 10))
    km = ko.build_kmap(coords, 2, 2, 0)
    nbmaps, nbsizes = ko.pairs_from_map(km["out_in_map"])
    a, qa = ko.scan_quantified(nbsizes)
    assert a[-1] == nbmaps.shape[0] and (qa % 128 == 0).all() and (np.diff(qa) >= np.diff(a)).all()
    n, m = km["sizes"]
    im, om = ko.masks_from_pairs(n, m, nbmaps, nbsizes)
    for k in range(8):
        seg = nbmaps[a[k]:a[k + 1]]
        assert np.array_equal(im[k * n + seg[:, 0]], np.arange(len(seg)))
        assert np.array_equal(om[k * m + seg[:, 1]], np.arange(len(seg)))
    # k2 s2: every input lands in exactly one output cell
    assert nbmaps.shape[0] <= coords.shape[0] and len(np.unique(nbmaps[:, 0])) == nbmaps.shape[0]


def test_empty_and_single_inputs():
    empty = np.zeros((0, 4), dtype=np.int32)
    m = ko.subm_map(empty, 3, (0, 0, 0, 0), (0, 0, 0, 0))
    assert m.shape == (0, 27)
    one = np.array([[0, 4, 5, 6]], dtype=np.int32)
    km = ko.build_kmap(one, 3, 1, 1)
    assert km["out_in_map"].shape == (128, 27)
    assert km["out_in_map"][0, 13] == 0 and (np.delete(km["out_in_map"][0], 13) == -1).all()
    kd = ko.build_kmap(one, 2, 2, 0)
    # x=4,y=5,z=6 -> output (2,2,3) exists only where the bound (max-1)//2 allows: x: (4-1)//2=1 < 2 -> dropped
    assert kd["sizes"][1] == 0


def test_oracle_backward_matches_autograd():
    """conv_backward_from_map against torch autograd through the same sum written with dense ops (fp64)."""
    import torch

    rng = np.random.default_rng(11)
    coords = random_coords(rng, 300, (9, 9, 9), 2)
    n = coords.shape[0]
    for ks, st, pd in ((3, 1, 1), (2, 2, 0), (3, 2, 1)):
        km = ko.build_kmap(coords, ks, st, pd)
        m = km["sizes"][1]
        kvol = km["out_in_map"].shape[1]
        x, w, gy = rng.standard_normal((n, 5)), rng.standard_normal((kvol, 5, 7)), rng.standard_normal((m, 7))
        dx, dw = ko.conv_backward_from_map(x, w, km["out_in_map"], m, gy)
        xt, wt = torch.tensor(x, requires_grad=True), torch.tensor(w, requires_grad=True)
        omap = torch.tensor(km["out_in_map"][:m]).long()
        y = torch.zeros(m, 7, dtype=torch.float64)
        for k in range(kvol):
            rows = (omap[:, k] >= 0).nonzero()[:, 0]
            y = y.index_add(0, rows, xt[omap[rows, k]] @ wt[k])
        assert np.allclose(y.detach().numpy(), ko.conv_from_map(x, w, km["out_in_map"], m), atol=1e-12)
        y.backward(torch.tensor(gy))
        assert np.abs(dx - xt.grad.numpy()).max() < 1e-12 and np.abs(dw - wt.grad.numpy()).max() < 1e-12


def test_oracle_hashmap_mode_agrees_with_on_the_fly_mode_where_both_are_defined():
    """Submanifold maps and stride = kernel maps without padding are the same in the two kernel-map
    modes of the reference (same output coordinates, same neighbours); the hashmap-mode restatement is
    checked against the on-the-fly one, which is pinned by the dense-convolution equivalence above."""
    rng = np.random.default_rng(12)
    coords = random_coords(rng, 1500, (16, 14, 12), 2)
    for ks, st, pd in ((3, 1, 1), (5, 1, 2), (2, 2, 0), ((1, 2, 2), (1, 2, 2), 0)):
        a = ko.build_kmap(coords, ks, st, pd)
        b = ko.build_kmap_hashmap_mode(coords, ks, st, pd)
        assert np.array_equal(a["coords"], b["coords"]), (ks, st)
        assert np.array_equal(a["out_in_map"], b["out_in_map"]), (ks, st)


def _dense_conv_at(coords, feats, w, ks, st, pd, out_coords):
    """Dense torch conv3d (fp64) of the scattered input with kernel `ks`, stride `st`, zero padding `pd`,
    sampled at out_coords; the weight of kernel index k sits at the digits the oracle assigns to k."""
    import torch

    ks3, st3, pd3 = ko._as3(ks), ko._as3(st), ko._as3(pd)
    b = int(coords[:, 0].max()) + 1
    size = [int(coords[:, 1 + i].max()) + 1 for i in range(3)]
    cin, cout = feats.shape[1], w.shape[2]
    dense = torch.zeros((b, cin, *size), dtype=torch.float64)
    dense[coords[:, 0], :, coords[:, 1], coords[:, 2], coords[:, 3]] = torch.from_numpy(feats)
    wd = torch.zeros((cout, cin, *ks3), dtype=torch.float64)
    for k, (dx, dy, dz) in enumerate(ko.kernel_digits(ks3)):
        wd[:, :, dx, dy, dz] = torch.from_numpy(w[k]).T
    out = torch.nn.functional.conv3d(dense, wd, stride=st3, padding=pd3)
    oc = out_coords
    return out[oc[:, 0], :, oc[:, 1], oc[:, 2], oc[:, 3]].numpy()


@pytest.mark.parametrize("ks,st,pd", [(3, 2, 1), ((1, 3, 1), (1, 2, 1), (0, 1, 0)), (3, 1, 1), (3, 3, 1)])
def test_oracle_hashmap_mode_pinned_by_dense_conv(ks, st, pd):
    """kmap_mode="hashmap" with stride != kernel looks neighbours up at  out * stride + digit - (kernel - 1) / 2
    (torchsparse/backend/hashmap/hashmap_cuda.cuh:213-232), which is a dense convolution with padding
    (kernel - 1) / 2: the restatement of that mode is pinned against torch's conv3d, the way the reference's
    own test pins its kernels (tests/python/test_single_layer_conv.py:111-220)."""
    rng = np.random.default_rng(21)
    coords = random_coords(rng, 900, (13, 12, 11), 2)
    feats = rng.standard_normal((coords.shape[0], 3))
    kvol = int(np.prod(ko._as3(ks)))
    w = rng.standard_normal((kvol, 3, 4))
    km = ko.build_kmap_hashmap_mode(coords, ks, st, pd)
    m = km["sizes"][1]
    assert m > 0
    y = ko.conv_from_map(feats, w, km["out_in_map"], m)
    want = _dense_conv_at(coords, feats, w, ks, st, pd, km["coords"])
    assert np.abs(y - want).max() < 1e-12


def test_generative_kernel_map_small_case():
    """One input voxel at (1, 1, 1) of a stride-2 tensor, kernel 2, stride 2, input range 16 per axis: the range the
    strided formula derives is 8, the eight generated voxels are (2..3)^3, and only the one that equals the scaled
    input is linked to it (the lookup adds the cell offset to the OUTPUT coordinate, hashmap_cuda.cuh:215-232)."""
    km = ko.build_kmap_generative(np.array([[0, 1, 1, 1]], dtype=np.int32), 2, 2, 0, (1, 16, 16, 16))
    assert km["spatial_range"] == (1, 8, 8, 8)
    want = np.array([[0, x, y, z] for x in (2, 3) for y in (2, 3) for z in (2, 3)], dtype=np.int32)
    assert np.array_equal(km["coords"], want)
    m = km["out_in_map"][:8]
    assert m[0, 0] == 0 and (m.ravel() >= 0).sum() == 1
    # two inputs one cell apart along z: the output between them (2, 2, 3) sees the second input at cell (0, 0, 1)
    km = ko.build_kmap_generative(np.array([[0, 1, 1, 1], [0, 1, 1, 2]], dtype=np.int32), 2, 2, 0, (1, 16, 16, 16))
    row = [tuple(c) for c in km["coords"].tolist()].index((0, 2, 2, 3))
    assert km["out_in_map"][row].tolist() == [-1, 1, -1, -1, -1, -1, -1, -1]
    # clamping: the generated coordinates never leave the derived range
    km = ko.build_kmap_generative(np.array([[0, 3, 3, 3]], dtype=np.int32), 2, 2, 0, (1, 8, 8, 8))
    assert km["spatial_range"] == (1, 4, 4, 4) and km["coords"].tolist() == [[0, 3, 3, 3]]


def test_bev_restatement_on_a_case_checked_by_hand():
    """Three voxels, two of them in one column along y: the four bird's-eye-view heads on numbers small enough to
    verify on paper (oracle/bev_oracle.py restates torchsparse/nn/modules/bev.py:17-222 on batch-first rows)."""
    from oracle import bev_oracle as bo

    coords = np.array([[0, 1, 0, 2], [0, 1, 3, 2], [0, 2, 1, 0]], dtype=np.int32)      # (batch, x, y, z)
    feats = np.array([[1.0, 2.0], [3.0, 6.0], [10.0, 20.0]], dtype=np.float32)
    c, f = bo.bev_reduction(coords, feats, dim=1)
    assert c.tolist() == [[0, 1, 0, 2], [0, 2, 0, 0]]
    assert f.tolist() == [[2.0, 4.0], [10.0, 20.0]]                                    # mean over the column
    kernel = np.zeros((4, 2, 1), dtype=np.float32)                                    # layer y: f . (y + 1, 0)
    kernel[:, 0, 0] = [1.0, 2.0, 3.0, 4.0]
    c, f, stride = bo.bev_convolution(coords, feats, (1, 1, 1), kernel, None, dim=1, stride=1)
    assert c.tolist() == [[0, 1, 0, 2], [0, 2, 0, 0]] and stride == (1, 1, 1)
    assert f.tolist() == [[1.0 * 1 + 3.0 * 4], [10.0 * 2]]
    c, f, stride = bo.bev_convolution(coords, feats, (1, 1, 1), kernel, np.array([[0.5]]), dim=1, stride=4)
    assert c.tolist() == [[0, 0, 0, 0]] and stride == (4, 4, 4)                        # one 4 x 4 column left
    assert f.tolist() == [[13.0 + 20.0 + 3 * 0.5]]                                     # the bias once per voxel
    dense = bo.dense_bev_convolution(coords, feats, (1, 1, 1), kernel, None, (3, 4, 3), (0, 0, 0), dim=1)
    assert dense.shape == (1, 1, 3, 3) and dense[0, 0, 1, 2] == 13.0 and dense[0, 0, 2, 0] == 20.0
    assert dense.sum() == 33.0
    hc = bo.bev_height_compression(coords, feats, (1, 1, 1), (3, 2, 3), (0, 0, 0), dim=1)
    assert hc.shape == (1, 4, 3, 3)                                                    # 2 layers x 2 channels
    assert hc[0, :, 1, 2].tolist() == [1.0, 2.0, 3.0, 6.0]                             # y = 3 clamped into layer 1
    assert hc[0, :, 2, 0].tolist() == [0.0, 0.0, 10.0, 20.0]
