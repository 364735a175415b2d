"""Generate the golden fixtures in this directory from the REFERENCE project itself.

Run in a container that has a checkout of the reference project (its path is the optional first argument):

    python oracle/build_ref.py            # compiles the reference's CPU sources -> oracle/_ref/
    python tests/golden/make_golden.py

What comes from reference code:
  * conv outputs: the reference's own CPU convolution
    (torchsparse/backend/convolution/convolution_gather_scatter_cpu.cpp), fed pair lists;
  * sparse_quantize: the reference's numpy routine (torchsparse/utils/quantize.py), imported by path;
  * kernel offsets: torchsparse/nn/utils/kernel.py:get_kernel_offsets, imported by path;
  * hash / count / voxelize / devoxelize: the reference's CPU sources.
The reference has no CPU kernel-map builder, so the pair lists come from oracle/kmap_oracle.py; they
are pinned the way the reference's own test pins them (tests/python/test_single_layer_conv.py):
by equality of the sparse result with a dense torch.nn.functional.conv3d on the densified input,
whose output at the sparse output coordinates is stored too.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"

from oracle import build_ref, kmap_oracle as ko  # noqa: E402


def _load_by_path(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_reference_python():
    """Import the pure-Python pieces of the reference without importing its package
    (the package needs a GPU and the absent `rootpath`)."""
    pkg = types.ModuleType("torchsparse")
    pkg.__path__ = []
    sys.modules["torchsparse"] = pkg
    utils_pkg = types.ModuleType("torchsparse.utils")
    utils_pkg.__path__ = []
    sys.modules["torchsparse.utils"] = utils_pkg
    u = _load_by_path("torchsparse.utils.utils", os.path.join(REF, "torchsparse/utils/utils.py"))
    utils_pkg.make_ntuple, utils_pkg.make_tensor = u.make_ntuple, u.make_tensor
    q = _load_by_path("torchsparse.utils.quantize", os.path.join(REF, "torchsparse/utils/quantize.py"))
    k = _load_by_path("ts_ref_kernel", os.path.join(REF, "torchsparse/nn/utils/kernel.py"))
    return q.sparse_quantize, k.get_kernel_offsets


def dense_conv_at(coords, feats, W, ks, st, pad, out_coords, shape, B):
    """Dense conv3d of the densified input, sampled at out_coords (fp64)."""
    ks, st = ko._as3(ks), ko._as3(st)
    cin, cout = W.shape[1], W.shape[2]
    dense = np.zeros((B, cin) + tuple(shape))
    dense[coords[:, 0], :, coords[:, 1], coords[:, 2], coords[:, 3]] = feats
    digits = ko.kernel_digits(ks)
    Wd = np.zeros((cout, cin) + ks)
    for k in range(W.shape[0]):
        Wd[:, :, digits[k, 0], digits[k, 1], digits[k, 2]] = W[k].T
    x = torch.from_numpy(dense)
    if all(s == 1 for s in st):
        padl = []
        for k in reversed(ks):
            padl += [(k - 1) // 2, (k - 1) // 2] if k % 2 == 1 else [0, k - 1]
        y = torch.nn.functional.conv3d(torch.nn.functional.pad(x, padl), torch.from_numpy(Wd))
    else:
        y = torch.nn.functional.conv3d(x, torch.from_numpy(Wd), stride=st, padding=ko._as3(pad))
    y = y.numpy()
    return y[out_coords[:, 0], :, out_coords[:, 1], out_coords[:, 2], out_coords[:, 3]]


def main():
    ref = build_ref.load()
    ref_quantize, ref_offsets = load_reference_python()
    rng = np.random.default_rng(20240521)
    out = {}

    cases = [("k3s1", 3, 1), ("k2s2", 2, 2), ("k3s2", 3, 2), ("k131s121", (1, 3, 1), (1, 2, 1)), ("k2s1", 2, 1),
             ("k5s1", 5, 1), ("k3s3", 3, 3)]
    shape, B, n_per, cin, cout = (11, 9, 10), 2, 170, 8, 16
    for name, ks, st in cases:
        ks3, st3 = ko._as3(ks), ko._as3(st)
        pad = tuple((k - 1) // 2 if (k % 2 == 1 and s == 1) else 0 for k, s in zip(ks3, st3))
        coords = []
        for b in range(B):
            lin = rng.choice(int(np.prod(shape)), n_per, replace=False)
            coords.append(np.concatenate([np.full((n_per, 1), b), np.stack(np.unravel_index(lin, shape), 1)], 1))
        coords = np.concatenate(coords).astype(np.int32)
        feats = rng.standard_normal((coords.shape[0], cin)).astype(np.float32)
        kvol = int(np.prod(ks3))
        W = (rng.standard_normal((kvol, cin, cout)) / np.sqrt(kvol * cin)).astype(np.float32)
        km = ko.build_kmap(coords, ks3, st3, pad)
        nbmaps, nbsizes = ko.pairs_from_map(km["out_in_map"])
        m = km["sizes"][1]
        y = torch.zeros(m, cout)
        ref.conv_forward_gather_scatter_cpu(torch.from_numpy(feats), y, torch.from_numpy(W),
                                            torch.from_numpy(nbmaps), torch.from_numpy(nbsizes), False)
        dense = dense_conv_at(coords, feats.astype(np.float64), W.astype(np.float64), ks3, st3, pad, km["coords"],
                              shape, B)
        assert np.abs(dense - y.numpy()).max() < 1e-4, name
        out[f"{name}/coords"], out[f"{name}/feats"], out[f"{name}/weight"] = coords, feats, W
        out[f"{name}/ref_cpu_out"] = y.numpy()
        out[f"{name}/dense_out"] = dense.astype(np.float32)
        out[f"{name}/out_coords"] = km["coords"].astype(np.int32)
        out[f"{name}/offsets"] = ref_offsets(ks3).numpy()
        if any(s > 1 for s in st3):
            # the matching transposed conv: input on the coarse coords, output on the fine ones
            xt = rng.standard_normal((m, cout)).astype(np.float32)
            Wt = (rng.standard_normal((kvol, cout, cin)) / np.sqrt(kvol * cout)).astype(np.float32)
            yt = torch.zeros(coords.shape[0], cin)
            ref.conv_forward_gather_scatter_cpu(torch.from_numpy(xt), yt, torch.from_numpy(Wt),
                                                torch.from_numpy(nbmaps), torch.from_numpy(nbsizes), True)
            out[f"{name}/t_feats"], out[f"{name}/t_weight"], out[f"{name}/t_ref_cpu_out"] = xt, Wt, yt.numpy()

    # sparse_quantize from the reference's numpy code
    pts = (rng.standard_normal((3000, 3)) * 3.0).astype(np.float32)
    pts[::7] = pts[1::7][: len(pts[::7])]  # duplicates
    for tag, vs in (("q05", 0.05), ("q37", (0.3, 0.7, 0.25))):
        c, idx, inv = ref_quantize(pts, vs, return_index=True, return_inverse=True)
        out[f"{tag}/points"], out[f"{tag}/coords"], out[f"{tag}/index"], out[f"{tag}/inverse"] = pts, c, idx, inv
    pts64 = rng.uniform(-20, 20, size=(2000, 3))
    c, idx, inv = ref_quantize(pts64, 0.1, return_index=True, return_inverse=True)
    out["q64/points"], out["q64/coords"], out["q64/index"], out["q64/inverse"] = pts64, c, idx, inv

    # hash / count / voxelize / devoxelize from the reference's CPU sources
    hc = rng.integers(-50, 1000, size=(500, 4)).astype(np.int32)
    out["hash/coords"] = hc
    out["hash/ref_cpu_fold60"] = ref.hash_cpu(torch.from_numpy(hc)).numpy()
    offs = ref_offsets(3).numpy()
    # the CPU kernel-hash shifts columns 0..2 and keeps column 3 (hash_cpu.cpp:26-41): feed it (x,y,z,b)
    out["hash/kernel_ref_cpu_fold60_xyzb"] = ref.kernel_hash_cpu(torch.from_numpy(hc), torch.from_numpy(offs)).numpy()
    n_pts, n_vox, c = 400, 90, 6
    idx = rng.integers(0, n_vox, size=n_pts).astype(np.int32)
    idx[::11] = -1
    cnt = ref.count_cpu(torch.from_numpy(idx), n_vox).numpy()
    pf = rng.standard_normal((n_pts, c)).astype(np.float32)
    idx_ok = np.where(idx < 0, 0, idx).astype(np.int32)
    vox = ref.voxelize_forward_cpu(torch.from_numpy(pf), torch.from_numpy(idx_ok), torch.from_numpy(cnt)).numpy()
    out["pts/idx"], out["pts/counts"], out["pts/feats"], out["pts/idx_nonneg"], out["pts/voxelized"] = idx, cnt, pf, idx_ok, vox
    di = rng.integers(-1, n_vox, size=(n_pts, 8)).astype(np.int32)
    dw = rng.uniform(0, 1, size=(n_pts, 8)).astype(np.float32)
    vf = rng.standard_normal((n_vox, c)).astype(np.float32)
    dv = ref.devoxelize_forward_cpu(torch.from_numpy(vf), torch.from_numpy(di), torch.from_numpy(dw)).numpy()
    out["devox/indices"], out["devox/weights"], out["devox/vox_feats"], out["devox/out"] = di, dw, vf, dv

    path = os.path.join(HERE, "golden_v1.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
