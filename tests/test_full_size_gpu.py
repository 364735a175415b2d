"""Parity at the sizes that are benchmarked: BASELINE config 2 (one full synthetic scan, ~110 k voxels,
SparseResUNet42 + head, fp16) and config 4 (SparseResNet21D on full 10-sweep scans, batch 2), each against the
CPU oracle executor (oracle kernel maps + the reference's own CPU convolution) on the same fp16-rounded weights.

Bars: coordinates of every level bit-exact; final features / logits relative L2 <= 2e-3 (fp16 operands, fp32
accumulation, one rounding per layer over a ~40-layer chain; the tolerance BASELINE states for fp16 network
outputs).  The CPU side runs single-threaded (the reference's OpenMP loops fork per row and get slower with
threads): about 15 s for config 2 and a minute for config 4."""
import copy

import numpy as np
import pytest
import torch

from conftest import rel_l2
from oracle import kmap_oracle as ko
from oracle import net_cpu

pytestmark = pytest.mark.gpu


def _bench():
    import bench
    return bench


@pytest.fixture(scope="module")
def config2():
    """The benchmark's own scan, model and CPU-oracle result (computed once for the tests below)."""
    b = _bench()
    pts = b.scan_points(0)
    model = b.make_model(None)                                   # fp32 on the CPU, the benchmark's initialisation
    vox, idx = ko.sparse_quantize(pts[:, :3], b.VOXEL, return_index=True)
    coords = np.concatenate([np.zeros((len(vox), 1), np.int32), vox], 1).astype(np.int32)
    feats = pts[idx].astype(np.float32)
    ref = copy.deepcopy(model).half().float()
    f_r = torch.from_numpy(feats).half().float().numpy()
    outs = net_cpu.forward_cpu(ref.backbone, coords, f_r, 1)
    logits = outs[-1].feats.numpy().astype(np.float64) @ ref.head.weight.detach().numpy().astype(np.float64).T \
        + ref.head.bias.detach().numpy().astype(np.float64)
    return {"pts": pts, "model": model, "coords": coords, "outs": outs, "logits": logits}


def _gpu_model(model, sorted_maps=True):
    """sorted_maps: False, True (submanifold maps up to stride 8) or "all" (every map of every level: the
    benchmark's setting)."""
    from torchsparse_b200.nn import InferenceEngine

    m = copy.deepcopy(model).cuda().half()
    if sorted_maps == "all":
        m.backbone = InferenceEngine(m.backbone, sorted_maps=True, sorted_max_stride=16, sorted_strided=True)
    else:
        m.backbone = InferenceEngine(m.backbone, sorted_maps=sorted_maps)
    return m


@pytest.mark.parametrize("sorted_maps", [True, False, "all"])
def test_config2_full_scan_eager_engine(config2, sorted_maps):
    """The benchmark's public-API path (bench.forward_scan without the head) at full size."""
    import torchsparse_b200 as ts

    b = _bench()
    m = _gpu_model(config2["model"], sorted_maps)
    pts = torch.from_numpy(config2["pts"]).cuda()
    vox, feats, vmax = b.scan_tensor(pts)
    coords = torch.nn.functional.pad(vox, (1, 0))
    assert np.array_equal(coords.cpu().numpy(), config2["coords"])          # voxelisation bit-exact
    x = ts.SparseTensor(feats, coords, coord_bounds=((0, 0, 0, 0), (0,) + tuple(vmax)))
    with torch.no_grad():
        outs = m.backbone(x)
        logits = m.head(outs[-1].feats)
    assert len(outs) == len(config2["outs"]) == 9
    for g, w in zip(outs, config2["outs"]):
        assert g.stride == w.stride
        assert np.array_equal(g.coords.cpu().numpy(), w.coords.numpy())   # coordinates of every level bit-exact
    assert rel_l2(outs[-1].feats.float().cpu().numpy(), config2["outs"][-1].feats.numpy()) < 2e-3
    assert rel_l2(logits.float().cpu().numpy(), config2["logits"]) < 2e-3


def test_config2_full_scan_graph_engine(config2):
    """What bench.py times: the CUDA-graph engine with the benchmark's bounds, on the benchmark's scan."""
    b = _bench()
    m = _gpu_model(config2["model"], "all")
    eng = b.make_engines(m, torch.device("cuda", 0), 1)[0]
    out, rec = eng(torch.from_numpy(config2["pts"]).cuda())
    eng.stream.synchronize()
    eng.check()
    n = int(rec[0].item())
    assert n == config2["coords"].shape[0]
    assert rel_l2(out[:n].float().cpu().numpy(), config2["logits"]) < 2e-3
    # a second scan through the same graph, then the first again: replays do not depend on what ran before
    first = out[:n].clone()
    eng(torch.from_numpy(b.scan_points(1)).cuda())
    out, rec = eng(torch.from_numpy(config2["pts"]).cuda())
    eng.stream.synchronize()
    assert int(rec[0].item()) == n and torch.equal(out[:n], first)


def test_config4_resnet21d_full_sweeps_batch2():
    """SparseResNet21D on two full 10-sweep scans collated with the config's spatial range (k3 s2 p0 strided
    maps that create more outputs than inputs, and the (1,3,1) / (1,2,1) last stage)."""
    b = _bench()
    model = b.make_model(None, kind="det")
    ref = copy.deepcopy(model).half().float()
    scans = [b.c4_points(7000 + i) for i in range(2)]
    rows, feats = [], []
    for i, pts in enumerate(scans):
        vox, idx = ko.sparse_quantize(pts[:, :3], b.C4_VOXEL, return_index=True)
        rows.append(np.concatenate([np.full((len(vox), 1), i, np.int32), vox], 1))
        feats.append(pts[idx])
    coords = np.concatenate(rows).astype(np.int32)
    feats = np.concatenate(feats).astype(np.float32)
    f_r = torch.from_numpy(feats).half().float().numpy()

    from torchsparse_b200.tensor import SparseTensor
    x_cpu = SparseTensor(torch.from_numpy(f_r), torch.from_numpy(coords), spatial_range=(2,) + b.C4_RANGE)
    torch.set_num_threads(1)
    with torch.no_grad(), net_cpu.cpu_conv():
        want = ref.backbone.cpu().float().eval()(x_cpu)

    m = _gpu_model(model)
    with torch.no_grad():
        got_feats = b.forward_batch(m, [torch.from_numpy(p).cuda() for p in scans], b.C4_VOXEL, b.C4_RANGE)
        # the same batch once more for the per-stage outputs
        import torchsparse_b200 as ts
        from torchsparse_b200.utils.collate import sparse_collate
        items = []
        for p in scans:
            vox, f, _ = b.scan_tensor(torch.from_numpy(p).cuda(), b.C4_VOXEL)
            items.append(ts.SparseTensor(f, vox))
        x = sparse_collate(items)
        x.spatial_range = (2,) + tuple(b.C4_RANGE)
        got = m.backbone(x)
    assert len(got) == len(want) == 5
    for g, w in zip(got, want):
        assert np.array_equal(g.coords.cpu().numpy(), w.coords.numpy())
        assert rel_l2(g.feats.float().cpu().numpy(), w.feats.numpy()) < 2e-3
    assert torch.equal(got_feats, got[-1].feats)
