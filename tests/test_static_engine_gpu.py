"""The CUDA-graph engine (sizes in device memory, one graph launch per scan) against the eager inference
engine on the same scans: the voxel count and the features of the finest decoder level must be bit-identical
for the valid rows (the same kernels run on the same rows; only where the row counts live differs), and one
captured graph must serve scans of different sizes.  (The linear head is left out of the comparison: a
library GEMM may pick another tiling for another row count.)"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
VOXEL = 0.05


def _net(width=0.5, in_channels=4):
    from torchsparse_b200.backbones import SparseResUNet42

    torch.manual_seed(0)
    net = SparseResUNet42(in_channels=in_channels, width_multiplier=width)
    g = torch.Generator().manual_seed(1)
    for m in net.modules():
        if isinstance(m, torch.nn.BatchNorm1d):
            m.weight.data.uniform_(0.8, 1.2, generator=g)
            m.bias.data.uniform_(-0.1, 0.1, generator=g)
            m.running_mean.uniform_(-0.1, 0.1, generator=g)
            m.running_var.uniform_(0.8, 1.2, generator=g)
    head = torch.nn.Linear(int(96 * width), 19)
    return net.eval().cuda().half(), head.cuda().half()


def _scan(seed, n_rays):
    from torchsparse_b200.utils.synthetic import lidar_scan

    pts = lidar_scan(seed, n_rays=n_rays)
    pts[:, :3] -= pts[:, :3].min(0, keepdims=True)
    return torch.from_numpy(pts).cuda()


def _eager(engine, head, pts):
    import torchsparse_b200 as ts
    from torchsparse_b200.utils import sparse_quantize

    vox, idx, (vmin, vmax) = sparse_quantize(pts[:, :3], VOXEL, return_index=True, return_bounds=True)
    coords = torch.nn.functional.pad(vox, (1, 0))
    feats = torch.nn.functional.pad(torch.index_select(pts, 0, idx).half(), (0, 4))
    x = ts.SparseTensor(feats, coords, coord_bounds=((0, 0, 0, 0), (0,) + tuple(vmax)))
    with torch.no_grad():
        outs = engine(x)
        return coords, outs[-1].feats


@pytest.mark.parametrize("overlap_maps", [True, False])
@pytest.mark.parametrize("sorted_maps", [True, False, "all"])
def test_static_engine_equals_eager_engine(sorted_maps, overlap_maps):
    """Bit-equal to the eager engine, with the kernel maps recorded on a side branch of the graph or in line."""
    from torchsparse_b200.nn import InferenceEngine, StaticEngine

    net, head = _net()
    # the first layer's kernel with its 4 input channels zero-padded to the 8 the engines feed it
    conv0 = net.stem[0]
    conv0.kernel = torch.nn.Parameter(torch.nn.functional.pad(conv0.kernel.data, (0, 0, 0, 4)), requires_grad=False)
    conv0.in_channels = 8
    if sorted_maps == "all":       # row-sorted copies of every map: strided, transposed and the coarsest level too
        engine = InferenceEngine(net, sorted_maps=True, sorted_max_stride=16, sorted_strided=True)
        sorted_maps = True
    else:
        engine = InferenceEngine(net, sorted_maps=sorted_maps)
    scans = [_scan(s, n) for s, n in ((0, 20000), (1, 12000), (2, 20000))]
    max_points = max(p.shape[0] for p in scans)
    ext = [int(max(float(p[:, d].max()) for p in scans) / VOXEL) + 8 for d in range(3)]
    static = StaticEngine(engine, lambda outs: outs[-1].feats, max_points=max_points, point_channels=4,
                          voxel_size=VOXEL, max_extent=ext, device=torch.device("cuda", 0), sorted_maps=sorted_maps,
                          overlap_maps=overlap_maps)
    static.capture()
    for pts in scans:
        coords, want = _eager(engine, head, pts)
        out, rec = static(pts)
        static.stream.synchronize()
        static.check()
        n = int(rec[0].item())
        assert n == want.shape[0]
        assert torch.equal(out[:n], want)


def test_static_engine_reports_a_scan_beyond_its_bounds():
    from torchsparse_b200.nn import InferenceEngine, StaticEngine

    net, head = _net()
    conv0 = net.stem[0]
    conv0.kernel = torch.nn.Parameter(torch.nn.functional.pad(conv0.kernel.data, (0, 0, 0, 4)), requires_grad=False)
    conv0.in_channels = 8
    engine = InferenceEngine(net)
    pts = _scan(0, 8000)
    static = StaticEngine(engine, lambda outs: outs[-1].feats, max_points=pts.shape[0], point_channels=4,
                          voxel_size=VOXEL, max_extent=[64, 64, 16], device=torch.device("cuda", 0))
    static(pts)
    static.stream.synchronize()
    with pytest.raises(RuntimeError):
        static.check()
