"""GPU parity of whole networks (the callers of the hot path) against the CPU oracle executor:
the package's own modules evaluated on CPU through oracle kernel maps + the reference CPU conv.

Tolerances are relative L2 of the final feature matrix / logits: fp32 1e-5 (stated in BASELINE for
network outputs), fp16 2e-3 per the same statement; the fp16 runs compare against an fp32 CPU run of
the SAME fp16-rounded weights, so what is measured is the arithmetic of the 42-layer chain."""
import numpy as np
import pytest
import torch

from conftest import rel_l2
from oracle import kmap_oracle as ko
from oracle import net_cpu

pytestmark = pytest.mark.gpu


def _scan_crop(n_target=6000, seed=0):
    from torchsparse_b200.utils.synthetic import lidar_scan

    pts = lidar_scan(seed)
    pts[:, :3] -= pts[:, :3].min(0, keepdims=True)
    vox, idx = ko.sparse_quantize(pts[:, :3], 0.05, return_index=True)
    centre = np.median(vox, axis=0)
    order = np.argsort(np.abs(vox - centre).max(axis=1), kind="stable")
    keep = np.sort(order[:n_target])
    coords = np.concatenate([np.zeros((len(keep), 1), np.int32), vox[keep]], 1).astype(np.int32)
    return coords, pts[idx[keep]].astype(np.float32)


def _randomise_bn(model):
    g = torch.Generator().manual_seed(1)
    for m in model.modules():
        if isinstance(m, torch.nn.BatchNorm1d):
            m.weight.data.uniform_(0.8, 1.2, generator=g)
            m.bias.data.uniform_(-0.1, 0.1, generator=g)
            m.running_mean.uniform_(-0.1, 0.1, generator=g)
            m.running_var.uniform_(0.8, 1.2, generator=g)


def _gpu_forward(model, coords, feats, dtype, engine):
    """engine: False = the module graph as written, True = fused inference engine (row-sorted
    column-major kernel maps, the default), "unsorted" = the engine on the maps as built."""
    import torchsparse_b200 as ts
    from torchsparse_b200.nn import InferenceEngine

    m = model.cuda().to(dtype).eval()
    if engine:
        m = InferenceEngine(m, sorted_maps=engine != "unsorted")
    x = ts.SparseTensor(torch.from_numpy(feats).cuda().to(dtype), torch.from_numpy(coords).cuda())
    with torch.no_grad():
        out = m(x)
        if engine:   # second call goes through the pre-built strided maps
            x2 = ts.SparseTensor(torch.from_numpy(feats).cuda().to(dtype), torch.from_numpy(coords).cuda())
            out2 = m(x2)
            assert torch.equal(out[-1].feats, out2[-1].feats)
    return out


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 2e-3)])
@pytest.mark.parametrize("engine", [False, True, "unsorted"])
def test_unet_matches_cpu_oracle(dtype, tol, engine):
    import copy
    from torchsparse_b200.backbones import SparseResUNet42

    torch.manual_seed(0)
    model = SparseResUNet42(in_channels=4, width_multiplier=0.5 if dtype == torch.float32 else 1.0)
    _randomise_bn(model)
    model.eval()
    coords, feats = _scan_crop()
    ref_model = copy.deepcopy(model).to(dtype).float()      # the rounded weights, evaluated in fp32 on CPU
    f_r = torch.from_numpy(feats).to(dtype).float().numpy()
    want = net_cpu.forward_cpu(ref_model, coords, f_r)
    got = _gpu_forward(copy.deepcopy(model), coords, feats, dtype, engine)
    assert len(got) == len(want) == 9
    for g, w in zip(got, want):
        assert np.array_equal(g.coords.cpu().numpy(), w.coords.numpy())     # coordinates bit-exact at every level
        assert g.stride == w.stride
    err = rel_l2(got[-1].feats.float().cpu().numpy(), want[-1].feats.numpy())
    assert err < tol, err
    err_mid = rel_l2(got[4].feats.float().cpu().numpy(), want[4].feats.numpy())   # bottleneck (stride 16)
    assert err_mid < tol, err_mid


def test_unet_fp32_tensors_under_tf32():
    """fp32 network with backends.allow_tf32 (the default on this hardware, as in the reference): every
    convolution multiplies as TF32 on the tensor cores; coordinates stay bit-exact, features within 1e-2
    of the exact-fp32 CPU evaluation after ~40 layers (10-bit mantissa operands, fp32 accumulation)."""
    import copy
    from torchsparse_b200 import backends
    from torchsparse_b200.backbones import SparseResUNet42

    torch.manual_seed(0)
    model = SparseResUNet42(in_channels=4, width_multiplier=0.5)
    _randomise_bn(model)
    model.eval()
    coords, feats = _scan_crop()
    want = net_cpu.forward_cpu(copy.deepcopy(model).float(), coords, feats)
    backends.allow_tf32 = True        # restored by the autouse fixture
    got = _gpu_forward(copy.deepcopy(model), coords, feats, torch.float32, True)
    for g, w in zip(got, want):
        assert np.array_equal(g.coords.cpu().numpy(), w.coords.numpy())
    err = rel_l2(got[-1].feats.cpu().numpy(), want[-1].feats.numpy())
    assert 1e-6 < err < 1e-2, err     # not exact (tensor cores ran), and close


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 2e-3)])
def test_resnet21d_matches_cpu_oracle(dtype, tol):
    import copy
    from torchsparse_b200.backbones import SparseResNet21D
    from torchsparse_b200.utils.synthetic import multisweep_scan

    torch.manual_seed(0)
    model = SparseResNet21D(in_channels=5)
    _randomise_bn(model)
    model.eval()
    pts = multisweep_scan(0, sweeps=3, n_rays=6000)
    xyz = pts[:, :3] - np.array([-54.0, -54.0, -5.0])
    q = np.floor(xyz / np.array([0.1, 0.1, 0.2])).astype(np.int64)
    _, idx = np.unique((q[:, 0] * 2000 + q[:, 1]) * 2000 + q[:, 2], return_index=True)
    coords = np.concatenate([np.zeros((len(idx), 1), np.int64), q[idx]], 1).astype(np.int32)
    feats = pts[idx].astype(np.float32)
    ref_model = copy.deepcopy(model).to(dtype).float()
    f_r = torch.from_numpy(feats).to(dtype).float().numpy()
    want = net_cpu.forward_cpu(ref_model, coords, f_r)
    for engine in (False, True):
        got = _gpu_forward(copy.deepcopy(model), coords, feats, dtype, engine)
        assert len(got) == len(want) == 5
        for g, w in zip(got, want):
            assert np.array_equal(g.coords.cpu().numpy(), w.coords.numpy())
            assert rel_l2(g.feats.float().cpu().numpy(), w.feats.numpy()) < tol


def test_batched_scans_equal_single_scans():
    """Scans in one batch do not interact, given a common spatial range: a 2-scan batch gives the
    concatenation of the single-scan results (what makes scan-sharding across GPUs exact).  Without a
    stated range the strided-conv output bound comes from the largest coordinate present in the whole
    batch (torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:33-37), so voxels on the
    upper boundary of one scan can depend on another scan; the range removes that coupling."""
    import torchsparse_b200 as ts
    from torchsparse_b200.backbones import SparseResUNet42

    torch.manual_seed(0)
    model = SparseResUNet42(in_channels=4, width_multiplier=0.5).cuda().eval()
    scans = [_scan_crop(3000, seed) for seed in (0, 1)]
    ext = np.max([c[:, 1:].max(0) for c, _ in scans], axis=0) + 1
    ext = tuple(int(v + (16 - v % 16) % 16) for v in ext)          # divisible by the total stride
    outs = []
    for coords, feats in scans:
        single = ts.SparseTensor(torch.from_numpy(feats).cuda(), torch.from_numpy(coords).cuda(),
                                 spatial_range=(1,) + ext)
        with torch.no_grad():
            outs.append(model(single)[-1])
    bc = np.concatenate([scans[0][0], scans[1][0] + np.array([1, 0, 0, 0], np.int32)])
    bf = np.concatenate([scans[0][1], scans[1][1]])
    batch = ts.SparseTensor(torch.from_numpy(bf).cuda(), torch.from_numpy(bc).cuda(), spatial_range=(2,) + ext)
    with torch.no_grad():
        y = model(batch)[-1]
    n0 = outs[0].feats.shape[0]
    assert y.feats.shape[0] == n0 + outs[1].feats.shape[0]
    assert torch.equal(y.coords[:n0, 1:], outs[0].coords[:, 1:]) and torch.equal(y.coords[n0:, 1:], outs[1].coords[:, 1:])
    assert bool((y.coords[n0:, 0] == 1).all())
    assert rel_l2(y.feats[:n0].cpu().numpy(), outs[0].feats.cpu().numpy()) < 1e-5
    assert rel_l2(y.feats[n0:].cpu().numpy(), outs[1].feats.cpu().numpy()) < 1e-5


def test_training_step_through_a_unet():
    """Forward + backward through the whole module graph (train mode, BatchNorm on batch statistics):
    every convolution kernel receives a finite, non-zero gradient and an SGD step lowers the loss."""
    import torchsparse_b200 as ts
    from torchsparse_b200.backbones import SparseResUNet42

    torch.manual_seed(0)
    model = SparseResUNet42(in_channels=4, width_multiplier=0.25).cuda().train()
    coords, feats = _scan_crop()
    c = torch.from_numpy(coords).cuda()
    f = torch.from_numpy(feats).cuda()
    target = torch.randn(c.shape[0], model(ts.SparseTensor(f, c))[-1].feats.shape[1], device="cuda")
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    losses = []
    for _ in range(3):
        opt.zero_grad()
        out = model(ts.SparseTensor(f, c))[-1].feats
        loss = torch.nn.functional.mse_loss(out, target)
        loss.backward()
        losses.append(float(loss.detach()))
        kernels = [p for n, p in model.named_parameters() if n.endswith("kernel")]
        assert kernels and all(p.grad is not None and torch.isfinite(p.grad).all() for p in kernels)
        assert all(float(p.grad.abs().max()) > 0 for p in kernels)
        opt.step()
    assert losses[-1] < losses[0], losses


@pytest.mark.parametrize("fused", [False, True])
def test_tune_assigns_a_config_per_group_and_keeps_results(fused):
    """utils.tune.tune_candidates: every group of convolutions sharing a kernel map gets one of the candidates,
    and the tuned model computes the same function."""
    import torchsparse_b200 as ts
    from torchsparse_b200.backbones import SparseResUNet42
    from torchsparse_b200.nn import InferenceEngine
    from torchsparse_b200.utils.tune import default_candidates, tune_candidates as tune

    torch.manual_seed(0)
    model = SparseResUNet42(in_channels=4, width_multiplier=0.5)
    _randomise_bn(model)
    model = model.cuda().half().eval()
    if fused:
        model = InferenceEngine(model)
    coords, feats = _scan_crop()
    c = torch.from_numpy(coords).cuda()
    f = torch.from_numpy(feats).cuda().half()
    with torch.no_grad():
        before = model(ts.SparseTensor(f, c))[-1].feats.float()
    choice = tune(model, [ts.SparseTensor(f, c)], warmup=1, iters=2)
    names = {name for name, _ in default_candidates()}
    assert len(choice) >= 8 and set(choice.values()) <= names
    assert any(key[3] for key in choice) and any(key[2] != (1, 1, 1) for key in choice)   # transposed, strided groups
    with torch.no_grad():
        after = model(ts.SparseTensor(f, c))[-1].feats.float()
    assert rel_l2(after.cpu().numpy(), before.cpu().numpy()) < 2e-3


def test_tuner_searches_the_reference_space_saves_and_reloads(tmp_path):
    """utils.tune.tune with the reference's arguments (torchsparse/utils/tune.py:373-386): the three dataflows with
    pruning, the table saved under save_dir/tune_tag in the reference's format, applied to the layers, the model
    unchanged in what it computes; a second call loads the table instead of measuring."""
    import torchsparse_b200 as ts
    from torchsparse_b200.backbones import SparseResUNet42
    from torchsparse_b200.nn import functional as F
    from torchsparse_b200.nn.modules.conv import Conv3d
    from torchsparse_b200.utils.tune import search_space, tune

    torch.manual_seed(0)
    model = SparseResUNet42(in_channels=4, width_multiplier=0.5)
    _randomise_bn(model)
    model = model.cuda().half().eval()
    coords, feats = _scan_crop()
    x = ts.SparseTensor(torch.from_numpy(feats).half(), torch.from_numpy(coords))
    loader = [{"input": x}, {"input": x}]
    with torch.no_grad():
        before = model(ts.SparseTensor(x.feats.cuda(), x.coords.cuda()))[-1].feats.float()
    flows = [F.Dataflow.ImplicitGEMM, F.Dataflow.FetchOnDemand, F.Dataflow.GatherScatter]
    assert len(search_space(flows)) == 8
    table = tune(model, loader, n_samples=1, collect_fn=lambda d: d["input"], enable_fp16=True, save_dir=str(tmp_path),
                 tune_tag="unet", dataflow_range=flows, dataflow_prune=True, verbose=False, skip_warning=True)
    assert len(table) >= 5
    fields = {"epsilon", "mm_thresh", "split_mask_num", "split_mask_num_bwd", "dataflow", "ifsort", "FOD_fusion"}
    assert all(set(cfg) == fields and cfg["dataflow"] in flows for cfg in table.values())
    name_to_group, saved = torch.load(tmp_path / "unet", weights_only=False)
    assert saved == table and all(g in table for g in name_to_group.values())
    convs = {n: m for n, m in model.named_modules() if isinstance(m, Conv3d) and m.kernel.dim() == 3}
    assert set(name_to_group) == set(convs)
    for n, m in convs.items():
        assert m._config["dataflow"] == table[name_to_group[n]]["dataflow"]
        assert m._config["ifsort"] == table[name_to_group[n]]["ifsort"]
    with torch.no_grad():
        after = model(ts.SparseTensor(x.feats.cuda(), x.coords.cuda()))[-1].feats.float()
    assert rel_l2(after.cpu().numpy(), before.cpu().numpy()) < 2e-3
    # the table on disk is applied to a fresh model without measuring (an empty loader would otherwise raise)
    fresh = SparseResUNet42(in_channels=4, width_multiplier=0.5).cuda().half().eval()
    again = tune(fresh, [], save_dir=str(tmp_path), tune_tag="unet", verbose=False, skip_warning=True)
    assert again == table
    got = {n: m._config["dataflow"] for n, m in fresh.named_modules() if isinstance(m, Conv3d) and m.kernel.dim() == 3}
    assert got == {n: table[name_to_group[n]]["dataflow"] for n in convs}
