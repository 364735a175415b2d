"""Per-group choice of the convolution configuration from measured timings
(``torchsparse.utils.tune.tune``, torchsparse/utils/tune.py:373-654).

The reference times every candidate configuration for every group of convolutions that share a kernel map
(tensor stride, kernel size, stride, dilation), stores the winner in each layer's config and saves the table under
``save_dir/tune_tag``.  :func:`tune` has that interface, search space (dataflows; sorted / unsorted implicit GEMM
with 1-4 mask splits; fused / unfused fetch-on-demand) and file format.  Where the reference runs the whole model
once per (group, candidate) and compares wall times, this module times every convolution module with its own pair
of CUDA events, so one pass per candidate serves all groups; the cost of whatever a candidate adds to the kernel-map
build (sorting, pair lists) falls on the first layer of the group that triggers it.

:func:`tune_candidates` is the same search over an explicit candidate list on explicit inputs; it also works on
the fused inference modules."""
import os
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
from torch import nn

from ..tensor import SparseTensor

__all__ = ["tune", "tune_candidates", "default_candidates", "search_space"]


def default_candidates() -> List[Tuple[str, Dict]]:
    from ..nn import functional as F

    unsorted = F.conv_config.get_default_conv_config()
    unsorted.ifsort = False
    srt = F.conv_config.get_default_conv_config()
    srt.ifsort, srt.split_mask_num = True, 1
    return [("implicit_gemm", unsorted), ("implicit_gemm_sorted", srt)]


def _conv_modules(model: nn.Module) -> List[nn.Module]:
    from ..nn.fused import FusedConv
    from ..nn.modules.conv import Conv3d

    out = []
    for m in model.modules():
        if isinstance(m, Conv3d) and m.kernel.dim() == 3:
            out.append(m)
        elif isinstance(m, FusedConv) and not m.pointwise:
            out.append(m)
    return out


def _fresh(x: SparseTensor) -> SparseTensor:
    """The same tensor with an empty kernel-map cache (every timed forward builds its maps)."""
    return SparseTensor(x.feats, x.coords, x.stride, x.spatial_range)


def _group_by_input(m: nn.Module, x) -> Tuple:
    return (tuple(x.stride), tuple(m.kernel_size), tuple(m.stride), bool(m.transposed))


def _group_like_reference(m: nn.Module, x) -> Tuple:
    """(tensor stride of the kernel map, kernel size, stride, dilation): a transposed convolution belongs to the
    group of the strided convolution whose map it reuses (torchsparse/utils/tune.py:420-431)."""
    from .utils import make_ntuple

    st = make_ntuple(m.stride, ndim=3)
    stride = tuple(x.stride) if not m.transposed else tuple(x.stride[k] // st[k] for k in range(3))
    return (stride, tuple(make_ntuple(m.kernel_size, ndim=3)), tuple(st), tuple(make_ntuple(m.dilation, ndim=3)))


def tune_candidates(model: nn.Module, inputs: Sequence[SparseTensor],
                    candidates: Optional[List[Tuple[str, Dict]]] = None, warmup: int = 1, iters: int = 3,
                    forward: Optional[Callable] = None, with_backward: bool = False, apply: bool = True,
                    group_key: Callable = _group_by_input, only_groups: Optional[Dict[Tuple, Sequence[str]]] = None,
                    fresh: Optional[Callable] = None) -> Dict:
    """Times ``model`` on ``inputs`` once per candidate configuration, groups its sparse convolutions by the kernel
    map they share and gives every group the candidate with the smallest summed time.  The choice is written into
    the modules' ``_config`` (``apply``) and returned as ``{group: candidate name}``.  ``forward(model, x)`` replaces
    the plain call when the model needs more than the tensor.  ``with_backward`` adds the time of a backward pass
    through the summed outputs (measured for the whole model, so it only separates candidates, not groups).
    ``only_groups`` maps a group to the candidate names it may choose from (dataflow pruning).  ``fresh(x)`` gives
    the input of one timed forward (default: the same tensor with an empty kernel-map cache)."""
    if not inputs:
        raise ValueError("tune needs at least one sample input")
    candidates = candidates or default_candidates()
    convs = _conv_modules(model)
    if not convs:
        return {}
    run = forward or (lambda mdl, x: mdl(x))
    fresh = fresh or _fresh
    records: List[Tuple[int, Tuple, torch.cuda.Event, torch.cuda.Event]] = []

    def instrument(idx: int, m: nn.Module):
        inner = m.forward

        def timed_forward(x, *args, **kwargs):
            key = group_key(m, x)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            y = inner(x, *args, **kwargs)
            e1.record()
            records.append((idx, key, e0, e1))
            return y

        m.forward = timed_forward          # instance attribute: shadows the class method

    def summed(out) -> torch.Tensor:
        if isinstance(out, SparseTensor):
            return out.feats.float().sum()
        if isinstance(out, torch.Tensor):
            return out.float().sum()
        if isinstance(out, dict):
            out = list(out.values())
        return sum(summed(o) for o in out)

    saved = [m._config for m in convs]
    for i, m in enumerate(convs):
        instrument(i, m)
    was_training = model.training
    if not with_backward:
        model.eval()
    group_of: Dict[int, Tuple] = {}
    per_candidate: List[Dict[int, float]] = []
    backward_ms: List[float] = []
    try:
        with torch.set_grad_enabled(with_backward):
            for _, cfg in candidates:
                for m in convs:
                    m._config = cfg
                total: Dict[int, float] = {}
                bwd = 0.0
                for it in range(warmup + iters):
                    records.clear()
                    b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    for x in inputs:
                        out = run(model, fresh(x))
                        if with_backward:
                            b0.record()
                            summed(out).backward()
                            b1.record()
                    torch.cuda.synchronize()
                    if it < warmup:
                        continue
                    if with_backward:
                        bwd += b0.elapsed_time(b1)
                    for idx, key, e0, e1 in records:
                        group_of[idx] = key
                        total[idx] = total.get(idx, 0.0) + e0.elapsed_time(e1)
                per_candidate.append(total)
                backward_ms.append(bwd)
    finally:
        for m, cfg in zip(convs, saved):
            m._config = cfg
            del m.forward                   # back to the class method
        model.train(was_training)
        if with_backward:
            model.zero_grad(set_to_none=True)

    groups: Dict[Tuple, List[int]] = {}
    for idx, key in group_of.items():
        groups.setdefault(key, []).append(idx)
    choice: Dict[Tuple, str] = {}
    for key, members in groups.items():
        allowed = None if only_groups is None else only_groups.get(key)
        sums = [sum(t.get(i, 0.0) for i in members) + backward_ms[c] for c, t in enumerate(per_candidate)]
        order = [c for c in range(len(candidates)) if allowed is None or candidates[c][0] in allowed]
        best = min(order or range(len(candidates)), key=lambda c: sums[c])
        choice[key] = candidates[best][0]
        if apply:
            for i in members:
                convs[i]._config = candidates[best][1]
    return choice


_CONFIG_FIELDS = ("epsilon", "mm_thresh", "split_mask_num", "split_mask_num_bwd", "dataflow", "ifsort", "FOD_fusion")


def search_space(dataflow_range: Optional[Sequence] = None) -> List[Tuple[str, Dict]]:
    """Candidate configurations of the reference's stage 2 (torchsparse/utils/tune.py:197-371): implicit GEMM on the
    unsorted map and on the sorted map with 1-4 mask splits; fetch-on-demand fused and unfused; gather-scatter.  The
    reference also sweeps ``epsilon`` x ``mm_thresh`` (60 points) for gather-scatter and ``split_mask_num_bwd`` 1-4
    when tuning with backward; in this library those three fields select nothing (pair lists are not regrouped, the
    weight gradient has no mask splits), so each sweep collapses to one candidate."""
    from ..nn import functional as F

    dataflow_range = list(dataflow_range) if dataflow_range else [F.Dataflow.ImplicitGEMM]
    out: List[Tuple[str, Dict]] = []

    def cand(name: str, **fields) -> None:
        cfg = F.conv_config.get_default_conv_config()
        for k, v in fields.items():
            setattr(cfg, k, v)
        out.append((name, cfg))

    if F.Dataflow.ImplicitGEMM in dataflow_range:
        cand("ImplicitGEMM/unsorted", dataflow=F.Dataflow.ImplicitGEMM, ifsort=False, split_mask_num=1)
        for split in range(1, 5):
            cand(f"ImplicitGEMM/sorted/split{split}", dataflow=F.Dataflow.ImplicitGEMM, ifsort=True, split_mask_num=split)
    if F.Dataflow.FetchOnDemand in dataflow_range:
        for fusion in (True, False):
            cand(f"FetchOnDemand/{'fused' if fusion else 'unfused'}", dataflow=F.Dataflow.FetchOnDemand, ifsort=False,
                 FOD_fusion=fusion)
    if F.Dataflow.GatherScatter in dataflow_range:
        cand("GatherScatter", dataflow=F.Dataflow.GatherScatter, ifsort=False)
    return out


def _representatives(dataflow_range: Sequence) -> List[Tuple[str, Dict]]:
    """Stage 1 of the reference (tune.py:113-190): per dataflow its representative settings (implicit GEMM: unsorted
    and sorted with 3 splits)."""
    keep = {"ImplicitGEMM/unsorted", "ImplicitGEMM/sorted/split3", "FetchOnDemand/fused", "GatherScatter"}
    return [c for c in search_space(dataflow_range) if c[0] in keep]


def _to_device(x: Any, half: bool) -> Any:
    if isinstance(x, SparseTensor):
        feats = x.feats.cuda()
        return SparseTensor(feats.half() if half else feats, x.coords.cuda(), x.stride, x.spatial_range)
    if isinstance(x, torch.Tensor):
        x = x.cuda()
        return x.half() if (half and x.is_floating_point()) else x
    if isinstance(x, dict):
        return {k: _to_device(v, half) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_to_device(v, half) for v in x)
    return x


def tune(model: nn.Module, data_loader: Iterable, n_samples: int = 100, collect_fn: Callable = lambda data: data,
         enable_fp16: bool = False, save_dir: str = ".torchsparse-tune", tune_tag: str = "temp",
         force_retune: bool = False, dataflow_range: Optional[List] = None, dataflow_prune: bool = False,
         tune_with_bwd: bool = False, verbose: bool = True, skip_warning: bool = False) -> Dict:
    """The reference's tuner (torchsparse/utils/tune.py:373-654), same arguments and the same file
    (``torch.save((name_to_group, group_configs), save_dir/tune_tag)``, group = (tensor stride, kernel size, stride,
    dilation), config = the seven fields of ``_CONFIG_FIELDS``).  A table found on disk is applied without measuring
    unless ``force_retune``.  ``model(collect_fn(data))`` is run on up to ``n_samples`` samples of ``data_loader``;
    with ``dataflow_prune`` and several dataflows, a first pass over the representative settings fixes each group's
    dataflow and the second pass searches only inside it.  Returns ``group_configs``."""
    from .. import backends
    from ..nn import functional as F
    from ..nn.modules.conv import Conv3d

    dataflow_range = list(dataflow_range) if dataflow_range else [F.Dataflow.ImplicitGEMM]
    if not backends.benchmark:
        if not skip_warning:
            print("Warning: to use tuning, torchsparse_b200.backends.benchmark is automatically set to be true.")
        backends.benchmark = True
    path = os.path.join(save_dir, tune_tag)
    named = {name: m for name, m in model.named_modules() if isinstance(m, Conv3d) and m.kernel.dim() == 3}
    if os.path.exists(path) and not force_retune:
        if verbose:
            print("Load existing tuned group configs")
        name_to_group, group_configs = torch.load(path, weights_only=False)
    else:
        model = model.cuda()
        if enable_fp16:
            model = model.half()
        samples = []
        for i, data in enumerate(data_loader):
            if i >= n_samples:
                break
            samples.append(_to_device(collect_fn(data), enable_fp16))
        if not samples:
            raise ValueError("tune needs at least one sample from data_loader")
        fwd = lambda mdl, x: mdl(x)
        # a sample that is not a bare SparseTensor is passed on as it is (its caches are then not reset)
        fresh = _fresh if all(isinstance(smp, SparseTensor) for smp in samples) else (lambda x: x)
        candidates = search_space(dataflow_range)
        by_name = dict(candidates)
        only = None
        if dataflow_prune and len(dataflow_range) > 1:
            first = tune_candidates(model, samples, _representatives(dataflow_range), warmup=1, iters=1, forward=fwd,
                                    with_backward=tune_with_bwd, apply=False, group_key=_group_like_reference,
                                    fresh=fresh)
            only = {g: [n for n, c in candidates if c["dataflow"] == by_name[w]["dataflow"]] for g, w in first.items()}
        elif dataflow_prune and verbose:
            print(f"Only 1 dataflow ({dataflow_range[0]}) is set. Skip dataflow selecting.")
        choice = tune_candidates(model, samples, candidates, warmup=1, iters=1, forward=fwd,
                                 with_backward=tune_with_bwd, apply=False, group_key=_group_like_reference,
                                 only_groups=only, fresh=fresh)
        group_configs = {g: {f: by_name[w][f] for f in _CONFIG_FIELDS} for g, w in choice.items()}
        # which group every named layer belongs to: one instrumented pass
        name_to_group: Dict[str, Tuple] = {}
        hooks = [m.register_forward_hook(lambda mod, inp, out, name=name: name_to_group.__setitem__(
            name, _group_like_reference(mod, inp[0]))) for name, m in named.items()]
        try:
            with torch.no_grad():
                fwd(model, fresh(samples[0]))
        finally:
            for h in hooks:
                h.remove()
        if verbose:
            print("Save tuned group configs to", path)
        os.makedirs(save_dir, exist_ok=True)
        torch.save((name_to_group, group_configs), path)

    for name, m in named.items():
        g = name_to_group.get(name)
        if g is None or g not in group_configs:
            continue
        cfg = m._config
        if cfg is None:
            glb = F.conv_config.get_global_conv_config()
            cfg = glb if glb is not None else F.conv_config.get_default_conv_config()
        cfg = cfg.copy() if hasattr(cfg, "copy") else cfg
        for f in _CONFIG_FIELDS:
            setattr(cfg, f, group_configs[g][f])
        m._config = cfg
    return group_configs
