"""Per-group choice of the convolution configuration from measured timings — a reduced form of
``torchsparse.utils.tune.tune`` (torchsparse/utils/tune.py:373-654).

The reference times every candidate configuration for every group of convolutions that share a
kernel map and stores the winner in each layer's config.  This module does the same search over a
small candidate list (by default: implicit GEMM on the unsorted map, implicit GEMM on the
row-sorted map) with CUDA events around every convolution module, the cost of whatever the
candidate adds to the kernel-map build (sorting, pair lists) included in the first layer of a
group that triggers it.  It works on a module graph of :class:`~torchsparse_b200.nn.Conv3d` and on
the fused inference modules alike."""
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
from torch import nn

from ..tensor import SparseTensor

__all__ = ["tune", "default_candidates"]


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


def tune(model: nn.Module, inputs: Sequence[SparseTensor], candidates: Optional[List[Tuple[str, Dict]]] = None,
         warmup: int = 1, iters: int = 3, forward: Optional[Callable] = None) -> Dict:
    """Times ``model`` on ``inputs`` once per candidate configuration, groups its sparse
    convolutions by the kernel map they share (input tensor stride, kernel size, stride, transposed)
    and gives every group the candidate with the smallest summed time.  The choice is written into
    the modules' ``_config`` and returned as ``{group: candidate name}``.  ``forward(model, x)``
    replaces the plain call when the model needs more than the tensor."""
    if not inputs:
        raise ValueError("tune needs at least one sample input")
    candidates = candidates or default_candidates()
    convs = _conv_modules(model)
    if not convs:
        return {}
    run = forward or (lambda mdl, x: mdl(x))
    records: List[Tuple[int, Tuple, torch.cuda.Event, torch.cuda.Event]] = []

    def instrument(idx: int, m: nn.Module):
        inner = m.forward

        def timed_forward(x, *args, **kwargs):
            key = (tuple(x.stride), tuple(m.kernel_size), tuple(m.stride), bool(m.transposed))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            y = inner(x, *args, **kwargs)
            e1.record()
            records.append((idx, key, e0, e1))
            return y

        m.forward = timed_forward          # instance attribute: shadows the class method

    saved = [m._config for m in convs]
    for i, m in enumerate(convs):
        instrument(i, m)
    was_training = model.training
    model.eval()
    group_of: Dict[int, Tuple] = {}
    per_candidate: List[Dict[int, float]] = []
    try:
        with torch.no_grad():
            for _, cfg in candidates:
                for m in convs:
                    m._config = cfg
                total: Dict[int, float] = {}
                for it in range(warmup + iters):
                    records.clear()
                    for x in inputs:
                        run(model, _fresh(x))
                    torch.cuda.synchronize()
                    if it < warmup:
                        continue
                    for idx, key, e0, e1 in records:
                        group_of[idx] = key
                        total[idx] = total.get(idx, 0.0) + e0.elapsed_time(e1)
                per_candidate.append(total)
    finally:
        for m, cfg in zip(convs, saved):
            m._config = cfg
            del m.forward                   # back to the class method
        model.train(was_training)

    groups: Dict[Tuple, List[int]] = {}
    for idx, key in group_of.items():
        groups.setdefault(key, []).append(idx)
    choice: Dict[Tuple, str] = {}
    for key, members in groups.items():
        sums = [sum(t.get(i, 0.0) for i in members) for t in per_candidate]
        best = min(range(len(candidates)), key=lambda c: sums[c])
        choice[key] = candidates[best][0]
        for i in members:
            convs[i]._config = candidates[best][1]
    return choice
