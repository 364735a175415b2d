"""Per-K-block timeline of one CTA of the implicit-GEMM kernel (a debugging aid).

Needs a library built with the trace points compiled in:

    TSB_NVCC_EXTRA=-DTSB_TRACE_BUILD python torchsparse_b200/csrc/build.py --force
    python torchsparse_b200/csrc/trace_blocks.py N CIN COUT OCCUPANCY [CTA]
    python torchsparse_b200/csrc/build.py --force          # back to the production build

Runs one k3 s1 fp16 convolution on N uniform voxels three times and prints, for the first 256 K blocks of
CTA number CTA (default 3) of the last launch, the %clock64 stamps of: gather side at the block / got
the stage / copies issued; MMA warp at the block / saw the stage full / committed; then the mean, median,
min and max of the intervals between them over the steady state."""
import os
import sys

import numpy as np
import torch


def main() -> None:
    n, cin, cout, occ = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), float(sys.argv[4])
    buf = torch.zeros(256 * 8, dtype=torch.int64, device="cuda")
    os.environ["TSB_UMMA_TRACE"] = str(buf.data_ptr())            # read by the library at every launch
    os.environ["TSB_UMMA_TRACE_CTA"] = sys.argv[5] if len(sys.argv) > 5 else "3"
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
    import torchsparse_b200 as ts
    from torchsparse_b200.nn import functional as F
    from torchsparse_b200.utils.synthetic import uniform_voxels

    coords = torch.from_numpy(uniform_voxels(0, n, occ)[0]).cuda()
    x = ts.SparseTensor(torch.randn(coords.shape[0], cin, device="cuda").half(), coords)
    w = (torch.randn(27, cin, cout, device="cuda") * 0.05).half()
    for _ in range(3):
        buf.zero_()
        F.conv3d(x, w, 3, None, 1, 1)
        torch.cuda.synchronize()
    t = buf.cpu().numpy().reshape(256, 8)
    blocks = int((t[:, 6] > 0).sum())
    if blocks == 0:
        raise SystemExit("no stamps: the library was not built with -DTSB_TRACE_BUILD (or the CTA ran no block)")
    t0 = t[:, :7][t[:, :7] > 0].min()
    print(f"voxels {coords.shape[0]}  {cin}->{cout}  blocks traced {blocks}")
    print("block | gather: at block, got stage, issued | - | mma: at block, full, committed")
    for b in range(blocks):
        print(b, *[int(v - t0) if v > 0 else -1 for v in t[b, :7]])
    lo, hi = 16, blocks - 8
    if hi - lo < 8:
        return
    rows = t[lo:hi]
    print("cycles/block", (t[hi - 1, 6] - t[lo, 6]) / (hi - 1 - lo))
    for name, a in (("gather wait for stage", rows[:, 1] - rows[:, 0]), ("gather issue", rows[:, 2] - rows[:, 1]),
                    ("issue -> mma sees full", rows[:, 5] - rows[:, 2]), ("mma wait", rows[:, 5] - rows[:, 4]),
                    ("mma issue + commit", rows[:, 6] - rows[:, 5])):
        print(f"{name:24s} mean {a.mean():8.0f} median {np.median(a):8.0f} min {a.min():8.0f} max {a.max():8.0f}")


if __name__ == "__main__":
    main()
