"""Worker of tests/test_multi_gpu.py (run under torch.distributed.run, one process per GPU): every rank pushes its
shard of the scans through the CUDA-graph engine and the logits are gathered with PaddedGather; rank 0 then runs
all scans by itself and compares, bit for bit, with what the gather delivered."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main() -> None:
    import bench
    from torchsparse_b200.sharding import PaddedGather, shard_range

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    n_scans = 2 * world
    rays = 30000                                             # small scans: the test is about the exchange
    from torchsparse_b200.utils.synthetic import lidar_scan

    def points(i):
        p = lidar_scan(100 + i, n_rays=rays)
        p[:, :3] -= p[:, :3].min(0, keepdims=True)
        return torch.from_numpy(p).to(device)

    model = bench.make_model(device)
    from torchsparse_b200.nn import StaticEngine
    max_points = int(rays * 1.2)
    eng = StaticEngine(model.backbone, lambda outs: model.head(outs[-1].feats), max_points=max_points, point_channels=4,
                       voxel_size=bench.VOXEL, max_extent=bench.MAX_EXTENT, device=device).capture()
    gather = PaddedGather(max_points, bench.NUM_CLASSES, torch.float16, device)
    lo, hi = shard_range(n_scans, world, rank)
    got = []
    for i in range(lo, hi):
        out, rec = eng(points(i))
        with torch.cuda.stream(eng.stream):
            buf, counts = gather(out, rec[:1])
            got.append((buf.clone(), counts.clone()))
        eng.stream.synchronize()
    eng.check()
    ok = True
    if rank == 0:
        for step, (buf, counts) in enumerate(got):
            for r in range(world):
                scan = shard_range(n_scans, world, r)[0] + step
                out, rec = eng(points(scan))
                eng.stream.synchronize()
                n = int(rec[0].item())
                ok = ok and n == int(counts[r].item()) and n > 1000 and torch.equal(buf[r, :n], out[:n])
    flag = torch.tensor([1 if ok else 0], device=device)
    dist.broadcast(flag, 0)
    dist.destroy_process_group()
    if rank == 0:
        print("SHARDED_OK" if ok else "SHARDED_MISMATCH", flush=True)
    sys.exit(0 if int(flag.item()) else 1)


if __name__ == "__main__":
    main()
