"""One rank of the multi-GPU batch test (started by tests/test_gpu_multi.py through torch.distributed.run):
renders its share of the views, takes part in the exchange step and, on rank 0, saves the reduced buffers."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def workload(device):
    import synthetic_workloads as syn
    tree = syn.adaptive_octree(4096, seed=1, min_level=3, max_level=6).to(device)
    n = 1 << 16
    feats = syn.sh_features(n, 12, "normal", 0.5).to(device)
    opac = syn.opacities_sigmoid(n, 13).to(device)
    views = [v.to(device) for v in syn.orbit_views(10, seed=2, width=256, height=160, focal=200.0)]
    g = torch.Generator().manual_seed(5)
    gi = (torch.randn((4, 160, 256), generator=g) * 1e-3).to(device)
    ga = (torch.randn((1, 160, 256), generator=g) * 1e-3).to(device)
    return tree, n, feats, opac, views, gi, ga


def run(rank, world, device):
    from inpc_b200.batch import ViewShardedTrainer
    tree, n, feats, opac, views, gi, ga = workload(device)
    tr = ViewShardedTrainer(tree, feats, opac, n, seed=0, n_appearance=1 << 12, n_streams=2)
    tr.run_batch(views, (gi, ga), rank, world)
    torch.cuda.synchronize()
    return tr.buffers.leaf.max_sampled.cpu(), tr.buffers.leaf.min_sampled.cpu(), tr.buffers.appearance.cpu()


if __name__ == "__main__":
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    out = run(rank, world, torch.device("cuda", local))
    if rank == 0:
        torch.save(out, sys.argv[1])
    dist.barrier()
    dist.destroy_process_group()
