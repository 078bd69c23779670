"""One rank of the two-process peer-window test (launched by
tests/test_gpu_ep.py through torch.distributed.run).  Writes this rank's
output rows of the last step to <outdir>/out_<rank>.npy."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tests.conftest import load_package  # noqa: E402


def main():
    outdir, T, steps = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    use_graph = len(sys.argv) > 4 and sys.argv[4] == "1"
    mode = sys.argv[5] if len(sys.argv) > 5 else "pull"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    os.environ["APUS_CUDA_DEVICE"] = str(local)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", local))
    pkg = load_package()
    from apus_b200 import ep, synth
    be = pkg.Backend()
    be.enable()
    cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128, top_k=8)
    W = synth.host_weights(be, cfg, seed=13, sigma=0.05)
    per = cfg["experts"] // world
    layer = be.layer_create(cfg, W, rank * per, (rank + 1) * per)
    blk = ep.PeerWindowBlock(be, layer, cfg, rank, world, T, device_epoch=use_graph,
                             mode=mode)
    out = None
    d_x = torch.empty((T, cfg["hidden"]), dtype=torch.int16, device="cuda")
    graph = None
    for s in range(steps):
        x = synth.host_x(be, T * world, cfg["hidden"], seed=100 + s)
        mine = np.ascontiguousarray(x[rank * T:(rank + 1) * T]).view(np.int16)
        d_x.copy_(torch.from_numpy(mine))
        if not use_graph:
            out = blk.forward(d_x)
        elif s == 0:
            out = blk.forward(d_x)             # workspaces grow outside the capture
            torch.cuda.synchronize()
            dist.barrier()
            stream = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                out = blk.forward(d_x)
        else:
            graph.replay()
    torch.cuda.synchronize()
    status = be.last_block_status()
    np.save(os.path.join(outdir, f"out_{rank}.npy"),
            out.cpu().numpy().view(np.uint16))
    dist.barrier()
    blk.close()
    dist.destroy_process_group()
    sys.exit(0 if status == 0 else 3)


if __name__ == "__main__":
    main()
