"""bench.py's multi-GPU arm: the expert-parallel block over NCCL, one process
per GPU (launched by torch.distributed.run)."""
import json
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist


def run(args, cfg, config, pkg, synth, metric, unit, peaks, clock_sampler=None):
    from . import ep
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    os.environ.setdefault("APUS_CUDA_DEVICE", str(local))
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", local))
    be = pkg.Backend()
    be.enable()
    H, E = cfg["hidden"], cfg["experts"]
    T = args.tokens                      # tokens per rank (weak scaling)
    per = E // world
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    sp = stream.cuda_stream
    # this rank's experts, generated in place in HBM
    layer = be.layer_create(cfg, None, rank * per, (rank + 1) * per)
    synth.device_weights(be, layer, cfg, seed=args.seed, layer=0,
                         expert_begin=rank * per, stream=sp)
    x_all = synth.host_x(be, T * world, H, seed=args.seed)
    x_host = np.ascontiguousarray(x_all[rank * T:(rank + 1) * T]).view(np.int16)
    d_x = torch.from_numpy(x_host).cuda()
    exchange = getattr(args, "exchange", "peer")
    exchange_note = None
    if exchange == "peer":
        # every rank must take the same arm: agree on whether the windows came up
        ok = torch.ones(1, device="cuda")
        try:
            blk = ep.PeerWindowBlock(be, layer, cfg, rank, world, T, device_epoch=True)
        except Exception as e:             # e.g. no peer access between two GPUs
            exchange_note = f"{type(e).__name__}: {e}"
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) == 0.0:
            if rank == 0:
                print(f"peer windows unavailable ({exchange_note}); using the NCCL "
                      "all-to-all exchange", file=sys.stderr)
            exchange = "nccl"
    if exchange != "peer":
        blk = ep.EPBlock(ep.CudaOps(be, layer, cfg), cfg, rank, world)

    def step():
        return blk.forward(d_x)

    out = step()
    l_one = be.launches()
    out = step()
    per_step = be.launches() - l_one        # kernels of one step (host launches)
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    # The window step has no host synchronisation and no collective call, and
    # its step number lives on the device: capture it once, replay it.
    use_graph = exchange == "peer" and not getattr(args, "no_graph", False)
    if use_graph:
        dist.barrier()
        ok = torch.ones(1, device="cuda")
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                out_g = blk.forward(d_x)
        except Exception as e:
            print(f"rank {rank}: graph capture failed ({type(e).__name__}: {e}); "
                  "host launches", file=sys.stderr)
            ok.zero_()
        torch.cuda.synchronize()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)      # all ranks take the same arm
        use_graph = float(ok.item()) != 0.0
    if use_graph:
        def step():
            graph.replay()
            return out_g
        for _ in range(2):
            step()
        torch.cuda.synchronize()
    sampler = None
    if rank == 0 and clock_sampler is not None:
        sampler = clock_sampler(local)       # SM clock and throttle reasons of GPU 0
        sampler.start()
    dist.barrier()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    l0 = be.launches()
    e0.record(stream)
    for _ in range(args.steps):
        out = step()
    e1.record(stream)
    # a replayed graph launches the kernels that one captured step launched
    n_launched = per_step * args.steps if use_graph else be.launches() - l0
    launches = torch.tensor([float(n_launched)], device="cuda")
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    status = be.last_block_status()

    # end to end: pinned host input -> device, block, result back to host
    xin = torch.from_numpy(x_host).pin_memory()
    hout = torch.empty_like(xin).pin_memory()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        d_x.copy_(xin, non_blocking=True)
        o = step()
        hout.copy_(o, non_blocking=True)
        torch.cuda.synchronize()
    e2e = torch.tensor([(time.perf_counter() - t0) * 1e3 / args.steps],
                       device="cuda")
    dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e.item())
    if exchange == "peer":
        # rows that left this GPU: assignments owned by another rank
        idx = torch.empty((T, cfg["top_k"]), dtype=torch.int32, device="cuda")
        w_ = torch.empty((T, cfg["top_k"]), dtype=torch.int16, device="cuda")
        sgl_ = torch.empty((T,), dtype=torch.int16, device="cuda")
        be.ep_route_dev(layer, d_x.data_ptr(), T, idx.data_ptr(), w_.data_ptr(),
                        sgl_.data_ptr(), stream=sp)
        torch.cuda.synchronize()
        sent = int(((idx // per) != rank).sum().item())
        rows = torch.tensor([sent, sent], dtype=torch.float64, device="cuda")
    else:
        rows = torch.tensor([blk.last_sent_rows, blk.last_recv_rows],
                            dtype=torch.float64, device="cuda")
    dist.all_reduce(rows, op=dist.ReduceOp.SUM)
    dist.all_reduce(launches, op=dist.ReduceOp.SUM)
    if sampler is not None:
        sampler.stop_flag = True
        sampler.join()
    if rank == 0:
        Tg = T * world
        cfgline = dict(config)
        cfgline["workload"] = (f"one MoE layer, expert-parallel over {world} "
                               f"GPUs ({per} experts per GPU), {T} tokens per "
                               f"GPU, uniform router, seed {args.seed}")
        cfgline["tokens_per_step"] = Tg
        cfgline["parallelism"] = f"ep{world}"
        cfgline["launch"] = "cuda graph replay" if use_graph else "host launches"
        line = {
            "metric": metric, "value": Tg / (ms * 1e-3), "unit": unit,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 storage, fp32 accumulate",
            "data": "synthetic", "config": cfgline,
            "e2e": {"value": Tg / (e2e_ms * 1e-3), "unit": unit,
                    "h2d_bytes_per_step": Tg * H * 2,
                    "d2h_bytes_per_step": Tg * H * 2, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches.item()),
            "exchange": {"rows_sent_per_step": float(rows[0]),
                         "bytes_each_way_per_step": float(rows[0]) * H * 2,
                         "requested": getattr(args, "exchange", "peer"),
                         "collective": ("none: kernels store rows into the owner's "
                                        "memory over NVLink (CUDA IPC windows)"
                                        if exchange == "peer" else
                                        "all_to_all_single (NCCL), rows as bytes")},
            "block": {"device_status": status},
        }
        if sampler is not None:
            line["clocks"] = sampler.summary()
        # what one GPU must read per step: its experts (all touched at these
        # sizes), the shared expert, the router, its token slice in and out
        I, Is = cfg["moe_inter"], cfg["shared_inter"]
        per_gpu = ((per * 3 * I * H + 3 * Is * H + E * H + H) * 2
                   + 2 * T * H * 2 + 2 * float(rows[0]) / world * H * 2)
        ach = per_gpu / (ms * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "kernel": "whole step on one GPU (all "
                            "kernels + exchange)", "achieved": ach,
                            "peak": peaks["hbm_gbs"], "peak_source": peaks["_source"],
                            "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                            "traffic": None,
                            "algorithmic_bytes_per_launch": per_gpu}
        print(json.dumps(line))
    dist.barrier()
    if exchange == "peer":
        blk.close()
    dist.destroy_process_group()
