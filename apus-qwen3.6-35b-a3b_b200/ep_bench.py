"""bench.py's multi-GPU arm: the expert-parallel block, one process per GPU
(launched by torch.distributed.run).

Strong scaling: the global batch is the same at every GPU count; rank r owns
tokens [r*T/N, (r+1)*T/N) and experts [r*E/N, (r+1)*E/N).  After the timed
region every rank's output is gathered on rank 0 and checked there: bit for bit
against the single-GPU block over the whole batch (all experts resident on GPU
0), and against the CPU checker on rows sampled from every rank's slice.
"""
import json
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

STAGES = ("route", "push", "shared", "wait_rows", "experts", "return",
          "wait_returns", "combine")


def run(args, cfg, config, pkg, synth, metric, unit, peaks, clock_sampler, wl):
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
    H, E, TK = cfg["hidden"], cfg["experts"], cfg["top_k"]
    Tg, skew = wl["T"], wl["skew"]
    if Tg % world or E % world:
        raise SystemExit(f"{Tg} tokens / {E} experts do not split over {world} GPUs")
    T = Tg // world                      # tokens per rank (strong scaling)
    per = E // world
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    sp = stream.cuda_stream
    # this rank's experts, generated in place in HBM; the router matrix (with
    # the skew's bias column) comes from the host
    layer = be.layer_create(cfg, None, rank * per, (rank + 1) * per)
    synth.device_weights(be, layer, cfg, seed=args.seed, layer=0,
                         expert_begin=rank * per, stream=sp)
    x_all = synth.host_x(be, Tg, H, seed=args.seed)
    rtr = None
    if skew:
        rtr = be.synth_fill_host(E * H, args.seed, 0, synth.T_RTR,
                                 synth.W_SIGMA).reshape(E, H)
        Wb, x_all = synth.apply_router_bias(
            {"rtr_w": rtr}, x_all,
            synth.zipf_bias(cfg, seed=args.seed, s=wl["zipf_s"], beta=wl["zipf_beta"]))
        rtr = Wb["rtr_w"]
        be.layer_upload(layer, "rtr_w", rtr)
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
    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    host_step = step
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

    def timed(n):
        dist.barrier()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        o = None
        for _ in range(n):
            o = step()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / n], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), o

    l0 = be.launches()
    ms, out = timed(args.steps)
    # a replayed graph launches the kernels that one captured step launched
    n_launched = per_step * args.steps if use_graph else be.launches() - l0
    launches = torch.tensor([float(n_launched)], device="cuda")
    out_keep = out.clone()
    clocks = sampler.finish() if sampler is not None else None
    # the same step for at least a second (every rank runs the same count)
    sustained = None
    if getattr(args, "sustain", 0) > 0:
        n_s = max(8, int(args.sustain * 1e3 / max(ms, 1e-3)) + 1)
        s2 = clock_sampler(local) if rank == 0 and clock_sampler is not None else None
        if s2 is not None:
            s2.start()
        sms, _ = timed(n_s)
        c2 = s2.finish() if s2 is not None else None
        sustained = {"steps": n_s, "ms_per_step": sms, "region_s": sms * n_s * 1e-3,
                     "clocks": c2,
                     "ms_x_sm_mhz": sms * c2["sm_mhz"] if c2 and c2.get("sm_mhz") else None}
    # per-stage device times of one rank's step (host launches, events between
    # the calls), max over ranks per stage; peer windows only
    stage_ms = None
    if exchange == "peer":
        acc = np.zeros(len(STAGES))
        reps = 5
        for _ in range(reps):
            evs = [torch.cuda.Event(enable_timing=True)]
            dist.barrier()
            torch.cuda.synchronize()
            evs[0].record(stream)

            def mark(_name):
                e = torch.cuda.Event(enable_timing=True)
                e.record(stream)
                evs.append(e)
            blk.forward(d_x, mark=mark)
            torch.cuda.synchronize()
            acc += np.array([evs[i].elapsed_time(evs[i + 1]) for i in range(len(STAGES))])
        st = torch.tensor(acc / reps, device="cuda", dtype=torch.float64)
        st_max = st.clone()
        dist.all_reduce(st_max, op=dist.ReduceOp.MAX)
        stage_ms = {"max_over_ranks": dict(zip(STAGES, (float(v) for v in st_max))),
                    "rank0": dict(zip(STAGES, (float(v) for v in st))),
                    "note": "one host-launched step bracketed by events; the two "
                            "wait stages contain the time a rank waits for its "
                            "slowest peer"}
    status_t = torch.tensor([float(be.last_block_status())], device="cuda")
    dist.all_reduce(status_t, op=dist.ReduceOp.MAX)
    status = int(status_t.item())

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
    dist.all_reduce(launches, op=dist.ReduceOp.SUM)

    # ---- output check on rank 0 -------------------------------------------
    gathered = [torch.empty_like(out_keep) for _ in range(world)] if rank == 0 else None
    dist.gather(out_keep, gathered, dst=0)
    parity, rows_per_rank, sent_rows = None, None, None
    if rank == 0 and not getattr(args, "no_check", False):
        ep_out = torch.cat(gathered).cpu().numpy().view(np.uint16)
        full = be.layer_create(cfg, None)
        synth.device_weights(be, full, cfg, seed=args.seed, layer=0, stream=sp)
        if rtr is not None:
            be.layer_upload(full, "rtr_w", rtr)
        d_all = torch.from_numpy(np.ascontiguousarray(x_all).view(np.int16)).cuda()
        d_ref = torch.empty_like(d_all)
        d_idx = torch.empty((Tg, TK), dtype=torch.int32, device="cuda")
        be.moe_block_dev(full, d_all.data_ptr(), d_ref.data_ptr(), Tg, stream=sp,
                         d_trace={"idx": d_idx.data_ptr()})
        torch.cuda.synchronize()
        one_gpu = d_ref.cpu().numpy().view(np.uint16)
        idx = d_idx.cpu().numpy()
        be.layer_destroy(full)
        owner = idx // per
        rows_per_rank = np.bincount(owner.ravel(), minlength=world)
        src_rank = np.repeat(np.arange(Tg) // T, TK).reshape(Tg, TK)
        sent_rows = int((owner != src_rank).sum())
        bad = int((ep_out != one_gpu).any(axis=1).sum())
        # CPU checker on rows sampled from every rank's slice
        from oracle import oracle
        orc = oracle.Restatement()
        W = synth.host_weights(be, cfg, seed=args.seed)
        if rtr is not None:
            W["rtr_w"] = rtr
        ridx, _ = orc.route_batch(x_all, W["rtr_w"], TK)
        rng = np.random.default_rng(args.seed)
        per_rank = []
        for r in range(world):
            rows = np.sort(r * T + rng.choice(T, 16, replace=False))
            exp = orc.moe_block(cfg, W, np.ascontiguousarray(x_all[rows]))
            a = synth.bf16_to_f32(ep_out[rows]).astype(np.float64)
            b = synth.bf16_to_f32(exp["out"]).astype(np.float64)
            per_rank.append({
                "rank": r, "rows": 16,
                "idx_exact": bool(np.array_equal(idx[rows], exp["idx"])),
                "max_abs": float(np.abs(a - b).max()),
                "rel_l2": float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-30))})
        parity = {
            "rows": 16 * world,
            "idx_exact": all(p["idx_exact"] for p in per_rank),
            "idx_exact_all_tokens": bool(np.array_equal(idx, ridx)),
            "max_abs": max(p["max_abs"] for p in per_rank),
            "rel_l2": max(p["rel_l2"] for p in per_rank),
            "tolerance": {"max_abs": 2e-2, "rel_l2": 1e-2},
            "per_rank": per_rank,
            "rows_differing_from_one_gpu_block": bad, "rows_compared_bitwise": int(Tg),
            "checker": "rank 0: apus_cuda_moe_block_dev over the whole batch "
                       "(bit equality of every row), oracle.Restatement() on 16 "
                       "sampled rows of every rank's slice and on every token's ids"}
        parity["ok"] = bool(parity["idx_exact"] and parity["idx_exact_all_tokens"]
                            and bad == 0 and parity["max_abs"] <= 2e-2
                            and parity["rel_l2"] <= 1e-2)
    if rank == 0:
        cfgline = dict(config)
        cfgline["parallelism"] = f"ep{world}"
        cfgline["tokens_per_gpu"] = T
        cfgline["experts_per_gpu"] = per
        I, Is = cfg["moe_inter"], cfg["shared_inter"]
        line = {
            "metric": metric, "value": Tg / (ms * 1e-3), "unit": unit,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": wl["dtype"],
            "data": "synthetic", "config": cfgline,
            "launch": "cuda graph replay" if use_graph else "host launches",
            "e2e": {"value": Tg / (e2e_ms * 1e-3), "unit": unit,
                    "h2d_bytes_per_step": Tg * H * 2,
                    "d2h_bytes_per_step": Tg * H * 2, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches.item()),
            "exchange": {"rows_sent_per_step": sent_rows,
                         "bytes_each_way_per_step":
                             sent_rows * H * 2 if sent_rows is not None else None,
                         "requested": getattr(args, "exchange", "peer"),
                         "collective": ("none: kernels store rows into the owner's "
                                        "memory over NVLink (CUDA IPC windows)"
                                        if exchange == "peer" else
                                        "all_to_all_single (NCCL), rows as bytes")},
            "block": {"device_status": status,
                      "weight_bytes_per_gpu": (per * 3 * I * H + 3 * Is * H + E * H + H) * 2},
        }
        if rows_per_rank is not None:
            line["block"]["expert_rows_per_rank"] = [int(v) for v in rows_per_rank]
            line["block"]["imbalance_max_over_mean"] = float(
                rows_per_rank.max() / rows_per_rank.mean())
        if stage_ms is not None:
            line["stage_ms"] = stage_ms
        if clocks is not None:
            line["clocks"] = clocks
        if sustained is not None:
            line["sustained"] = sustained
        if parity is not None:
            line["parity"] = parity
        # The batch is tensor-bound at these sizes: all flops of the step over
        # what N GPUs could do at the measured dense rate in the step's time.
        ach = wl["flops"] / (ms * 1e-3) / 1e12
        line["roofline"] = {"bound": "tensor",
                            "kernel": "whole step on all GPUs (all kernels + exchange)",
                            "achieved": ach, "peak": world * peaks["bf16_tflops"],
                            "peak_source": peaks["_source"], "unit": "TFLOP/s",
                            "frac": ach / (world * peaks["bf16_tflops"]),
                            "traffic": None,
                            "algorithmic_flops_per_launch": wl["flops"]}
        print(json.dumps(line))
    dist.barrier()
    if exchange == "peer":
        blk.close()
    dist.destroy_process_group()
    if status != 0:
        raise SystemExit(f"device status {status} on some rank (a bounded wait gave up)")
    if rank == 0 and parity is not None and not parity["ok"]:
        raise SystemExit("expert-parallel output check failed: " + json.dumps(parity))
