#!/usr/bin/env python3
"""Benchmark of the MoE-block hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T]
                  [--impl ours|reference]

One "step" is one pass of the MoE block (router -> top-8 -> dispatch -> routed
SwiGLU experts + shared expert -> weighted combine) over one batch of T
synthetic tokens at the Qwen3.6-35B-A3B dimensions (H 2048, 256 experts, top-8,
I 512).  Default workload: T=512 prefill, one layer, seed 0, weights resident
in HBM.  Prints ONE JSON line.

  value      tokens/s with inputs already in HBM (CUDA events, max over ranks)
  e2e        tokens/s through the host-pointer C-ABI call the engine would
             make (pinned host input, host output, copies inside the timing)
  roofline   the dominant kernel's algorithmic bytes / its own measured time,
             against the measured HBM copy bandwidth
  cpu_baseline  the reference's own C code (oracle/_ref) on this box's cores

--impl reference times only the reference CPU arm and prints the same line
shape with "impl": "reference".
"""
import argparse
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.join(ROOT, "apus-qwen3.6-35b-a3b_b200")
sys.path.insert(0, ROOT)

METRIC = "moe_layer_prefill_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0,
                      bf16_tflops_sustained=1400.0)


def load_package():
    spec = importlib.util.spec_from_file_location(
        "apus_b200", os.path.join(PKG_DIR, "__init__.py"),
        submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["apus_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


def algorithmic_bytes(cfg, T, unique_experts):
    """Bytes the block must move once: router matrix, every touched expert's
    weights, the shared expert, the shared gate row, activations in and out."""
    H, E, I, Is = cfg["hidden"], cfg["experts"], cfg["moe_inter"], cfg["shared_inter"]
    slab = (2 * I * H + H * I) * 2
    shared = (2 * Is * H + H * Is) * 2
    return E * H * 2 + unique_experts * slab + shared + H * 2 + 2 * T * H * 2


def flops(cfg, T):
    H, E, I, Is, TK = (cfg["hidden"], cfg["experts"], cfg["moe_inter"],
                       cfg["shared_inter"], cfg["top_k"])
    per_tok = 2 * (E * H + TK * 3 * I * H + 3 * Is * H + H)
    return T * per_tok


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons with nvidia-smi while the timed
    region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.maxmhz = None
        self.stop_flag = False

    def run(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                 "sw_power_cap"]
        while not self.stop_flag:
            try:
                out = subprocess.run(
                    ["nvidia-smi", "-i", str(self.index),
                     "--query-gpu=" + self.Q, "--format=csv,noheader,nounits"],
                    capture_output=True, text=True, timeout=5).stdout.strip()
                f = [s.strip() for s in out.split(",")]
                self.samples.append(float(f[0]))
                self.maxmhz = float(f[1])
                for n, v in zip(names, f[2:]):
                    if v.lower().startswith("active"):
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.05)

    def summary(self):
        s = sorted(self.samples)
        return dict(sm_mhz=s[len(s) // 2] if s else None,
                    sm_max_mhz=self.maxmhz, reasons=sorted(self.reasons),
                    samples=len(s))


def cpu_reference_arm(cfg, T, seed, steps, warmup, be, synth, min_seconds=0.0):
    """Times the reference's own MoE block (apus_layer_moe_batch, AVX2 rows
    over its pthread pool) on this host.  Returns (tokens/s, threads,
    sample-description, ms_per_step).  With min_seconds the timed loop keeps
    going (up to 64 steps) until that much CPU time has been sampled."""
    from oracle import oracle
    if not oracle.Reference.available():
        return None
    ref = oracle.Reference()
    W = synth.host_weights(be, cfg, seed=seed)
    x = synth.host_x(be, T, cfg["hidden"], seed=seed)
    # bound the sample: the full batch when it is cheap, else a slice of it
    Ts = T
    t0 = time.perf_counter()
    ref.moe_block(cfg, W, x[:min(T, 16)])
    est = (time.perf_counter() - t0) * T / min(T, 16)
    while Ts > 16 and est * Ts / T * (steps + warmup) > 60.0:
        Ts //= 2
    xs = x[:Ts]
    for _ in range(warmup):
        ref.moe_block(cfg, W, xs)
    best, spent, done = None, 0.0, 0
    while done < steps or (spent < min_seconds and done < 64):
        t0 = time.perf_counter()
        ref.moe_block(cfg, W, xs)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        spent += dt
        done += 1
    sample = (f"{Ts} of {T} tokens, one layer, apus_layer_moe_batch, "
              f"best of {done} ({spent:.1f} s sampled)")
    return Ts / best, ref.threads(), sample, best * 1e3

L2_BYTES = 126 << 20


def run_stack(args, cfg, config, pkg, synth, L):
    """A stack of L MoE layers with independent seeded weights, generated in
    place in HBM.  Every step runs every layer's block once, so nothing a step
    needs is left in L2 by the previous one.  Layer l reads its own seeded
    token batch; with --chain the layers are chained as the engine chains them
    (c/layer.h:386-388): ln2 = rmsnorm(h); h = rnd(h + moe_l(ln2)), and the
    two elementwise kernels are inside the timed region."""
    import numpy as np
    import torch
    torch.cuda.set_device(0)
    be = pkg.Backend()
    be.enable()
    T, H, TK = args.tokens, cfg["hidden"], cfg["top_k"]
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    sp = stream.cuda_stream
    layers = []
    for l in range(L):
        h = be.layer_create(cfg, None)
        synth.device_weights(be, h, cfg, seed=args.seed, layer=l, stream=sp)
        layers.append(h)
    be.reserve(cfg, T)
    chain = args.chain
    n_in = 1 if chain else L
    x_host = np.stack([synth.host_x(be, T, H, seed=args.seed, layer=l)
                       for l in range(n_in)])
    d_x = torch.from_numpy(x_host.view(np.int16)).cuda()      # [n_in, T, H]
    d_h = torch.empty_like(d_x)                               # chain state / outputs
    d_ln = torch.empty((T, H), dtype=torch.int16, device="cuda")
    d_moe = torch.empty((T, H), dtype=torch.int16, device="cuda")
    d_idx = torch.empty((T, TK), dtype=torch.int32, device="cuda")
    row = T * H * 2

    def one_pass(trace_uniq=None, timing=None):
        if chain:
            d_h.copy_(d_x)
        for l, lay in enumerate(layers):
            tr = {"idx": d_idx.data_ptr()} if trace_uniq is not None else None
            if chain:
                be.rmsnorm_dev(d_h.data_ptr(), None, d_ln.data_ptr(), T, H, stream=sp)
                be.moe_block_dev(lay, d_ln.data_ptr(), d_moe.data_ptr(), T,
                                 stream=sp, d_trace=tr)
            else:
                be.moe_block_dev(lay, d_x.data_ptr() + l * row,
                                 d_h.data_ptr() + l * row, T, stream=sp, d_trace=tr)
            if timing is not None:
                for k, v in be.last_stage_ms().items():
                    timing[k] = timing.get(k, 0.0) + v
            if trace_uniq is not None:
                torch.cuda.synchronize()
                trace_uniq.append(int(torch.unique(d_idx).numel()))
            if chain:
                be.resadd_dev(d_h.data_ptr(), d_moe.data_ptr(), d_h.data_ptr(),
                              T * H, stream=sp)

    uniq = []
    one_pass(trace_uniq=uniq)
    torch.cuda.synchronize()
    launches_per_layer = be.last_block_launches() + (2 if chain else 0)
    step = one_pass
    launch_mode = "host launches"
    if not args.no_graph:
        try:
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=stream):
                one_pass()
            step = g.replay
            launch_mode = "cuda graph replay"
        except Exception as e:
            launch_mode = f"host launches (graph capture failed: {e})"
            torch.cuda.synchronize()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    status = be.last_block_status()
    # stage times (host launches, events / device timeline per layer)
    be.stage_timing(True)
    acc = {}
    one_pass(timing=acc)
    be.stage_timing(False)
    stage_ms = {k: v / L for k, v in acc.items()}
    # end to end: pinned host tokens in, result back to host, every step
    xin = torch.from_numpy(x_host.view(np.int16)).pin_memory()
    hout = torch.empty_like(xin).pin_memory()
    for _ in range(3):
        d_x.copy_(xin, non_blocking=True); step(); hout.copy_(d_h, non_blocking=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        d_x.copy_(xin, non_blocking=True)
        step()
        hout.copy_(d_h, non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    sampler.stop_flag = True
    sampler.join()

    pk = peaks()
    bytes_pass = sum(algorithmic_bytes(cfg, T, u) for u in uniq)
    tok_layers = T * L
    cfgline = dict(config)
    cfgline.update({
        "workload": f"stack of {L} MoE layers (independent weights"
                    + (", chained x <- x + moe(rmsnorm(x))" if chain else
                       ", one token batch per layer")
                    + f"), {T} tokens per layer per step, uniform router, "
                    f"seed {args.seed}, H2048 E256 top8 I512",
        "layers": L, "launch": launch_mode,
        "l2_policy": f"inputs larger than L2: one pass reads "
                     f"{bytes_pass / 1e6:.0f} MB of weights across {L} layers"})
    kms = sum(stage_ms.values())
    fused = be.last_block_launches() == 1
    line = {
        "metric": METRIC, "value": tok_layers / (ms * 1e-3), "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 storage, fp32 accumulate",
        "data": "synthetic", "config": cfgline, "clocks": sampler.summary(),
        "e2e": {"value": tok_layers / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": n_in * T * H * 2,
                "d2h_bytes_per_step": n_in * T * H * 2,
                "ms_per_step": e2e_ms},
        "gpu_launches": launches_per_layer * L * args.steps,
        "roofline": {"bound": "hbm",
                     "kernel": "decode_fused_kernel" if fused else "whole layer (all kernels)",
                     "achieved": bytes_pass / L / (kms * 1e-3) / 1e9 if kms else None,
                     "peak": pk["hbm_gbs"], "peak_source": pk["_source"],
                     "unit": "GB/s",
                     "frac": (bytes_pass / L / (kms * 1e-3) / 1e9 / pk["hbm_gbs"]) if kms else None,
                     "traffic": None,
                     "algorithmic_bytes_per_launch": bytes_pass / L},
        "block": {"algorithmic_bytes_per_layer": bytes_pass / L,
                  "hbm_frac_of_measured": bytes_pass / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                  "unique_experts_mean": sum(uniq) / L, "stage_ms_per_layer": stage_ms,
                  "us_per_token_layer": ms * 1e3 / tok_layers,
                  "device_status": status},
    }
    if not args.no_cpu_baseline:
        r = cpu_reference_arm(cfg, T, args.seed, 3, 1, be, synth, min_seconds=10.0)
        if r is not None:
            v, threads, sample, _ = r
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads,
                                    "kind": "reference",
                                    "sample": sample + " (one layer of the stack)"}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=0,
                    help="run a stack of this many MoE layers with independent "
                         "weights, chained as x <- x + moe(rmsnorm(x)); default: "
                         "1, or as many as it takes for one pass to read more "
                         "than four times the L2 capacity (small token counts)")
    ap.add_argument("--chain", action="store_true",
                    help="with a layer stack: chain the layers through rmsnorm "
                         "and the residual add instead of one batch per layer")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="multi-GPU arm: rows exchanged by kernels that store into "
                         "the peers' memory (default), or by NCCL all-to-all")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every step from the host instead of "
                         "replaying a captured CUDA graph")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pkg = load_package()
    import apus_b200.synth as synth
    cfg = dict(synth.QWEN_CFG)
    T = args.tokens
    config = {"workload": f"one MoE layer, prefill T={T}, uniform router, seed "
                          f"{args.seed}, H2048 E256 top8 I512",
              "tokens_per_step": T, "layers": 1,
              "l2_policy": "inputs larger than L2 (1.6 GB of weights per step)"}

    if args.impl == "reference":
        if rank != 0:
            return
        be = pkg.Backend()
        steps = max(1, min(args.steps, 5))
        warm = max(1, min(args.warmup, 2))
        r = cpu_reference_arm(cfg, T, args.seed, steps, warm, be, synth)
        if r is None:
            print(json.dumps({"impl": "reference",
                              "unavailable": "oracle/_ref was not built"}))
            return
        v, threads, sample, ms = r
        line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT,
                "n_gpus": args.gpus, "steps": steps, "warmup": warm,
                "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16 storage, fp32 arithmetic",
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads,
                                 "kind": "reference", "sample": sample},
                "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    import numpy as np
    import torch
    if world > 1:
        from apus_b200 import ep_bench
        ep_bench.run(args, cfg, config, pkg, synth, METRIC, UNIT, peaks(), ClockSampler)
        return

    # small token counts touch few experts: one layer's working set would sit
    # in L2 from step to step, so they run as a stack of independent layers
    L = args.layers
    if L <= 0:
        est_uniq = min(cfg["experts"], T * cfg["top_k"])
        per_layer = algorithmic_bytes(cfg, T, est_uniq)
        L = 1 if per_layer >= 4 * L2_BYTES else -(-4 * L2_BYTES // per_layer)
    if L > 1:
        run_stack(args, cfg, config, pkg, synth, L)
        return

    torch.cuda.set_device(0)
    be = pkg.Backend()
    be.enable()
    H = cfg["hidden"]
    W = synth.host_weights(be, cfg, seed=args.seed)
    x_host = synth.host_x(be, T, H, seed=args.seed)
    layer = be.layer_create(cfg, W)
    be.reserve(cfg, T)
    stream = torch.cuda.Stream()       # every launch and event goes here
    torch.cuda.set_stream(stream)
    d_x = torch.from_numpy(x_host.view(np.int16)).cuda()
    d_out = torch.empty_like(d_x)
    d_idx = torch.empty((T, cfg["top_k"]), dtype=torch.int32, device="cuda")
    sp = stream.cuda_stream

    def step():
        be.moe_block_dev(layer, d_x.data_ptr(), d_out.data_ptr(), T, stream=sp)

    # unique experts touched (for the algorithmic byte count)
    be.moe_block_dev(layer, d_x.data_ptr(), d_out.data_ptr(), T, stream=sp,
                     d_trace={"idx": d_idx.data_ptr()})
    torch.cuda.synchronize()
    uniq = int(torch.unique(d_idx).numel())
    launches_per_step = be.last_block_launches()

    # one block call captured into a CUDA graph: the replay is what a serving
    # loop would issue per layer (no per-launch host work)
    launch_mode = "host launches"
    if not args.no_graph:
        try:
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=stream):
                be.moe_block_dev(layer, d_x.data_ptr(), d_out.data_ptr(), T,
                                 stream=torch.cuda.current_stream().cuda_stream)
            direct = step
            step = g.replay
            launch_mode = "cuda graph replay"
        except Exception as e:          # capture unsupported: say so, go on
            launch_mode = f"host launches (graph capture failed: {e})"
            torch.cuda.synchronize()
    config["launch"] = launch_mode

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    status = be.last_block_status()

    # per-stage times, measured live with CUDA events on the launching stream
    if launch_mode.startswith("cuda graph"):
        step = direct
    be.stage_timing(True)
    acc = {}
    for _ in range(args.steps):
        step()
        for k, v in be.last_stage_ms().items():
            acc[k] = acc.get(k, 0.0) + v
    be.stage_timing(False)
    stage_ms = {k: v / args.steps for k, v in acc.items()}

    # end to end through the host-pointer entry point (pinned host buffers)
    xin = torch.from_numpy(x_host.view(np.int16)).pin_memory()
    xout = torch.empty_like(xin).pin_memory()
    xin_np, xout_np = xin.numpy().view(np.uint16), xout.numpy().view(np.uint16)
    c_cfg = pkg.backend.MoeCfg.from_dict(cfg)
    c_w = pkg.backend.MoeW(*[W[k].ctypes.data for k in
                             ("rtr_w", "exp_gu", "exp_d", "sh_g", "sh_u",
                              "sh_d", "sh_gate")])
    import ctypes as C

    def e2e_step():
        rc = be.lib.apus_cuda_moe_block(
            C.byref(c_cfg), C.byref(c_w),
            xin_np.ctypes.data_as(C.POINTER(C.c_uint16)),
            xout_np.ctypes.data_as(C.POINTER(C.c_uint16)), T, None)
        if rc:
            raise RuntimeError(be.last_error())
    for _ in range(max(3, args.warmup)):
        e2e_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    sampler.stop_flag = True
    sampler.join()
    assert np.array_equal(xout_np, d_out.cpu().numpy().view(np.uint16)), \
        "host-pointer and device-pointer entry points disagree"

    pk = peaks()
    slab_gu = 2 * cfg["moe_inter"] * H * 2
    slab_d = H * cfg["moe_inter"] * 2
    A = T * cfg["top_k"]
    I = cfg["moe_inter"]
    hbm_ideal = algorithmic_bytes(cfg, T, uniq) / (pk["hbm_gbs"] * 1e9)
    tc_ideal = flops(cfg, T) / (pk["bf16_tflops"] * 1e12)
    if launches_per_step == 1:
        # the one-kernel decode path: the kernel IS the block; its duration is
        # the device-timeline sum of its phases
        dom = "decode_fused_kernel"
        kbytes = algorithmic_bytes(cfg, T, uniq)
        kms = sum(stage_ms.values())
        roof = {"bound": "hbm", "kernel": dom,
                "achieved": kbytes / (kms * 1e-3) / 1e9 if kms else None,
                "peak": pk["hbm_gbs"], "unit": "GB/s", "traffic": None,
                "algorithmic_bytes_per_launch": kbytes}
    else:
        dom = max(("gate_up", "down"), key=lambda k: stage_ms.get(k, 0.0))
        kname = ("grouped_gemm_kernel<gate_up>" if dom == "gate_up"
                 else "grouped_gemm_kernel<down>")
        if T <= 4:
            kname = "decode_" + dom + "_kernel"
        if dom == "gate_up":
            kbytes = (uniq + 1) * slab_gu + (A + T) * H * 2 + (A + T) * I * 2
            kflops = 2 * (A + T) * 2 * I * H
        else:
            kbytes = (uniq + 1) * slab_d + (A + T) * I * 2 + (A + T) * H * 2
            kflops = 2 * (A + T) * H * I
        kms = stage_ms.get(dom, 0.0)
        if tc_ideal > hbm_ideal:
            roof = {"bound": "tensor", "kernel": kname,
                    "achieved": kflops / (kms * 1e-3) / 1e12 if kms else None,
                    "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "traffic": None,
                    "algorithmic_flops_per_launch": kflops}
        else:
            # ncu dram__bytes_read+write of this launch at the default workload
            # (profiles/grouped_gemm_t512_prefill.md); other sizes not captured
            traffic = None
            if T == 512 and uniq == 256:
                traffic = 1.1005e9 + 7.5e6 if dom == "gate_up" else 0.5439e9 + 17.2e6
            roof = {"bound": "hbm", "kernel": kname,
                    "achieved": kbytes / (kms * 1e-3) / 1e9 if kms else None,
                    "peak": pk["hbm_gbs"], "unit": "GB/s", "traffic": traffic,
                    "algorithmic_bytes_per_launch": kbytes}
    roof["peak_source"] = pk["_source"]
    roof["frac"] = roof["achieved"] / roof["peak"] if roof["achieved"] else None
    block_bytes = algorithmic_bytes(cfg, T, uniq)
    line = {
        "metric": METRIC, "value": T / (ms * 1e-3), "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 storage, fp32 accumulate",
        "data": "synthetic", "config": config,
        "clocks": sampler.summary(),
        "e2e": {"value": T / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": T * H * 2, "d2h_bytes_per_step": T * H * 2,
                "ms_per_step": e2e_ms},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": roof,
        "block": {"algorithmic_bytes": block_bytes,
                  "hbm_frac_of_measured": block_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                  "tensor_frac_of_measured": flops(cfg, T) / (ms * 1e-3) / 1e12 / pk["bf16_tflops"],
                  "unique_experts": uniq, "stage_ms": stage_ms,
                  "us_per_token": ms * 1e3 / T, "device_status": status},
    }
    if not args.no_cpu_baseline:
        r = cpu_reference_arm(cfg, T, args.seed, 3, 1, be, synth, min_seconds=10.0)
        if r is not None:
            v, threads, sample, _ = r
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads,
                                    "kind": "reference", "sample": sample}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
