"""Expert-parallel entry points on one GPU: N ranks emulated in one process
(each with its own partial layer; the two all-to-alls done by slicing), and
the real torch.distributed path at world size 1.  The result must equal the
single-GPU block bit for bit."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def emulate(be, ep, torch, cfg, W, x, N):
    T, H = x.shape
    per, E, TK = T // N, cfg["experts"], cfg["top_k"]
    layers = [be.layer_create(cfg, W, r * E // N, (r + 1) * E // N)
              for r in range(N)]
    ops = [ep.CudaOps(be, layers[r], cfg) for r in range(N)]
    xs = [torch.from_numpy(x[r * per:(r + 1) * per].view(np.int16).copy()).cuda()
          for r in range(N)]
    routed = [ops[r].route(xs[r]) for r in range(N)]
    packed = [ops[r].pack(xs[r], routed[r][0], N) for r in range(N)]
    torch.cuda.synchronize()
    counts = [p[2].cpu().numpy() for p in packed]          # [src][dst]
    offs = [np.concatenate([[0], np.cumsum(c)]) for c in counts]
    back = [torch.empty((per * TK, H), dtype=torch.int16, device="cuda")
            for _ in range(N)]
    for dst in range(N):
        rx = torch.cat([packed[src][0][offs[src][dst]:offs[src][dst + 1]]
                        for src in range(N)])
        re = torch.cat([packed[src][1][offs[src][dst]:offs[src][dst + 1]]
                        for src in range(N)])
        assert int(re.min()) >= dst * E // N and int(re.max()) < (dst + 1) * E // N
        y = ops[dst].experts(rx, re)
        o = 0
        for src in range(N):
            n = counts[src][dst]
            back[src][offs[src][dst]:offs[src][dst + 1]] = y[o:o + n]
            o += n
    outs = [ops[r].finish(xs[r], back[r], packed[r][3], routed[r][1],
                          routed[r][2]) for r in range(N)]
    torch.cuda.synchronize()
    assert be.last_block_status() == 0
    out = np.concatenate([o.cpu().numpy().view(np.uint16) for o in outs])
    for l in layers:
        be.layer_destroy(l)
    return out


@pytest.mark.parametrize("path", ["gemm", "gemv"])
@pytest.mark.parametrize("N,T", [(2, 20), (2, 200), (4, 400), (8, 1024)])
def test_ep_emulated_ranks_equal_single_gpu(be, synth, N, T, path, monkeypatch):
    """With both sides pinned to the same expert kernels (a row's result does
    not depend on which other rows share its tile or group), the N-rank result
    is the single-GPU result bit for bit."""
    import torch
    from apus_b200 import ep
    monkeypatch.setenv("APUS_CUDA_DECODE_MAX_T",
                       "0" if path == "gemm" else "1000000")
    be.enable()
    try:
        cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128,
                   top_k=8)
        W = synth.host_weights(be, cfg, seed=13, sigma=0.05)
        x = synth.host_x(be, T, cfg["hidden"], seed=13)
        whole = be.moe_block(cfg, W, x, trace=False)["out"]
        got = emulate(be, ep, torch, cfg, W, x, N)
        assert np.array_equal(got, whole)
    finally:
        be.disable()


def test_ep_matches_checker(gpu, orc, be, synth):
    import torch
    from apus_b200 import ep
    cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128, top_k=8)
    W = synth.host_weights(be, cfg, seed=14, sigma=0.05)
    x = synth.host_x(be, 96, cfg["hidden"], seed=14)
    got = emulate(be, ep, torch, cfg, W, x, 2)
    exp = orc.moe_block(cfg, W, x)["out"]
    a, b = synth.bf16_to_f32(got), synth.bf16_to_f32(exp)
    assert np.abs(a - b).max() <= 2e-2
    assert np.linalg.norm(a - b) / np.linalg.norm(b) <= 1e-2


def test_ep_world_size_one_process_group(gpu, be, synth):
    """The torch.distributed path itself (NCCL, one rank)."""
    import torch
    import torch.distributed as dist
    from apus_b200 import ep
    cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128, top_k=8)
    W = synth.host_weights(be, cfg, seed=15, sigma=0.05)
    x = synth.host_x(be, 150, cfg["hidden"], seed=15)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(29700 + os.getpid() % 1000))
    dist.init_process_group("nccl", rank=0, world_size=1)
    try:
        layer = be.layer_create(cfg, W)
        blk = ep.EPBlock(ep.CudaOps(be, layer, cfg), cfg, 0, 1)
        out = blk.forward(torch.from_numpy(x.view(np.int16).copy()).cuda())
        torch.cuda.synchronize()
        whole = gpu.moe_block(cfg, W, x, trace=False)["out"]
        assert np.array_equal(out.cpu().numpy().view(np.uint16), whole)
    finally:
        dist.destroy_process_group()


def emulate_windows(be, ep, torch, cfg, W, x, N, steps=1, device_epoch=False,
                    mode="push"):
    """N ranks in this process, one peer window each, attached to one another
    by pointer.  All pushes are launched before the first wait, all returns
    before the first wait for them, so no kernel ever waits on a later one."""
    T, H = x.shape
    per, E = T // N, cfg["experts"]
    layers = [be.layer_create(cfg, W, r * E // N, (r + 1) * E // N)
              for r in range(N)]
    wins = [be.ep_window_create(per, cfg["top_k"], H, E, N, r) for r in range(N)]
    for r in range(N):
        for q in range(N):
            if q != r:
                be.ep_window_attach_local(wins[r], q, wins[q])
    blks = [ep.PeerWindowBlock(be, layers[r], cfg, r, N, per, window=wins[r],
                               device_epoch=device_epoch, mode=mode)
            for r in range(N)]
    xs = [torch.from_numpy(x[r * per:(r + 1) * per].view(np.int16).copy()).cuda()
          for r in range(N)]
    for _ in range(steps):
        sts = [blks[r].begin(xs[r]) for r in range(N)]
        for r in range(N):
            blks[r].middle()
        outs = [blks[r].end(sts[r]) for r in range(N)]
    torch.cuda.synchronize()
    assert be.last_block_status() == 0
    out = np.concatenate([o.cpu().numpy().view(np.uint16) for o in outs])
    for w in wins:
        be.ep_window_destroy(w)
    for l in layers:
        be.layer_destroy(l)
    return out


@pytest.mark.parametrize("mode,path", [("push", "gemm"), ("push", "gemv"),
                                       ("pull", "gemm")])
@pytest.mark.parametrize("N,T", [(2, 20), (2, 200), (4, 400), (8, 1024), (4, 2400)])
def test_peer_window_ranks_equal_single_gpu(be, synth, N, T, path, mode, monkeypatch):
    """The exchange through peer windows gives the single-GPU block bit for
    bit; three steps in a row reuse the windows.  push: rows stored straight
    into the owner's memory, outputs stored straight back by kernels of their
    own.  pull: rows gathered from the publishers' windows, outputs stored by
    the down GEMM's epilogue (always the tensor-core kernels)."""
    import torch
    from apus_b200 import ep
    monkeypatch.setenv("APUS_CUDA_DECODE_MAX_T",
                       "0" if path == "gemm" else "1000000")
    be.enable()
    try:
        cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128,
                   top_k=8)
        W = synth.host_weights(be, cfg, seed=13, sigma=0.05)
        x = synth.host_x(be, T, cfg["hidden"], seed=13)
        whole = be.moe_block(cfg, W, x, trace=False)["out"]
        got = emulate_windows(be, ep, torch, cfg, W, x, N, steps=3, mode=mode)
        assert np.array_equal(got, whole)
    finally:
        be.disable()


@pytest.mark.parametrize("min_rows", ["192", "32"])
def test_peer_window_pull_real_dims(be, synth, min_rows, monkeypatch):
    """The real layer shape (H 2048, 256 experts, top-8, I 512), two ranks of 1024
    tokens: the one-SM GEMMs (64 rows per resident expert on average) and, with
    the threshold lowered, the two-SM GEMMs store their outputs into the owners'
    windows; every row equals the one-GPU block on the same weights."""
    import torch
    from apus_b200 import ep
    monkeypatch.setenv("APUS_CUDA_PAIR_MIN_ROWS", min_rows)
    be.enable()
    try:
        cfg = dict(synth.QWEN_CFG)
        N, per, H, E = 2, 1024, cfg["hidden"], cfg["experts"]
        sp = torch.cuda.current_stream().cuda_stream
        whole = be.layer_create(cfg, None, 0, E)
        synth.device_weights(be, whole, cfg, seed=5, stream=sp)
        layers = []
        for r in range(N):
            h = be.layer_create(cfg, None, r * E // N, (r + 1) * E // N)
            synth.device_weights(be, h, cfg, seed=5, expert_begin=r * E // N, stream=sp)
            layers.append(h)
        x = synth.host_x(be, N * per, H, seed=5)
        d_x = torch.from_numpy(x.view(np.int16).copy()).cuda()
        d_ref = torch.empty_like(d_x)
        be.moe_block_dev(whole, d_x.data_ptr(), d_ref.data_ptr(), N * per, stream=sp)
        wins = [be.ep_window_create(per, cfg["top_k"], H, E, N, r) for r in range(N)]
        for r in range(N):
            be.ep_window_attach_local(wins[r], 1 - r, wins[1 - r])
        blks = [ep.PeerWindowBlock(be, layers[r], cfg, r, N, per, window=wins[r])
                for r in range(N)]
        xs = [d_x[r * per:(r + 1) * per].contiguous() for r in range(N)]
        for _ in range(2):
            sts = [blks[r].begin(xs[r]) for r in range(N)]
            for r in range(N):
                blks[r].middle()
            outs = [blks[r].end(sts[r]) for r in range(N)]
        torch.cuda.synchronize()
        assert be.last_block_status() == 0
        assert torch.equal(torch.cat(outs), d_ref)
        for w in wins:
            be.ep_window_destroy(w)
        for l in layers + [whole]:
            be.layer_destroy(l)
    finally:
        be.disable()


@pytest.mark.parametrize("mode,overlap", [("push", False), ("pull", True),
                                          ("pull", False)])
def test_peer_window_ragged_ranks(be, synth, mode, overlap):
    """Ranks with different token counts (5, 200, 37, 128; windows sized for
    200): the unused tail of a rank's region holds no assignment.  overlap: the
    rows are stored on a second stream beside the router."""
    import torch
    from apus_b200 import ep
    be.enable()
    try:
        cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128,
                   top_k=8)
        counts, N, cap_t = [5, 200, 37, 128], 4, 200
        T, H, E = sum(counts), cfg["hidden"], cfg["experts"]
        W = synth.host_weights(be, cfg, seed=31, sigma=0.05)
        x = synth.host_x(be, T, H, seed=31)
        whole = be.moe_block(cfg, W, x, trace=False)["out"]
        layers = [be.layer_create(cfg, W, r * E // N, (r + 1) * E // N)
                  for r in range(N)]
        wins = [be.ep_window_create(cap_t, cfg["top_k"], H, E, N, r) for r in range(N)]
        for r in range(N):
            for q in range(N):
                if q != r:
                    be.ep_window_attach_local(wins[r], q, wins[q])
        blks = [ep.PeerWindowBlock(be, layers[r], cfg, r, N, cap_t, window=wins[r],
                                   mode=mode, overlap=overlap) for r in range(N)]
        lo = np.concatenate([[0], np.cumsum(counts)])
        xs = [torch.from_numpy(x[lo[r]:lo[r + 1]].view(np.int16).copy()).cuda()
              for r in range(N)]
        for _ in range(2):
            sts = [blks[r].begin(xs[r]) for r in range(N)]
            for r in range(N):
                blks[r].middle()
            outs = [blks[r].end(sts[r]) for r in range(N)]
        torch.cuda.synchronize()
        assert be.last_block_status() == 0
        got = np.concatenate([o.cpu().numpy().view(np.uint16) for o in outs])
        assert np.array_equal(got, whole)
        for w in wins:
            be.ep_window_destroy(w)
        for l in layers:
            be.layer_destroy(l)
    finally:
        be.disable()


@pytest.mark.parametrize("N,T", [(2, 4096), (8, 8192)])
def test_peer_window_pull_two_sm_kernels(be, synth, N, T, monkeypatch):
    """Enough rows per resident expert for the two-SM GEMMs (and the one-SM
    kernels on the remainders): their down epilogues store to the sources'
    windows too."""
    import torch
    from apus_b200 import ep
    monkeypatch.setenv("APUS_CUDA_PAIR_MIN_ROWS", "64")
    be.enable()
    try:
        cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128,
                   top_k=8)
        W = synth.host_weights(be, cfg, seed=29, sigma=0.05)
        x = synth.host_x(be, T, cfg["hidden"], seed=29)
        whole = be.moe_block(cfg, W, x, trace=False)["out"]
        got = emulate_windows(be, ep, torch, cfg, W, x, N, steps=2, mode="pull")
        assert np.array_equal(got, whole)
    finally:
        be.disable()


@pytest.mark.parametrize("mode", ["push", "pull"])
def test_peer_window_skewed_router_one_owner(be, synth, mode):
    """Every assignment of every token goes to experts of rank 0: the other
    ranks receive nothing and return nothing."""
    import torch
    from apus_b200 import ep
    be.enable()
    try:
        cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128,
                   top_k=8)
        W = synth.host_weights(be, cfg, seed=17, sigma=0.05)
        # router rows of experts 0..15 get a large positive last column
        rw = synth.bf16_to_f32(W["rtr_w"]).copy()
        rw[:16, -1] = 4.0
        rw[16:, -1] = -4.0
        W = dict(W)
        W["rtr_w"] = synth.f32_to_bf16(rw)
        x = synth.bf16_to_f32(synth.host_x(be, 64, 512, seed=17)).copy()
        x[:, -1] = 8.0
        x = synth.f32_to_bf16(x)
        whole = be.moe_block(cfg, W, x, trace=True)
        assert int(whole["idx"].max()) < 16
        got = emulate_windows(be, ep, torch, cfg, W, x, 4, mode=mode)
        assert np.array_equal(got, whole["out"])
    finally:
        be.disable()


@pytest.mark.parametrize("mode", ["push", "pull"])
@pytest.mark.parametrize("T,graph", [(24, 0), (300, 0), (300, 1)])
def test_peer_window_two_processes(be, synth, T, graph, mode, tmp_path):
    """Two real ranks, one per GPU, windows mapped through CUDA IPC: the rows
    cross NVLink by the kernels' own stores.  Three steps (graph = 1: the step
    captured once in a CUDA graph and replayed, its number kept on the device);
    the last one must equal the single-GPU block bit for bit."""
    import subprocess
    import sys
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)),
                          "ep_peer_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    port = 29800 + os.getpid() % 100
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
         "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
         "--master-port", str(port), worker, str(tmp_path), str(T), "3",
         str(graph), mode],
        env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    got = np.concatenate([np.load(tmp_path / f"out_{k}.npy") for k in range(2)])
    be.enable()
    try:
        cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128,
                   top_k=8)
        W = synth.host_weights(be, cfg, seed=13, sigma=0.05)
        x = synth.host_x(be, 2 * T, cfg["hidden"], seed=102)
        whole = be.moe_block(cfg, W, x, trace=False)["out"]
        assert np.array_equal(got, whole)
    finally:
        be.disable()


@pytest.mark.parametrize("mode", ["push", "pull"])
def test_peer_window_step_number_on_the_device(be, synth, mode):
    """Epoch 0 in every call: the windows count the steps themselves (what a
    captured CUDA graph of the step needs).  Four steps, four ranks."""
    import torch
    from apus_b200 import ep
    be.enable()
    try:
        cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128,
                   top_k=8)
        W = synth.host_weights(be, cfg, seed=21, sigma=0.05)
        x = synth.host_x(be, 160, cfg["hidden"], seed=21)
        whole = be.moe_block(cfg, W, x, trace=False)["out"]
        got = emulate_windows(be, ep, torch, cfg, W, x, 4, steps=4,
                              device_epoch=True, mode=mode)
        assert np.array_equal(got, whole)
    finally:
        be.disable()


def test_peer_window_wait_gives_up(be, synth):
    """A peer that never pushes: the wait runs out after about two seconds,
    the status word says so (6), and the context and the windows stay usable."""
    import time
    import torch
    from apus_b200 import ep
    be.enable()
    try:
        cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128,
                   top_k=8)
        wins = [be.ep_window_create(16, 8, 512, 64, 2, r) for r in range(2)]
        be.ep_window_attach_local(wins[0], 1, wins[1])
        be.ep_window_attach_local(wins[1], 0, wins[0])
        t0 = time.time()
        be.ep_wait_dev(wins[0], 0, 7)            # nobody ever announces step 7
        torch.cuda.synchronize()
        assert time.time() - t0 < 30
        assert be.last_block_status() == 6
        assert be.last_block_status() == 0       # read once, then clear
        for w in wins:
            be.ep_window_destroy(w)
        W = synth.host_weights(be, cfg, seed=23, sigma=0.05)
        x = synth.host_x(be, 32, cfg["hidden"], seed=23)
        whole = be.moe_block(cfg, W, x, trace=False)["out"]
        got = emulate_windows(be, ep, torch, cfg, W, x, 2)
        assert np.array_equal(got, whole)
    finally:
        be.disable()
