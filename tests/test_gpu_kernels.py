"""GPU parity tests, kernel level, all through the C-ABI: the per-matmul
hooks, the router and the dispatch against the CPU checker.  Integer and
index results are compared bit for bit."""
import os

import numpy as np
import pytest

from test_oracle_cpu import rd, manifest, f32, tol_ok, rng_codes

pytestmark = pytest.mark.gpu


# ---- per-matmul hooks: bitwise the CPU anchor (tests/m10/test_kernels.c) ----

@pytest.mark.parametrize("O,K", [(1, 1), (3, 5), (7, 1), (33, 100), (64, 256),
                                 (256, 2048), (1024, 2048), (2048, 512),
                                 (512, 2048), (1, 2048)])
def test_hook_gemv_matvec_bitwise(gpu, orc, O, K):
    rng = np.random.default_rng(O * 131 + K)
    w, x = rng_codes(rng, (O, K), 0.5), rng_codes(rng, K, 1.0)
    assert np.array_equal(gpu.bf16_gemv(w, x), orc.gemv(w, x))
    assert np.array_equal(gpu.bf16_matvec_f32(w, x), orc.matvec_f32(w, x))


@pytest.mark.parametrize("M", [1, 2, 3, 5, 64, 300])
def test_hook_gemm_bitwise(gpu, orc, M):
    rng = np.random.default_rng(M)
    O, K = 96, 200
    w, x = rng_codes(rng, (O, K), 0.5), rng_codes(rng, (M, K), 1.0)
    assert np.array_equal(gpu.bf16_gemm(w, x), orc.gemm(w, x))


def test_hook_zero_dims_and_counters(gpu):
    assert gpu.lib.apus_cuda_bf16_gemv(None, None, None, 0, 8) != 0
    assert gpu.lib.apus_cuda_bf16_gemm(None, None, None, 1, 0, 8) != 0
    rng = np.random.default_rng(1)
    w, x = rng_codes(rng, (64, 64), 0.5), rng_codes(rng, 64, 1.0)
    up0, l0 = gpu.bytes_uploaded(), gpu.launches()
    gpu.bf16_gemv(w, x)
    gpu.bf16_gemv(w, x)      # second call reuses the resident copy
    assert gpu.bytes_uploaded() - up0 == w.nbytes
    assert gpu.launches() - l0 == 2


def test_hooks_inside_the_reference_engine(gpu, ref, be, synth):
    """Drop-in: the backend's three entry points installed into the
    reference's own hook table; the reference's MoE block, run through its own
    layer code, must reproduce its CPU result bit for bit (the per-op hooks
    keep the anchor's order)."""
    cfg = synth.MINI_CFG
    W = synth.host_weights(be, cfg, seed=21, sigma=0.08)
    x = synth.host_x(be, 5, cfg["hidden"], seed=21)
    cpu = ref.moe_block(cfg, W, x)
    l0 = gpu.launches()
    ref.set_hooks(gpu.lib.apus_cuda_bf16_gemv, gpu.lib.apus_cuda_bf16_gemm,
                  gpu.lib.apus_cuda_bf16_matvec_f32)
    try:
        for batched in (False, True):
            hooked = ref.moe_block(cfg, W, x, batched=batched)
            for k in ("idx", "w", "routed", "shared", "out"):
                assert np.array_equal(cpu[k], hooked[k]), (k, batched)
    finally:
        ref.set_hooks(None, None, None)
    assert gpu.launches() > l0       # the GPU really ran them


# ---- router ----------------------------------------------------------------------

def test_router_golden(gpu):
    m = manifest()
    E, K, TK = m["RTR_E"], m["RTR_K"], m["RTR_TK"]
    x = rd("moe_rtr_x.bin", np.uint16)
    wg = rd("moe_rtr_wg.bin", np.uint16).reshape(E, K)
    idx, w = gpu.moe_route(x, wg, TK)
    assert idx[0].tolist() == rd("moe_rtr_idx.bin", np.int64).tolist()
    assert tol_ok(f32(w[0]).astype(np.float64), rd("moe_rtr_w.bin", np.float64),
                  0.02, 0.008, 0.008).all()
    assert gpu.moe_route_topn(x, wg, TK).tolist() == idx[0].tolist()
    assert gpu.moe_route_topn(x, wg, TK + 4)[:TK].tolist() == idx[0].tolist()


def test_router_tie_kats(gpu):
    E, K, TK = 16, 4, 8
    x = np.array([0x3F80, 0, 0, 0], np.uint16)
    wg = np.zeros((E, K), np.uint16)
    wg[:, 0] = 0x3F00
    idx, w = gpu.moe_route(x, wg, TK)
    assert idx[0].tolist() == list(range(8))
    assert (w[0] == 0x3E00).all()
    wg[:, 0] = 0
    wg[:9, 0] = 0x3F80
    idx, _ = gpu.moe_route(x, wg, TK)
    assert idx[0].tolist() == list(range(8))


@pytest.mark.parametrize("T,E,K,TK,sx,sw", [
    (1, 256, 2048, 8, 1.0, 0.02), (2, 256, 2048, 8, 1.0, 0.02),
    (5, 16, 128, 4, 1.0, 0.08), (64, 256, 2048, 8, 1.0, 0.02),
    (300, 256, 2048, 8, 1.0, 0.02), (1111, 256, 2048, 8, 1.0, 0.02),
    (37, 100, 72, 6, 1.0, 0.1), (9, 33, 37, 5, 1.0, 0.1),
    (300, 256, 2048, 8, 1e-19, 1e-19),      # products underflow: literal chain
])
def test_router_bit_exact(gpu, orc, T, E, K, TK, sx, sw):
    """Selected ids, BF16 logits and BF16 routing weights against the CPU
    checker.  Logit ties are frequent here (256 BF16 logits per token), so
    the lowest-index rule is exercised on almost every token."""
    rng = np.random.default_rng(T * 7 + E)
    x = rng_codes(rng, (T, K), 0.4 * sx)
    wg = rng_codes(rng, (E, K), sw * 0.5)
    idx, w, lg = gpu.moe_route(x, wg, TK, want_logits=True)
    oi, ow, ol = orc.route_batch(x, wg, TK, want_logits=True)
    assert np.array_equal(lg, ol)            # logits: bit-exact chains
    assert np.array_equal(idx, oi)           # selection: bit-exact
    # weights: expf last-bit class only — at most one BF16 ulp, and rare
    d = np.abs(w.astype(np.int32) - ow.astype(np.int32))
    assert d.max() <= 1
    assert (d != 0).mean() <= 0.002


# ---- dispatch ------------------------------------------------------------------------

@pytest.mark.parametrize("T,TK,E,skew", [
    (1, 8, 256, False), (3, 8, 256, False), (5, 4, 16, False),
    (64, 8, 256, False), (300, 8, 256, False), (512, 8, 256, False),
    (513, 8, 256, True), (1000, 8, 256, True), (8192, 8, 256, True),
    (8448, 8, 256, False), (700, 6, 1000, False)])
def test_dispatch_bit_exact(gpu, orc, T, TK, E, skew):
    rng = np.random.default_rng(T + E)
    p = None
    if skew:
        p = np.arange(1, E + 1, dtype=np.float64) ** -1.1
        p = p[rng.permutation(E)]
        p /= p.sum()
    idx = np.stack([rng.choice(E, TK, replace=False, p=p) for _ in range(T)]
                   ).astype(np.int32)
    counts, offsets, perm = gpu.moe_dispatch(idx, E)
    oc, oo, op = orc.dispatch(idx, E)
    assert np.array_equal(counts, oc)
    assert np.array_equal(offsets, oo)
    assert np.array_equal(perm, op)


def test_dispatch_rejects_bad_expert_id(gpu):
    idx = np.array([[0, 1, 2, 999]], np.int32)
    with pytest.raises(Exception):
        gpu.moe_dispatch(idx, 16)
    # the context stays usable
    c, o, p = gpu.moe_dispatch(np.array([[3, 1, 2, 0]], np.int32), 16)
    assert p.tolist() == [3, 1, 2, 0]


# --- many-token router: fast logits + exact chains for the candidates ---------
def _route_dev(gpu, synth, cfg, W, x):
    """idx [T, TK], w [T, TK] from apus_cuda_route_dev on a resident layer."""
    import torch
    T = x.shape[0]
    layer = gpu.layer_create(cfg, W)
    d_x = torch.from_numpy(x.view(np.int16)).cuda()
    d_idx = torch.full((T, cfg["top_k"]), -1, dtype=torch.int32, device="cuda")
    d_w = torch.zeros((T, cfg["top_k"]), dtype=torch.int16, device="cuda")
    torch.cuda.synchronize()
    gpu.route_dev(layer, d_x.data_ptr(), T, d_idx.data_ptr(), d_w.data_ptr(),
                  stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return d_idx.cpu().numpy(), d_w.cpu().numpy().view(np.uint16)


CERT_CFG = dict(hidden=512, experts=128, moe_inter=128, shared_inter=128,
                top_k=8)


@pytest.mark.parametrize("T", [65, 257, 1000])
@pytest.mark.parametrize("case", ["plain", "tied_rows", "tiny_logits", "skewed"])
def test_router_certified_selection_is_exact(gpu, orc, be, synth, T, case):
    """Above 64 tokens the router scores all experts on the tensor cores and
    walks the exact chain only for experts that can still reach the top_k.
    The selection must equal the exact router's bit for bit, also when rows of
    the router matrix are identical (every logit tied with its neighbour), when
    all logits are tiny, and when a few experts dominate."""
    cfg = CERT_CFG
    W = synth.host_weights(be, cfg, seed=900 + T, sigma=0.05)
    x = synth.host_x(be, T, cfg["hidden"], seed=900 + T)
    rtr = W["rtr_w"]
    if case == "tied_rows":
        rtr[1::2] = rtr[0::2]
    elif case == "tiny_logits":
        rtr[:] = synth.f32_to_bf16(synth.bf16_to_f32(rtr) * 2.0 ** -20)
    elif case == "skewed":
        W, x = synth.apply_router_bias(W, x, synth.zipf_bias(cfg, seed=3))
        rtr = W["rtr_w"]
    before = gpu.router_exact_chains()
    idx, w = _route_dev(gpu, synth, cfg, W, x)
    chains = gpu.router_exact_chains() - before
    assert gpu.last_block_status() == 0          # includes the error-bound check
    eidx, ew = orc.route_batch(x, rtr, cfg["top_k"])
    assert np.array_equal(idx, eidx)
    d = np.abs(w.astype(np.int32) - ew.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() <= 0.002
    # the certified path ran, and it ran far fewer chains than E per token
    assert cfg["top_k"] * T <= chains
    if case in ("plain", "skewed"):
        assert chains <= 4 * cfg["top_k"] * T


def test_router_certified_can_be_switched_off(be, orc, synth, monkeypatch):
    monkeypatch.setenv("APUS_CUDA_ROUTER_CERTIFY", "0")
    be.enable()
    try:
        cfg = CERT_CFG
        W = synth.host_weights(be, cfg, seed=77, sigma=0.05)
        x = synth.host_x(be, 130, cfg["hidden"], seed=77)
        before = be.router_exact_chains()
        idx, w = _route_dev(be, synth, cfg, W, x)
        assert be.router_exact_chains() == before
        eidx, _ = orc.route_batch(x, W["rtr_w"], cfg["top_k"])
        assert np.array_equal(idx, eidx)
    finally:
        be.disable()


# --- the callers either side of the block: rmsnorm before, residual add after ---
@pytest.mark.parametrize("T,N", [(1, 2048), (5, 2048), (33, 512), (3, 130), (2, 24)])
def test_rmsnorm_and_residual_add_bitwise(gpu, orc, be, synth, T, N):
    """apus_cuda_rmsnorm_dev / apus_cuda_resadd_dev against the checker
    (c/attn.h:175-186 with its sequential sum of squares; c/layer.h:230-234):
    bit for bit, with and without a gain vector, rows that are not a multiple
    of the vector width included."""
    import torch
    x = synth.f32_to_bf16(
        synth.bf16_to_f32(be.synth_fill_host(T * N, 5, 0, 0, 1.0)).reshape(T, N) * 3.0)
    gw = be.synth_fill_host(N, 5, 1, 1, 0.3)
    sp = torch.cuda.current_stream().cuda_stream
    d_x = torch.from_numpy(x.view(np.int16)).cuda()
    d_w = torch.from_numpy(gw.view(np.int16)).cuda()
    d_y = torch.empty_like(d_x)
    for w_dev, w_host in ((d_w, gw), (None, None)):
        gpu.rmsnorm_dev(d_x.data_ptr(), w_dev.data_ptr() if w_dev is not None else None,
                        d_y.data_ptr(), T, N, stream=sp)
        torch.cuda.synchronize()
        assert np.array_equal(d_y.cpu().numpy().view(np.uint16), orc.rmsnorm(x, w_host))
    b = be.synth_fill_host(T * N, 6, 0, 0, 1.0).reshape(T, N)
    d_b = torch.from_numpy(b.view(np.int16)).cuda()
    gpu.resadd_dev(d_x.data_ptr(), d_b.data_ptr(), d_y.data_ptr(), T * N, stream=sp)
    torch.cuda.synchronize()
    assert np.array_equal(d_y.cpu().numpy().view(np.uint16), orc.resadd(x, b))


# ---- the dense weight stream on device pointers --------------------------------

@pytest.mark.parametrize("M,O,K", [(1, 4096, 2048), (3, 1000, 512), (8, 777, 256),
                                   (1, 1, 256), (2, 33, 2048)])
def test_gemv_stream_dev(gpu, orc, M, O, K):
    """apus_cuda_bf16_gemv_dev against the CPU anchor: same products, another
    summation order, so BF16 tolerance (the hooks keep the exact bits)."""
    import torch
    rng = np.random.default_rng(M * 1000 + O)
    w, x = rng_codes(rng, (O, K), 0.05), rng_codes(rng, (M, K), 1.0)
    d_w = torch.from_numpy(w.view(np.int16)).cuda()
    d_x = torch.from_numpy(x.view(np.int16)).cuda()
    d_y = torch.zeros((M, O), dtype=torch.int16, device="cuda")
    gpu.bf16_gemv_dev(d_w.data_ptr(), d_x.data_ptr(), d_y.data_ptr(), M, O, K,
                      stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    got = f32(d_y.cpu().numpy().view(np.uint16))
    exp = f32(orc.gemm(w, x))
    scale = np.abs(exp).max() + 1e-9
    assert np.abs(got - exp).max() <= 1e-2 * scale
    assert (got.view(np.uint32) != exp.view(np.uint32)).mean() <= 0.2
