"""Edge behaviour the reference pins in tests/m4a/test_moe.c (:230-263 equal
logits, :370-374 silu(0) = +0, :433-446 zero weights and k = 1), exercised on
the GPU through the C-ABI; an RNE-narrowing sweep of the device's bf16_bits
against the reference's; the fail-soft knobs of the enable call
(tests/m10/test_kernels.c:194-238 is the reference's idiom for them); the
ordering of calls that arrive on different streams; workspace growth after a
graph capture."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def f32(c):
    return (np.asarray(c, np.uint16).astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("T", [1, 3, 9, 80])
def test_zero_input_gives_plus_zero_and_first_experts(gpu, be, synth, T):
    """x = 0: every logit is 0, so idx = 0..k-1 and w = 1/k exactly
    (k a power of two); silu(0) = +0 makes every expert output +0, the shared
    gate is rnd(0.5) times +0: moe_out is the code 0x0000, never -0."""
    cfg = dict(hidden=256, experts=32, moe_inter=128, shared_inter=128, top_k=8)
    W = synth.host_weights(be, cfg, seed=2, sigma=0.05)
    x = np.zeros((T, cfg["hidden"]), np.uint16)
    got = gpu.moe_block(cfg, W, x)
    assert (got["idx"] == np.arange(8)[None, :]).all()
    assert (got["w"] == 0x3E00).all()
    for k in ("routed", "shared", "out"):
        assert (got[k] == 0).all(), k
    assert gpu.last_block_status() == 0


@pytest.mark.parametrize("T", [2, 70])
def test_zero_weights_give_plus_zero(gpu, be, synth, T):
    cfg = dict(hidden=256, experts=32, moe_inter=128, shared_inter=128, top_k=4)
    W = {k: np.zeros_like(v) for k, v in
         synth.host_weights(be, cfg, seed=2, sigma=0.05).items()}
    x = synth.host_x(be, T, cfg["hidden"], seed=4)
    got = gpu.moe_block(cfg, W, x)
    assert (got["idx"] == np.arange(4)[None, :]).all()
    assert (got["w"] == 0x3E80).all()          # 0.25
    for k in ("routed", "shared", "out"):
        assert (got[k] == 0).all(), k


@pytest.mark.parametrize("T", [1, 6, 72])
def test_single_slot_combine_is_the_weighted_row(gpu, orc, be, synth, T):
    """top_k = 1: the renormalised weight is exactly 1.0 and the routed row is
    rnd(1.0 * y) = the expert's own BF16 output."""
    cfg = dict(hidden=256, experts=16, moe_inter=128, shared_inter=128, top_k=1)
    W = synth.host_weights(be, cfg, seed=6, sigma=0.06)
    x = synth.host_x(be, T, cfg["hidden"], seed=6)
    got, exp = gpu.moe_block(cfg, W, x), orc.moe_block(cfg, W, x)
    assert np.array_equal(got["idx"], exp["idx"])
    assert (got["w"] == 0x3F80).all() and (exp["w"] == 0x3F80).all()
    assert np.abs(f32(got["routed"]) - f32(exp["routed"])).max() <= 2e-2
    assert np.abs(f32(got["out"]) - f32(exp["out"])).max() <= 2e-2


def test_device_narrowing_equals_the_reference(gpu, orc):
    """bf16_bits on the device against the checker's (c/bf16.h:268-274), over
    sums a + b of BF16 values that land on and around rounding ties, through
    the public GEMV hook (K = 8: y = rnd(a*1 + b*1))."""
    rng = np.random.default_rng(9)
    n = 1 << 17
    a = rng.integers(0, 1 << 16, n).astype(np.uint16)
    # b a small multiple of a's half-ulp: exact ties, just below, just above
    ea = ((a >> 7) & 0xFF).astype(np.int32)
    k = rng.integers(-3, 4, n)
    eb = np.clip(ea - 8 - rng.integers(0, 3, n), 1, 254)
    b = ((eb << 7) | (rng.integers(0, 2, n) << 15) | (np.abs(k) << 4)).astype(np.uint16)
    finite = (ea < 255) & (ea > 0)
    a, b = a[finite], b[finite]
    O = a.size
    w = np.zeros((O, 8), np.uint16)
    w[:, 0], w[:, 1] = a, b
    x = np.zeros(8, np.uint16)
    x[0] = x[1] = 0x3F80
    got = gpu.bf16_gemv(w, x)
    s = f32(a) + f32(b)                       # fp32 sum, as the chain computes it
    exp = np.array([orc.bf16_bits(v) for v in s[:4096]], np.uint16)
    assert np.array_equal(got[:4096], exp)
    assert np.array_equal(got, orc.gemv(w, x))
    # ties really occur in the sweep
    u = s.view(np.uint32)
    assert ((u & 0xFFFF) == 0x8000).sum() > 100


def test_dense_budget_makes_a_hook_decline(be, monkeypatch):
    """APUS_CUDA_DENSE_MB: past the budget a per-matmul entry point returns
    nonzero (the engine then runs its CPU kernel); within it, it works."""
    monkeypatch.setenv("APUS_CUDA_DENSE_MB", "1")
    be.enable()
    try:
        rng = np.random.default_rng(3)
        small = rng.integers(0x3C00, 0x3F00, (64, 512)).astype(np.uint16)
        big = rng.integers(0x3C00, 0x3F00, (1024, 1024)).astype(np.uint16)   # 2 MiB
        x = rng.integers(0x3C00, 0x3F00, 1024).astype(np.uint16)
        be.bf16_gemv(small, x[:512])
        with pytest.raises(Exception) as ei:
            be.bf16_gemv(big, x)
        assert "budget" in str(ei.value)
        be.bf16_gemv(small, x[:512])           # still usable
    finally:
        be.disable()


def test_no_moe_knob_leaves_the_block_slot_empty(be, monkeypatch):
    import ctypes as C
    hooks = C.c_void_p.in_dll(be.lib, "apus_cuda_block_hooks")
    monkeypatch.setenv("APUS_CUDA_NO_MOE", "1")
    be.enable()
    try:
        assert hooks.value is None
    finally:
        be.disable()
    monkeypatch.delenv("APUS_CUDA_NO_MOE")
    be.enable()
    try:
        assert hooks.value is not None
    finally:
        be.disable()
    assert C.c_void_p.in_dll(be.lib, "apus_cuda_block_hooks").value is None


def test_calls_on_two_streams_are_ordered(gpu, orc, be, synth):
    """All device-pointer calls share one workspace; the library orders a call
    behind the previous one when it arrives on another stream.  Two layers,
    two streams, calls interleaved without any synchronisation in between:
    each result must equal the one computed alone."""
    import torch
    cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128, top_k=8)
    layers, xs, alone = [], [], []
    for i, T in enumerate((3, 200)):           # one-kernel path and GEMM path
        W = synth.host_weights(be, cfg, seed=40 + i, sigma=0.05)
        layers.append(gpu.layer_create(cfg, W))
        x = synth.host_x(be, T, cfg["hidden"], seed=40 + i)
        xs.append(torch.from_numpy(x.view(np.int16)).cuda())
    outs = [torch.empty_like(x) for x in xs]
    for i in range(2):
        gpu.moe_block_dev(layers[i], xs[i].data_ptr(), outs[i].data_ptr(),
                          xs[i].shape[0])
        torch.cuda.synchronize()
        alone.append(outs[i].cpu().numpy().copy())
        outs[i].zero_()
    s = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for rep in range(6):
        for i in range(2):
            gpu.moe_block_dev(layers[i], xs[i].data_ptr(), outs[i].data_ptr(),
                              xs[i].shape[0], stream=s[i].cuda_stream)
    torch.cuda.synchronize()
    assert gpu.last_block_status() == 0
    for i in range(2):
        assert np.array_equal(outs[i].cpu().numpy(), alone[i]), i


def test_graph_survives_workspace_growth(gpu, be, synth):
    """A graph captured at a small size keeps replaying correctly after a
    later, larger call has grown the workspace (the outgrown arena stays
    allocated), and growth inside a capture is refused, not performed."""
    import torch
    cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128, top_k=8)
    W = synth.host_weights(be, cfg, seed=50, sigma=0.05)
    layer = gpu.layer_create(cfg, W)
    T = 96
    x = torch.from_numpy(synth.host_x(be, T, cfg["hidden"], seed=50).view(np.int16)).cuda()
    out = torch.empty_like(x)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        gpu.moe_block_dev(layer, x.data_ptr(), out.data_ptr(), T,
                          stream=stream.cuda_stream)
        torch.cuda.synchronize()
        want = out.cpu().numpy().copy()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            gpu.moe_block_dev(layer, x.data_ptr(), out.data_ptr(), T,
                              stream=torch.cuda.current_stream().cuda_stream)
        # a much larger call grows the arena
        Tb = 3000
        xb = torch.from_numpy(synth.host_x(be, Tb, cfg["hidden"], seed=51).view(np.int16)).cuda()
        ob = torch.empty_like(xb)
        gpu.moe_block_dev(layer, xb.data_ptr(), ob.data_ptr(), Tb,
                          stream=stream.cuda_stream)
        torch.cuda.synchronize()
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want)
        assert gpu.last_block_status() == 0
        # growth inside a capture: refused with a message that names the cure
        Tc = 9000
        xc = torch.zeros((Tc, cfg["hidden"]), dtype=torch.int16, device="cuda")
        oc = torch.empty_like(xc)
        g2 = torch.cuda.CUDAGraph()
        msg = ""
        try:
            with torch.cuda.graph(g2, stream=stream):
                try:
                    gpu.moe_block_dev(layer, xc.data_ptr(), oc.data_ptr(), Tc,
                                      stream=torch.cuda.current_stream().cuda_stream)
                except Exception as e:
                    msg = str(e)
        except Exception:
            pass                      # an empty capture may itself be refused
        torch.cuda.synchronize()
        assert "apus_cuda_reserve" in msg


def test_host_call_in_two_halves_gives_the_same_bits(be, synth, monkeypatch):
    """From 4096 tokens the host-pointer call runs as two half calls whose PCIe
    copies overlap the other half's kernels (APUS_CUDA_HOST_SPLIT_T): every
    output and trace array equals the single call bit for bit, odd token count
    included."""
    cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128, top_k=8)
    W = synth.host_weights(be, cfg, seed=41, sigma=0.05)
    x = synth.host_x(be, 4101, cfg["hidden"], seed=41)
    res = {}
    for split in ("0", "4096"):
        monkeypatch.setenv("APUS_CUDA_HOST_SPLIT_T", split)
        be.enable()
        try:
            res[split] = be.moe_block(cfg, W, x)
            assert be.last_block_status() == 0
        finally:
            be.disable()
    for k in ("idx", "w", "shared", "routed", "out"):
        assert np.array_equal(res["0"][k], res["4096"][k]), k


def test_no_token_is_a_successful_no_op(gpu, be, synth):
    """T = 0: the engine's loops run zero times (c/layer.h:589); the block call
    returns success and writes nothing, host and device entry points alike."""
    import ctypes as C
    import torch
    cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128, top_k=8)
    W = synth.host_weights(be, cfg, seed=43, sigma=0.05)
    layer = gpu.layer_create(cfg, W)
    d = torch.full((4, cfg["hidden"]), 0x1234, dtype=torch.int16, device="cuda")
    rc = gpu.lib.apus_cuda_moe_block_dev(layer, d.data_ptr(), d.data_ptr(), 0, None, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert int((d != 0x1234).sum()) == 0
    gpu.layer_destroy(layer)
    x = synth.host_x(be, 1, cfg["hidden"], seed=43)
    res = gpu.moe_block(cfg, W, x[:0])              # host pointers, T = 0
    assert res["out"].shape == (0, cfg["hidden"]) and res["idx"].shape == (0, 8)
