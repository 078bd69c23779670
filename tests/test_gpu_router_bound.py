"""The many-token router decides which experts need the engine's exact
sequential chain (c/moe.h:289-291) from fast tensor-core logits widened by an
error bound B(t, e) = cbound * ||x_t|| * ||w_e||.  The kernel checks the bound
only on the pairs it evaluates exactly; a pair it excludes is never looked at
again, so the bound itself is checked here on EVERY (token, expert) pair at the
real dimensions, against the exact fp32 chain of the CPU checker, for inputs
that stress it in different ways.  Through the C-ABI
(apus_cuda_debug_fast_logits)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

E, H, T = 256, 2048, 1024


def _inputs(be, synth, kind):
    cfg = synth.QWEN_CFG
    x = synth.host_x(be, T, H, seed=77)
    wg = be.synth_fill_host(E * H, 77, 0, synth.T_RTR, synth.W_SIGMA).reshape(E, H)
    if kind == "same_sign":
        # every product positive: no cancellation, the sums are as large as
        # the bound's sum of magnitudes
        x = x & 0x7FFF
        wg = wg & 0x7FFF
    elif kind == "wide_range":
        # token channels scaled by 2^-12 .. 2^12: a few huge terms among many
        # tiny ones
        rng = np.random.default_rng(5)
        sc = np.exp2(rng.integers(-12, 13, size=H)).astype(np.float32)
        x = synth.f32_to_bf16(synth.bf16_to_f32(x) * sc[None, :])
    elif kind == "zipf":
        W, x = synth.apply_router_bias({"rtr_w": wg}, x,
                                       synth.zipf_bias(cfg, seed=77, beta=0.27))
        wg = W["rtr_w"]
    return np.ascontiguousarray(x), np.ascontiguousarray(wg)


@pytest.mark.parametrize("kind", ["plain", "same_sign", "wide_range", "zipf"])
def test_fast_logits_within_the_bound_on_every_pair(gpu, orc, be, synth, kind):
    x, wg = _inputs(be, synth, kind)
    fast, xnorm, wnorm, cbound = gpu.debug_fast_logits(x, wg)
    exact = np.stack([orc.matvec_f32(wg, x[t]) for t in range(T)])   # fp32 chains
    # the chains really are the router's logits before narrowing
    _, _, lg = orc.route_batch(x[:8], wg, 8, want_logits=True)
    assert np.array_equal(synth.f32_to_bf16(exact[:8]), lg)
    B = (np.float32(cbound) * xnorm)[:, None] * wnorm[None, :E]
    err = np.abs(fast.astype(np.float64) - exact.astype(np.float64))
    ratio = float((err / B).max())
    print(f"[{kind}] max |fast - exact| / B over {T * E} pairs: {ratio:.3g} "
          f"(max err {err.max():.3g}, min B {B.min():.3g})")
    assert np.isfinite(fast).all()
    assert (err <= B).all(), ratio
    # the norms the bound uses are upper bounds of the true norms
    xf = synth.bf16_to_f32(x).astype(np.float64)
    wf = synth.bf16_to_f32(wg).astype(np.float64)
    assert (xnorm >= np.sqrt((xf * xf).sum(1))).all()
    assert (wnorm[:E] >= np.sqrt((wf * wf).sum(1))).all()
    assert wnorm[E] == wnorm[:E].max()


@pytest.mark.parametrize("kind", ["plain", "same_sign", "wide_range", "zipf"])
def test_certified_selection_equals_the_exact_router(gpu, orc, be, synth, kind):
    """Same inputs through the router proper: ids of every token bit-exact."""
    x, wg = _inputs(be, synth, kind)
    cfg = synth.QWEN_CFG
    import torch
    layer = gpu.layer_create(cfg, None)
    gpu.layer_upload(layer, "rtr_w", wg)
    d_x = torch.from_numpy(x.view(np.int16)).cuda()
    d_idx = torch.empty((T, 8), dtype=torch.int32, device="cuda")
    d_w = torch.empty((T, 8), dtype=torch.int16, device="cuda")
    c0 = gpu.router_exact_chains()
    gpu.route_dev(layer, d_x.data_ptr(), T, d_idx.data_ptr(), d_w.data_ptr(),
                  stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert gpu.last_block_status() == 0
    chains = gpu.router_exact_chains() - c0
    # the certified path ran; on ordinary inputs it walks a small fraction of
    # the T * E chains (same-sign inputs put most logits within rounding
    # distance of each other, where nearly every chain is needed)
    assert 0 < chains <= T * (E + 1)
    if kind in ("plain", "zipf"):
        assert chains < T * E // 8
    idx, _ = orc.route_batch(x, wg, 8)
    assert np.array_equal(d_idx.cpu().numpy(), idx)
    gpu.layer_destroy(layer)
