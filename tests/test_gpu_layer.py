"""The block with its two neighbours folded in (c/layer.h:386-388):
res_out = rnd(res + moe_block(rmsnorm(res, 1 + ln_w))), one entry point, and a
stack of such layers in place on one residual stream.  Must equal, bit for bit,
the three separate calls (rmsnorm, block, residual add), which are themselves
checked against the CPU checker; and the CPU checker's chain directly."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MID = dict(hidden=512, experts=64, moe_inter=128, shared_inter=128, top_k=8)


def f32(c):
    return (np.asarray(c, np.uint16).astype(np.uint32) << 16).view(np.float32)


def _dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()


def _three_calls(gpu, torch, layer, d_res, d_w, T, H):
    ln = torch.empty_like(d_res)
    moe = torch.empty_like(d_res)
    out = torch.empty_like(d_res)
    gpu.rmsnorm_dev(d_res.data_ptr(), d_w.data_ptr() if d_w is not None else None,
                    ln.data_ptr(), T, H)
    gpu.moe_block_dev(layer, ln.data_ptr(), moe.data_ptr(), T)
    gpu.resadd_dev(d_res.data_ptr(), moe.data_ptr(), out.data_ptr(), T * H)
    torch.cuda.synchronize()
    return moe.cpu().numpy().view(np.uint16), out.cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("T", [1, 2, 4, 5, 9, 80, 300])
@pytest.mark.parametrize("gains", [False, True])
def test_layer_equals_three_calls_and_the_checker(gpu, orc, be, synth, T, gains):
    import torch
    cfg, H = MID, MID["hidden"]
    W = synth.host_weights(be, cfg, seed=80, sigma=0.05)
    layer = gpu.layer_create(cfg, W)
    rng = np.random.default_rng(T)
    res = synth.f32_to_bf16(rng.normal(0, 1.7, (T, H)).astype(np.float32))
    lnw = synth.f32_to_bf16(rng.normal(0, 0.1, H).astype(np.float32)) if gains else None
    d_res = _dev(torch, res)
    d_w = _dev(torch, lnw) if gains else None
    moe3, out3 = _three_calls(gpu, torch, layer, d_res, d_w, T, H)
    d_out = torch.empty_like(d_res)
    d_tr = torch.empty_like(d_res)
    gpu.moe_layer_dev(layer, d_res.data_ptr(), d_w.data_ptr() if gains else None,
                      d_out.data_ptr(), T, d_trace={"out": d_tr.data_ptr()})
    torch.cuda.synchronize()
    assert gpu.last_block_status() == 0
    assert gpu.last_block_launches() == (1 if T <= 4 else gpu.last_block_launches())
    assert np.array_equal(d_out.cpu().numpy().view(np.uint16), out3)
    assert np.array_equal(d_tr.cpu().numpy().view(np.uint16), moe3)
    # the CPU checker's chain
    ln = orc.rmsnorm(res, lnw)
    exp = orc.resadd(res, orc.moe_block(cfg, W, ln)["out"])
    assert np.abs(f32(out3) - f32(exp)).max() <= 4e-2      # a BF16 step of |res + moe| ~ 4
    # in place
    d_in = d_res.clone()
    gpu.moe_layer_dev(layer, d_in.data_ptr(), d_w.data_ptr() if gains else None,
                      d_in.data_ptr(), T)
    torch.cuda.synchronize()
    assert np.array_equal(d_in.cpu().numpy().view(np.uint16), out3)


@pytest.mark.parametrize("T", [1, 3, 40])
def test_stack_in_place_equals_the_chain_of_calls(gpu, be, synth, T):
    import torch
    cfg, H, L = MID, MID["hidden"], 3
    layers = [gpu.layer_create(cfg, synth.host_weights(be, cfg, seed=81, layer=l, sigma=0.05))
              for l in range(L)]
    res = synth.host_x(be, T, H, seed=81)
    d = _dev(torch, res)
    ref = d.clone()
    for lay in layers:
        _, out = _three_calls(gpu, torch, lay, ref, None, T, H)
        ref = _dev(torch, out)
    gpu.moe_stack_dev(layers, d.data_ptr(), T)
    torch.cuda.synchronize()
    assert gpu.last_block_status() == 0
    assert np.array_equal(d.cpu().numpy(), ref.cpu().numpy())
    if T <= 4:
        assert gpu.last_block_launches() == L          # one kernel per layer


def test_layer_at_the_real_dimensions_one_token(gpu, orc, be, synth):
    import torch
    cfg = synth.QWEN_CFG
    layer = gpu.layer_create(cfg, None)
    synth.device_weights(gpu, layer, cfg, seed=5, layer=0)
    H = cfg["hidden"]
    res = synth.f32_to_bf16(np.random.default_rng(5).normal(0, 2.0, (1, H)).astype(np.float32))
    d_res = _dev(torch, res)
    moe3, out3 = _three_calls(gpu, torch, layer, d_res, None, 1, H)
    d_out = torch.empty_like(d_res)
    gpu.moe_layer_dev(layer, d_res.data_ptr(), None, d_out.data_ptr(), 1)
    torch.cuda.synchronize()
    assert gpu.last_block_launches() == 1
    assert np.array_equal(d_out.cpu().numpy().view(np.uint16), out3)
