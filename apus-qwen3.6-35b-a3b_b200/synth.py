"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (random-init weights ~N(0, 0.02), activations
~N(0, 1) then RMS-normalised).  Every tensor is a counter-based stream
(csrc/synth.h), so the same (seed, layer, tensor) can be produced on the host
for the CPU checker and directly in HBM for the GPU without copying.
"""
import numpy as np

QWEN_CFG = dict(hidden=2048, experts=256, moe_inter=512, shared_inter=512,
                top_k=8)
MINI_CFG = dict(hidden=128, experts=16, moe_inter=32, shared_inter=32,
                top_k=4)

T_X, T_RTR, T_GU, T_D, T_SG, T_SU, T_SD, T_SGATE, T_BIAS = range(9)
W_SIGMA = 0.02


def weight_shapes(cfg):
    H, E, I, Is = (cfg["hidden"], cfg["experts"], cfg["moe_inter"],
                   cfg["shared_inter"])
    return dict(rtr_w=(T_RTR, (E, H)), exp_gu=(T_GU, (E, 2 * I, H)),
                exp_d=(T_D, (E, H, I)), sh_g=(T_SG, (Is, H)),
                sh_u=(T_SU, (Is, H)), sh_d=(T_SD, (H, Is)),
                sh_gate=(T_SGATE, (1, H)))


def bf16_to_f32(codes):
    return (np.asarray(codes, np.uint16).astype(np.uint32) << 16).view(
        np.float32)


def f32_to_bf16(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7fffffff) > 0x7f800000
    r = (u + 0x7fff + ((u >> 16) & 1)) >> 16
    return np.where(nan, u >> 16, r).astype(np.uint16)


def host_weights(be, cfg, seed=0, layer=0, sigma=W_SIGMA):
    """All MoE weights of one layer as host uint16 arrays."""
    W = {}
    for name, (tid, shape) in weight_shapes(cfg).items():
        n = int(np.prod(shape))
        W[name] = be.synth_fill_host(n, seed, layer, tid, sigma).reshape(shape)
    return W


def device_weights(be, layer_handle, cfg, seed=0, layer=0, sigma=W_SIGMA,
                   expert_begin=0, expert_end=None, stream=None):
    """Fill a device-resident layer (created with W=None) in place."""
    H, I = cfg["hidden"], cfg["moe_inter"]
    for name, (tid, shape) in weight_shapes(cfg).items():
        p, n = be.layer_tensor(layer_handle, name)
        first = 0
        if name == "exp_gu":
            first = expert_begin * 2 * I * H
        elif name == "exp_d":
            first = expert_begin * H * I
        be.synth_fill_dev(p, n, seed, layer, tid, sigma, first=first,
                          stream=stream)
    be.layer_refresh(layer_handle)


def host_x(be, T, H, seed=0, layer=0):
    """x ~ N(0,1) per element, each row scaled to unit RMS (the engine's
    RMSNorm with zero gain offset, c/attn.h:175-186, evaluated in float64),
    rounded to BF16."""
    raw = bf16_to_f32(be.synth_fill_host(T * H, seed, layer, T_X, 1.0))
    v = raw.reshape(T, H).astype(np.float64)
    rs = 1.0 / np.sqrt((v * v).mean(axis=1, keepdims=True) + 1e-6)
    return f32_to_bf16((v * rs).astype(np.float32))


def zipf_bias(cfg, seed=0, s=1.1, beta=1.0):
    """Per-expert router bias b_e = beta * ln p_e with p_e ~ rank^-s over a
    seeded permutation of the experts."""
    E = cfg["experts"]
    rng = np.random.default_rng(seed + 7919)
    order = rng.permutation(E)
    p = np.empty(E)
    p[order] = (np.arange(1, E + 1, dtype=np.float64)) ** (-s)
    p /= p.sum()
    return beta * np.log(p)


def apply_router_bias(W, x, bias):
    """The engine's router takes no bias (c/moe.h:35-36), so a bias is
    realised inside its own API: the last hidden channel of every token is
    set to 1.0 and the bias goes into that column of the router matrix."""
    W = dict(W)
    rtr = W["rtr_w"].copy()
    rtr[:, -1] = f32_to_bf16(np.asarray(bias, np.float32))
    W["rtr_w"] = rtr
    x = x.copy()
    x[:, -1] = 0x3F80
    return W, x
