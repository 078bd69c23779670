"""CPU suite: pins the plain-C restatement (oracle/moe_oracle.c) against the
reference's golden vectors, its known-answer tests, and bit-for-bit against the
reference's own compiled code (oracle/_ref).  Mirrors tests/m4a/test_moe.c,
tests/m9c (batched == per-token) and tests/m12 (hot == scalar anchor) of the
reference.  No GPU involved."""
import hashlib
import os

import numpy as np
import pytest

G = os.path.join(os.path.dirname(__file__), "golden")


def rd(name, dt):
    return np.fromfile(os.path.join(G, "m4a", name), dtype=dt)


def manifest():
    out = {}
    for line in open(os.path.join(G, "m4a", "manifest.txt")):
        k, v = line.strip().split("=")
        out[k] = int(v)
    return out


def f32(codes):
    return (np.asarray(codes, np.uint16).astype(np.uint32) << 16).view(np.float32)


def tol_ok(c, gold, esc, rel, escfrac):
    return np.abs(c - gold) <= rel * np.abs(gold) + escfrac * esc + 1e-30


def rng_codes(rng, shape, scale):
    x = (rng.random(shape) * 8.0 - 4.0).astype(np.float32) * np.float32(scale)
    u = x.view(np.uint32).astype(np.uint64)
    return ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)


# ---- reference golden vectors (tests/m4a/test_moe.c:160-226,275-457) -------

@pytest.mark.parametrize("which", ["orc", "ref"])
def test_router_golden(which, request):
    o = request.getfixturevalue(which)
    m = manifest()
    E, K, TK = m["RTR_E"], m["RTR_K"], m["RTR_TK"]
    x = rd("moe_rtr_x.bin", np.uint16)
    wg = rd("moe_rtr_wg.bin", np.uint16).reshape(E, K)
    gi = rd("moe_rtr_idx.bin", np.int64)
    gw = rd("moe_rtr_w.bin", np.float64)
    idx, w = o.route(x, wg, TK)
    assert idx.tolist() == gi.tolist()          # selection EXACT
    assert tol_ok(f32(w).astype(np.float64), gw, 0.02, 0.008, 0.008).all()
    # topn == route prefix (tests/m4a/test_moe.c:215-223)
    assert o.route_topn(x, wg, TK).tolist() == idx.tolist()
    assert o.route_topn(x, wg, TK + 4)[:TK].tolist() == idx.tolist()


def test_router_logits_golden(orc):
    m = manifest()
    E, K, TK = m["RTR_E"], m["RTR_K"], m["RTR_TK"]
    x = rd("moe_rtr_x.bin", np.uint16)
    wg = rd("moe_rtr_wg.bin", np.uint16).reshape(E, K)
    gl = rd("moe_rtr_logits.bin", np.uint16)
    _, _, lg = orc.route_batch(x[None, :], wg, TK, want_logits=True)
    # f64-accumulated golden vs fp32 sequential: codes may differ by one ulp
    d = np.abs(lg[0].astype(np.int32) - gl.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 0.01


@pytest.mark.parametrize("which", ["orc", "ref"])
def test_router_tie_kats(which, request):
    """tests/m4a/test_moe.c:230-263"""
    o = request.getfixturevalue(which)
    E, K, TK = 16, 4, 8
    one, half = 0x3F80, 0x3F00
    x = np.array([one, 0, 0, 0], np.uint16)
    wg = np.zeros((E, K), np.uint16)
    wg[:, 0] = half
    idx, w = o.route(x, wg, TK)
    assert idx.tolist() == list(range(8))
    assert (w == 0x3E00).all()                   # 0.125 exactly
    wg[:, 0] = 0
    wg[:9, 0] = one
    idx, _ = o.route(x, wg, TK)
    assert idx.tolist() == list(range(8))        # row 8 loses the cut tie


@pytest.mark.parametrize("which", ["orc", "ref"])
def test_act_silu_combine_golden(which, request):
    o = request.getfixturevalue(which)
    m = manifest()
    gu = rd("moe_act_gu.bin", np.uint16)
    ga = rd("moe_act_act.bin", np.float64)
    act = o.silu_act(gu)
    assert act.size == m["ACT_I"]
    assert tol_ok(f32(act).astype(np.float64), ga, 0.02, 0.008, 0.008).all()
    g, u = rd("moe_silu_g.bin", np.uint16), rd("moe_silu_u.bin", np.uint16)
    gy = rd("moe_silu_y.bin", np.float64)
    assert tol_ok(f32(o.silu_mul(g, u)).astype(np.float64), gy, 0.02, 0.008,
                  0.008).all()
    k, N = m["COMB_K"], m["COMB_N"]
    y = rd("moe_comb_y.bin", np.uint16).reshape(k, N)
    w = rd("moe_comb_w.bin", np.uint16)
    go, ge = rd("moe_comb_out.bin", np.float64), rd("moe_comb_esc.bin", np.float64)
    out = o.combine(y, w)
    assert tol_ok(f32(out).astype(np.float64), go, ge, 0.008, 0.008).all()


@pytest.mark.parametrize("which", ["orc", "ref"])
def test_specials(which, request):
    """silu(0)=+0; zero weights -> +0 codes; k=1 combine == rnd(w*y)
    (tests/m4a/test_moe.c:370-374,433-446)."""
    o = request.getfixturevalue(which)
    assert o.silu_mul(np.array([0], np.uint16),
                      np.array([0x4040], np.uint16))[0] == 0
    rng = np.random.default_rng(5)
    y = rng_codes(rng, (8, 767), 2.0)
    assert (o.combine(y, np.zeros(8, np.uint16)) == 0).all()
    w = rng_codes(rng, 8, 0.4)
    one = o.combine(y[:1, :4], w[:1])
    exp = [o.bf16_bits(float(f32(w[:1])[0] * f32(y[0, i:i + 1])[0]))
           for i in range(4)]
    assert one.tolist() == exp


# ---- restatement == reference, bit for bit ---------------------------------

SHAPES = [(1, 1), (3, 5), (7, 1), (33, 100), (64, 256), (256, 2048),
          (1024, 2048), (2048, 512), (512, 2048), (1, 2048)]


@pytest.mark.parametrize("O,K", SHAPES)
def test_gemv_bitwise(orc, ref, O, K):
    rng = np.random.default_rng(O * 131 + K)
    w, x = rng_codes(rng, (O, K), 0.5), rng_codes(rng, K, 1.0)
    a = orc.gemv(w, x)
    assert np.array_equal(a, ref.gemv(w, x, hot=False))   # scalar anchor
    assert np.array_equal(a, ref.gemv(w, x, hot=True))    # AVX2 pool path
    assert np.array_equal(orc.matvec_f32(w, x), ref.matvec_f32(w, x))
    assert np.array_equal(orc.matvec_f32(w, x), ref.matvec_f32_hot(w, x))


@pytest.mark.parametrize("M,O,K", [(2, 3, 5), (5, 33, 100), (9, 64, 256),
                                   (37, 128, 512), (64, 256, 128)])
def test_gemm_bitwise_and_m_independence(orc, ref, M, O, K):
    rng = np.random.default_rng(M + O + K)
    w, x = rng_codes(rng, (O, K), 0.5), rng_codes(rng, (M, K), 1.0)
    a = orc.gemm(w, x)
    assert np.array_equal(a, ref.gemm(w, x, hot=True))
    for m in (0, M - 1):                       # GEMM row == GEMV row
        assert np.array_equal(a[m], orc.gemv(w, x[m]))


def test_pointwise_bitwise(orc, ref):
    rng = np.random.default_rng(3)
    gu = rng_codes(rng, 2 * 767, 3.0)
    assert np.array_equal(orc.silu_act(gu), ref.silu_act(gu))
    g, u = rng_codes(rng, 767, 3.0), rng_codes(rng, 767, 3.0)
    assert np.array_equal(orc.silu_mul(g, u), ref.silu_mul(g, u))
    y, w = rng_codes(rng, (8, 767), 2.0), rng_codes(rng, 8, 0.4)
    assert np.array_equal(orc.combine(y, w), ref.combine(y, w))
    x, gw = rng_codes(rng, (5, 2048), 1.0), rng_codes(rng, 2048, 0.1)
    assert np.array_equal(orc.rmsnorm(x, gw), ref.rmsnorm(x, gw))
    assert np.array_equal(orc.resadd(x, x[::-1].copy()),
                          ref.resadd(x, x[::-1].copy()))


@pytest.mark.parametrize("T", [1, 2, 7, 33])
def test_block_bitwise_mini(orc, ref, be, synth, T):
    cfg = synth.MINI_CFG
    W = synth.host_weights(be, cfg, seed=100 + T, sigma=0.08)
    x = synth.host_x(be, T, cfg["hidden"], seed=100 + T)
    a = orc.moe_block(cfg, W, x)
    for batched in (False, True):             # tests/m9c: batched == per-token
        r = ref.moe_block(cfg, W, x, batched=batched)
        for k in a:
            assert np.array_equal(a[k], r[k]), (k, batched)


def test_block_bitwise_medium(orc, ref, be, synth):
    cfg = dict(hidden=512, experts=64, moe_inter=128, shared_inter=64, top_k=8)
    W = synth.host_weights(be, cfg, seed=9, sigma=0.05)
    x = synth.host_x(be, 40, cfg["hidden"], seed=9)
    a, r = orc.moe_block(cfg, W, x), ref.moe_block(cfg, W, x)
    for k in a:
        assert np.array_equal(a[k], r[k]), k


# ---- committed block goldens -------------------------------------------------

def digest(W):
    h = hashlib.sha256()
    for k in sorted(W):
        h.update(W[k].tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("name", ["block_mini_t1", "block_mini_t7",
                                  "block_qwen_t3"])
def test_block_golden(orc, be, synth, name):
    g = np.load(os.path.join(G, name + ".npz"))
    cfg = dict(zip(("hidden", "experts", "moe_inter", "shared_inter", "top_k"),
                   (int(v) for v in g["cfg"])))
    W = synth.host_weights(be, cfg, seed=int(g["seed"]), sigma=float(g["sigma"]))
    assert digest(W) == str(g["digest"]), "synthetic weight stream drifted"
    x = g["x"]
    assert np.array_equal(x, synth.host_x(be, x.shape[0], cfg["hidden"],
                                          seed=int(g["seed"])))
    a = orc.moe_block(cfg, W, x)
    for k in ("idx", "w", "routed", "shared", "out"):
        assert np.array_equal(a[k], g[k]), k


def test_numpy_oracle_golden(orc, be, synth):
    """The reference's independent numpy oracle on the mini configuration:
    selection identical; outputs inside the f64-matmul-vs-fp32 envelope the
    reference's own layer test uses (tests/m4c/README.md:49-57)."""
    g = np.load(os.path.join(G, "npblock_mini_t7.npz"))
    cfg = synth.MINI_CFG
    W = synth.host_weights(be, cfg, seed=11, sigma=0.08)
    x = synth.host_x(be, 7, cfg["hidden"], seed=11)
    a = orc.moe_block(cfg, W, x)
    assert np.array_equal(a["idx"], g["idx"])
    out = f32(a["out"]).astype(np.float64)
    scale = np.abs(g["out"]).max()
    assert np.abs(out - g["out"]).max() <= 0.01 * scale


# ---- dispatch restatement ------------------------------------------------------

@pytest.mark.parametrize("T,TK,E", [(1, 8, 256), (5, 4, 16), (300, 8, 256),
                                    (1000, 8, 256)])
def test_dispatch_is_stable_sort(orc, T, TK, E):
    rng = np.random.default_rng(T)
    idx = np.stack([rng.choice(E, TK, replace=False) for _ in range(T)]
                   ).astype(np.int32)
    counts, offsets, perm = orc.dispatch(idx, E)
    flat = idx.ravel()
    assert np.array_equal(counts, np.bincount(flat, minlength=E))
    assert offsets[0] == 0 and np.array_equal(np.diff(offsets), counts)
    assert np.array_equal(perm, np.argsort(flat, kind="stable"))
    # the literal loop order of c/layer.h:599-606
    exp = [t * TK + j for e in range(E) for t in range(T) for j in range(TK)
           if idx[t, j] == e] if T <= 300 else None
    if exp is not None:
        assert perm.tolist() == exp
