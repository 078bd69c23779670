"""ctypes loaders for the two CPU checkers.  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module; the product (the CUDA library and its Python binding) never does.

  * ``Restatement`` — oracle/liboracle.so, the plain-C restatement of the
    reference's MoE arithmetic (oracle/moe_oracle.c).
  * ``Reference``   — oracle/_ref/libapus_ref.so, the reference engine's own
    code compiled from its sources (oracle/ref_harness.c).  Present whenever
    the tree was built where the reference checkout exists.

Both expose the same method names, mirroring the reference's C entry points
(apus_moe_route, apus_moe_silu_act, apus_bf16_gemv_hot, ...) with numpy
arrays of uint16 BF16 codes.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
u16p = C.POINTER(C.c_uint16)
i32p = C.POINTER(C.c_int32)
f32p = C.POINTER(C.c_float)
sz = C.c_size_t


def build(quiet=True):
    """Compile liboracle.so (and _ref/libapus_ref.so where the reference
    checkout is present)."""
    subprocess.run(["make", "-C", HERE], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _p(a, t):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(t)


def _u16(a):
    return np.ascontiguousarray(a, dtype=np.uint16)


class _Base:
    prefix = ""

    def __init__(self, path):
        self.lib = C.CDLL(path)
        self.path = path

    def _fn(self, name, argtypes, restype=None):
        f = getattr(self.lib, self.prefix + name)
        f.argtypes = argtypes
        f.restype = restype
        return f

    # ---- scalar helpers -------------------------------------------------
    def bf16_bits(self, x):
        f = self._fn("bf16_bits", [C.c_float], C.c_uint16)
        return f(float(x))

    def bf16_f32(self, b):
        f = self._fn("bf16_f32", [C.c_uint16], C.c_float)
        return f(int(b))

    # ---- per-op kernels --------------------------------------------------
    def route(self, x, wg, topk):
        x, wg = _u16(x), _u16(wg)
        E, K = wg.shape
        idx = np.zeros(topk, np.int32)
        w = np.zeros(topk, np.uint16)
        self._fn("moe_route", [u16p, u16p, i32p, u16p, sz, sz, sz])(
            _p(x, u16p), _p(wg, u16p), _p(idx, i32p), _p(w, u16p), E, K, topk)
        return idx, w

    def route_topn(self, x, wg, n):
        x, wg = _u16(x), _u16(wg)
        E, K = wg.shape
        idx = np.zeros(n, np.int32)
        self._fn("moe_route_topn", [u16p, u16p, i32p, sz, sz, sz])(
            _p(x, u16p), _p(wg, u16p), _p(idx, i32p), n, E, K)
        return idx

    def silu_act(self, gu):
        gu = _u16(gu)
        I = gu.size // 2
        act = np.zeros(I, np.uint16)
        self._fn("moe_silu_act", [u16p, u16p, sz])(_p(gu, u16p), _p(act, u16p), I)
        return act

    def silu_mul(self, g, u):
        g, u = _u16(g), _u16(u)
        y = np.zeros(g.size, np.uint16)
        self._fn("moe_silu_mul", [u16p, u16p, u16p, sz])(
            _p(g, u16p), _p(u, u16p), _p(y, u16p), g.size)
        return y

    def combine(self, y, w):
        y, w = _u16(y), _u16(w)
        k, N = y.shape
        out = np.zeros(N, np.uint16)
        self._fn("moe_combine", [u16p, u16p, u16p, sz, sz])(
            _p(y, u16p), _p(w, u16p), _p(out, u16p), k, N)
        return out

    def matvec_f32(self, w, x):
        w, x = _u16(w), _u16(x)
        O, K = w.shape
        y = np.zeros(O, np.float32)
        self._fn("matvec_f32", [u16p, u16p, f32p, sz, sz])(
            _p(w, u16p), _p(x, u16p), _p(y, f32p), O, K)
        return y

    def rmsnorm(self, x, w=None):
        x = _u16(x)
        N = x.shape[-1]
        xs = x.reshape(-1, N)
        y = np.zeros_like(xs)
        wz = _u16(w) if w is not None else np.zeros(N, np.uint16)
        f = self._fn("rmsnorm", [u16p, u16p, u16p, sz])
        for t in range(xs.shape[0]):
            f(_p(xs[t], u16p), _p(wz, u16p), _p(y[t], u16p), N)
        return y.reshape(x.shape)

    def resadd(self, a, b):
        a, b = _u16(a), _u16(b)
        out = np.zeros_like(a)
        self._fn("resadd", [u16p, u16p, u16p, sz])(
            _p(a, u16p), _p(b, u16p), _p(out, u16p), a.size)
        return out


class Restatement(_Base):
    prefix = "orc_"

    def __init__(self):
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        super().__init__(path)

    def threads(self):
        return self._fn("threads", [], C.c_int)()

    def synth_fill_host(self, n, seed, layer, tensor_id, sigma, first=0):
        """The seeded tensor stream of the package (csrc/synth.h), host-only
        build: same signature as Backend.synth_fill_host, so synth.host_x /
        host_weights take this object in place of the CUDA binding."""
        out = np.empty(n, np.uint16)
        self._fn("synth_fill", [u16p, sz, C.c_uint64, C.c_uint32, C.c_uint32,
                                C.c_uint64, C.c_double])(
            _p(out, u16p), n, seed, layer, tensor_id, first, sigma)
        return out

    def gemv(self, w, x):
        w, x = _u16(w), _u16(x)
        O, K = w.shape
        y = np.zeros(O, np.uint16)
        self._fn("bf16_gemv", [u16p, u16p, u16p, sz, sz])(
            _p(w, u16p), _p(x, u16p), _p(y, u16p), O, K)
        return y

    def gemm(self, w, x):
        w, x = _u16(w), _u16(x)
        O, K = w.shape
        M = x.shape[0]
        y = np.zeros((M, O), np.uint16)
        self._fn("bf16_gemm", [u16p, u16p, u16p, sz, sz, sz])(
            _p(w, u16p), _p(x, u16p), _p(y, u16p), M, O, K)
        return y

    def route_batch(self, x, wg, topk, want_logits=False):
        x, wg = _u16(x), _u16(wg)
        E, K = wg.shape
        T = x.shape[0]
        idx = np.zeros((T, topk), np.int32)
        w = np.zeros((T, topk), np.uint16)
        lg = np.zeros((T, E), np.uint16) if want_logits else None
        self._fn("moe_route_batch",
                 [u16p, u16p, i32p, u16p, u16p, sz, sz, sz, sz])(
            _p(x, u16p), _p(wg, u16p), _p(idx, i32p), _p(w, u16p),
            _p(lg, u16p), T, E, K, topk)
        return (idx, w, lg) if want_logits else (idx, w)

    def dispatch(self, idx, E):
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        T, TK = idx.shape
        counts = np.zeros(E, np.int32)
        offsets = np.zeros(E + 1, np.int32)
        perm = np.zeros(T * TK, np.int32)
        self._fn("dispatch", [i32p, sz, sz, sz, i32p, i32p, i32p])(
            _p(idx, i32p), T, TK, E, _p(counts, i32p), _p(offsets, i32p),
            _p(perm, i32p))
        return counts, offsets, perm

    def moe_block(self, cfg, W, ln2):
        """cfg: dict(hidden, experts, moe_inter, shared_inter, top_k);
        W: dict of uint16 arrays; ln2 [T,H].  Returns dict(out, idx, w,
        routed, shared)."""
        ln2 = _u16(ln2)
        T, H = ln2.shape
        TK = cfg["top_k"]
        out = np.zeros((T, H), np.uint16)
        idx = np.zeros((T, TK), np.int32)
        w = np.zeros((T, TK), np.uint16)
        routed = np.zeros((T, H), np.uint16)
        shared = np.zeros((T, H), np.uint16)
        self._fn("moe_block", [sz] * 5 + [u16p] * 9 + [sz, i32p, u16p, u16p,
                                                        u16p])(
            H, cfg["experts"], cfg["moe_inter"], cfg["shared_inter"], TK,
            *[_p(_keep(W, k), u16p) for k in
              ("rtr_w", "exp_gu", "exp_d", "sh_g", "sh_u", "sh_d", "sh_gate")],
            _p(ln2, u16p), _p(out, u16p), T, _p(idx, i32p), _p(w, u16p),
            _p(routed, u16p), _p(shared, u16p))
        return dict(out=out, idx=idx, w=w, routed=routed, shared=shared)


def _keep(W, k):
    a = W[k]
    assert a.dtype == np.uint16 and a.flags["C_CONTIGUOUS"], k
    return a


class Reference(_Base):
    prefix = "ref_"

    @staticmethod
    def available():
        return os.path.exists(os.path.join(HERE, "_ref", "libapus_ref.so"))

    def __init__(self):
        super().__init__(os.path.join(HERE, "_ref", "libapus_ref.so"))

    def threads(self):
        return self._fn("pool_threads", [], C.c_int)()

    def have_avx2(self):
        return bool(self._fn("have_avx2", [], C.c_int)())

    def gemv(self, w, x, hot=True):
        w, x = _u16(w), _u16(x)
        O, K = w.shape
        y = np.zeros(O, np.uint16)
        self._fn("bf16_gemv_hot" if hot else "bf16_gemv_scalar",
                 [u16p, u16p, u16p, sz, sz])(
            _p(w, u16p), _p(x, u16p), _p(y, u16p), O, K)
        return y

    def gemm(self, w, x, hot=True):
        w, x = _u16(w), _u16(x)
        O, K = w.shape
        M = x.shape[0]
        y = np.zeros((M, O), np.uint16)
        self._fn("bf16_gemm_hot" if hot else "bf16_gemm_scalar",
                 [u16p, u16p, u16p, sz, sz, sz])(
            _p(w, u16p), _p(x, u16p), _p(y, u16p), M, O, K)
        return y

    def matvec_f32_hot(self, w, x):
        w, x = _u16(w), _u16(x)
        O, K = w.shape
        y = np.zeros(O, np.float32)
        self._fn("matvec_f32_hot", [u16p, u16p, f32p, sz, sz])(
            _p(w, u16p), _p(x, u16p), _p(y, f32p), O, K)
        return y

    def moe_block(self, cfg, W, ln2, batched=None):
        ln2 = _u16(ln2)
        T, H = ln2.shape
        TK = cfg["top_k"]
        if batched is None:
            batched = T > 1
        out = np.zeros((T, H), np.uint16)
        idx = np.zeros((T, TK), np.int32)
        w = np.zeros((T, TK), np.uint16)
        routed = np.zeros((T, H), np.uint16)
        shared = np.zeros((T, H), np.uint16)
        self._fn("moe_block", [sz] * 5 + [u16p] * 9 + [sz, C.c_int, i32p, u16p,
                                                        u16p, u16p])(
            H, cfg["experts"], cfg["moe_inter"], cfg["shared_inter"], TK,
            *[_p(_keep(W, k), u16p) for k in
              ("rtr_w", "exp_gu", "exp_d", "sh_g", "sh_u", "sh_d", "sh_gate")],
            _p(ln2, u16p), _p(out, u16p), T, 1 if batched else 0,
            _p(idx, i32p), _p(w, u16p), _p(routed, u16p), _p(shared, u16p))
        return dict(out=out, idx=idx, w=w, routed=routed, shared=shared)

    def set_hooks(self, gemv, gemm, matvec):
        """Install three C function pointers (ctypes function objects or
        None) into the reference's own hook table."""
        f = self._fn("set_hooks", [C.c_void_p, C.c_void_p, C.c_void_p])
        cast = lambda fn: C.cast(fn, C.c_void_p) if fn is not None else None
        f(cast(gemv), cast(gemm), cast(matvec))
