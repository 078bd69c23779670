"""ctypes binding of include/backend_cuda.h.

Method names and argument meaning follow the C entry points one for one
(apus_cuda_moe_route -> Backend.moe_route, ...), which in turn mirror the
reference engine's operator surface (c/moe.h, c/layer.h, c/backend_metal.h).
Host-pointer methods take and return numpy arrays of uint16 BF16 codes;
``*_dev`` methods take raw device addresses (ints) and a CUDA stream handle.

The library must exist: importing never builds, and every compute call raises
``BackendError`` when the CUDA library reports failure (there is no CPU path).
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libapus_cuda.so")

u16p = C.POINTER(C.c_uint16)
i32p = C.POINTER(C.c_int32)
f32p = C.POINTER(C.c_float)
sz = C.c_size_t
vp = C.c_void_p


class BackendError(RuntimeError):
    pass


class MoeCfg(C.Structure):
    """ApusCudaMoeCfg"""
    _fields_ = [("hidden", sz), ("experts", sz), ("moe_inter", sz),
                ("shared_inter", sz), ("top_k", sz)]

    @classmethod
    def from_dict(cls, d):
        return cls(d["hidden"], d["experts"], d["moe_inter"],
                   d["shared_inter"], d["top_k"])


class MoeW(C.Structure):
    """ApusCudaMoeW"""
    _fields_ = [(k, vp) for k in ("rtr_w", "exp_gu", "exp_d", "sh_g", "sh_u",
                                  "sh_d", "sh_gate")]


class MoeTrace(C.Structure):
    """ApusCudaMoeTrace"""
    _fields_ = [(k, vp) for k in ("rtr_idx", "rtr_w", "moe_routed",
                                  "moe_shared", "moe_out")]


# every symbol include/backend_cuda.h declares
SYMBOLS = [
    "apus_cuda_enable", "apus_cuda_disable", "apus_cuda_is_enabled",
    "apus_cuda_bytes_resident", "apus_cuda_bytes_uploaded",
    "apus_cuda_launches", "apus_cuda_last_error", "apus_cuda_bf16_gemv",
    "apus_cuda_bf16_gemm", "apus_cuda_bf16_matvec_f32", "apus_cuda_moe_route",
    "apus_cuda_moe_route_topn", "apus_cuda_moe_dispatch",
    "apus_cuda_moe_block", "apus_cuda_block_hooks", "apus_cuda_layer_create",
    "apus_cuda_layer_destroy", "apus_cuda_layer_tensor",
    "apus_cuda_layer_refresh", "apus_cuda_layer_upload",
    "apus_cuda_layer_load_slabs", "apus_cuda_register_layer_slabs",
    "apus_cuda_debug_fast_logits", "apus_cuda_moe_block_dev",
    "apus_cuda_moe_layer_dev", "apus_cuda_moe_stack_dev", "apus_cuda_reserve",
    "apus_cuda_last_block_launches", "apus_cuda_last_block_path",
    "apus_cuda_last_block_status",
    "apus_cuda_stage_timing", "apus_cuda_last_stage_ms",
    "apus_cuda_fused_timeline", "apus_cuda_router_exact_chains",
    "apus_cuda_router_timeline",
    "apus_cuda_ep_route_dev", "apus_cuda_ep_pack_dev", "apus_cuda_experts_dev",
    "apus_cuda_ep_finish_dev",
    "apus_cuda_ep_window_create", "apus_cuda_ep_window_destroy",
    "apus_cuda_ep_window_handle_bytes", "apus_cuda_ep_window_handle",
    "apus_cuda_ep_window_attach", "apus_cuda_ep_window_attach_local",
    "apus_cuda_ep_push_dev", "apus_cuda_ep_wait_dev",
    "apus_cuda_ep_window_experts_dev", "apus_cuda_ep_return_dev",
    "apus_cuda_ep_shared_dev", "apus_cuda_ep_combine_dev",
    "apus_cuda_ep_publish_dev", "apus_cuda_ep_publish_rows_dev",
    "apus_cuda_ep_pull_experts_dev",
    "apus_cuda_route_dev", "apus_cuda_dispatch_dev",
    "apus_cuda_dispatch_dev_static", "apus_cuda_rmsnorm_dev",
    "apus_cuda_resadd_dev", "apus_cuda_bf16_gemv_dev", "apus_synth_fill_host",
    "apus_synth_fill_dev",
]

STAGES = ("router", "dispatch", "gather", "gate_up", "down", "finalize")
TENSOR_IDS = dict(rtr_w=1, exp_gu=2, exp_d=3, sh_g=4, sh_u=5, sh_d=6, sh_gate=7)


def _ptr(a, t=vp):
    if a is None:
        return None
    if isinstance(a, int):
        return C.cast(a, t) if t is not vp else a
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(t) if t is not vp else a.ctypes.data


def _u16(a):
    return np.ascontiguousarray(a, dtype=np.uint16)


class Backend:
    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise BackendError(
                f"{path} is missing: build it first (build.build()); "
                "there is no CPU fallback")
        self.lib = L = C.CDLL(path)
        L.apus_cuda_last_error.restype = C.c_char_p
        L.apus_cuda_enable.argtypes = [C.c_char_p, sz]
        for n in ("bytes_resident", "bytes_uploaded", "launches"):
            getattr(L, "apus_cuda_" + n).restype = C.c_uint64
        L.apus_cuda_bf16_gemv.argtypes = [u16p, u16p, u16p, sz, sz]
        L.apus_cuda_bf16_gemm.argtypes = [u16p, u16p, u16p, sz, sz, sz]
        L.apus_cuda_bf16_matvec_f32.argtypes = [u16p, u16p, f32p, sz, sz]
        L.apus_cuda_moe_route.argtypes = [u16p, u16p, i32p, u16p, u16p, sz, sz,
                                          sz, sz]
        L.apus_cuda_moe_route_topn.argtypes = [u16p, u16p, i32p, sz, sz, sz]
        L.apus_cuda_moe_dispatch.argtypes = [i32p, sz, sz, sz, i32p, i32p, i32p]
        L.apus_cuda_moe_block.argtypes = [C.POINTER(MoeCfg), C.POINTER(MoeW),
                                          u16p, u16p, sz, C.POINTER(MoeTrace)]
        L.apus_cuda_layer_create.argtypes = [C.POINTER(MoeCfg),
                                             C.POINTER(MoeW), sz, sz,
                                             C.POINTER(vp)]
        L.apus_cuda_layer_destroy.argtypes = [vp]
        L.apus_cuda_layer_destroy.restype = None
        L.apus_cuda_layer_tensor.argtypes = [vp, C.c_int, C.POINTER(sz)]
        L.apus_cuda_layer_tensor.restype = vp
        L.apus_cuda_layer_refresh.argtypes = [vp]
        L.apus_cuda_layer_upload.argtypes = [vp, C.c_int, u16p, sz, sz]
        L.apus_cuda_layer_load_slabs.argtypes = [vp, C.c_char_p, C.c_int]
        L.apus_cuda_register_layer_slabs.argtypes = [C.POINTER(MoeCfg), C.POINTER(MoeW),
                                                     C.c_char_p, C.c_int]
        L.apus_cuda_debug_fast_logits.argtypes = [u16p, u16p, sz, sz, sz, f32p,
                                                  f32p, f32p, f32p]
        L.apus_cuda_moe_block_dev.argtypes = [vp, vp, vp, sz,
                                              C.POINTER(MoeTrace), vp]
        L.apus_cuda_moe_layer_dev.argtypes = [vp, vp, vp, vp, sz, C.POINTER(MoeTrace), vp]
        L.apus_cuda_moe_stack_dev.argtypes = [C.POINTER(vp), C.POINTER(vp), sz, vp, sz, vp]
        L.apus_cuda_reserve.argtypes = [C.POINTER(MoeCfg), sz]
        L.apus_cuda_last_stage_ms.argtypes = [C.POINTER(C.c_float), C.c_int]
        L.apus_cuda_route_dev.argtypes = [vp, vp, sz, vp, vp, vp]
        L.apus_cuda_dispatch_dev.argtypes = [vp, sz, sz, sz, vp, vp, vp, vp]
        L.apus_cuda_dispatch_dev_static.argtypes = [vp, sz, sz, sz, vp, vp, vp,
                                                    vp]
        L.apus_cuda_ep_route_dev.argtypes = [vp, vp, sz, vp, vp, vp, vp]
        L.apus_cuda_ep_pack_dev.argtypes = [vp, vp, sz, sz, sz, sz, sz, vp, vp,
                                            vp, vp, vp]
        L.apus_cuda_experts_dev.argtypes = [vp, vp, vp, sz, vp, vp]
        L.apus_cuda_ep_finish_dev.argtypes = [vp, vp, sz, vp, vp, vp, vp, vp,
                                              C.POINTER(MoeTrace), vp]
        L.apus_cuda_ep_window_create.argtypes = [sz, sz, sz, sz, sz, sz,
                                                 C.POINTER(vp)]
        L.apus_cuda_ep_window_destroy.argtypes = [vp]
        L.apus_cuda_ep_window_destroy.restype = None
        L.apus_cuda_ep_window_handle_bytes.argtypes = []
        L.apus_cuda_ep_window_handle_bytes.restype = sz
        L.apus_cuda_ep_window_handle.argtypes = [vp, vp]
        L.apus_cuda_ep_window_attach.argtypes = [vp, sz, vp]
        L.apus_cuda_ep_window_attach_local.argtypes = [vp, sz, vp]
        L.apus_cuda_ep_push_dev.argtypes = [vp, vp, vp, sz, C.c_uint32, vp, vp]
        L.apus_cuda_ep_wait_dev.argtypes = [vp, C.c_int, C.c_uint32, vp]
        L.apus_cuda_ep_window_experts_dev.argtypes = [vp, vp, vp]
        L.apus_cuda_ep_return_dev.argtypes = [vp, C.c_uint32, vp]
        L.apus_cuda_ep_shared_dev.argtypes = [vp, vp, sz, vp, vp]
        L.apus_cuda_ep_publish_dev.argtypes = [vp, vp, vp, sz, C.c_uint32, vp]
        L.apus_cuda_ep_publish_rows_dev.argtypes = [vp, vp, sz, vp]
        L.apus_cuda_ep_pull_experts_dev.argtypes = [vp, vp, C.c_uint32, vp, sz, vp, vp]
        L.apus_cuda_ep_combine_dev.argtypes = [vp, vp, sz, vp, vp, vp, vp, vp, vp]
        L.apus_cuda_rmsnorm_dev.argtypes = [vp, vp, vp, sz, sz, vp]
        L.apus_cuda_resadd_dev.argtypes = [vp, vp, vp, sz, vp]
        L.apus_cuda_bf16_gemv_dev.argtypes = [vp, vp, vp, sz, sz, sz, vp]
        L.apus_synth_fill_host.argtypes = [u16p, sz, C.c_uint64, C.c_uint32,
                                           C.c_uint32, C.c_uint64, C.c_double]
        L.apus_synth_fill_host.restype = None
        L.apus_synth_fill_dev.argtypes = [vp, sz, C.c_uint64, C.c_uint32,
                                          C.c_uint32, C.c_uint64, C.c_double,
                                          vp]

    # ---- errors -----------------------------------------------------------
    def last_error(self):
        return self.lib.apus_cuda_last_error().decode()

    def _check(self, rc, what):
        if rc != 0:
            raise BackendError(f"{what} failed (rc={rc}): {self.last_error()}")

    # ---- lifecycle ----------------------------------------------------------
    def enable(self):
        buf = C.create_string_buffer(512)
        rc = self.lib.apus_cuda_enable(buf, 512)
        if rc != 0:
            raise BackendError("apus_cuda_enable: " + buf.value.decode())

    def disable(self):
        self.lib.apus_cuda_disable()

    def is_enabled(self):
        return bool(self.lib.apus_cuda_is_enabled())

    def bytes_resident(self):
        return int(self.lib.apus_cuda_bytes_resident())

    def bytes_uploaded(self):
        return int(self.lib.apus_cuda_bytes_uploaded())

    def launches(self):
        return int(self.lib.apus_cuda_launches())

    # ---- per-matmul entry points (host arrays) -----------------------------
    def bf16_gemv(self, w, x):
        w, x = _u16(w), _u16(x)
        O, K = w.shape
        y = np.zeros(O, np.uint16)
        rc = self.lib.apus_cuda_bf16_gemv(_ptr(w, u16p), _ptr(x, u16p),
                                          _ptr(y, u16p), O, K)
        self._check(rc, "apus_cuda_bf16_gemv")
        return y

    def bf16_gemm(self, w, x):
        w, x = _u16(w), _u16(x)
        O, K = w.shape
        M = x.shape[0]
        y = np.zeros((M, O), np.uint16)
        rc = self.lib.apus_cuda_bf16_gemm(_ptr(w, u16p), _ptr(x, u16p),
                                          _ptr(y, u16p), M, O, K)
        self._check(rc, "apus_cuda_bf16_gemm")
        return y

    def bf16_matvec_f32(self, w, x):
        w, x = _u16(w), _u16(x)
        O, K = w.shape
        y = np.zeros(O, np.float32)
        rc = self.lib.apus_cuda_bf16_matvec_f32(_ptr(w, u16p), _ptr(x, u16p),
                                                _ptr(y, f32p), O, K)
        self._check(rc, "apus_cuda_bf16_matvec_f32")
        return y

    # ---- router / dispatch (host arrays) -----------------------------------
    def moe_route(self, x, wg, topk, want_logits=False):
        x, wg = _u16(x), _u16(wg)
        if x.ndim == 1:
            x = x[None, :]
        T, K = x.shape
        E = wg.shape[0]
        idx = np.zeros((T, topk), np.int32)
        w = np.zeros((T, topk), np.uint16)
        lg = np.zeros((T, E), np.uint16) if want_logits else None
        rc = self.lib.apus_cuda_moe_route(_ptr(x, u16p), _ptr(wg, u16p),
                                          _ptr(idx, i32p), _ptr(w, u16p),
                                          _ptr(lg, u16p), T, E, K, topk)
        self._check(rc, "apus_cuda_moe_route")
        return (idx, w, lg) if want_logits else (idx, w)

    def moe_route_topn(self, x, wg, n):
        x, wg = _u16(x), _u16(wg)
        E, K = wg.shape
        idx = np.zeros(n, np.int32)
        rc = self.lib.apus_cuda_moe_route_topn(_ptr(x, u16p), _ptr(wg, u16p),
                                               _ptr(idx, i32p), n, E, K)
        self._check(rc, "apus_cuda_moe_route_topn")
        return idx

    def moe_dispatch(self, idx, E):
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        T, TK = idx.shape
        counts = np.zeros(E, np.int32)
        offsets = np.zeros(E + 1, np.int32)
        perm = np.zeros(T * TK, np.int32)
        rc = self.lib.apus_cuda_moe_dispatch(_ptr(idx, i32p), T, TK, E,
                                             _ptr(counts, i32p),
                                             _ptr(offsets, i32p),
                                             _ptr(perm, i32p))
        self._check(rc, "apus_cuda_moe_dispatch")
        return counts, offsets, perm

    # ---- the block, host arrays ---------------------------------------------
    def moe_block(self, cfg, W, ln2, trace=True):
        """cfg: dict; W: dict of uint16 arrays (kept alive by the caller: the
        rtr_w address is the residency key); ln2 [T,H].  Returns dict(out,
        idx, w, routed, shared)."""
        ln2 = _u16(ln2)
        T, H = ln2.shape
        TK = cfg["top_k"]
        c = MoeCfg.from_dict(cfg)
        w = MoeW(*[W[k].ctypes.data if W.get(k) is not None else None for k in
                   ("rtr_w", "exp_gu", "exp_d", "sh_g", "sh_u", "sh_d",
                    "sh_gate")])
        out = np.zeros((T, H), np.uint16)
        res = dict(out=out)
        tr = None
        if trace:
            res["idx"] = np.zeros((T, TK), np.int32)
            res["w"] = np.zeros((T, TK), np.uint16)
            res["routed"] = np.zeros((T, H), np.uint16)
            res["shared"] = np.zeros((T, H), np.uint16)
            tr = MoeTrace(res["idx"].ctypes.data, res["w"].ctypes.data,
                          res["routed"].ctypes.data, res["shared"].ctypes.data,
                          None)
        rc = self.lib.apus_cuda_moe_block(C.byref(c), C.byref(w),
                                          _ptr(ln2, u16p), _ptr(out, u16p), T,
                                          C.byref(tr) if tr else None)
        self._check(rc, "apus_cuda_moe_block")
        return res

    # ---- device-resident form -------------------------------------------------
    def layer_create(self, cfg, W=None, expert_begin=0, expert_end=None):
        c = MoeCfg.from_dict(cfg)
        if expert_end is None:
            expert_end = cfg["experts"]
        w = None
        if W is not None:
            w = MoeW(*[W[k].ctypes.data for k in
                       ("rtr_w", "exp_gu", "exp_d", "sh_g", "sh_u", "sh_d",
                        "sh_gate")])
        h = vp()
        rc = self.lib.apus_cuda_layer_create(C.byref(c),
                                             C.byref(w) if w else None,
                                             expert_begin, expert_end,
                                             C.byref(h))
        self._check(rc, "apus_cuda_layer_create")
        return h.value

    def layer_destroy(self, layer):
        self.lib.apus_cuda_layer_destroy(layer)

    def layer_tensor(self, layer, name):
        n = sz()
        p = self.lib.apus_cuda_layer_tensor(layer, TENSOR_IDS[name],
                                            C.byref(n))
        return p, int(n.value)

    def layer_refresh(self, layer):
        self._check(self.lib.apus_cuda_layer_refresh(layer),
                    "apus_cuda_layer_refresh")

    def layer_upload(self, layer, name, src, first=0):
        """Host uint16 array -> elements [first, first + src.size) of a
        resident tensor of the layer."""
        src = _u16(src)
        self._check(self.lib.apus_cuda_layer_upload(
            layer, TENSOR_IDS[name], _ptr(src, u16p), first, src.size),
            "apus_cuda_layer_upload")

    def layer_load_slabs(self, layer, container_dir, layer_index):
        """Routed experts of the layer's resident range from the engine's
        weight container (apus.index.json + shards)."""
        self._check(self.lib.apus_cuda_layer_load_slabs(
            layer, str(container_dir).encode(), layer_index),
            "apus_cuda_layer_load_slabs")

    def register_layer_slabs(self, cfg, W, container_dir, layer_index):
        """Tiered mode: W holds router / shared expert / gate host arrays (the
        rtr_w address is the key), the routed experts come from the container."""
        c = MoeCfg.from_dict(cfg)
        w = MoeW(W["rtr_w"].ctypes.data, None, None, W["sh_g"].ctypes.data,
                 W["sh_u"].ctypes.data, W["sh_d"].ctypes.data, W["sh_gate"].ctypes.data)
        self._check(self.lib.apus_cuda_register_layer_slabs(
            C.byref(c), C.byref(w), str(container_dir).encode(), layer_index),
            "apus_cuda_register_layer_slabs")

    def debug_fast_logits(self, x, wg):
        """(fast [T,E] f32, xnorm [T], wnorm [E+1], cbound) of the many-token
        router's tensor-core scoring."""
        x, wg = _u16(x), _u16(wg)
        T, K = x.shape
        E = wg.shape[0]
        fast = np.zeros((T, E), np.float32)
        xn = np.zeros(T, np.float32)
        wn = np.zeros(E + 1, np.float32)
        cb = np.zeros(1, np.float32)
        self._check(self.lib.apus_cuda_debug_fast_logits(
            _ptr(x, u16p), _ptr(wg, u16p), T, E, K, _ptr(fast, f32p),
            _ptr(xn, f32p), _ptr(wn, f32p), _ptr(cb, f32p)),
            "apus_cuda_debug_fast_logits")
        return fast, xn, wn, float(cb[0])

    def reserve(self, cfg, T):
        c = MoeCfg.from_dict(cfg)
        self._check(self.lib.apus_cuda_reserve(C.byref(c), T),
                    "apus_cuda_reserve")

    def moe_block_dev(self, layer, d_ln2, d_out, T, stream=None, d_trace=None):
        tr = None
        if d_trace:
            tr = MoeTrace(d_trace.get("idx"), d_trace.get("w"),
                          d_trace.get("routed"), d_trace.get("shared"),
                          d_trace.get("out"))
        rc = self.lib.apus_cuda_moe_block_dev(layer, d_ln2, d_out, T,
                                              C.byref(tr) if tr else None,
                                              stream)
        self._check(rc, "apus_cuda_moe_block_dev")

    def moe_layer_dev(self, layer, d_res, d_ln_w, d_res_out, T, stream=None, d_trace=None):
        """d_res_out = rnd(d_res + moe_block(rmsnorm(d_res, 1 + d_ln_w)))"""
        tr = None
        if d_trace:
            tr = MoeTrace(d_trace.get("idx"), d_trace.get("w"), d_trace.get("routed"),
                          d_trace.get("shared"), d_trace.get("out"))
        self._check(self.lib.apus_cuda_moe_layer_dev(
            layer, d_res, d_ln_w, d_res_out, T, C.byref(tr) if tr else None, stream),
            "apus_cuda_moe_layer_dev")

    def moe_stack_dev(self, layers, d_res, T, d_ln_w=None, stream=None):
        """In place over a stack of layers: d_res <- d_res + moe_l(rmsnorm(d_res))."""
        n = len(layers)
        arr = (vp * n)(*layers)
        gains = (vp * n)(*d_ln_w) if d_ln_w is not None else None
        self._check(self.lib.apus_cuda_moe_stack_dev(arr, gains, n, d_res, T, stream),
                    "apus_cuda_moe_stack_dev")

    def stage_timing(self, enable):
        self._check(self.lib.apus_cuda_stage_timing(1 if enable else 0),
                    "apus_cuda_stage_timing")

    def last_stage_ms(self):
        ms = (C.c_float * len(STAGES))()
        n = self.lib.apus_cuda_last_stage_ms(ms, len(STAGES))
        if n < 0:
            raise BackendError("apus_cuda_last_stage_ms failed")
        return dict(zip(STAGES, (float(v) for v in ms)))

    def fused_timeline(self):
        """[n_cta, 8] global-timer stamps of the one-kernel path's phases."""
        buf = (C.c_ulonglong * (256 * 8))()
        n = self.lib.apus_cuda_fused_timeline(buf, 256 * 8)
        if n < 0:
            return None
        return np.array(buf[:n], dtype=np.uint64).reshape(-1, 8)

    def router_timeline(self):
        """(ns from start: candidates known, chains done, end; chains walked)
        of the certified router's first CTA in its last launch."""
        out = (C.c_uint * 5)()
        if self.lib.apus_cuda_router_timeline(out) != 0:
            return None
        t0 = out[0]
        return [(int(out[i]) - int(t0)) & 0xffffffff for i in (1, 2, 3)] + [int(out[4])]

    def router_exact_chains(self):
        self.lib.apus_cuda_router_exact_chains.restype = C.c_long
        return int(self.lib.apus_cuda_router_exact_chains())

    def last_block_launches(self):
        return int(self.lib.apus_cuda_last_block_launches())

    def last_block_path(self):
        """0 one-kernel, 1 grouped GEMV, 2 one-SM GEMM, 3 two-SM GEMM."""
        return int(self.lib.apus_cuda_last_block_path())

    def last_block_status(self):
        return int(self.lib.apus_cuda_last_block_status())

    def route_dev(self, layer, d_x, T, d_idx, d_w, stream=None):
        self._check(self.lib.apus_cuda_route_dev(layer, d_x, T, d_idx, d_w,
                                                 stream),
                    "apus_cuda_route_dev")

    def dispatch_dev(self, d_idx, T, topk, E, d_counts, d_offsets, d_perm,
                     stream=None):
        self._check(self.lib.apus_cuda_dispatch_dev(d_idx, T, topk, E,
                                                    d_counts, d_offsets,
                                                    d_perm, stream),
                    "apus_cuda_dispatch_dev")

    def dispatch_dev_static(self, d_idx, T, topk, E, d_counts, d_offsets,
                            d_perm, stream=None):
        """apus_cuda_dispatch_dev_static: the dispatch with its scratch in
        the library's built-in array; never allocates."""
        self._check(self.lib.apus_cuda_dispatch_dev_static(
            d_idx, T, topk, E, d_counts, d_offsets, d_perm, stream),
            "apus_cuda_dispatch_dev_static")

    # ---- expert parallelism ---------------------------------------------------
    def ep_route_dev(self, layer, d_x, T, d_idx, d_w, d_sgl, stream=None):
        self._check(self.lib.apus_cuda_ep_route_dev(layer, d_x, T, d_idx, d_w,
                                                    d_sgl, stream),
                    "apus_cuda_ep_route_dev")

    def ep_pack_dev(self, d_x, d_idx, T, topk, H, E, n_ranks, d_send_x,
                    d_send_e, d_send_counts, d_pos, stream=None):
        self._check(self.lib.apus_cuda_ep_pack_dev(
            d_x, d_idx, T, topk, H, E, n_ranks, d_send_x, d_send_e,
            d_send_counts, d_pos, stream), "apus_cuda_ep_pack_dev")

    def experts_dev(self, layer, d_x, d_e, R, d_y, stream=None):
        self._check(self.lib.apus_cuda_experts_dev(layer, d_x, d_e, R, d_y,
                                                   stream),
                    "apus_cuda_experts_dev")

    def ep_finish_dev(self, layer, d_x, T, d_y_sorted, d_pos, d_w, d_sgl,
                      d_out, stream=None, d_trace=None):
        tr = None
        if d_trace:
            tr = MoeTrace(None, None, d_trace.get("routed"),
                          d_trace.get("shared"), d_trace.get("out"))
        self._check(self.lib.apus_cuda_ep_finish_dev(
            layer, d_x, T, d_y_sorted, d_pos, d_w, d_sgl, d_out,
            C.byref(tr) if tr else None, stream), "apus_cuda_ep_finish_dev")

    # ---- expert parallelism through peer memory ---------------------------
    def ep_window_create(self, max_tokens, topk, H, E, n_ranks, rank):
        w = vp()
        self._check(self.lib.apus_cuda_ep_window_create(
            max_tokens, topk, H, E, n_ranks, rank, C.byref(w)),
            "apus_cuda_ep_window_create")
        return w

    def ep_window_destroy(self, w):
        self.lib.apus_cuda_ep_window_destroy(w)

    def ep_window_handle(self, w):
        buf = C.create_string_buffer(self.lib.apus_cuda_ep_window_handle_bytes())
        self._check(self.lib.apus_cuda_ep_window_handle(w, buf),
                    "apus_cuda_ep_window_handle")
        return buf.raw

    def ep_window_attach(self, w, peer, handle):
        self._check(self.lib.apus_cuda_ep_window_attach(
            w, peer, C.c_char_p(handle)), "apus_cuda_ep_window_attach")

    def ep_window_attach_local(self, w, peer, other):
        self._check(self.lib.apus_cuda_ep_window_attach_local(w, peer, other),
                    "apus_cuda_ep_window_attach_local")

    def ep_push_dev(self, w, d_x, d_idx, T, epoch, d_pos, stream=None):
        self._check(self.lib.apus_cuda_ep_push_dev(w, d_x, d_idx, T, epoch,
                                                   d_pos, stream),
                    "apus_cuda_ep_push_dev")

    def ep_wait_dev(self, w, which, epoch, stream=None):
        self._check(self.lib.apus_cuda_ep_wait_dev(w, which, epoch, stream),
                    "apus_cuda_ep_wait_dev")

    def ep_window_experts_dev(self, w, layer, stream=None):
        self._check(self.lib.apus_cuda_ep_window_experts_dev(w, layer, stream),
                    "apus_cuda_ep_window_experts_dev")

    def ep_return_dev(self, w, epoch, stream=None):
        self._check(self.lib.apus_cuda_ep_return_dev(w, epoch, stream),
                    "apus_cuda_ep_return_dev")

    def ep_publish_dev(self, w, d_x, d_idx, T, epoch, stream=None):
        self._check(self.lib.apus_cuda_ep_publish_dev(w, d_x, d_idx, T, epoch,
                                                      stream),
                    "apus_cuda_ep_publish_dev")

    def ep_publish_rows_dev(self, w, d_x, T, stream=None):
        self._check(self.lib.apus_cuda_ep_publish_rows_dev(w, d_x, T, stream),
                    "apus_cuda_ep_publish_rows_dev")

    def ep_pull_experts_dev(self, w, layer, epoch, d_x=None, T=0, d_sy=None,
                            stream=None):
        self._check(self.lib.apus_cuda_ep_pull_experts_dev(w, layer, epoch, d_x,
                                                           T, d_sy, stream),
                    "apus_cuda_ep_pull_experts_dev")

    def ep_shared_dev(self, layer, d_x, T, d_sy, stream=None):
        self._check(self.lib.apus_cuda_ep_shared_dev(layer, d_x, T, d_sy,
                                                     stream),
                    "apus_cuda_ep_shared_dev")

    def ep_combine_dev(self, w, layer, T, d_pos, d_w, d_sy, d_sgl, d_out,
                       stream=None):
        self._check(self.lib.apus_cuda_ep_combine_dev(
            w, layer, T, d_pos, d_w, d_sy, d_sgl, d_out, stream),
            "apus_cuda_ep_combine_dev")

    def rmsnorm_dev(self, d_x, d_w, d_y, T, N, stream=None):
        self._check(self.lib.apus_cuda_rmsnorm_dev(d_x, d_w, d_y, T, N,
                                                   stream),
                    "apus_cuda_rmsnorm_dev")

    def resadd_dev(self, d_a, d_b, d_out, n, stream=None):
        self._check(self.lib.apus_cuda_resadd_dev(d_a, d_b, d_out, n, stream),
                    "apus_cuda_resadd_dev")

    def bf16_gemv_dev(self, d_w, d_x, d_y, M, O, K, stream=None):
        self._check(self.lib.apus_cuda_bf16_gemv_dev(d_w, d_x, d_y, M, O, K, stream),
                    "apus_cuda_bf16_gemv_dev")

    # ---- synthetic tensors -------------------------------------------------------
    def synth_fill_host(self, n, seed, layer, tensor_id, sigma, first=0):
        out = np.empty(n, np.uint16)
        self.lib.apus_synth_fill_host(_ptr(out, u16p), n, seed, layer,
                                      tensor_id, first, sigma)
        return out

    def synth_fill_dev(self, d_dst, n, seed, layer, tensor_id, sigma, first=0,
                       stream=None):
        self._check(self.lib.apus_synth_fill_dev(d_dst, n, seed, layer,
                                                 tensor_id, first, sigma,
                                                 stream),
                    "apus_synth_fill_dev")
