"""Expert-parallel MoE block: one process per GPU, experts [r*E/N, (r+1)*E/N)
resident on rank r, tokens data-parallel, two all-to-alls per block.

The reference engine is a single process; what is mirrored here is only the
math of its batched MoE body (c/layer.h:570-651).  The compute steps are the
C entry points apus_cuda_ep_route_dev / _ep_pack_dev / _experts_dev /
_ep_finish_dev; this module adds the exchange with torch.distributed
(all_to_all_single over NCCL on GPUs, over gloo in the CPU tests).

`ops` is the object that provides those four steps on torch tensors; the
product implementation is CudaOps below.  (Tests drive the same exchange logic
over gloo with a CPU stand-in for `ops`.)
"""
import numpy as np
import torch
import torch.distributed as dist


def split_sizes(counts):
    """all_to_all_single split lists from a per-destination count vector."""
    return [int(c) for c in counts]


class EPBlock:
    def __init__(self, ops, cfg, rank, world, group=None):
        assert cfg["experts"] % world == 0
        self.ops, self.cfg, self.rank, self.world = ops, cfg, rank, world
        self.group = group
        self.last_sent_rows = 0
        self.last_recv_rows = 0

    def forward(self, x):
        """x: [T_local, H] int16 tensor of BF16 codes on the ops' device.
        Returns [T_local, H]."""
        cfg, N = self.cfg, self.world
        T, H = x.shape
        TK, E = cfg["top_k"], cfg["experts"]
        idx, w, sgl = self.ops.route(x)
        send_x, send_e, send_counts, pos = self.ops.pack(x, idx, N)
        # counts exchange (tiny), then rows + expert ids
        sc = send_counts.to(torch.int64)
        rc = torch.empty_like(sc)
        dist.all_to_all_single(rc, sc, group=self.group)
        in_splits = split_sizes(sc.cpu().numpy())
        out_splits = split_sizes(rc.cpu().numpy())
        R = sum(out_splits)
        recv_x = x.new_empty((R, H))
        recv_e = send_e.new_empty((R,))
        # rows travel as bytes: 16-bit integer tensors are not a collective
        # datatype in NCCL or gloo
        dist.all_to_all_single(recv_x.view(torch.uint8), send_x.view(torch.uint8),
                               out_splits, in_splits, group=self.group)
        dist.all_to_all_single(recv_e, send_e, out_splits, in_splits,
                               group=self.group)
        recv_y = self.ops.experts(recv_x, recv_e)
        back_y = x.new_empty((T * TK, H))
        dist.all_to_all_single(back_y.view(torch.uint8),
                               recv_y.view(torch.uint8), in_splits, out_splits,
                               group=self.group)
        self.last_sent_rows = T * TK - in_splits[self.rank]
        self.last_recv_rows = R - out_splits[self.rank]
        return self.ops.finish(x, back_y, pos, w, sgl)


class CudaOps:
    """The four compute steps on CUDA tensors through the C-ABI."""

    def __init__(self, be, layer, cfg):
        self.be, self.layer, self.cfg = be, layer, cfg

    def _s(self):
        return torch.cuda.current_stream().cuda_stream

    def route(self, x):
        T = x.shape[0]
        TK = self.cfg["top_k"]
        idx = torch.empty((T, TK), dtype=torch.int32, device=x.device)
        w = torch.empty((T, TK), dtype=torch.int16, device=x.device)
        sgl = torch.empty((T,), dtype=torch.int16, device=x.device)
        self.be.ep_route_dev(self.layer, x.data_ptr(), T, idx.data_ptr(),
                             w.data_ptr(), sgl.data_ptr(), stream=self._s())
        return idx, w, sgl

    def pack(self, x, idx, n_ranks):
        T, H = x.shape
        TK, E = self.cfg["top_k"], self.cfg["experts"]
        A = T * TK
        send_x = torch.empty((A, H), dtype=torch.int16, device=x.device)
        send_e = torch.empty((A,), dtype=torch.int32, device=x.device)
        counts = torch.empty((n_ranks,), dtype=torch.int32, device=x.device)
        pos = torch.empty((A,), dtype=torch.int32, device=x.device)
        self.be.ep_pack_dev(x.data_ptr(), idx.data_ptr(), T, TK, H, E, n_ranks,
                            send_x.data_ptr(), send_e.data_ptr(),
                            counts.data_ptr(), pos.data_ptr(), stream=self._s())
        return send_x, send_e, counts, pos

    def experts(self, rx, re):
        R, H = rx.shape
        y = torch.empty((R, H), dtype=torch.int16, device=rx.device)
        if R:
            self.be.experts_dev(self.layer, rx.data_ptr(), re.data_ptr(), R,
                                y.data_ptr(), stream=self._s())
        return y

    def finish(self, x, y_sorted, pos, w, sgl):
        T, H = x.shape
        out = torch.empty_like(x)
        self.be.ep_finish_dev(self.layer, x.data_ptr(), T, y_sorted.data_ptr(),
                              pos.data_ptr(), w.data_ptr(), sgl.data_ptr(),
                              out.data_ptr(), stream=self._s())
        return out


_SIDE_STREAMS = {}


class PeerWindowBlock:
    """The same block step with the two exchanges done by kernels that load from
    and store into the peers' memory: no collective on the data path and no host
    synchronisation inside a step.  torch.distributed is used once, to hand
    round the windows' IPC handles.

    mode "pull" (default): a rank publishes its rows in its own window; the
    expert ranks gather what they need from there and the down GEMM's epilogue
    stores the outputs straight into the source's window
    (apus_cuda_ep_publish_dev / _pull_experts_dev).
    mode "push": exchange kernels of their own before and after the experts
    (apus_cuda_ep_push_dev / _return_dev)."""

    def __init__(self, be, layer, cfg, rank, world, max_tokens, group=None,
                 window=None, device_epoch=False, mode="pull", overlap=True):
        import torch.distributed as dist
        assert cfg["experts"] % world == 0
        assert mode in ("pull", "push")
        self.mode = mode
        # pull: the rows are stored into the peers' windows on a second stream
        # while the router runs (they need nothing from it)
        self.overlap = overlap and mode == "pull"
        self._side = None
        self.be, self.layer, self.cfg = be, layer, cfg
        self.rank, self.world, self.max_tokens = rank, world, max_tokens
        self.epoch = 0
        # step number kept on the device: the step can be captured in a CUDA graph
        self.device_epoch = device_epoch
        self.owns = window is None
        self.win = window
        if window is not None:
            return
        # every rank goes through the same collective calls whatever fails on
        # it, so that a rank without peer access cannot leave the others waiting
        err, mine = None, None
        try:
            self.win = be.ep_window_create(max_tokens, cfg["top_k"], cfg["hidden"],
                                           cfg["experts"], world, rank)
            mine = be.ep_window_handle(self.win)
        except Exception as e:
            err = e
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, mine, group=group)
            if err is None and all(h is not None for h in handles):
                try:
                    for r in range(world):
                        if r != rank:
                            be.ep_window_attach(self.win, r, handles[r])
                except Exception as e:
                    err = e
            oks = [None] * world
            dist.all_gather_object(oks, err is None, group=group)
            if err is None and not all(oks):
                err = RuntimeError("a peer could not map the windows")
        if err is not None:
            self.close()
            raise RuntimeError(f"peer windows: {err}")

    def close(self):
        if self.owns and self.win:
            self.be.ep_window_destroy(self.win)
        self.win = None

    def _s(self):
        return torch.cuda.current_stream().cuda_stream

    # the step in three parts, so that a test can run several ranks in one
    # process: all `begin`s before any `middle`, all `middle`s before any `end`
    def begin(self, x, mark=None):
        """mark (optional): called with a stage name after each stage's launch,
        so that a benchmark can bracket the stages with events."""
        mark = mark or (lambda name: None)
        T, H = x.shape
        TK = self.cfg["top_k"]
        assert T <= self.max_tokens
        if not self.device_epoch:
            self.epoch += 1
        st = dict(x=x)
        st["idx"] = torch.empty((T, TK), dtype=torch.int32, device=x.device)
        st["w"] = torch.empty((T, TK), dtype=torch.int16, device=x.device)
        st["sgl"] = torch.empty((T,), dtype=torch.int16, device=x.device)
        st["pos"] = torch.empty((T * TK,), dtype=torch.int32, device=x.device) \
            if self.mode == "push" else None
        st["sy"] = torch.empty((T, H), dtype=torch.int16, device=x.device)
        be, s = self.be, self._s()
        if self.overlap:
            if self._side is None:
                # one second stream per device, shared by every block (a stack of
                # layers forks and joins the same stream forty times per step)
                dev = x.device.index or 0
                if dev not in _SIDE_STREAMS:
                    _SIDE_STREAMS[dev] = torch.cuda.Stream(device=x.device)
                self._side = _SIDE_STREAMS[dev]
            main = torch.cuda.current_stream()
            self._side.wait_stream(main)          # after the previous step's combine
            be.ep_publish_rows_dev(self.win, x.data_ptr(), T,
                                   stream=self._side.cuda_stream)
        be.ep_route_dev(self.layer, x.data_ptr(), T, st["idx"].data_ptr(),
                        st["w"].data_ptr(), st["sgl"].data_ptr(), stream=s)
        mark("route")
        if self.mode == "push":
            be.ep_push_dev(self.win, x.data_ptr(), st["idx"].data_ptr(), T,
                           self.epoch, st["pos"].data_ptr(), stream=s)
        elif self.overlap:
            main.wait_stream(self._side)          # the rows are in the windows
            be.ep_publish_dev(self.win, None, st["idx"].data_ptr(), T,
                              self.epoch, stream=s)
        else:
            be.ep_publish_dev(self.win, x.data_ptr(), st["idx"].data_ptr(), T,
                              self.epoch, stream=s)
        mark("push")
        if self.mode == "push":
            be.ep_shared_dev(self.layer, x.data_ptr(), T, st["sy"].data_ptr(),
                             stream=s)
        # pull: the shared expert rides in the routed experts' launches
        mark("shared")
        self._st = st
        return st

    def middle(self, mark=None):
        mark = mark or (lambda name: None)
        be, s = self.be, self._s()
        be.ep_wait_dev(self.win, 0, self.epoch, stream=s)
        mark("wait_rows")
        if self.mode == "push":
            be.ep_window_experts_dev(self.win, self.layer, stream=s)
            mark("experts")
            be.ep_return_dev(self.win, self.epoch, stream=s)
        else:
            st = self._st
            be.ep_pull_experts_dev(self.win, self.layer, self.epoch,
                                   st["x"].data_ptr(), st["x"].shape[0],
                                   st["sy"].data_ptr(), stream=s)
            mark("experts")
        mark("return")

    def end(self, st, mark=None):
        mark = mark or (lambda name: None)
        be, s = self.be, self._s()
        x = st["x"]
        out = torch.empty_like(x)
        be.ep_wait_dev(self.win, 1, self.epoch, stream=s)
        mark("wait_returns")
        be.ep_combine_dev(self.win, self.layer, x.shape[0],
                          st["pos"].data_ptr() if st["pos"] is not None else None,
                          st["w"].data_ptr(), st["sy"].data_ptr(),
                          st["sgl"].data_ptr(), out.data_ptr(), stream=s)
        mark("combine")
        return out

    def forward(self, x, mark=None):
        st = self.begin(x, mark)
        self.middle(mark)
        return self.end(st, mark)
