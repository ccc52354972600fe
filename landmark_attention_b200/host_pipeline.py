"""Forward + backward of fused landmark attention for tensors that live in (pinned) host memory.

Attention is independent per (batch, head), so the heads are cut into chunks and three CUDA streams overlap the
host-to-device copy of chunk i+1, the kernels of chunk i and the device-to-host copy of chunk i-1.  PCIe is full
duplex, so a step costs about max(bytes in, bytes out) / link bandwidth instead of their sum plus the kernel time.
"""
import math

import torch

from . import _lib as L


class HostAttentionPipeline:
    """Reusable buffers and streams for `run` (shapes are fixed at construction).

    q/k/v/dO and the results o/dq/dk/dv are [B, H, L, D] tensors in pinned host memory; heads are processed in
    `chunks` groups of H // chunks heads."""

    def __init__(self, B, H, Lq, Lk, D, dtype=torch.bfloat16, block_size=64, chunks=4, device="cuda", sm_scale=None):
        assert H % chunks == 0
        self.B, self.H, self.Lq, self.Lk, self.D = B, H, Lq, Lk, D
        self.block, self.chunks, self.hc = block_size, chunks, H // chunks
        self.scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)
        self.dev = torch.device(device)
        self.dtype = dtype
        n_buf = 4                                  # device buffer sets, used in rotation across chunks and steps
        mk = lambda L_: torch.empty((B, self.hc, L_, D), dtype=dtype, device=self.dev)
        self.bufs = [dict(q=mk(Lq), k=mk(Lk), v=mk(Lk), do=mk(Lq), o=mk(Lq), dq=mk(Lq), dk=mk(Lk), dv=mk(Lk),
                          l=torch.empty((B * self.hc, Lq), dtype=torch.float32, device=self.dev),
                          m=torch.empty((B * self.hc, Lq), dtype=torch.float32, device=self.dev))
                     for _ in range(n_buf)]
        code = L._DTYPES[dtype]
        need = L.lib().lmk_attn_bwd_workspace(B, self.hc, Lq, Lk, D, block_size, code, L.PATH_AUTO)
        self.ws = [torch.empty(max(int(need), 256), dtype=torch.uint8, device=self.dev) for _ in range(n_buf)]
        self.code = code
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))

    def run(self, q, k, v, do, o, dq, dk, dv, use_graph=False, wait=True):
        """All eight arguments are pinned host tensors [B, H, L, D]; returns after enqueueing (call
        torch.cuda.synchronize() before reading the outputs).

        wait=True makes the current stream wait for the step's last device-to-host copy, so that work enqueued on it
        afterwards sees the outputs.  wait=False leaves the step on the pipeline's own streams and returns the event of
        its last copy: consecutive steps then overlap (the host-to-device copies of step i+1 run while step i's results
        are still leaving the device; the device buffers are handed over through events), which is how a loop over
        many problems should call it; wait on the returned event, or synchronise the device, before reading.

        With use_graph=True the step is captured into a CUDA graph after one eager run (keyed by the host buffers'
        addresses) and replayed; on PCIe-bound shapes this measures the same as the eager path, which is the default."""
        if not use_graph:
            return self._enqueue(q, k, v, do, o, dq, dk, dv, wait)
        key = tuple(t.data_ptr() for t in (q, k, v, do, o, dq, dk, dv))
        if getattr(self, "_graph_key", None) != key:
            self._enqueue(q, k, v, do, o, dq, dk, dv)          # eager once: validates arguments, warms everything up
            torch.cuda.synchronize(self.dev)
            graph = torch.cuda.CUDAGraph()
            cap = torch.cuda.Stream(self.dev)
            cap.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(cap):
                with torch.cuda.graph(graph, stream=cap):
                    self._enqueue(q, k, v, do, o, dq, dk, dv)
            torch.cuda.current_stream(self.dev).wait_stream(cap)
            self._graph, self._graph_key = graph, key
            self._keep = (q, k, v, do, o, dq, dk, dv)          # the graph holds raw host pointers
        self._graph.replay()
        return None

    def _enqueue(self, q, k, v, do, o, dq, dk, dv, wait=True):
        lib = L.lib()
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        nb = len(self.bufs)
        capturing = torch.cuda.is_current_stream_capturing()
        if capturing or not hasattr(self, "_free"):
            free, first = [None] * nb, 0           # per device buffer set: its last results have left the device
        else:
            free, first = self._free, self._next
        copied = [None] * self.chunks
        done = [None] * self.chunks
        drained = [None] * self.chunks
        for c in range(self.chunks):
            bi = (first + c) % nb
            buf, ws = self.bufs[bi], self.ws[bi]
            hs = slice(c * self.hc, (c + 1) * self.hc)
            with torch.cuda.stream(self.s_in):
                if free[bi] is not None:           # the buffer's previous results must have left the device
                    self.s_in.wait_event(free[bi])
                for name, src in (("q", q), ("k", k), ("v", v), ("do", do)):
                    buf[name].copy_(src[:, hs], non_blocking=True)
                copied[c] = torch.cuda.Event()
                copied[c].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(copied[c])
                st = L.c_void_p(self.s_run.cuda_stream)
                s3q, s3k = L.strides3(buf["q"]), L.strides3(buf["k"])
                L.check(lib.lmk_attn_fwd(L.ptr(buf["q"]), L.ptr(buf["k"]), L.ptr(buf["v"]), L.ptr(buf["o"]),
                                         L.ptr(buf["l"]), L.ptr(buf["m"]), self.B, self.hc, self.Lq, self.Lk, self.D,
                                         s3q, s3k, s3k, self.block, self.scale, self.code, L.PATH_AUTO, st),
                        "lmk_attn_fwd")
                L.check(lib.lmk_attn_bwd(L.ptr(buf["q"]), L.ptr(buf["k"]), L.ptr(buf["v"]), L.ptr(buf["o"]),
                                         L.ptr(buf["do"]), L.ptr(buf["l"]), L.ptr(buf["m"]), L.ptr(buf["dq"]),
                                         L.ptr(buf["dk"]), L.ptr(buf["dv"]), L.ptr(ws), ws.numel(), self.B, self.hc,
                                         self.Lq, self.Lk, self.D, s3q, s3k, s3k, self.block, self.scale, self.code,
                                         L.PATH_AUTO, st), "lmk_attn_bwd")
                done[c] = torch.cuda.Event()
                done[c].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done[c])
                for name, dst in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
                    dst[:, hs].copy_(buf[name], non_blocking=True)
                drained[c] = torch.cuda.Event()
                drained[c].record(self.s_out)
                free[bi] = drained[c]
        if not capturing:
            self._free, self._next = free, (first + self.chunks) % nb
        if wait or capturing:
            cur.wait_stream(self.s_out)
        return drained[-1]
