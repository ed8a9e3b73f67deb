"""Expert-parallel MoE layer: one process per GPU, experts sharded across ranks.

Follows the partition of the reference's (dormant) expert-parallel branch
(moe_gen/models/deepseek/deepseekv3/modeling_deepseek_v3.py:574-592,636-672,692-700): rank r
owns experts [r*E/N, (r+1)*E/N); every rank gates its own tokens.  The exchange is not three
all-to-all collectives with host-side split sizes: every rank maps the other ranks' receive and
output buffers (CUDA IPC over NVLink) and the permute scatter / combine gather kernels write
and read them directly.  torch.distributed (NCCL) carries only the count all-gather and two
one-element all-reduces that act as barriers.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from . import lib as L
from .layer import MoELayer, _ptr

PEER_SHIFT = 24
TILE_M = 128


def ep_layout_reference(counts_all: np.ndarray, rank: int, e_local: int, cap_rows: int):
    """Host restatement of the device layout step (ep_layout_kernel), used by tests.

    counts_all[s, e] = picks of global expert e among rank s's tokens.  Returns
    (send_base[E], recv_counts[e_local], recv_pad[e_local+1], overflow[N]): send_base[e] =
    owner << 24 | first row, in the owner's buffers, of this rank's rows of expert e; inside an
    expert's 128-padded segment source rank 0 comes first."""
    n, E = counts_all.shape
    tot = counts_all.sum(axis=0)
    before = counts_all[:rank].sum(axis=0)
    send_base = np.empty(E, dtype=np.int64)
    over = np.zeros(n, dtype=bool)
    recv_counts = np.zeros(e_local, dtype=np.int64)
    recv_pad = np.zeros(e_local + 1, dtype=np.int64)
    for d in range(n):
        seg = (tot[d * e_local:(d + 1) * e_local] + TILE_M - 1) // TILE_M * TILE_M
        pad = np.concatenate([[0], np.cumsum(seg)])
        over[d] = pad[-1] > cap_rows
        for j in range(e_local):
            e = d * e_local + j
            send_base[e] = -(1 << 30) if over[d] else ((d << PEER_SHIFT) | (pad[j] + before[e]))
        if d == rank and not over[d]:
            recv_counts[:] = tot[d * e_local:(d + 1) * e_local]
            recv_pad[:] = pad
    return send_base, recv_counts, recv_pad, over


def ep_copy_plan_reference(counts_all: np.ndarray, rank: int, e_local: int, cap_rows: int):
    """Host restatement of the copy-engine return as owner `rank` issues it (api.cu: copy_part), used by tests:
    a list of (destination rank, first row in its return buffer, first row in this owner's out_rows, rows),
    one entry per (local expert, source rank) that has rows.  The destination row is the first row of the
    expert in the source rank's own expert-sorted, unpadded order."""
    n, E = counts_all.shape
    tot = counts_all.sum(axis=0)
    seg = (tot[rank * e_local:(rank + 1) * e_local] + TILE_M - 1) // TILE_M * TILE_M
    if seg.sum() > cap_rows:
        return []
    own = np.cumsum(counts_all, axis=1) - counts_all          # [s, e]: first row of expert e in rank s's order
    plan, pad = [], 0
    for j in range(e_local):
        e = rank * e_local + j
        row = pad
        for s in range(n):
            if counts_all[s, e] > 0:
                plan.append((s, int(own[s, e]), int(row), int(counts_all[s, e])))
            row += int(counts_all[s, e])
        pad += int(seg[j])
    return plan


def ep_mirror_delta_reference(counts_all: np.ndarray, rank: int, e_local: int):
    """Host restatement of ep_mirror_delta_kernel: per global expert, (first row of the expert in this rank's own
    order) - (first row of this rank's rows of the expert in the owner's buffer)."""
    n, E = counts_all.shape
    own = np.cumsum(counts_all[rank]) - counts_all[rank]
    base, *_ = ep_layout_reference(counts_all, rank, e_local, 1 << 40)
    return own - (base & ((1 << PEER_SHIFT) - 1))


class _MicroBatch:
    """Buffers, stream and process group of one token micro-batch of the expert-parallel forward."""
    pass


class EPMoELayer:
    """Wraps a MoELayer created with ep_rank/ep_size and runs the expert-parallel forward.

    n_micro > 1 splits the local tokens into micro-batches that are pipelined: while the experts
    of one micro-batch run on the tensor cores, the next one's rows travel over NVLink and the
    previous one's results are gathered back, each micro-batch on its own stream with its own
    shared buffers and its own NCCL group (so their barriers do not queue behind each other)."""

    PHASES = ["route_dispatch", "expert_ffn", "combine"]

    def __init__(self, layer: MoELayer, group: Optional[dist.ProcessGroup] = None, capacity_factor: float = 2.0,
                 n_micro: int = 1, dedup: bool = True, min_headroom: int = 4096, push_return: Optional[bool] = None,
                 return_parts: int = 4, copy_return: bool = False):
        self.layer = layer
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        assert layer.desc.ep_size == self.world and layer.desc.ep_rank == self.rank
        # a rank's receive buffers hold max(capacity_factor * mean rows, mean rows + min_headroom) rows
        # (plus padding; min_headroom = 0 leaves the factor alone); more rows than that raise
        # MG_DEV_CAPACITY, reported by check_status()
        self.capacity_factor = capacity_factor
        self.min_headroom = min_headroom
        self.n_micro = max(1, n_micro)
        # one row per (token, destination rank) over NVLink; the owner copies the rows of a token's
        # further experts on that rank (pays off when top_k exceeds the number of ranks a token reaches)
        self.dedup = dedup
        # the owners push their experts' outputs into the token owners' return buffers part by part while the
        # next part's down projection runs, and the combine is local; False = the combine gathers the rows
        # from the owners' buffers after the experts have finished
        # None = off: measured at 2 GPUs the pushes slow the experts beside them by about their own duration
        # (24.5 against 21.4 ms) while the combine gets 2.2 ms shorter: 30.2 against 29.4 ms per step
        self.push_return = False if push_return is None else push_return
        self.return_parts = return_parts
        # the owners' copy engines carry every (expert, source rank) segment of the results into the source
        # rank's return buffer, in that rank's own expert-sorted order, part by part beside the down projection;
        # the combine is local.  Needs the gathered counts on the host: one small synchronising read per
        # forward, taken after the dispatch has been enqueued.  Wins over push_return when both are set.
        self.copy_return = copy_return
        self.lib = layer.lib
        self.dev = layer.device
        self._mbs: List[_MicroBatch] = []
        self._tokens = -1
        self.timing = False                # record CUDA events around the phases of forward()
        self._events: List[list] = []
        self._side = torch.cuda.Stream(device=self.dev)   # shared expert runs beside the dispatch
        ranks = list(range(self.world)) if group is None else dist.get_process_group_ranks(group)
        self._groups = [group] + [dist.new_group(ranks) for _ in range(self.n_micro - 1)]
        self._streams = [torch.cuda.Stream(device=self.dev) for _ in range(self.n_micro)]
        self.deq = None
        self._batch_tokens = 0             # local tokens of the batch forward_host is feeding in parts
        # device status word mirrored into pinned host memory behind every forward (no synchronisation):
        # a receive buffer that was too small drops picks, and the caller must hear about it
        self._status_host = torch.zeros(2, dtype=torch.int32).pin_memory()
        self._status_event: Optional[torch.cuda.Event] = None

    # ------------------------------------------------------------------ buffers
    def _setup(self, T: int):
        """(Re)allocates the shared buffers for T local tokens and exchanges their handles."""
        self._release()
        lay = self.layer
        E, El, k = lay.E, lay.e_local, lay.k
        n = self.n_micro if T >= 2 * self.n_micro else 1
        bounds = [T * i // n for i in range(n + 1)]
        handles = []
        with torch.cuda.device(self.dev):
            for i in range(n):
                mb = _MicroBatch()
                mb.t0, mb.t1 = bounds[i], bounds[i + 1]
                Tm = mb.t1 - mb.t0
                avg_rows = Tm * k                              # rows a rank receives when load is even
                floor = avg_rows + self.min_headroom if self.min_headroom > 0 else 0
                cap = int(min(Tm * self.world * k, max(avg_rows * self.capacity_factor, floor)))
                cap = (cap + TILE_M - 1) // TILE_M * TILE_M + El * TILE_M
                assert cap < (1 << PEER_SHIFT)
                mb.cap = cap
                mb.own = []
                # recv_x, out_rows, duplicate table, return table, return buffer
                for nbytes in (cap * lay.H * 2, cap * lay.H * 2, cap * 4, cap * 4, max(Tm * k, 1) * lay.H * 2):
                    p = C.c_void_p()
                    L.check(self.lib.mg_ep_alloc(nbytes, C.byref(p)))
                    hd = (C.c_ubyte * 64)()
                    L.check(self.lib.mg_ep_export(p, hd))
                    mb.own.append(p.value)
                    handles.append(bytes(hd))
                i32 = dict(dtype=torch.int32, device=self.dev)
                mb.counts = torch.empty(E, **i32)
                mb.counts_all = torch.empty(self.world, E, **i32)
                mb.recv_counts = torch.empty(El, **i32)
                mb.recv_pad = torch.empty(El + 1, **i32)
                mb.dst = torch.empty(Tm, k, **i32)
                mb.idx = torch.empty(Tm, k, **i32)
                mb.w = torch.empty(Tm, k, dtype=torch.float32, device=self.dev)
                mb.logits = torch.empty(Tm, E, dtype=torch.float32, device=self.dev)
                nf = C.c_size_t()
                L.check(self.lib.mg_route_fix_bytes(Tm, C.byref(nf)))
                mb.fix = torch.zeros(nf.value // 4, **i32)
                nb = C.c_size_t()
                L.check(self.lib.mg_plan_ws_bytes(lay._h, Tm, C.byref(nb)))
                mb.plan_ws = torch.empty(nb.value, dtype=torch.uint8, device=self.dev)
                mb.h_buf = torch.empty(cap, lay.I, dtype=torch.bfloat16, device=self.dev)
                mb.flag = torch.zeros(1, dtype=torch.int32, device=self.dev)
                mb.delta = torch.zeros(E, **i32)
                mb.counts_host = torch.zeros(self.world, E, dtype=torch.int32).pin_memory()
                mb.counts_event = torch.cuda.Event()
                mb.stream = self._streams[i]
                mb.group = self._groups[i]
                mb.imported = []
                self._mbs.append(mb)
            gathered: List[Optional[list]] = [None] * self.world
            dist.all_gather_object(gathered, handles, group=self.group)
            for i, mb in enumerate(self._mbs):
                tables = [(C.c_void_p * self.world)() for _ in range(5)]
                for r in range(self.world):
                    if r == self.rank:
                        for which, table in enumerate(tables):
                            table[r] = mb.own[which]
                        continue
                    for which, table in enumerate(tables):
                        p = C.c_void_p()
                        buf = (C.c_ubyte * 64).from_buffer_copy(gathered[r][5 * i + which])
                        L.check(self.lib.mg_ep_import(buf, C.byref(p)))
                        table[r] = p.value
                        mb.imported.append(p.value)
                mb.peer_recv, mb.peer_out, mb.peer_dup, mb.peer_back, mb.peer_ret = tables
            self.hs = torch.empty(T, max(lay.Is, 1), dtype=torch.bfloat16, device=self.dev)
            self.shared_out = torch.empty(T, lay.H, dtype=torch.bfloat16, device=self.dev) if lay.Is else None
            nd = C.c_size_t()
            L.check(self.lib.mg_dequant_ws_bytes(lay._h, C.byref(nd)))
            # FP8: scratch for the library's FP8 mode (the L2-resident ring from 1024 rows per expert on, or
            # the bf16 copy of pre-dequantise mode); below that the GEMMs convert in shared memory
            mode = lay.options.get(L.OPT_FP8_MODE, 0)
            Tb = max(T, self._batch_tokens)    # parts of one batch share the de-quantised copy
            use_deq = nd.value > 0 and (mode in (L.FP8_PREDEQUANT, L.FP8_RING) or
                                        (mode == L.FP8_AUTO and Tb * self.world * k >= 1024 * E))
            self.deq = torch.empty(nd.value, dtype=torch.uint8, device=self.dev) if use_deq else None
            if nd.value > 0 and L.OPT_FP8_M256 not in lay.options:
                # the library picks the tile height of its convert-in-the-GEMM kernels from the rows of
                # the buffer it is given; here that is the receive capacity, so decide from the batch
                L.check(self.lib.mg_set_option(lay._h, L.OPT_FP8_M256, 2 if T * self.world * k >= 120 * E else 0))
            # rows the dispatch, duplicate-fill and combine kernels may address in a rank's buffers (looked at by
            # a -DMG_BOUNDS_CHECK build of the library only)
            L.check(self.lib.mg_set_option(lay._h, L.OPT_ROWS_BOUND, max(mb.cap for mb in self._mbs)))
        self._tokens = T
        dist.barrier(group=self.group)

    def _release(self):
        if not self._mbs:
            return
        torch.cuda.synchronize(self.dev)
        if dist.is_initialized():
            dist.barrier(group=self.group)       # nobody may still be reading our buffers
        for mb in self._mbs:
            for p in mb.imported:
                self.lib.mg_ep_unimport(C.c_void_p(p))
        if dist.is_initialized():
            dist.barrier(group=self.group)       # every mapping of our buffers is closed
        for mb in self._mbs:
            for p in mb.own:
                self.lib.mg_ep_free(C.c_void_p(p))
        self._mbs = []
        self._tokens = -1

    def close(self):
        self._release()

    def reconfigure(self, capacity_factor: Optional[float] = None):
        """Changes the receive-buffer capacity (in multiples of the mean rows per rank); the shared
        buffers are re-allocated by the next forward.  Collective: every rank must call it."""
        if capacity_factor is not None:
            self.capacity_factor = capacity_factor
        self._release()

    def check_status(self, wait: bool = False):
        """Raises if a forward whose status has reached the host reported a device-side problem.
        wait=False looks only at forwards that have already finished (no synchronisation); forward()
        calls it on entry, forward_host() with wait=True before it returns.  MG_DEV_CAPACITY means a
        rank's receive buffer was too small for the rows routed to its experts: the picks sent to that
        rank were dropped from dispatch and combine, so that forward's output lacks their contributions."""
        ev = self._status_event
        if ev is None:
            return
        if wait:
            ev.synchronize()
        elif not ev.query():
            return
        self._status_event = None
        code, detail = int(self._status_host[0]), int(self._status_host[1])
        if code == L.DEV_OK:
            return
        self.layer.device_status()                      # fetch and clear on the device
        if code == L.DEV_CAPACITY:
            raise RuntimeError(
                f"expert-parallel receive buffer of rank {detail} overflowed (capacity_factor="
                f"{self.capacity_factor}): the picks routed to that rank were dropped and the output of that "
                "forward is incomplete; raise capacity_factor (reconfigure) and run the batch again")
        raise RuntimeError(f"device status {code} (detail {detail}) reported by an expert-parallel forward")

    @staticmethod
    def _barrier(mb):
        # a stream-ordered collective: kernels launched after it on this rank start only after
        # every rank's earlier kernels on the micro-batch's stream have finished
        dist.all_reduce(mb.flag, group=mb.group)

    def _mark(self, evs, stream):
        if evs is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record(stream)
            evs.append(e)

    def phase_times(self) -> dict:
        """Mean milliseconds of the first micro-batch's phases over the forwards run with timing on
        (call after synchronising).  With pipelining the phases of different micro-batches overlap."""
        out = {p: 0.0 for p in self.PHASES}
        for evs in self._events:
            for i, p in enumerate(self.PHASES):
                out[p] += evs[i].elapsed_time(evs[i + 1]) / len(self._events)
        return out

    # ------------------------------------------------------------------ forward
    def forward_host(self, x_host: torch.Tensor, y_host: Optional[torch.Tensor] = None,
                     n_chunks: int = 2) -> torch.Tensor:
        """This rank's tokens from (pinned) host memory and the result back to it: the local tokens
        go through forward() in n_chunks equal parts, copy-in, compute and copy-out on three streams.
        Every rank must call it with the same token count and n_chunks (each part is a collective
        forward).  FP8 layers de-quantise once for all parts."""
        T = x_host.shape[0]
        if y_host is None:
            y_host = torch.empty_like(x_host, pin_memory=x_host.is_pinned())
        n = n_chunks if n_chunks > 1 and T % n_chunks == 0 and T >= 2 * n_chunks else 1
        cs = T // n
        H = self.layer.H
        with torch.cuda.device(self.dev):
            if getattr(self, "_hb", None) is None or self._hb[0].shape[0] != cs:
                self._hb = [torch.empty(cs, H, dtype=torch.bfloat16, device=self.dev) for _ in range(4)]
                self._hs = [torch.cuda.Stream(device=self.dev), torch.cuda.Stream(device=self.dev)]
            xin, yout = self._hb[:2], self._hb[2:]
            s_in, s_out = self._hs
            comp = torch.cuda.current_stream()
            ev_in = [torch.cuda.Event() for _ in range(2)]
            ev_done = [torch.cuda.Event() for _ in range(2)]
            ev_out = [torch.cuda.Event() for _ in range(2)]
            s_in.wait_stream(comp)
            s_out.wait_stream(comp)
            self._batch_tokens = T
            for c in range(n):
                b, t0 = c & 1, c * cs
                if c >= 2:
                    s_in.wait_event(ev_done[b])
                with torch.cuda.stream(s_in):
                    xin[b].copy_(x_host[t0:t0 + cs], non_blocking=True)
                    ev_in[b].record(s_in)
                comp.wait_event(ev_in[b])
                if c >= 2:
                    comp.wait_event(ev_out[b])
                self.forward(xin[b], out=yout[b], _first=(c == 0), _last=(c == n - 1))
                ev_done[b].record(comp)
                s_out.wait_event(ev_done[b])
                with torch.cuda.stream(s_out):
                    y_host[t0:t0 + cs].copy_(yout[b], non_blocking=True)
                    ev_out[b].record(s_out)
            self._batch_tokens = 0
            s_out.synchronize()
        self.check_status(wait=True)
        return y_host

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, _first: bool = True,
                _last: bool = True) -> torch.Tensor:
        """_first / _last: set by forward_host for the parts of one batch; the FP8 weights are
        de-quantised in the first part and the copy is released after the last."""
        lay, lib = self.layer, self.lib
        self.check_status()
        x2 = x.reshape(-1, lay.H)
        T = x2.shape[0]
        if T != self._tokens:
            self._setup(T)
        y = torch.empty_like(x2) if out is None else out
        h = lay._h
        cur = torch.cuda.current_stream()
        evs = [] if self.timing else None
        H2 = lay.H * 2
        with torch.cuda.device(self.dev):
            for mb in self._mbs:
                mb.stream.wait_stream(cur)
            s0 = self._mbs[0].stream
            if self.deq is not None and _first:
                # weights do not depend on the routing: de-quantise once per forward, starting now
                L.check(lib.mg_set_option(h, L.OPT_KEEP_DEQUANT, 2))
                L.check(lib.mg_dequant_start(h, lay.packed.data_ptr(), self.deq.data_ptr(), s0.cuda_stream))
            self._mark(evs, s0)
            # ---- routing and dispatch of every micro-batch, each on its own stream; the dispatches
            # follow one another so that the first one has the whole NVLink bandwidth and its experts
            # can start while the next micro-batch is still travelling
            sent = None
            for i, mb in enumerate(self._mbs):
                st = mb.stream.cuda_stream
                Tm = mb.t1 - mb.t0
                xp = x2.data_ptr() + mb.t0 * H2
                with torch.cuda.stream(mb.stream):
                    # tables other ranks write during the dispatch: reset before this rank joins the count
                    # exchange, i.e. before any rank can dispatch
                    if self.dedup:
                        L.check(lib.mg_ep_clear_duplicates(h, mb.own[2], mb.cap, st))
                    if self.push_return and not self.copy_return:
                        L.check(lib.mg_ep_clear_duplicates(h, mb.own[3], mb.cap, st))
                    L.check(lib.mg_gate_route_topk(h, xp, lay.gate_w.data_ptr(), _ptr(lay.bias), Tm,
                                                   mb.logits.data_ptr(), mb.idx.data_ptr(), mb.w.data_ptr(),
                                                   mb.fix.data_ptr(), st))
                    L.check(lib.mg_ep_count(h, mb.idx.data_ptr(), Tm, mb.counts.data_ptr(), mb.plan_ws.data_ptr(), st))
                    dist.all_gather_into_tensor(mb.counts_all, mb.counts, group=mb.group)
                    if self.copy_return:
                        mb.counts_host.copy_(mb.counts_all, non_blocking=True)
                        mb.counts_event.record(mb.stream)
                        L.check(lib.mg_ep_mirror_delta(h, mb.counts_all.data_ptr(), mb.delta.data_ptr(), st))
                    L.check(lib.mg_ep_place(h, mb.idx.data_ptr(), Tm, mb.counts_all.data_ptr(), mb.cap,
                                            mb.plan_ws.data_ptr(), mb.recv_counts.data_ptr(), mb.recv_pad.data_ptr(),
                                            mb.dst.data_ptr(), st))
                    if i == 0 and lay.Is:
                        # the shared expert needs only local data: a side stream, ordered after the first
                        # routing kernels, runs its GEMMs while the dispatch is bound by NVLink
                        self._side.wait_stream(mb.stream)
                        L.check(lib.mg_shared_ffn(h, x2.data_ptr(), T, lay.packed.data_ptr(), self.hs.data_ptr(),
                                                  self.shared_out.data_ptr(), self._side.cuda_stream))
                    if sent is not None:
                        mb.stream.wait_event(sent)
                    if self.push_return and not self.copy_return:
                        L.check(lib.mg_ep_dispatch_back(h, xp, mb.dst.data_ptr(), Tm, mb.peer_recv,
                                                        mb.peer_dup if self.dedup else None, mb.peer_back, st))
                    elif self.dedup:
                        L.check(lib.mg_ep_dispatch_dedup(h, xp, mb.dst.data_ptr(), Tm, mb.peer_recv, mb.peer_dup, st))
                    else:
                        L.check(lib.mg_ep_dispatch(h, xp, mb.dst.data_ptr(), Tm, mb.peer_recv, st))
                    sent = torch.cuda.Event()
                    sent.record(mb.stream)
                    self._barrier(mb)                # all rows have landed in the owners' recv_x
                    if self.dedup:
                        L.check(lib.mg_ep_fill_duplicates(h, mb.own[0], mb.own[2], mb.cap, st))
            self._mark(evs, s0)
            # ---- experts, one micro-batch after the other on the tensor cores
            prev = None
            for mb in self._mbs:
                with torch.cuda.stream(mb.stream):
                    if prev is not None:
                        mb.stream.wait_event(prev)   # also orders the reuse of the de-quantised weights
                    if self.copy_return:
                        mb.counts_event.synchronize()         # long done: the dispatch and a barrier were enqueued since
                        L.check(lib.mg_ep_expert_ffn_copy_return(h, mb.own[0], mb.recv_pad.data_ptr(),
                                                                 mb.recv_counts.data_ptr(), mb.cap, lay.packed.data_ptr(),
                                                                 mb.h_buf.data_ptr(), mb.own[1], _ptr(self.deq),
                                                                 mb.counts_host.data_ptr(), mb.peer_ret,
                                                                 self.return_parts, mb.stream.cuda_stream))
                    elif self.push_return:
                        L.check(lib.mg_ep_expert_ffn_return(h, mb.own[0], mb.recv_pad.data_ptr(),
                                                            mb.recv_counts.data_ptr(), mb.cap, lay.packed.data_ptr(),
                                                            mb.h_buf.data_ptr(), mb.own[1], _ptr(self.deq), mb.own[3],
                                                            mb.peer_ret, self.return_parts, mb.stream.cuda_stream))
                    else:
                        L.check(lib.mg_expert_ffn(h, mb.own[0], mb.recv_pad.data_ptr(), mb.recv_counts.data_ptr(),
                                                  mb.cap, lay.packed.data_ptr(), mb.h_buf.data_ptr(), mb.own[1],
                                                  _ptr(self.deq), mb.stream.cuda_stream))
                    prev = torch.cuda.Event()
                    prev.record(mb.stream)
                    self._barrier(mb)                # all owners' out_rows of this micro-batch are complete
            self._mark(evs, s0)
            # ---- return + combine
            for mb in self._mbs:
                with torch.cuda.stream(mb.stream):
                    if lay.Is:
                        mb.stream.wait_stream(self._side)
                    sh = self.shared_out.data_ptr() + mb.t0 * H2 if lay.Is else None
                    if self.copy_return:
                        L.check(lib.mg_ep_combine_mirror(h, mb.own[4], mb.dst.data_ptr(), mb.delta.data_ptr(),
                                                         mb.idx.data_ptr(), mb.w.data_ptr(), sh, mb.t1 - mb.t0,
                                                         y.data_ptr() + mb.t0 * H2, mb.stream.cuda_stream))
                    elif self.push_return:
                        L.check(lib.mg_ep_combine_slots(h, mb.own[4], mb.own[1], mb.dst.data_ptr(), mb.idx.data_ptr(),
                                                        mb.w.data_ptr(), sh, mb.t1 - mb.t0, y.data_ptr() + mb.t0 * H2,
                                                        mb.stream.cuda_stream))
                    else:
                        L.check(lib.mg_ep_combine(h, mb.peer_out, mb.dst.data_ptr(), mb.idx.data_ptr(), mb.w.data_ptr(),
                                                  sh, mb.t1 - mb.t0, y.data_ptr() + mb.t0 * H2, mb.stream.cuda_stream))
            self._mark(evs, s0)
            if self.deq is not None and _last:
                L.check(lib.mg_set_option(h, L.OPT_KEEP_DEQUANT, 0))
            for mb in self._mbs:
                cur.wait_stream(mb.stream)
            # the status word follows the result to the host; the next call (or check_status) reads it
            L.check(lib.mg_device_status_async(h, self._status_host.data_ptr(), cur.cuda_stream))
            self._status_event = torch.cuda.Event()
            self._status_event.record(cur)
        if evs is not None:
            self._events.append(evs)
        return y.view(x.shape)

    __call__ = forward
