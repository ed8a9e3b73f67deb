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


class EPMoELayer:
    """Wraps a MoELayer created with ep_rank/ep_size and runs the expert-parallel forward."""

    def __init__(self, layer: MoELayer, group: Optional[dist.ProcessGroup] = None, capacity_factor: float = 2.0):
        self.layer = layer
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        assert layer.desc.ep_size == self.world and layer.desc.ep_rank == self.rank
        self.capacity_factor = capacity_factor
        self.lib = layer.lib
        self.dev = layer.device
        self._cap_rows = 0
        self._own: List[int] = []          # [recv_x, out_rows] device addresses owned by this rank
        self._peer_recv = None
        self._peer_out = None
        self._imported: List[int] = []
        self._tokens = -1
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.timing = False                # record CUDA events around the phases of forward()
        self._events: List[list] = []
        self._side = torch.cuda.Stream(device=self.dev)   # shared expert runs beside the dispatch

    # ------------------------------------------------------------------ buffers
    def _setup(self, T: int):
        """(Re)allocates the shared buffers for T local tokens and exchanges their handles."""
        self._release()
        lay = self.layer
        avg_rows = T * lay.k                               # rows a rank receives when load is even
        cap = int(min(T * self.world * lay.k, max(avg_rows * self.capacity_factor, avg_rows + 4096)))
        cap = (cap + TILE_M - 1) // TILE_M * TILE_M + lay.e_local * TILE_M
        assert cap < (1 << PEER_SHIFT)
        self._cap_rows = cap
        nbytes = cap * lay.H * 2
        handles = []
        with torch.cuda.device(self.dev):
            for _ in range(2):
                p = C.c_void_p()
                L.check(self.lib.mg_ep_alloc(nbytes, C.byref(p)))
                hd = (C.c_ubyte * 64)()
                L.check(self.lib.mg_ep_export(p, hd))
                self._own.append(p.value)
                handles.append(bytes(hd))
            gathered: List[Optional[list]] = [None] * self.world
            dist.all_gather_object(gathered, handles, group=self.group)
            recv = (C.c_void_p * self.world)()
            out = (C.c_void_p * self.world)()
            for r in range(self.world):
                if r == self.rank:
                    recv[r], out[r] = self._own[0], self._own[1]
                    continue
                for which, table in ((0, recv), (1, out)):
                    p = C.c_void_p()
                    buf = (C.c_ubyte * 64).from_buffer_copy(gathered[r][which])
                    L.check(self.lib.mg_ep_import(buf, C.byref(p)))
                    table[r] = p.value
                    self._imported.append(p.value)
            self._peer_recv, self._peer_out = recv, out
            E, El, k = lay.E, lay.e_local, lay.k
            i32 = dict(dtype=torch.int32, device=self.dev)
            self.counts = torch.empty(E, **i32)
            self.counts_all = torch.empty(self.world, E, **i32)
            self.recv_counts = torch.empty(El, **i32)
            self.recv_pad = torch.empty(El + 1, **i32)
            self.dst = torch.empty(T, k, **i32)
            self.idx = torch.empty(T, k, **i32)
            self.w = torch.empty(T, k, dtype=torch.float32, device=self.dev)
            self.logits = torch.empty(T, E, dtype=torch.float32, device=self.dev)
            nb = C.c_size_t()
            L.check(self.lib.mg_plan_ws_bytes(lay._h, T, C.byref(nb)))
            self.plan_ws = torch.empty(nb.value, dtype=torch.uint8, device=self.dev)
            self.h_buf = torch.empty(cap, lay.I, dtype=torch.bfloat16, device=self.dev)
            self.hs = torch.empty(T, max(lay.Is, 1), dtype=torch.bfloat16, device=self.dev)
            self.shared_out = torch.empty(T, lay.H, dtype=torch.bfloat16, device=self.dev) if lay.Is else None
            nd = C.c_size_t()
            L.check(self.lib.mg_dequant_ws_bytes(lay._h, C.byref(nd)))
            # FP8: pre-dequantise when an expert sees many rows (same rule as the single-GPU path)
            use_deq = nd.value > 0 and T * self.world * k > 256 * E
            self.deq = torch.empty(nd.value, dtype=torch.uint8, device=self.dev) if use_deq else None
        self._tokens = T
        dist.barrier(group=self.group)

    def _release(self):
        for p in self._imported:
            self.lib.mg_ep_unimport(C.c_void_p(p))
        self._imported = []
        if self._own:
            torch.cuda.synchronize(self.dev)
            if dist.is_initialized():
                dist.barrier(group=self.group)       # nobody may still be reading our buffers
            for p in self._own:
                self.lib.mg_ep_free(C.c_void_p(p))
        self._own = []

    def close(self):
        self._release()

    def _barrier(self):
        # a stream-ordered collective: kernels launched after it on this rank start only after
        # every rank's earlier kernels have finished
        dist.all_reduce(self._flag, group=self.group)

    PHASES = ["gate_route", "count_gather_place", "dispatch", "shared_ffn", "barrier_1", "expert_ffn", "barrier_2",
              "combine"]

    def _mark(self, evs):
        if evs is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            evs.append(e)

    def phase_times(self) -> dict:
        """Mean milliseconds per phase over the forwards run with timing on (call after synchronising)."""
        out = {p: 0.0 for p in self.PHASES}
        for evs in self._events:
            for i, p in enumerate(self.PHASES):
                out[p] += evs[i].elapsed_time(evs[i + 1]) / len(self._events)
        return out

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        lay, lib = self.layer, self.lib
        x2 = x.reshape(-1, lay.H)
        T = x2.shape[0]
        if T != self._tokens:
            self._setup(T)
        y = torch.empty_like(x2) if out is None else out
        st = torch.cuda.current_stream().cuda_stream
        h = lay._h
        evs = [] if self.timing else None
        with torch.cuda.device(self.dev):
            self._mark(evs)
            L.check(lib.mg_gate_logits(h, x2.data_ptr(), lay.gate_w.data_ptr(), T, self.logits.data_ptr(), st))
            L.check(lib.mg_route_topk(h, self.logits.data_ptr(), _ptr(lay.bias), T, self.idx.data_ptr(),
                                      self.w.data_ptr(), st))
            self._mark(evs)
            L.check(lib.mg_ep_count(h, self.idx.data_ptr(), T, self.counts.data_ptr(), self.plan_ws.data_ptr(), st))
            dist.all_gather_into_tensor(self.counts_all, self.counts, group=self.group)
            L.check(lib.mg_ep_place(h, self.idx.data_ptr(), T, self.counts_all.data_ptr(), self._cap_rows,
                                    self.plan_ws.data_ptr(), self.recv_counts.data_ptr(), self.recv_pad.data_ptr(),
                                    self.dst.data_ptr(), st))
            self._mark(evs)
            if lay.Is:
                # the shared expert needs only local data: it goes to a side stream (ordered after the
                # routing kernels, before the dispatch is enqueued) so that its GEMMs run while the
                # dispatch below is bound by NVLink
                self._side.wait_stream(torch.cuda.current_stream())
                L.check(lib.mg_shared_ffn(h, x2.data_ptr(), T, lay.packed.data_ptr(), self.hs.data_ptr(),
                                          self.shared_out.data_ptr(), self._side.cuda_stream))
            L.check(lib.mg_ep_dispatch(h, x2.data_ptr(), self.dst.data_ptr(), T, self._peer_recv, st))
            self._mark(evs)
            self._mark(evs)
            self._barrier()                      # all rows have landed in the owners' recv_x
            self._mark(evs)
            L.check(lib.mg_expert_ffn(h, self._own[0], self.recv_pad.data_ptr(), self.recv_counts.data_ptr(),
                                      self._cap_rows, lay.packed.data_ptr(), self.h_buf.data_ptr(), self._own[1],
                                      _ptr(self.deq), st))
            self._mark(evs)
            self._barrier()                      # all owners' out_rows are complete
            if lay.Is:
                torch.cuda.current_stream().wait_stream(self._side)
            self._mark(evs)
            L.check(lib.mg_ep_combine(h, self._peer_out, self.dst.data_ptr(), self.idx.data_ptr(),
                                      self.w.data_ptr(), _ptr(self.shared_out), T, y.data_ptr(), st))
            self._mark(evs)
        if evs is not None:
            self._events.append(evs)
        return y.view(x.shape)

    __call__ = forward
