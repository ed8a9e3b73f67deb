"""Expert weights streamed from host memory: a MoE layer whose packed expert weights do not stay on
the GPU.

MoE-Gen keeps all expert weights in pinned host memory and cycles them through a few per-expert GPU
slots: a worker thread copies the next expert into a free slot (core/HtoD_Engine/HtoD_Engine.cpp:201-267),
the expert call waits for its slot and releases it afterwards
(core/GPU_Weight_Buffer/GPU_Weight_Buffer.cpp:144-169,261-308; moe_gen/models/Wrapper.py:476-527).
Here the unit is a group of experts in the packed layout: the layer's experts are cut into groups, each
group's packed bytes sit in pinned host memory, the GPU holds `slots` group-sized buffers, and one
forward walks the groups: the copy of group g+1 runs on a copy stream while the grouped GEMMs of group
g run (events order the two, nothing blocks the host).  Router, plan, scatter and combine run once
over all experts, so the result is bit-identical to the resident layer's.  With `routing_aware` the
per-group row counts are read back once per forward and groups nobody routed to are neither copied
nor computed (small batches, skewed routing).
"""
import ctypes as C
from typing import List, Optional, Tuple

import torch

from . import lib as L
from .layer import MoELayer, _ptr


class StreamedMoELayer:
    def __init__(self, *, group_experts: int, slots: int = 2, routing_aware: bool = False, device=None,
                 **layer_kwargs):
        E = layer_kwargs["n_experts"]
        if group_experts < 1 or E % group_experts:
            raise ValueError(f"group_experts={group_experts} must divide n_experts={E}")
        if slots < 2:
            raise ValueError("at least two slots (one being filled, one being read)")
        self.groups = E // group_experts
        self.n = group_experts
        self.slots = min(slots, self.groups)
        self.routing_aware = routing_aware
        # a handle whose "local experts" are one group: its packed layout is the layout of a slot
        self.layer = MoELayer(ep_rank=0, ep_size=self.groups, device=device, **layer_kwargs)
        lay = self.layer
        self.device = lay.device
        self.group_bytes = lay.packed.numel()
        self.host: List[torch.Tensor] = [torch.empty(self.group_bytes, dtype=torch.uint8).pin_memory()
                                         for _ in range(self.groups)]
        with torch.cuda.device(self.device):
            # slot 0 is the layer's own packed buffer (it also holds the shared expert, which stays)
            self.slot = [lay.packed] + [torch.zeros(self.group_bytes, dtype=torch.uint8, device=self.device)
                                        for _ in range(self.slots - 1)]
            self.copy_stream = torch.cuda.Stream(device=self.device)
            self.ready = [torch.cuda.Event() for _ in range(self.slots)]
            self.free = [torch.cuda.Event() for _ in range(self.slots)]
        nb = C.c_size_t()
        L.check(lay.lib.mg_dequant_ws_bytes(lay._h, C.byref(nb)))
        self._deq_bytes = nb.value
        self._deq: Optional[torch.Tensor] = None
        self._shared_loaded = False
        self.last_groups_moved = 0
        self.last_group_order: List[int] = []
        self._counts_host = None
        self._counts_event = None

    # ------------------------------------------------------------------ weights
    def set_router(self, gate_weight, bias=None):
        self.layer.set_router(gate_weight, bias)

    def load_shared(self, gate, up, down):
        """Shared expert: resident, in every slot's shared section (the GEMM reads it from slot 0)."""
        self.layer.load_shared(gate, up, down)
        self._shared_loaded = True

    def load_expert(self, expert: int, gate, up, down, scales: Optional[Tuple] = None):
        """Packs global expert `expert` on the device and stores its group's bytes in host memory once
        the group is complete (call in ascending expert order within a group)."""
        g, i = divmod(expert, self.n)
        self.layer.load_expert(i, gate, up, down, scales)
        if i == self.n - 1:
            self.host[g].copy_(self.layer.packed)
            torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        lay, lib = self.layer, self.layer.lib
        shape = x.shape
        x2 = x.reshape(-1, lay.H)
        T, E, k, n = x2.shape[0], lay.E, lay.k, self.n
        y = torch.empty_like(x2) if out is None else out.reshape(-1, lay.H)
        if T == 0:
            return y.view(shape)
        dev = self.device
        with torch.cuda.device(dev):
            comp = torch.cuda.current_stream()
            st = comp.cuda_stream
            idx, w = lay.gate_route(x2)[:2]
            counts, offsets, pad, dst = lay.permute_plan(idx, 0, E)
            rows = (-(-T * k // 128) + E) * 128
            perm = torch.empty(rows, lay.H, dtype=torch.bfloat16, device=dev)
            hbuf = torch.empty(rows, lay.I, dtype=torch.bfloat16, device=dev)
            outr = torch.empty(rows, lay.H, dtype=torch.bfloat16, device=dev)
            shared = None
            if not self.routing_aware:
                L.check(lib.mg_permute_rows(lay._h, x2.data_ptr(), dst.data_ptr(), T, perm.data_ptr(), st))
                if lay.Is:
                    # before the slots start to rotate: slot 0 still holds whatever group was last there,
                    # its shared section is never overwritten by a group copy (see _copy_group)
                    shared = lay.shared_ffn(x2)
            todo = list(range(self.groups))
            if self.routing_aware:
                # The order of the copies follows the routing: the rows per group travel to pinned host
                # memory behind the plan kernels (a few hundred bytes, asynchronous); the host waits for that
                # one event only, while the scatter and the shared expert's GEMMs keep the GPU busy.  Groups
                # without rows are neither copied nor computed; the others go by falling row count, so that
                # the long GEMMs run first and hide the copies of the groups behind them.
                per_group = counts.view(self.groups, n).sum(1, dtype=torch.int32)
                if self._counts_host is None:
                    self._counts_host = torch.empty(self.groups, dtype=torch.int32).pin_memory()
                    self._counts_event = torch.cuda.Event()
                self._counts_host.copy_(per_group, non_blocking=True)
                self._counts_event.record(comp)
                L.check(lib.mg_permute_rows(lay._h, x2.data_ptr(), dst.data_ptr(), T, perm.data_ptr(), st))
                if lay.Is:
                    shared = lay.shared_ffn(x2)
                self._counts_event.synchronize()
                rows_of = self._counts_host.tolist()
                todo = sorted((g for g in todo if rows_of[g] > 0), key=lambda g: (-rows_of[g], g))
            self.last_groups_moved = len(todo)
            self.last_group_order = list(todo)
            # FP8: de-quantise a group ahead of its GEMMs when it sees many rows, else convert in the GEMM
            use_deq = self._deq_bytes > 0 and T * k >= 1024 * E
            if use_deq and self._deq is None:
                self._deq = torch.empty(self._deq_bytes, dtype=torch.uint8, device=dev)
            deq = self._deq if use_deq else None
            self.copy_stream.wait_stream(comp)
            for j, g in enumerate(todo[:self.slots]):
                self._copy_group(g, j)
            for j, g in enumerate(todo):
                b = j % self.slots
                comp.wait_event(self.ready[b])
                L.check(lib.mg_expert_ffn(lay._h, perm.data_ptr(), pad.data_ptr() + 4 * g * n,
                                          counts.data_ptr() + 4 * g * n, rows, self.slot[b].data_ptr(),
                                          hbuf.data_ptr(), outr.data_ptr(), _ptr(deq), st))
                self.free[b].record(comp)
                if j + self.slots < len(todo):
                    self.copy_stream.wait_event(self.free[b])
                    self._copy_group(todo[j + self.slots], b)
            L.check(lib.mg_combine(lay._h, outr.data_ptr(), dst.data_ptr(), idx.data_ptr(), w.data_ptr(),
                                   _ptr(shared), T, y.data_ptr(), st))
            # the buffers above are freed when this returns; keep the allocator from handing them to
            # another stream's work before the copy stream is done with the slots
            comp.wait_stream(self.copy_stream)
        return y.view(shape)

    __call__ = forward

    def _copy_group(self, g: int, b: int):
        """Host group g -> slot b on the copy stream.  Only the expert sections travel: the shared
        expert's section at the end of a slot is left alone."""
        nbytes = self._expert_bytes()
        with torch.cuda.stream(self.copy_stream):
            self.slot[b][:nbytes].copy_(self.host[g][:nbytes], non_blocking=True)
            self.ready[b].record(self.copy_stream)

    def _expert_bytes(self) -> int:
        if getattr(self, "_eb", None) is None:
            lay = self.layer
            # the shared expert's two sections (SH13 [2 I_s, H], SH2 [H, I_s], bf16) are the last ones of
            # the packed layout, each rounded up to 256 bytes
            r256 = lambda b: (b + 255) // 256 * 256                  # noqa: E731
            self._eb = self.group_bytes - r256(2 * lay.Is * lay.H * 2) - r256(lay.H * lay.Is * 2)
            assert self._eb > 0
        return self._eb

    def close(self):
        self.layer.close()
