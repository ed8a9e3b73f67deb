"""Host-side MoE layer object: owns the native handle, the packed weight buffer and
the workspace (all torch CUDA tensors — torch is used for device memory and streams
only), and calls the C ABI for every computation.

The staged methods mirror the steps of the reference's layer
(moe_gen/models/deepseek/deepseekv3/modeling_deepseek_v3.py: MoEGate.forward
:500-561, DeepseekV3MoE.moe_infer :628-711) so tests can compare stage by stage.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import lib as L


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class MoELayer:
    def __init__(self, *, hidden: int, inter: int, n_experts: int, top_k: int, inter_shared: int = 0,
                 n_group: int = 1, topk_group: int = 1, gating: int = L.GATE_SOFTMAX_GREEDY,
                 norm_topk_prob: bool = False, routed_scale: float = 1.0,
                 weight_format: int = L.WEIGHT_BF16, combine_mode: int = L.COMBINE_FP32,
                 ep_rank: int = 0, ep_size: int = 1, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("moe_gen_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.lib = L.load()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.desc = L.LayerDesc(C.sizeof(L.LayerDesc), hidden, inter, inter_shared, n_experts, top_k, n_group,
                                topk_group, gating, int(bool(norm_topk_prob)), float(routed_scale),
                                weight_format, combine_mode, ep_rank, ep_size)
        self.H, self.I, self.Is, self.E, self.k = hidden, inter, inter_shared, n_experts, top_k
        self.e_local = n_experts // ep_size
        self.expert_lo = ep_rank * self.e_local
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_create(C.byref(self.desc), C.byref(self._h)))
            n = C.c_size_t()
            L.check(self.lib.mg_packed_weight_bytes(self._h, C.byref(n)))
            # zeroed: the alignment gaps between its sections are never written
            self.packed = torch.zeros(n.value, dtype=torch.uint8, device=self.device)
        self.gate_w: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self._ws: Optional[torch.Tensor] = None
        self._ws_tokens = -1
        self.options = {}                       # option id -> last value set

    # ------------------------------------------------------------------ lifetime
    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self.lib.mg_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    def _check_in(self, t: torch.Tensor, dtype, what: str):
        if t.device != self.device or t.dtype != dtype or not t.is_contiguous():
            raise ValueError(f"{what}: expected contiguous {dtype} tensor on {self.device}, got "
                             f"{t.dtype} on {t.device} contiguous={t.is_contiguous()}")

    # ------------------------------------------------------------------ weights
    def set_router(self, gate_weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        """gate.weight [E,H] (kept as bf16) and, for noaux_tc, e_score_correction_bias [E] (fp32)."""
        self.gate_w = gate_weight.detach().to(self.device, torch.bfloat16).contiguous()
        assert self.gate_w.shape == (self.E, self.H)
        self.bias = None if bias is None else bias.detach().to(self.device, torch.float32).contiguous()

    def load_expert(self, local_expert: int, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
                    scales: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None):
        """Packs one expert ([I,H], [I,H], [H,I] as nn.Linear stores them).  local_expert = -1 is
        the shared expert.  FP8 layers pass float8_e4m3fn matrices plus their fp32 scales."""
        fp8 = self.desc.weight_format == L.WEIGHT_FP8_BLOCK128 and local_expert >= 0
        dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
        mats = [m.detach().to(self.device).contiguous() for m in (gate, up, down)]
        I = self.Is if local_expert < 0 else self.I
        for m, shp in zip(mats, ((I, self.H), (I, self.H), (self.H, I))):
            if m.dtype != dt or tuple(m.shape) != shp:
                raise ValueError(f"expert matrix {tuple(m.shape)} {m.dtype}, expected {shp} {dt}")
        sc = [None, None, None]
        if fp8:
            if scales is None:
                raise ValueError("FP8 layer: scales=(gate_scale, up_scale, down_scale) required")
            sc = [s.detach().to(self.device, torch.float32).contiguous() for s in scales]
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_pack_expert(self._h, local_expert, mats[0].data_ptr(), mats[1].data_ptr(),
                                            mats[2].data_ptr(), _ptr(sc[0]), _ptr(sc[1]), _ptr(sc[2]),
                                            self.packed.data_ptr(), self._stream()))
            torch.cuda.current_stream().synchronize()   # sources may be temporaries

    def load_shared(self, gate, up, down):
        self.load_expert(-1, gate, up, down)

    # ------------------------------------------------------------------ sizes
    def padded_rows(self, n_rows: int) -> int:
        out = C.c_int64()
        L.check(self.lib.mg_padded_rows(self._h, n_rows, C.byref(out)))
        return out.value

    def _workspace(self, T: int) -> torch.Tensor:
        if self._ws is None or T > self._ws_tokens:
            n = C.c_size_t()
            L.check(self.lib.mg_workspace_bytes(self._h, T, 0, C.byref(n)))
            self._ws = None
            self._ws = torch.empty(max(n.value, 256), dtype=torch.uint8, device=self.device)
            self._ws_tokens = T
        return self._ws

    def workspace_view(self, which: int, T: int) -> int:
        p = C.c_void_p()
        L.check(self.lib.mg_workspace_ptr(self._h, self._ws.data_ptr(), self._ws_tokens, 0, which, C.byref(p)))
        return p.value

    def device_status(self) -> Tuple[int, int]:
        code, detail = C.c_int32(), C.c_int32()
        L.check(self.lib.mg_device_status(self._h, C.byref(code), C.byref(detail)))
        return code.value, detail.value

    def set_option(self, option: int, value: int):
        L.check(self.lib.mg_set_option(self._h, option, value))
        self.options[option] = value
        if option != L.OPT_KEEP_DEQUANT:
            self._ws, self._ws_tokens = None, -1    # workspace layout may depend on options
            self._hws = None

    def set_stage_timing(self, enable: bool):
        L.check(self.lib.mg_set_stage_timing(self._h, int(enable)))

    def stage_times(self) -> dict:
        """Milliseconds per stage of the last forward (call after synchronising)."""
        ms = (C.c_float * len(L.STAGES))()
        L.check(self.lib.mg_stage_times(self._h, ms, len(L.STAGES)))
        return dict(zip(L.STAGES, [float(v) for v in ms]))

    def last_launch_count(self) -> int:
        n = C.c_int32()
        L.check(self.lib.mg_last_launch_count(self._h, C.byref(n)))
        return n.value

    # ------------------------------------------------------------------ whole layer
    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: [..., H] bf16 on the layer's device -> same shape.  Asynchronous on the current stream."""
        shape = x.shape
        x2 = x.reshape(-1, self.H)
        self._check_in(x2, torch.bfloat16, "hidden_states")
        T = x2.shape[0]
        ws = self._workspace(T)
        y = torch.empty_like(x2) if out is None else out
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_moe_forward(self._h, x2.data_ptr(), T, self.gate_w.data_ptr(), _ptr(self.bias),
                                            self.packed.data_ptr(), ws.data_ptr(), ws.numel(), y.data_ptr(),
                                            self._stream()))
        return y.view(shape)

    __call__ = forward

    def forward_from_logits(self, x: torch.Tensor, logits: torch.Tensor, out: Optional[torch.Tensor] = None):
        """The layer on router logits the caller computed ([T,E] fp32, e.g. F.linear(x.float(),
        W.float()) as the reference's MoEGate does, modeling_deepseek_v3.py:503-508): the routing is
        then an exact function of those logits."""
        shape = x.shape
        x2 = x.reshape(-1, self.H)
        self._check_in(x2, torch.bfloat16, "hidden_states")
        self._check_in(logits, torch.float32, "logits")
        T = x2.shape[0]
        if tuple(logits.shape) != (T, self.E):
            raise ValueError(f"logits {tuple(logits.shape)}, expected {(T, self.E)}")
        ws = self._workspace(T)
        y = torch.empty_like(x2) if out is None else out
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_moe_forward_from_logits(self._h, x2.data_ptr(), T, logits.data_ptr(), _ptr(self.bias),
                                                        self.packed.data_ptr(), ws.data_ptr(), ws.numel(),
                                                        y.data_ptr(), self._stream()))
        return y.view(shape)

    # ------------------------------------------------------------------ decoder-layer glue
    def rmsnorm(self, x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """weight * bf16(x * rsqrt(mean(x^2) + eps)): the reference's DeepseekV3RMSNorm
        (modeling_deepseek_v3.py:125-150) with the bf16 weight of a bfloat16 model."""
        x2 = x.reshape(-1, self.H)
        self._check_in(x2, torch.bfloat16, "hidden_states")
        self._check_in(weight, torch.bfloat16, "norm weight")
        if weight.numel() != self.H:
            raise ValueError(f"norm weight has {weight.numel()} elements, hidden size is {self.H}")
        y = torch.empty_like(x2) if out is None else out
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_rmsnorm(self._h, x2.data_ptr(), weight.data_ptr(), float(eps), x2.shape[0],
                                        y.data_ptr(), self._stream()))
        return y.view(x.shape)

    def block_forward(self, hidden: torch.Tensor, norm_weight: torch.Tensor, eps: float = 1e-6,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """hidden + moe(rmsnorm(hidden)): the decoder layer's second half
        (modeling_deepseek_v3.py:1361-1365) with the residual add done by the combine kernel.
        out may be hidden itself (in-place update of the residual stream)."""
        shape = hidden.shape
        h2 = hidden.reshape(-1, self.H)
        self._check_in(h2, torch.bfloat16, "hidden_states")
        self._check_in(norm_weight, torch.bfloat16, "norm weight")
        if norm_weight.numel() != self.H:
            raise ValueError(f"norm weight has {norm_weight.numel()} elements, hidden size is {self.H}")
        T = h2.shape[0]
        ws = self._workspace(T)
        if getattr(self, "_xnorm", None) is None or self._xnorm.shape[0] < T:
            self._xnorm = torch.empty(max(T, 1), self.H, dtype=torch.bfloat16, device=self.device)
        y = torch.empty_like(h2) if out is None else out.reshape(-1, self.H)
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_moe_block_forward(self._h, h2.data_ptr(), norm_weight.data_ptr(), float(eps), T,
                                                  self.gate_w.data_ptr(), _ptr(self.bias), self.packed.data_ptr(),
                                                  self._xnorm.data_ptr(), ws.data_ptr(), ws.numel(), y.data_ptr(),
                                                  self._stream()))
        return y.view(shape)

    @staticmethod
    def host_chunks(T: int, chunk_tokens: int) -> list:
        """Token counts of the chunks the host-buffer forward uses (mg_host_chunk_plan): the copy-in of
        the first chunk and the copy-out of the last one cannot overlap with compute, so those two are
        half a chunk; the ones between them are one and a half, because every chunk streams all expert
        weights once."""
        lib = L.load()
        n = C.c_int32()
        L.check(lib.mg_host_chunk_plan(T, max(1, chunk_tokens), None, 0, C.byref(n)))
        sizes = (C.c_int64 * max(n.value, 1))()
        L.check(lib.mg_host_chunk_plan(T, max(1, chunk_tokens), sizes, n.value, C.byref(n)))
        return [int(v) for v in sizes[:n.value]]

    def forward_host(self, x_host: torch.Tensor, y_host: Optional[torch.Tensor] = None,
                     chunk_tokens: int = 8192) -> torch.Tensor:
        """Host-buffer entry (mg_moe_forward_host): x_host [T,H] bf16 in (preferably pinned) host memory
        -> y_host.  The library copies chunks in, computes and copies out on three streams; returns
        after the last copy has finished."""
        T = x_host.shape[0]
        if x_host.dtype != torch.bfloat16 or not x_host.is_contiguous() or x_host.is_cuda:
            raise ValueError("x_host: expected a contiguous bfloat16 tensor in host memory")
        if y_host is None:
            y_host = torch.empty_like(x_host, pin_memory=x_host.is_pinned())
        if T == 0:
            return y_host
        with torch.cuda.device(self.device):
            n = C.c_size_t()
            L.check(self.lib.mg_host_workspace_bytes(self._h, T, chunk_tokens, C.byref(n)))
            if getattr(self, "_hws", None) is None or self._hws.numel() < n.value:
                self._hws = None
                self._hws = torch.empty(n.value, dtype=torch.uint8, device=self.device)
            L.check(self.lib.mg_moe_forward_host(self._h, x_host.data_ptr(), T, self.gate_w.data_ptr(), _ptr(self.bias),
                                                 self.packed.data_ptr(), self._hws.data_ptr(), self._hws.numel(),
                                                 y_host.data_ptr(), chunk_tokens, self._stream()))
            torch.cuda.current_stream().synchronize()
        return y_host

    # ------------------------------------------------------------------ stages
    def gate_logits(self, x: torch.Tensor) -> torch.Tensor:
        self._check_in(x, torch.bfloat16, "hidden_states")
        T = x.shape[0]
        logits = torch.empty(T, self.E, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_gate_logits(self._h, x.data_ptr(), self.gate_w.data_ptr(), T, logits.data_ptr(),
                                            self._stream()))
        return logits

    def route_topk(self, logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        self._check_in(logits, torch.float32, "logits")
        T = logits.shape[0]
        idx = torch.empty(T, self.k, dtype=torch.int32, device=self.device)
        w = torch.empty(T, self.k, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_route_topk(self._h, logits.data_ptr(), _ptr(self.bias), T, idx.data_ptr(),
                                           w.data_ptr(), self._stream()))
        return idx, w

    def gate_route(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        """The routing mg_moe_forward uses: router product on the tensor cores, top-k, and near-tie tokens
        re-routed from exactly recomputed logits.  -> topk_idx, topk_w, logits (recomputed entries included),
        fix (int32: [0] tokens routed again, [1] of which with the whole row recomputed, [2] single logits
        recomputed; tokens from [4], row tokens from [4+T], (token, expert) pairs from [4+2T])."""
        self._check_in(x, torch.bfloat16, "hidden_states")
        T = x.shape[0]
        logits = torch.empty(T, self.E, dtype=torch.float32, device=self.device)
        idx = torch.empty(T, self.k, dtype=torch.int32, device=self.device)
        w = torch.empty(T, self.k, dtype=torch.float32, device=self.device)
        n = C.c_size_t()
        L.check(self.lib.mg_route_fix_bytes(T, C.byref(n)))
        fix = torch.zeros(n.value // 4, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_gate_route_topk(self._h, x.data_ptr(), self.gate_w.data_ptr(), _ptr(self.bias), T,
                                                logits.data_ptr(), idx.data_ptr(), w.data_ptr(), fix.data_ptr(),
                                                self._stream()))
        return idx, w, logits, fix

    def permute_plan(self, topk_idx: torch.Tensor, expert_lo: int = 0, n_plan: Optional[int] = None):
        """-> counts [n], offsets [n+1], pad_offsets [n+1], dst_row [T,k] (all int32)."""
        self._check_in(topk_idx, torch.int32, "topk_idx")
        n = self.E if n_plan is None else n_plan
        T = topk_idx.shape[0]
        dev = self.device
        counts = torch.empty(n, dtype=torch.int32, device=dev)
        offsets = torch.empty(n + 1, dtype=torch.int32, device=dev)
        pad = torch.empty(n + 1, dtype=torch.int32, device=dev)
        dst = torch.empty(T, self.k, dtype=torch.int32, device=dev)
        nb = C.c_size_t()
        L.check(self.lib.mg_plan_ws_bytes(self._h, T, C.byref(nb)))
        ws = torch.empty(max(nb.value, 4), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            L.check(self.lib.mg_permute_plan(self._h, topk_idx.data_ptr(), T, expert_lo, n, counts.data_ptr(),
                                             offsets.data_ptr(), pad.data_ptr(), dst.data_ptr(), ws.data_ptr(),
                                             self._stream()))
        return counts, offsets, pad, dst

    def permute_rows(self, x: torch.Tensor, dst_row: torch.Tensor, rows_padded: int) -> torch.Tensor:
        self._check_in(x, torch.bfloat16, "hidden_states")
        perm = torch.zeros(rows_padded, self.H, dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_permute_rows(self._h, x.data_ptr(), dst_row.data_ptr(), x.shape[0],
                                             perm.data_ptr(), self._stream()))
        return perm

    def expert_ffn(self, perm_x: torch.Tensor, pad_offsets: torch.Tensor, counts: torch.Tensor,
                   predequant: bool = False):
        """-> (h_buf [rows,I], out_rows [rows,H]) over the padded expert-sorted rows.
        predequant=True (FP8 layers) de-quantises the weights into scratch first."""
        rows = perm_x.shape[0]
        hbuf = torch.zeros(rows, self.I, dtype=torch.bfloat16, device=self.device)
        out = torch.zeros(rows, self.H, dtype=torch.bfloat16, device=self.device)
        nb = C.c_size_t()
        L.check(self.lib.mg_dequant_ws_bytes(self._h, C.byref(nb)))
        deq = torch.empty(nb.value, dtype=torch.uint8, device=self.device) if (nb.value and predequant) else None
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_expert_ffn(self._h, perm_x.data_ptr(), pad_offsets.data_ptr(), counts.data_ptr(),
                                           rows, self.packed.data_ptr(), hbuf.data_ptr(), out.data_ptr(),
                                           _ptr(deq), self._stream()))
            if deq is not None:
                torch.cuda.current_stream().synchronize()
        return hbuf, out

    def shared_ffn(self, x: torch.Tensor) -> torch.Tensor:
        self._check_in(x, torch.bfloat16, "hidden_states")
        T = x.shape[0]
        hs = torch.empty(T, self.Is, dtype=torch.bfloat16, device=self.device)
        out = torch.empty(T, self.H, dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_shared_ffn(self._h, x.data_ptr(), T, self.packed.data_ptr(), hs.data_ptr(),
                                           out.data_ptr(), self._stream()))
        return out

    def combine(self, out_rows: torch.Tensor, dst_row: torch.Tensor, topk_idx: torch.Tensor,
                topk_w: torch.Tensor, shared_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        T = topk_idx.shape[0]
        y = torch.empty(T, self.H, dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_combine(self._h, out_rows.data_ptr(), dst_row.data_ptr(), topk_idx.data_ptr(),
                                        topk_w.data_ptr(), _ptr(shared_out), T, y.data_ptr(), self._stream()))
        return y

    def dequant_fp8(self, q: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
        """bf16(float(q) * scale[r/128][c/128]) (moe_gen/models/Wrapper.py:109-138)."""
        q = q.to(self.device).contiguous()
        s = scale_inv.to(self.device, torch.float32).contiguous()
        out = torch.empty(q.shape, dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            L.check(self.lib.mg_dequant_fp8_block128(q.data_ptr(), s.data_ptr(), q.shape[0], q.shape[1],
                                                     out.data_ptr(), self._stream()))
        return out
