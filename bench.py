#!/usr/bin/env python
"""Benchmark of the MoE-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload v3|v2_236b|mixtral8x7b|v2lite] [--tokens T] [--zipf A]

One step = one forward of one MoE layer over T tokens of synthetic hidden states.
Default workload: DeepSeek-V3/R1 layer shape, W8A16 (FP8-e4m3 expert weights with 128x128
block scales), T = 65536 tokens, seed 3.  Rank 0 prints ONE JSON line.

  value     tokens/s with inputs resident in HBM (CUDA events, max over ranks)
  e2e       tokens/s through MoELayer.forward_host: pinned host input -> device -> layer ->
            host output, copies inside the timed region
  roofline  the dominant kernel (routed gate/up grouped GEMM with the SiLU*mul epilogue):
            algorithmic FLOPs per launch / mean device time of that stage, against the measured
            sustained bf16 GEMM throughput of this pool
  cpu_baseline  the CPU restatement of the reference layer (oracle/moe_oracle.py, torch CPU ops,
            all host threads) on a bounded token sample of the same layer

--impl reference times that CPU restatement alone (the reference ships no device code for
this path; its layer is PyTorch arithmetic, which the oracle restates and which cannot be
imported on the benchmark machine).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (hidden, inter, n_experts, top_k, inter_shared, n_group, topk_group, gating, norm, scale, wfmt, combine, T, seed)
    "v3": (7168, 2048, 256, 8, 2048, 8, 4, 2, True, 2.5, 1, 0, 65536, 3),
    "v2_236b": (5120, 1536, 160, 6, 3072, 8, 3, 1, False, 16.0, 0, 1, 32768, 2),
    "mixtral8x7b": (4096, 14336, 8, 2, 0, 1, 1, 3, True, 1.0, 0, 2, 16384, 1),
    "v2lite": (2048, 1408, 64, 6, 2816, 1, 1, 0, False, 1.0, 0, 1, 2048, 0),
    # the V3 layer with 32 experts and 4096 tokens: same kernels, same rows per expert per tile wave,
    # a few GB on the device -- the case profiler captures are taken on
    "v3_small": (7168, 2048, 32, 8, 2048, 8, 4, 2, True, 2.5, 1, 0, 4096, 3),
}
WORKLOAD_TEXT = {
    "v3": "DeepSeek-V3/R1 MoE layer W8A16: H=7168 E=256 k=8 I=2048 shared I=2048, sigmoid+bias noaux_tc G=8 keep 4",
    "v2_236b": "DeepSeek-V2-236B MoE layer bf16: H=5120 E=160 k=6 I=1536 shared I=3072, softmax group-limited G=8 keep 3",
    "mixtral8x7b": "Mixtral-8x7B MoE layer bf16: H=4096 E=8 k=2 I=14336, softmax top-2 renormalised",
    "v2lite": "DeepSeek-V2-Lite MoE layer bf16: H=2048 E=64 k=6 I=1408 shared I=2816, softmax greedy",
    "v3_small": "DeepSeek-V3 layer shape cut to 32 experts (profiling case): H=7168 E=32 k=8 I=2048 shared I=2048",
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# --------------------------------------------------------------------------------------
# synthetic layer on the device
# --------------------------------------------------------------------------------------
def quantize_fp8_block128_gpu(w: torch.Tensor):
    """Per-128x128-block e4m3 quantisation with scale = amax/448 (the DeepSeek-V3 checkpoint
    format: moe_gen/models/deepseek/deepseekv3/deepseekv3_initializer.py:191-205)."""
    m, n = w.shape
    v = w.view(m // 128, 128, n // 128, 128)
    amax = v.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    q = (v * (448.0 / amax)).to(torch.float8_e4m3fn)
    return q.view(m, n).contiguous(), (amax / 448.0).view(m // 128, n // 128).contiguous()


def router_tensors(name: str, device, zipf=0.0):
    H, I, E, k, Is, G, keep, gating, norm, scale, wfmt, comb, _, seed = WORKLOADS[name]
    g = torch.Generator(device=device).manual_seed(seed)           # same on every rank
    gate_w = (torch.randn(E, H, generator=g, device=device) * 0.02).to(torch.bfloat16)
    bias = torch.randn(E, generator=g, device=device) * 0.01 if gating == 2 else None
    if zipf > 0:
        # per-expert logit offset through hidden column 0 (set to 1.0 in the inputs)
        perm = torch.randperm(E, generator=g, device=device)
        pmf = 1.0 / torch.arange(1, E + 1, dtype=torch.float64, device=device) ** zipf
        b = (pmf / pmf.sum()).log()
        col = torch.empty(E, device=device)
        col[perm] = (b - b.mean()).float()
        gate_w[:, 0] = col.to(torch.bfloat16)
    return gate_w, bias


def expert_tensors(name: str, device, e: int):
    """Global expert e (e = -1: the shared expert): bf16 matrices, or (fp8, scale) pairs for W8A16 layers."""
    H, I, E, k, Is, G, keep, gating, norm, scale, wfmt, comb, _, seed = WORKLOADS[name]
    ge = torch.Generator(device=device)
    if e < 0:
        ge.manual_seed(seed * 100003 + 99991)
        return [(torch.randn(r, c, generator=ge, device=device) * 0.02).to(torch.bfloat16)
                for r, c in ((Is, H), (Is, H), (H, Is))]
    ge.manual_seed(seed * 100003 + e)                               # per global expert id
    mats = [(torch.randn(r, c, generator=ge, device=device) * 0.02).to(torch.bfloat16)
            for r, c in ((I, H), (I, H), (H, I))]
    return [quantize_fp8_block128_gpu(m) for m in mats] if wfmt == 1 else mats


def build_layer(name: str, device, ep_rank=0, ep_size=1, zipf=0.0, load=True):
    from moe_gen_b200 import MoELayer
    H, I, E, k, Is, G, keep, gating, norm, scale, wfmt, comb, _, seed = WORKLOADS[name]
    layer = MoELayer(hidden=H, inter=I, n_experts=E, top_k=k, inter_shared=Is, n_group=G, topk_group=keep,
                     gating=gating, norm_topk_prob=norm, routed_scale=scale, weight_format=wfmt,
                     combine_mode=comb, ep_rank=ep_rank, ep_size=ep_size, device=device)
    if not load:
        return layer
    layer.set_router(*router_tensors(name, device, zipf))
    for i in range(layer.e_local):
        ws = expert_tensors(name, device, layer.expert_lo + i)
        if wfmt == 1:
            layer.load_expert(i, ws[0][0], ws[1][0], ws[2][0], (ws[0][1], ws[1][1], ws[2][1]))
        else:
            layer.load_expert(i, *ws)
    if Is:
        layer.load_shared(*expert_tensors(name, device, -1))
    return layer


def write_layer_checkpoint(name: str, path: str, device, zipf=0.0):
    """The workload's layer as one safetensors shard in the DeepSeek naming (block 0)."""
    from moe_gen_b200 import ingest as ING
    E, Is = WORKLOADS[name][2], WORKLOADS[name][4]
    gate_w, bias = router_tensors(name, device, zipf)

    def cpu(ws):
        return [tuple(t.cpu() for t in w) if isinstance(w, tuple) else w.cpu() for w in ws]
    experts = [cpu(expert_tensors(name, device, e)) for e in range(E)]
    shared = cpu(expert_tensors(name, device, -1)) if Is else None
    ING.export_moe_layer(path, 0, gate_w.cpu(), None if bias is None else bias.cpu(), experts, shared)


def make_tokens(name: str, T: int, device, rank=0, zipf=0.0):
    H = WORKLOADS[name][0]
    seed = WORKLOADS[name][13]
    g = torch.Generator(device=device).manual_seed(seed * 7919 + 17 + rank)
    x = torch.randn(T, H, generator=g, device=device).to(torch.bfloat16)
    if zipf > 0:
        x[:, 0] = 1.0
    return x


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); pw.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------
# CPU restatement of the reference layer (baseline leg and --impl reference)
# --------------------------------------------------------------------------------------
def reference_sample(name: str, t_sample: int) -> dict:
    """What one step of the CPU reference arm covers, relative to one forward of the named workload."""
    E, wfmt, T_full = WORKLOADS[name][2], WORKLOADS[name][10], WORKLOADS[name][12]
    t_sample = min(t_sample, T_full)
    n_deq = max(1, round(E * t_sample / T_full)) if wfmt == 1 else 0
    return {"tokens_timed": t_sample, "fraction_of_forward": t_sample / T_full,
            "experts_dequantised_per_step": n_deq, "distinct_expert_sets": min(E, 16),
            "extrapolated": t_sample < T_full}


def cpu_reference(name: str, t_sample: int, steps: int, warmup: int, zipf=0.0):
    """Times the CPU restatement of the reference layer (oracle.layer_forward, bf16, as the reference
    modules run on CPU) on a bounded sample: t_sample tokens of the workload's T through the full
    router and all experts, and, for W8A16 layers, the per-call FP8 de-quantisation the reference's
    Expert_Wrapper performs (moe_gen/models/Wrapper.py:481-491) for the same fraction of the experts
    (E * t_sample / T of them: a full forward de-quantises each expert once, whatever T is).
    Expert weights: N(0,0.02) drawn once for min(E,16) distinct experts and reused cyclically (each
    expert's matrices are far larger than the host caches, so reuse 16 experts apart does not change
    the memory behaviour; it only bounds set-up time and host memory)."""
    from oracle import moe_oracle as O
    H, I, E, k, Is, G, keep, gating, norm, scale, wfmt, comb = WORKLOADS[name][:12]
    spec = O.LayerSpec(H, I, E, k, Is, G, keep, gating, norm, scale, wfmt, comb, name)
    info = reference_sample(name, t_sample)
    t_sample, n_deq = info["tokens_timed"], info["experts_dequantised_per_step"]
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(WORKLOADS[name][13])
    x = torch.randn(t_sample, H, generator=g).to(torch.bfloat16)
    gate_w = (torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16)
    bias = torch.randn(E, generator=g) * 0.01 if spec.gating == O.GATE_SIGMOID_NOAUX_TC else None
    W = O.LayerWeights(gate_w, bias)
    distinct = min(E, 16)
    base = [[(torch.randn(r, c, generator=g) * 0.02).to(torch.bfloat16) for r, c in ((I, H), (I, H), (H, I))]
            for _ in range(distinct)]
    base_q = None
    if wfmt == 1:
        base_q = [[O.quantize_fp8_block128(m) for m in mats] for mats in base]
        base = [[O.dequantize_fp8_block128(q, s_) for q, s_ in mats] for mats in base_q]
    for e in range(E):
        m = base[e % distinct]
        W.w_gate.append(m[0]); W.w_up.append(m[1]); W.w_down.append(m[2])
    if spec.inter_shared:
        W.shared = tuple((torch.randn(r, c, generator=g) * 0.02).to(torch.bfloat16)
                         for r, c in ((Is, H), (Is, H), (H, Is)))
    if zipf > 0:
        x[:, 0] = 1.0

    def step():
        O.layer_forward(spec, x, W)
        for i in range(n_deq):
            for q, s_ in base_q[i % distinct]:
                O.dequantize_fp8_block128(q, s_)
    with torch.no_grad():
        for _ in range(warmup):
            step()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        dt = (time.perf_counter() - t0) / max(steps, 1)
    return {"tokens_per_s": t_sample / dt, "ms_per_step": dt * 1e3, "cores": threads,
            "sample": f"{t_sample} of the {WORKLOADS[name][12]} tokens of the {name} layer per step through the full "
                      f"router and expert count ({distinct} distinct expert weight sets reused cyclically)"
                      + (f", plus the per-call FP8 de-quantisation of {n_deq} of the {E} experts (the same fraction of a forward)"
                         if n_deq else "")
                      + f", torch CPU bf16, {steps} timed steps after {warmup} warm-up"}


def cuda_eager_baseline(name: str, x: torch.Tensor, zipf: float, steps: int = 2):
    """The same restatement of the reference layer run on the GPU as the reference would run it there:
    eager PyTorch + cuBLAS, the Python loop over experts, the row-count read-back, FP8 weights
    de-quantised on every expert call (modeling_deepseek_v3.py:675-691, Wrapper.py:481-491)."""
    from oracle import moe_oracle as O
    H, I, E, k, Is, G, keep, gating, norm, scale, wfmt, comb = WORKLOADS[name][:12]
    spec = O.LayerSpec(H, I, E, k, Is, G, keep, gating, norm, scale, wfmt, comb, name)
    dev = x.device
    gate_w, bias = router_tensors(name, dev, zipf)
    W = O.LayerWeights(gate_w, bias)
    if wfmt == 1:
        W.q_gate, W.q_up, W.q_down = [], [], []
    for e in range(E):
        ws = expert_tensors(name, dev, e)
        if wfmt == 1:
            W.q_gate.append(ws[0]); W.q_up.append(ws[1]); W.q_down.append(ws[2])
            W.w_gate.append(None); W.w_up.append(None); W.w_down.append(None)
        else:
            W.w_gate.append(ws[0]); W.w_up.append(ws[1]); W.w_down.append(ws[2])
    if Is:
        W.shared = tuple(expert_tensors(name, dev, -1))
    with torch.no_grad():
        y = O.layer_forward(spec, x, W, dequant_per_call=(wfmt == 1))["y"]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            y = O.layer_forward(spec, x, W, dequant_per_call=(wfmt == 1))["y"]
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"value": x.shape[0] / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms, "steps": steps,
            "what": "CPU restatement of the reference layer executed on this GPU: eager torch + cuBLAS, Python "
                    "expert loop with a host read of the row counts" +
                    (", FP8 weights de-quantised on every expert call" if wfmt == 1 else "")}, y


# --------------------------------------------------------------------------------------
# correctness gate printed beside the timing (single GPU): a few tokens recomputed with plain
# torch fp32 ops on the device from the same seeded weights
# --------------------------------------------------------------------------------------
def sample_check(name: str, layer, x: torch.Tensor, y: torch.Tensor, zipf: float, n_tokens: int = 16):
    import torch.nn.functional as F
    H, I, E, k, Is, G, keep, gating, norm, scale, wfmt, comb, _, seed = WORKLOADS[name]
    dev = x.device
    T = x.shape[0]
    idx, w, _, fix = layer.gate_route(x)
    # routing from fp32 (CUDA-core) logits, as the reference computes them
    if gating == 3:
        lg = F.linear(x, layer.gate_w).float()
    else:
        lg = F.linear(x.float(), layer.gate_w.float())
    idx2, _ = layer.route_topk(lg.contiguous())
    differ = int((idx.sort(1).values != idx2.sort(1).values).any(1).sum())
    # ... and from the correctly rounded logits (fp64 product, rounded once), which the layer's routing
    # has to equal token for token where the router works in fp32
    differ_exact = None
    if gating != 3:
        lg = F.linear(x.double(), layer.gate_w.double()).float()
        idx3, _ = layer.route_topk(lg.contiguous())
        differ_exact = int((idx.sort(1).values != idx3.sort(1).values).any(1).sum())
        del idx3
    del lg

    def fp32_mats(e):
        ws = expert_tensors(name, dev, e)
        if isinstance(ws[0], tuple):
            ws = [layer.dequant_fp8(q, s_) for q, s_ in ws]
        return [m.float() for m in ws]

    def mlp(xt, g_, u_, d_):
        return F.linear(F.silu(F.linear(xt, g_)) * F.linear(xt, u_), d_)

    tokens = torch.linspace(0, T - 1, min(n_tokens, T)).round().long().unique().to(dev)
    xs = x[tokens].float()
    ref = mlp(xs, *fp32_mats(-1)) if Is else torch.zeros(len(tokens), H, device=dev)
    pe, pw = idx[tokens].long(), w[tokens]
    for e in pe.unique().tolist():                      # every needed expert regenerated once from the seed
        rows, slots = (pe == e).nonzero(as_tuple=True)
        ref.index_add_(0, rows, mlp(xs[rows], *fp32_mats(e)) * pw[rows, slots].unsqueeze(1))
    err = (y[tokens].float() - ref).norm(dim=1) / ref.norm(dim=1).clamp_min(1e-30)
    return {"sampled_tokens": int(len(tokens)), "worst_rel_l2_vs_torch_fp32": float(err.max()), "tolerance": 1e-2,
            "tokens_routed_differently_from_fp32_logits": differ,
            "tokens_routed_differently_from_exact_logits": differ_exact, "tokens_rerouted_by_fixup": int(fix[0]),
            "tokens": T}


def quick_config(name: str, T: int, zipf: float, world: int, rank: int, device, steps: int = 5, reuse=None):
    """One compact line for a named configuration other than the headline: device-timed tokens/s at
    `world` GPUs and the sampled correctness gate.  `reuse`: an already built layer of this workload
    (its router is swapped for the Zipf cases and put back)."""
    import torch.distributed as dist
    layer = reuse
    if layer is None:
        base = build_layer(name, device, rank, world, zipf)
        if world > 1:
            from moe_gen_b200.ep import EPMoELayer
            layer = EPMoELayer(base, capacity_factor=float(world) if zipf > 0 else 2.0)
        else:
            layer = base
    else:
        base = layer.layer if world > 1 else layer
        base.set_router(*router_tensors(name, device, zipf))
        if world > 1:
            layer.reconfigure(capacity_factor=float(world) if zipf > 0 else 2.0)
    x = make_tokens(name, T // world, device, rank, zipf)
    for _ in range(3):
        y = layer.forward(x)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        y = layer.forward(x)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1) / steps
    code, detail = base.device_status()
    chk = sample_check(name, base, x, y, zipf, n_tokens=8)
    if world > 1:
        t = torch.tensor([ms, chk["worst_rel_l2_vs_torch_fp32"], float(code),
                          float(chk["tokens_routed_differently_from_exact_logits"] or 0)], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, chk["worst_rel_l2_vs_torch_fp32"], code = float(t[0]), float(t[1]), int(t[2])
        if chk["tokens_routed_differently_from_exact_logits"] is not None:
            chk["tokens_routed_differently_from_exact_logits"] = int(t[3])
        chk["sampled_tokens"] *= world
    if reuse is None:
        if world > 1:
            layer.close()
        base.close()
    out = {"workload": name, "tokens": T, "zipf_alpha": zipf, "ms_per_step": round(ms, 4),
           "tokens_per_s": round(T / (ms * 1e-3), 1), "device_status": code,
           "check": {"sampled_tokens": chk["sampled_tokens"],
                     "worst_rel_l2_vs_torch_fp32": round(chk["worst_rel_l2_vs_torch_fp32"], 6),
                     "tokens_routed_differently_from_fp32_logits": chk["tokens_routed_differently_from_fp32_logits"],
                     "tokens_routed_differently_from_exact_logits": chk["tokens_routed_differently_from_exact_logits"]}}
    if code != 0 or chk["worst_rel_l2_vs_torch_fp32"] > 1e-2 or chk["tokens_routed_differently_from_exact_logits"]:
        raise SystemExit(f"correctness gate failed for {out}")
    return out


def host_copy_ceiling(xh: torch.Tensor, yh: torch.Tensor, device, world: int, reps: int = 5):
    """Pinned-host <-> device copies of one step's input and output, all ranks at once, max over ranks."""
    import torch.distributed as dist
    xd = torch.empty_like(xh, device=device)
    yd = torch.empty_like(yh, device=device)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def timed(do_in: bool, do_out: bool) -> float:
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        s_in.wait_stream(torch.cuda.current_stream())
        s_out.wait_stream(torch.cuda.current_stream())
        for _ in range(reps):
            if do_in:
                with torch.cuda.stream(s_in):
                    xd.copy_(xh, non_blocking=True)
            if do_out:
                with torch.cuda.stream(s_out):
                    yh.copy_(yd, non_blocking=True)
        torch.cuda.current_stream().wait_stream(s_in)
        torch.cuda.current_stream().wait_stream(s_out)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    yd.zero_()
    timed(True, True)                                    # warm-up
    h2d, d2h, both = timed(True, False), timed(False, True), timed(True, True)
    nbytes = xh.numel() * 2
    return {"bytes_per_rank_each_way": nbytes, "h2d_ms": round(h2d, 3), "d2h_ms": round(d2h, 3), "both_ms": round(both, 3),
            "h2d_gbs_per_rank": round(nbytes / h2d / 1e6, 1), "d2h_gbs_per_rank": round(nbytes / d2h / 1e6, 1),
            "both_gbs_per_rank_each_way": round(nbytes / both / 1e6, 1),
            "note": "all ranks copy at once; slowest rank; the step's e2e time cannot be below both_ms, nor below "
                    "the device step plus the first chunk in and the last chunk out"}


def algorithmic(name: str, T: int):
    H, I, E, k, Is = WORKLOADS[name][:5]
    R = T * k
    return {
        "gemm1_flops": 4.0 * R * H * I, "gemm2_flops": 2.0 * R * H * I,
        "shared_flops": 6.0 * T * H * Is, "gate_flops": 2.0 * T * H * E,
        "permute_bytes": T * H * 2 + R * H * 2 + R * 4 + (E + 1) * 4,
        "combine_bytes": R * H * 2 + R * 4 + T * H * 2 + (T * H * 2 if Is else 0),
        "gate_bytes": T * H * 2 + E * H * 2 + T * E * 4,
        "topk_bytes": T * E * 4 + T * k * 8,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="v3", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--zipf", type=float, default=0.0)
    ap.add_argument("--cpu-sample-tokens", type=int, default=4096)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true",
                    help="skip the compact lines of the other named configurations")
    ap.add_argument("--no-eager-baseline", action="store_true",
                    help="skip the eager torch + cuBLAS restatement of the reference layer on this GPU")
    ap.add_argument("--stream-groups", type=int, default=0,
                    help="also time the layer with its expert weights streamed from pinned host memory in this many groups")
    ap.add_argument("--ingest", action="store_true",
                    help="also time checkpoint ingest: the layer written as a safetensors shard, then file -> packed buffer")
    ap.add_argument("--no-glue", action="store_true", help="skip the RMSNorm / residual-add measurement")
    ap.add_argument("--chunk-tokens", type=int, default=16384)
    ap.add_argument("--micro", type=int, default=1, help="token micro-batches pipelined in the expert-parallel forward")
    ap.add_argument("--capacity-factor", type=float, default=0.0,
                    help="expert-parallel receive buffers, in multiples of the mean rows per GPU (default 2, 8 with --zipf)")
    ap.add_argument("--ep-chunks", type=int, default=0,
                    help="expert parallel, host-buffer path: parts each rank's tokens are fed in")
    ap.add_argument("--ep-dedup", type=int, default=1,
                    help="expert parallel: 1 sends one row per (token, destination GPU), 0 one per (token, expert)")
    ap.add_argument("--ep-push", type=int, default=-1,
                    help="expert parallel: 1 owners push results home part by part beside the down projection, "
                         "0 the combine gathers them after the experts (-1: the library's default, 0)")
    ap.add_argument("--ep-parts", type=int, default=4, help="expert parallel: parts of the pushed return")
    ap.add_argument("--ep-copy", type=int, default=-1,
                    help="expert parallel: 1 = the results travel home through the copy engines beside the down "
                         "projection, 0 = the combine gathers them")
    ap.add_argument("--shared-early", type=int, default=-1,
                    help="1/0 shared expert beside the routing kernels / after the routed experts")
    ap.add_argument("--pair-gemm", type=int, default=-1, help="1/0 force the SM-pair expert GEMM on/off")
    ap.add_argument("--route-fixup", type=int, default=-1,
                    help="0 = route every token from the tensor-core router product as it is (no near-tie fix-up)")
    ap.add_argument("--fp8-mode", type=int, default=-1, help="0 auto, 1 pre-dequantise, 2 convert in the GEMM")
    ap.add_argument("--fp8-tall", type=int, default=-1, help="convert-in-GEMM tile height: 0 128 rows, 1 auto, 2 256 rows")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    name = args.workload
    T = args.tokens or WORKLOADS[name][12]
    H, I, E, k, Is = WORKLOADS[name][:5]
    warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    wbytes = WORKLOADS[name][2] * 3 * I * H * (1 if WORKLOADS[name][10] == 1 else 2)   # expert weights read every step
    big = T * H * 2 + wbytes > 126e6
    config = {"workload": WORKLOAD_TEXT[name], "tokens": T, "seed": WORKLOADS[name][13],
              "parallelism": f"ep{world}, {args.micro} micro-batches" if world > 1 else "single GPU",
              "zipf_alpha": args.zipf, "reference_sample": reference_sample(name, args.cpu_sample_tokens), "l2": f"inputs exceed L2: {wbytes / 1e9:.2f} GB of expert weights and {T * H * 2 / 1e6:.0f} MB of "
                    "hidden states are read every step" if big else "L2 flushed between steps by writing a 256 MB buffer"}

    # ------------------------------------------------------------------ reference arm (CPU)
    if args.impl == "reference":
        if rank != 0:
            return
        r = cpu_reference(name, args.cpu_sample_tokens, max(args.steps, 1), args.warmup, args.zipf)
        out = {"impl": "reference", "metric": "MoE-layer tokens/s", "value": r["tokens_per_s"], "unit": "tokens/s",
               "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
               "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
               "data": "synthetic", "config": config,
               "cpu_baseline": {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["cores"],
                                "kind": "port", "sample": r["sample"]},
               "e2e": {"value": r["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                       "d2h_bytes_per_step": 0}, "gpu_launches": 0}
        print(json.dumps(out), flush=True)
        return

    # ------------------------------------------------------------------ our arm
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    peaks, peak_kind = measured_peaks()

    if world == 1:
        layer = build_layer(name, device, zipf=args.zipf)
        x = make_tokens(name, T, device, 0, args.zipf)
        step = lambda: layer.forward(x)                                   # noqa: E731
        T_total = T
    else:
        from moe_gen_b200.ep import EPMoELayer
        assert T % world == 0
        # skewed routing can send most rows to one GPU: size the receive buffers for it
        cap = args.capacity_factor if args.capacity_factor > 0 else (float(world) if args.zipf > 0 else 2.0)
        layer = EPMoELayer(build_layer(name, device, rank, world, args.zipf), capacity_factor=cap, n_micro=args.micro,
                           dedup=bool(args.ep_dedup), push_return=None if args.ep_push < 0 else bool(args.ep_push), return_parts=args.ep_parts,
                           copy_return=args.ep_copy > 0)
        x = make_tokens(name, T // world, device, rank, args.zipf)
        step = lambda: layer.forward(x)                                   # noqa: E731
        T_total = T
    flush = None if big else torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def run_step():
        if flush is not None:
            flush.zero_()
        return step()

    base = layer.layer if world > 1 else layer
    if args.pair_gemm >= 0:
        base.set_option(2, args.pair_gemm)
    if args.route_fixup >= 0:
        base.set_option(10, args.route_fixup)
    if args.fp8_mode >= 0:
        base.set_option(1, args.fp8_mode)
    if args.fp8_tall >= 0:
        base.set_option(4, args.fp8_tall)
    if args.shared_early >= 0:
        base.set_option(6, args.shared_early)
    for _ in range(warmup):
        y = run_step()
    torch.cuda.synchronize()
    code, detail = base.device_status()
    if code != 0:
        raise SystemExit(f"device status {code} (detail {detail}) after warm-up")
    if world == 1:
        base.set_stage_timing(True)
    else:
        layer.timing = True
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        y = run_step()
    ev1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if world == 1:
        stage_ms = base.stage_times()
        base.set_stage_timing(False)
        launches = base.last_launch_count() + (1 if flush is not None else 0)
        phases = None
    else:
        layer.timing = False
        phases = layer.phase_times()
        n_micro_batches = max(len(layer._mbs), 1)       # read now: later legs re-allocate the buffers
        all_phases = [None] * world
        dist.all_gather_object(all_phases, {k_: round(v, 3) for k_, v in phases.items()})
        stage_ms = {"expert_gemm1": 0.0}
        # router product, top-k + the three fix-up kernels, count + scan, layout + place, dispatch (+ duplicate
        # table fill), [shared 2], experts (2, or 2 GEMMs + 2 de-quantisations per chunk of experts when FP8
        # weights are pre-dequantised; the down projection in parts, each followed by a return kernel, when the
        # return is pushed; in parts and one offset kernel when the copy engines carry it), combine; NCCL
        # kernels, memsets and copy-engine copies not counted
        parts = min(layer.return_parts, base.e_local, 8)
        pushed = layer.push_return and not layer.copy_return
        if layer.deq is not None:
            experts = 16 + 16 + (8 if pushed else 0)
        else:
            experts = 1 + (2 * parts if pushed else parts if layer.copy_return else 1)
        fixup = 3 if WORKLOADS[name][7] != 3 else 0
        launches = (7 + fixup + (1 if layer.dedup else 0) + (2 if Is else 0) + experts + 1
                    + (1 if layer.copy_return else 0))
    code, detail = base.device_status()
    if code != 0:
        raise SystemExit(f"device status {code} (detail {detail}) in the timed region")
    ms_per_step = ms / args.steps
    value = T_total / (ms_per_step * 1e-3)

    # ------------------------------------------------------------------ e2e: host buffers in and out
    e2e = None
    if not args.no_e2e and world == 1:
        xh = x.cpu().pin_memory()
        yh = torch.empty_like(xh).pin_memory()
        for _ in range(2):
            layer.forward_host(xh, yh, chunk_tokens=args.chunk_tokens)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            layer.forward_host(xh, yh, chunk_tokens=args.chunk_tokens)
        e1.record()
        torch.cuda.synchronize()
        e_ms = e0.elapsed_time(e1) / args.steps
        same = torch.equal(yh.view(torch.int16), y.cpu().view(torch.int16))
        e2e = {"value": T / (e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e_ms,
               "h2d_bytes_per_step": xh.numel() * 2, "d2h_bytes_per_step": yh.numel() * 2,
               "equals_device_path": bool(same), "chunk_tokens": args.chunk_tokens}
    elif not args.no_e2e:
        # every rank brings its own token shard from pinned host memory and takes its result back
        xh = x.cpu().pin_memory()
        yh = torch.empty_like(xh).pin_memory()

        # parts of at least 8192 tokens, two at least (measured at two GPUs: 4 parts of 8192 tokens 38.7 ms,
        # 2 parts 40.2 ms, 1 part 49.7 ms)
        ep_chunks = args.ep_chunks if args.ep_chunks > 0 else max(2, xh.shape[0] // 8192)
        while ep_chunks > 1 and xh.shape[0] % ep_chunks:
            ep_chunks -= 1

        def host_step():
            layer.forward_host(xh, yh, n_chunks=ep_chunks)
        for _ in range(2):
            host_step()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            host_step()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e_ms = float(t.item())
        e2e = {"value": T_total / (e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e_ms,
               "h2d_bytes_per_step": xh.numel() * 2 * world, "d2h_bytes_per_step": yh.numel() * 2 * world,
               "equals_device_path": bool(torch.equal(yh.view(torch.int16), y.cpu().view(torch.int16))),
               "chunks_per_rank": ep_chunks}

    # what the host link delivers for this step's buffers with all ranks copying at once: H2D alone, D2H
    # alone and both directions together (the e2e path's floor is the last of the three, fully overlapped)
    if e2e is not None:
        e2e["host_copy"] = host_copy_ceiling(xh, yh, device, world)

    # rows each GPU's experts receive (all ranks' picks), for the load-balance figures
    ep_load = None
    if world > 1:
        idx_l, _ = base.gate_route(x)[:2]
        hist = torch.bincount(idx_l.view(-1).long(), minlength=E).to(torch.int64)
        dist.all_reduce(hist)
        per_gpu = hist.view(world, E // world).sum(1).cpu().tolist()
        ep_load = {"rows_per_gpu": per_gpu, "max_over_mean": max(per_gpu) * world / max(sum(per_gpu), 1),
                   "capacity_factor": cap}

    # ---- correctness gate beside the timing, on every rank: sampled tokens of this rank's shard
    # recomputed with plain torch fp32 ops from the seeded weights (any global expert regenerates from
    # its id), worst case over the ranks
    check = None
    if not args.no_check:
        check = sample_check(name, base, x, y, args.zipf)
        if world > 1:
            t = torch.tensor([check["worst_rel_l2_vs_torch_fp32"], float(check["tokens_routed_differently_from_fp32_logits"]),
                              float(check["tokens_routed_differently_from_exact_logits"] or 0),
                              float(check["tokens_rerouted_by_fixup"])], device=device)
            worst = t.clone()
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            check["worst_rel_l2_vs_torch_fp32"] = float(worst[0])
            check["tokens_routed_differently_from_fp32_logits"] = int(t[1])
            if check["tokens_routed_differently_from_exact_logits"] is not None:
                check["tokens_routed_differently_from_exact_logits"] = int(t[2])
            check["tokens_rerouted_by_fixup"] = int(t[3])
            check["sampled_tokens"] *= world
            check["tokens"] = T_total
            check["note"] = "every rank checks sampled tokens of its own shard against its own output; worst over ranks"
        if check["worst_rel_l2_vs_torch_fp32"] > 1e-2 or check["tokens_routed_differently_from_exact_logits"]:
            raise SystemExit(f"correctness gate failed: {check}")
    code, detail = base.device_status()
    if world > 1:
        t = torch.tensor([float(code)], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        code = int(t[0])
    if code != 0:
        raise SystemExit(f"device status {code} (detail {detail}) on some rank after the correctness check")

    # ---- the other named configurations, one compact line each (same gate), at this GPU count
    others = None
    if not args.no_other_configs and name == "v3" and args.zipf == 0 and T == WORKLOADS["v3"][12]:
        others = []

        def side_entry(oname, oT, ozipf, **kw):
            # a side entry that fails its gate is reported as failed in its own line (the gate's verdict is
            # all-reduced, so every rank takes the same branch); the headline's own gate above ends the run
            try:
                others.append(quick_config(oname, oT, ozipf, world, rank, device, **kw))
            except SystemExit as e:
                others.append({"workload": oname, "tokens": oT, "zipf_alpha": ozipf, "failed": str(e)[:400]})

        for oname, oT in (("v2lite", 2048), ("mixtral8x7b", 16384), ("v2_236b", 32768), ("v2_236b", 512)):
            if oT % world == 0 and WORKLOADS[oname][2] % world == 0:
                side_entry(oname, oT, 0.0)
        for oT in (64, 256, 1024, 4096, 16384):
            side_entry("v3", oT, 1.2, reuse=layer)
        base.set_router(*router_tensors(name, device, args.zipf))
        if world > 1:
            layer.reconfigure(capacity_factor=cap)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    alg = algorithmic(name, T_total)
    if world > 1:
        # expert phase of the first micro-batch = gate/up GEMM + down GEMM (+ FP8 conversion) of this
        # rank's experts over 1/n_micro of the rows
        t_g1 = phases["expert_ffn"] * 1e-3
        n_mb = n_micro_batches
        tf = (alg["gemm1_flops"] + alg["gemm2_flops"]) / world / n_mb / t_g1 / 1e12 if t_g1 > 0 else 0.0
    else:
        t_g1 = stage_ms["expert_gemm1"] * 1e-3
        tf = alg["gemm1_flops"] / world / t_g1 / 1e12 if t_g1 > 0 else 0.0
    peak_tf = peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"])
    roofline = {"kernel": "grouped_gemm_kernel<SWIGLU> (routed gate/up projections + SiLU*mul)" if world == 1 else
                "grouped_gemm_kernel, both expert GEMMs of rank 0 (expert phase of the expert-parallel forward)",
                "bound": "tensor", "achieved": tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": tf / peak_tf,
                "peak_kind": f"of {peak_kind} sustained bf16 GEMM", "frac_of_burst": tf / peaks.get("bf16_tflops", 1590.0),
                "traffic": None}
    if world == 1 and name == "v3" and args.fp8_mode in (-1, 0, 1) and T == WORKLOADS["v3"][12]:
        # not measured by this run: DRAM bytes of one launch of this kernel (one chunk of 32 experts) as ncu
        # counted them on this workload (dram__bytes_read.sum + dram__bytes_write.sum, 1-pass counters, mean
        # of the 8 launches of a forward), recorded once; the same launch moves 3.09 GB algorithmically
        roofline["traffic"] = 4.88e9
        roofline["traffic_recorded"] = {"captured": "2026-11-25, commit eea7afe", "algorithmic_bytes": 3.09e9,
                                        "ratio": round(4.88 / 3.09, 2),
                                        "note": "bytes per launch from a recorded ncu capture of this workload, not "
                                                "from this run; the kernel's tile order is unchanged since"}
    hbm = peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"])
    Tl = T_total // world
    algl = algorithmic(name, Tl)
    stages = {}
    for st, num, unit in (("permute_rows", algl["permute_bytes"], "GB/s"), ("combine", algl["combine_bytes"], "GB/s"),
                          ("route_topk", algl["topk_bytes"], "GB/s"), ("gate_logits", algl["gate_bytes"], "GB/s"),
                          ("expert_gemm1", alg["gemm1_flops"] / world, "TFLOP/s"),
                          ("expert_gemm2", alg["gemm2_flops"] / world, "TFLOP/s"),
                          ("shared_gemm1", algl["shared_flops"] * 2 / 3, "TFLOP/s"),
                          ("shared_gemm2", algl["shared_flops"] / 3, "TFLOP/s")):
        t = stage_ms.get(st, 0.0) * 1e-3
        if st.startswith("shared_gemm") and t < 2e-5:
            # the shared expert ran on the library's side stream beside the routing kernels
            stages[st] = {"ms": round(t * 1e3, 4), "note": "overlapped with top-k, plan and scatter"}
            continue
        if t > 0 and num > 0:
            rate = num / t / (1e9 if unit == "GB/s" else 1e12)
            stages[st] = {"ms": round(t * 1e3, 4), "achieved": round(rate, 1), "unit": unit,
                          "frac": round(rate / (hbm if unit == "GB/s" else peak_tf), 3)}
    for st in ("permute_plan", "dequant"):
        if stage_ms.get(st, 0.0) > 0:
            stages[st] = {"ms": round(stage_ms[st], 4)}
    if phases is not None:
        stages = {k_: {"ms": round(v, 4)} for k_, v in phases.items()}
        stages["by_rank_ms"] = all_phases
        stages["note"] = (f"phases of the first of {n_micro_batches} pipelined micro-batches on its stream; "
                          f"each rank fetches {Tl * k * H * 2 * (world - 1) / world / 1e6:.0f} MB over NVLink per step in the combine "
                          f"and sends at most that in the dispatch (one row per token and destination GPU)")

    # ---- decoder-layer glue: RMSNorm in front of the block, residual add inside the combine ----
    glue = None
    if world == 1 and not args.no_glue:
        gw = (1.0 + 0.1 * torch.randn(H, device=device)).to(torch.bfloat16)
        xn = torch.empty_like(x)
        for _ in range(3):
            layer.rmsnorm(x, gw, 1e-6, out=xn)
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(20):
            layer.rmsnorm(x, gw, 1e-6, out=xn)
        g1.record()
        torch.cuda.synchronize()
        n_ms = g0.elapsed_time(g1) / 20
        yb = torch.empty_like(x)
        for _ in range(2):
            layer.block_forward(x, gw, 1e-6, out=yb)
        g0.record()
        for _ in range(max(2, args.steps // 4)):
            layer.block_forward(x, gw, 1e-6, out=yb)
        g1.record()
        torch.cuda.synchronize()
        b_ms = g0.elapsed_time(g1) / max(2, args.steps // 4)
        want = (x.float() + layer.forward(xn).float()).to(torch.bfloat16)
        nbytes = 2 * T * H * 2 + H * 2
        glue = {"rmsnorm_ms": round(n_ms, 4), "rmsnorm_gbs": round(nbytes / n_ms / 1e6, 1),
                "rmsnorm_frac_of_hbm": round(nbytes / n_ms / 1e6 / hbm, 3), "block_ms": round(b_ms, 3),
                "block_equals_norm_forward_add": bool(torch.equal(yb.view(torch.int16), want.view(torch.int16))),
                "note": "block = hidden + moe(rmsnorm(hidden)); rmsnorm moves T*H*2 bytes in and out"}
    # ---- checkpoint ingest: safetensors shard (page cache) -> pinned staging -> packed expert buffer ----
    ing = None
    if world == 1 and args.ingest:
        import tempfile
        from moe_gen_b200 import ingest as ING
        with tempfile.TemporaryDirectory() as td:
            path = os.path.join(td, "model-00001-of-00001.safetensors")
            write_layer_checkpoint(name, path, device, args.zipf)
            fresh = build_layer(name, device, zipf=args.zipf, load=False)
            ck = ING.Checkpoint(path)
            ING.load_moe_layer(fresh, ck, 0)                      # first pass warms the page cache
            st_ = ING.load_moe_layer(fresh, ck, 0)
            ck.close()
            same = bool(torch.equal(fresh.packed, layer.packed))
            yi = fresh.forward(x)
            ing = {"gb_per_s": round(st_["gb_per_s"], 2), "seconds": round(st_["seconds"], 3), "bytes": st_["bytes"],
                   "packed_equals_direct_load": same,
                   "forward_equals": bool(torch.equal(yi.view(torch.int16), y.view(torch.int16))),
                   "note": "file in the page cache; 8 copy threads into pinned staging, H2D and packing overlapped"}
            del fresh
    # ---- expert weights streamed from pinned host memory, group by group, beside the GEMMs ----
    streamed = None
    if world == 1 and args.stream_groups > 0:
        from moe_gen_b200.stream import StreamedMoELayer
        Hh, Ii, Ee, kk, Iss, Gg, keep, gating, norm, scale, wfmt, comb = WORKLOADS[name][:12]
        sl = StreamedMoELayer(group_experts=Ee // args.stream_groups, slots=2, device=device, hidden=Hh, inter=Ii,
                              n_experts=Ee, top_k=kk, inter_shared=Iss, n_group=Gg, topk_group=keep, gating=gating,
                              norm_topk_prob=norm, routed_scale=scale, weight_format=wfmt, combine_mode=comb)
        sl.set_router(*router_tensors(name, device, args.zipf))
        if Iss:
            sl.load_shared(*expert_tensors(name, device, -1))
        for e in range(Ee):
            ws_ = expert_tensors(name, device, e)
            if wfmt == 1:
                sl.load_expert(e, ws_[0][0], ws_[1][0], ws_[2][0], (ws_[0][1], ws_[1][1], ws_[2][1]))
            else:
                sl.load_expert(e, *ws_)
        for _ in range(2):
            ys = sl.forward(x)
        torch.cuda.synchronize()
        n_s = max(2, args.steps // 4)
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(n_s):
            ys = sl.forward(x)
        s1.record()
        torch.cuda.synchronize()
        s_ms = s0.elapsed_time(s1) / n_s
        moved = sl._expert_bytes() * sl.groups
        streamed = {"groups": sl.groups, "slots": sl.slots, "ms_per_step": round(s_ms, 3),
                    "tokens_per_s": round(T / (s_ms * 1e-3), 1), "h2d_bytes_per_step": moved,
                    "h2d_gb_per_s": round(moved / s_ms / 1e6, 2),
                    "equals_resident_path": bool(torch.equal(ys.view(torch.int16), y.view(torch.int16))),
                    "note": "expert weights cross PCIe on every step; the copy of a group overlaps the previous group's GEMMs"}
        sl.close()
        del sl
    eager = None
    if world == 1 and not args.no_eager_baseline:
        if hasattr(layer, "_ws"):
            layer._ws, layer._ws_tokens = None, -1          # make room: the eager layer keeps its own copies
        torch.cuda.empty_cache()
        eager, y_eager = cuda_eager_baseline(name, x, args.zipf)
        eager["rel_l2_of_this_library_vs_eager_bf16"] = float(
            (y.float() - y_eager.float()).norm() / y_eager.float().norm())
        del y_eager
        torch.cuda.empty_cache()
    cpu = None
    if not args.no_cpu_baseline:
        r = cpu_reference(name, args.cpu_sample_tokens, 2, 1, args.zipf)
        cpu = {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["cores"], "kind": "port",
               "sample": r["sample"]}

    out = {"metric": "MoE-layer tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
           "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config, "clocks": clocks,
           "e2e": e2e, "gpu_launches": launches * args.steps, "roofline": roofline, "cpu_baseline": cpu,
           "stages": stages, "check": check, "ep_load": ep_load, "glue": glue, "ingest": ing, "streamed": streamed,
           "other_configs": others, "cuda_eager_baseline": eager,
           "layer_tflops": (alg["gemm1_flops"] + alg["gemm2_flops"] + alg["shared_flops"] + alg["gate_flops"])
           / (ms_per_step * 1e-3) / 1e12 / world}
    print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
