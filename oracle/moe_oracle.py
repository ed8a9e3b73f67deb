"""CPU oracle for the MoE-layer path (TEST INFRASTRUCTURE, not product code).

This file restates, with plain torch CPU ops, the arithmetic of the reference's
MoE layer so that the CUDA path can be checked against it.  Only tests, the
smoke check and the CPU-baseline leg of the benchmark may import it; the
library itself never does.

Reference functions followed (paths inside the MoE-Gen project):

* gate logits + softmax scoring + greedy / group-limited top-k:
  moe_gen/models/deepseek/deepseekv2/modeling_deepseek_v2.py:483-533
* sigmoid scoring + correction bias + noaux_tc group top-k:
  moe_gen/models/deepseek/deepseekv3/modeling_deepseek_v3.py:500-561
* histogram / sort / gather (permute), expert loop, unpermute + combine:
  modeling_deepseek_v2.py:670-758, modeling_deepseek_v3.py:628-711
* SwiGLU expert: modeling_deepseek_v2.py:449-453, modeling_deepseek_v3.py:463-467
* shared-expert add: modeling_deepseek_v2.py:666-667, modeling_deepseek_v3.py:624-625
* FP8 128x128 block de-quantisation: moe_gen/models/Wrapper.py:109-138
* FP8 block quantisation recipe: deepseekv3_initializer.py:191-205
* Mixtral block: third-party transformers==4.42.0 (requirements.txt:8),
  MixtralSparseMoeBlock.forward.  Its source is not part of the reference
  tree, so the Mixtral functions below restate the published algorithm
  (softmax in fp32 over all experts, top-2, renormalise over the chosen two,
  cast to the activation dtype, per-expert SwiGLU scaled by the weight and
  index-added in ascending expert order).  PARITY UNPINNED for Mixtral: the
  reference holds no test or vector at that boundary; the restatement is only
  cross-checked against the transformers release installed next to torch.

Pinning: every DeepSeek function here is compared with the reference modules
themselves (imported from the reference tree) by tests/golden/make_golden.py,
which also writes the fixtures that tests/test_oracle_golden.py replays.

Canonical choices where the reference is under-specified
(torch.topk(sorted=False) and argsort() without stable=True):
  * top-k order: score descending, ties -> lower expert id;
  * permutation: experts ascending, tokens ascending inside an expert.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

# gating modes (values shared with include/moegen_b200.h)
GATE_SOFTMAX_GREEDY = 0      # DeepSeek-V2 "greedy"
GATE_SOFTMAX_GROUP_MAX = 1   # DeepSeek-V2 "group_limited_greedy"
GATE_SIGMOID_NOAUX_TC = 2    # DeepSeek-V3 "noaux_tc"
GATE_SOFTMAX_TOPK_RENORM = 3 # Mixtral: softmax, top-k, renormalise

# combine modes
COMBINE_FP32 = 0             # V3: fp32 products and sum, one rounding
COMBINE_BF16_PROD = 1        # V2: bf16 weight, bf16-rounded products, fp32 sum
COMBINE_BF16_SEQ = 2         # Mixtral: bf16 products index-added one by one

WEIGHT_BF16 = 0
WEIGHT_FP8_BLOCK128 = 1


@dataclass
class LayerSpec:
    hidden: int
    inter: int
    n_experts: int
    top_k: int
    inter_shared: int = 0
    n_group: int = 1
    topk_group: int = 1
    gating: int = GATE_SOFTMAX_GREEDY
    norm_topk_prob: bool = False
    routed_scale: float = 1.0
    weight_format: int = WEIGHT_BF16
    combine_mode: int = COMBINE_FP32
    name: str = ""


# ----------------------------------------------------------------------------
# named configurations (the five workloads the benchmark and tests refer to)
# ----------------------------------------------------------------------------
def named_spec(name: str) -> LayerSpec:
    if name == "v2lite":
        return LayerSpec(2048, 1408, 64, 6, 2816, 1, 1, GATE_SOFTMAX_GREEDY, False, 1.0,
                         WEIGHT_BF16, COMBINE_BF16_PROD, name)
    if name == "mixtral8x7b":
        return LayerSpec(4096, 14336, 8, 2, 0, 1, 1, GATE_SOFTMAX_TOPK_RENORM, True, 1.0,
                         WEIGHT_BF16, COMBINE_BF16_SEQ, name)
    if name == "v2_236b":
        return LayerSpec(5120, 1536, 160, 6, 3072, 8, 3, GATE_SOFTMAX_GROUP_MAX, False, 16.0,
                         WEIGHT_BF16, COMBINE_BF16_PROD, name)
    if name == "v3":
        return LayerSpec(7168, 2048, 256, 8, 2048, 8, 4, GATE_SIGMOID_NOAUX_TC, True, 2.5,
                         WEIGHT_FP8_BLOCK128, COMBINE_FP32, name)
    raise KeyError(name)


# ----------------------------------------------------------------------------
# gating
# ----------------------------------------------------------------------------
def gate_logits(x: torch.Tensor, gate_w: torch.Tensor, bf16_out: bool = False) -> torch.Tensor:
    """fp32 logits = x.float() @ W.float().T  (v2:484-492, v3:501-508).

    bf16_out=True is the Mixtral router: a bf16 nn.Linear whose output is
    rounded to bf16 before the fp32 softmax; returned widened to fp32."""
    x2 = x.reshape(-1, x.shape[-1])
    if bf16_out:
        return F.linear(x2, gate_w, None).to(torch.float32)
    return F.linear(x2.to(torch.float32), gate_w.to(torch.float32), None)


def topk_lower_id(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Canonical top-k: score descending, equal scores -> lower index first."""
    return torch.sort(scores, dim=-1, descending=True, stable=True).indices[:, :k]


def _mask_groups(scores: torch.Tensor, group_scores: torch.Tensor, topk_group: int) -> torch.Tensor:
    """Keep the topk_group best groups, set every other candidate to 0.0
    (not -inf: v2:509-523, v3:531-543)."""
    T, E = scores.shape
    G = group_scores.shape[1]
    gidx = topk_lower_id(group_scores, topk_group)
    gmask = torch.zeros_like(group_scores).scatter_(1, gidx, 1.0).bool()
    return scores.view(T, G, E // G).masked_fill(~gmask.unsqueeze(-1), 0.0).view(T, E)


def route(spec: LayerSpec, logits: torch.Tensor, bias: Optional[torch.Tensor] = None
          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Scores + top-k from fp32 logits [T,E] -> (idx int64 [T,k], weight fp32 [T,k]).

    Slot order is canonical (selection score descending, ties -> lower id)."""
    T, E = logits.shape
    k = spec.top_k
    if spec.gating in (GATE_SOFTMAX_GREEDY, GATE_SOFTMAX_GROUP_MAX, GATE_SOFTMAX_TOPK_RENORM):
        s = logits.softmax(dim=-1, dtype=torch.float32)
        if spec.gating == GATE_SOFTMAX_GROUP_MAX:
            gs = s.view(T, spec.n_group, -1).max(dim=-1).values            # v2:506-508
            choice = _mask_groups(s, gs, spec.topk_group)
        else:
            choice = s
        idx = topk_lower_id(choice, k)
        w = choice.gather(1, idx)                                           # v2:501-526 (values of topk)
        if spec.gating == GATE_SOFTMAX_TOPK_RENORM:
            w = w / w.sum(dim=-1, keepdim=True)                             # Mixtral renormalisation
        elif k > 1 and spec.norm_topk_prob:
            w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)                   # v2:529-531
        else:
            w = w * spec.routed_scale                                       # v2:532-533
        return idx, w
    if spec.gating == GATE_SIGMOID_NOAUX_TC:
        s = logits.sigmoid()                                                # v3:509-510
        c = s + bias.to(torch.float32).unsqueeze(0)                         # v3:519-521
        gs = c.view(T, spec.n_group, -1).topk(2, dim=-1)[0].sum(dim=-1)     # v3:522-526
        choice = _mask_groups(c, gs, spec.topk_group)
        idx = topk_lower_id(choice, k)
        w = s.gather(1, idx)                                                # v3:547 (un-biased)
        if k > 1 and spec.norm_topk_prob:
            w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)                   # v3:553-556
        w = w * spec.routed_scale                                           # v3:557-559 (always)
        return idx, w
    raise ValueError(spec.gating)


def kth_gap(spec: LayerSpec, logits: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per token: selection score of the k-th pick minus that of the (k+1)-th
    candidate.  Tokens whose gap is ~0 are ties the reference resolves
    arbitrarily; parity tests exempt them."""
    T, E = logits.shape
    if spec.gating == GATE_SIGMOID_NOAUX_TC:
        s = logits.sigmoid()
        c = s + bias.to(torch.float32).unsqueeze(0)
        gs = c.view(T, spec.n_group, -1).topk(2, dim=-1)[0].sum(dim=-1)
        choice = _mask_groups(c, gs, spec.topk_group)
        gsort = gs.sort(dim=-1, descending=True).values
        ggap = gsort[:, spec.topk_group - 1] - gsort[:, spec.topk_group] if spec.topk_group < spec.n_group else None
    else:
        s = logits.softmax(dim=-1, dtype=torch.float32)
        ggap = None
        if spec.gating == GATE_SOFTMAX_GROUP_MAX:
            gs = s.view(T, spec.n_group, -1).max(dim=-1).values
            choice = _mask_groups(s, gs, spec.topk_group)
            gsort = gs.sort(dim=-1, descending=True).values
            ggap = gsort[:, spec.topk_group - 1] - gsort[:, spec.topk_group]
        else:
            choice = s
    srt = choice.sort(dim=-1, descending=True).values
    gap = srt[:, spec.top_k - 1] - srt[:, spec.top_k] if spec.top_k < E else torch.full((T,), float("inf"))
    # relative to the magnitude of the k-th score
    gap = gap / srt[:, spec.top_k - 1].abs().clamp_min(1e-30)
    if ggap is not None:
        gap = torch.minimum(gap, ggap / gsort[:, spec.topk_group - 1].abs().clamp_min(1e-30))
    return gap


def canonical_sets(idx: torch.Tensor, w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sort each token's picks by expert id (weights follow)."""
    o = idx.sort(dim=-1)
    return o.values, w.gather(1, o.indices)


# ----------------------------------------------------------------------------
# permute plan
# ----------------------------------------------------------------------------
def permute_plan(topk_idx: torch.Tensor, n_experts: int):
    """Histogram + stable sort of the flattened picks (v3:630-635).

    Returns counts [E] int64, offsets [E+1] int64 (exclusive scan),
    order [R] int64 (flattened (token*k+slot) index of each sorted row) and
    src_token [R] = order // k."""
    T, k = topk_idx.shape
    flat = topk_idx.reshape(-1)
    counts = torch.bincount(flat, minlength=n_experts)
    offsets = torch.zeros(n_experts + 1, dtype=torch.int64)
    offsets[1:] = counts.cumsum(0).cpu()          # read on the host (the reference's .cpu() at v3:673)
    order = flat.argsort(stable=True)
    return counts, offsets, order, order // k


# ----------------------------------------------------------------------------
# experts
# ----------------------------------------------------------------------------
def swiglu_mlp(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) with bias-free linears, in the dtype of the
    operands (v2:449-453).  bf16 operands reproduce the module's roundings;
    fp32 operands give the fp32-accumulated gold."""
    return F.linear(F.silu(F.linear(x, wg)) * F.linear(x, wu), wd)


def quantize_fp8_block128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-128x128-block e4m3 quantisation, scale = amax/448 (fp32)
    (recipe of deepseekv3_initializer.py:191-205)."""
    m, n = w.shape
    mp, np_ = (m + 127) // 128 * 128, (n + 127) // 128 * 128
    wp = torch.zeros(mp, np_, dtype=w.dtype)
    wp[:m, :n] = w
    v = wp.view(mp // 128, 128, np_ // 128, 128)
    amax = v.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    q = (v * (448.0 / amax)).to(torch.float8_e4m3fn)
    return q.view(mp, np_)[:m, :n].contiguous(), (amax / 448.0).view(mp // 128, np_ // 128)


def dequantize_fp8_block128(q: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    """bf16(float(q) * scale[r/128][c/128])  (Wrapper.py:109-138)."""
    rows, cols = q.shape
    w = q.to(torch.float32)
    s = scale_inv.repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)[:rows, :cols]
    return (w * s).to(torch.bfloat16)


# ----------------------------------------------------------------------------
# combine
# ----------------------------------------------------------------------------
def combine(spec: LayerSpec, rows_by_slot: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor
            ) -> torch.Tensor:
    """rows_by_slot: [T,k,H] bf16 expert outputs in the slot order of topk_idx."""
    if spec.combine_mode == COMBINE_FP32:                                   # v3:704-710
        return (rows_by_slot.float() * topk_w.unsqueeze(-1)).sum(dim=1).to(rows_by_slot.dtype)
    if spec.combine_mode == COMBINE_BF16_PROD:                              # v2:746-757
        w = topk_w.to(rows_by_slot.dtype)
        return rows_by_slot.clone().mul_(w.unsqueeze(-1)).sum(dim=1).to(rows_by_slot.dtype)
    if spec.combine_mode == COMBINE_BF16_SEQ:                               # Mixtral index_add order
        T, k, H = rows_by_slot.shape
        w = topk_w.to(rows_by_slot.dtype)
        order = topk_idx.argsort(dim=-1, stable=True)                       # experts ascending
        y = torch.zeros(T, H, dtype=rows_by_slot.dtype, device=rows_by_slot.device)
        ar = torch.arange(T, device=rows_by_slot.device)
        for j in range(k):
            sel = order[:, j]
            r = rows_by_slot[ar, sel]
            y = y + r * w[ar, sel].unsqueeze(-1)
        return y
    raise ValueError(spec.combine_mode)


# ----------------------------------------------------------------------------
# whole layer
# ----------------------------------------------------------------------------
@dataclass
class LayerWeights:
    gate_w: torch.Tensor                       # [E,H] bf16
    bias: Optional[torch.Tensor]               # [E] fp32 (V3) or None
    w_gate: List[torch.Tensor] = field(default_factory=list)   # E x [I,H] bf16 (de-quantised if FP8)
    w_up: List[torch.Tensor] = field(default_factory=list)
    w_down: List[torch.Tensor] = field(default_factory=list)   # E x [H,I]
    shared: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None  # ([Is,H],[Is,H],[H,Is])
    # FP8 originals (None for bf16 layers): lists of (q, scale_inv)
    q_gate: Optional[list] = None
    q_up: Optional[list] = None
    q_down: Optional[list] = None


def make_inputs(spec: LayerSpec, T: int, seed: int, zipf_alpha: float = 0.0):
    """Seeded synthetic tensors.  Order of draws is fixed: x, gate W, bias,
    experts 0..E-1 (gate, up, down), shared (gate, up, down).

    zipf_alpha > 0 biases the router: hidden column 0 is set to 1.0 and
    gate_w[:,0] to log Zipf pmf over a seeded expert permutation, which adds a
    per-expert constant to every token's logits through the gate product."""
    g = torch.Generator().manual_seed(seed)
    H, I, E = spec.hidden, spec.inter, spec.n_experts
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    gate_w = (torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16)
    bias = (torch.randn(E, generator=g) * 0.01) if spec.gating == GATE_SIGMOID_NOAUX_TC else None
    W = LayerWeights(gate_w, bias)
    fp8 = spec.weight_format == WEIGHT_FP8_BLOCK128
    if fp8:
        W.q_gate, W.q_up, W.q_down = [], [], []
    for _ in range(E):
        mats = [(torch.randn(I, H, generator=g) * 0.02).to(torch.bfloat16),
                (torch.randn(I, H, generator=g) * 0.02).to(torch.bfloat16),
                (torch.randn(H, I, generator=g) * 0.02).to(torch.bfloat16)]
        if fp8:
            qs = [quantize_fp8_block128(m) for m in mats]
            W.q_gate.append(qs[0]); W.q_up.append(qs[1]); W.q_down.append(qs[2])
            mats = [dequantize_fp8_block128(q, s) for q, s in qs]
        W.w_gate.append(mats[0]); W.w_up.append(mats[1]); W.w_down.append(mats[2])
    if spec.inter_shared:
        Is = spec.inter_shared
        W.shared = ((torch.randn(Is, H, generator=g) * 0.02).to(torch.bfloat16),
                    (torch.randn(Is, H, generator=g) * 0.02).to(torch.bfloat16),
                    (torch.randn(H, Is, generator=g) * 0.02).to(torch.bfloat16))
    if zipf_alpha > 0.0:
        perm = torch.randperm(E, generator=g)
        pmf = 1.0 / torch.arange(1, E + 1, dtype=torch.float64) ** zipf_alpha
        pmf = pmf / pmf.sum()
        b = pmf.log()
        b = (b - b.mean()).to(torch.float32)
        col = torch.empty(E)
        col[perm] = b
        x[:, 0] = 1.0
        W.gate_w[:, 0] = col.to(torch.bfloat16)
    return x, W


def layer_forward(spec: LayerSpec, x: torch.Tensor, W: LayerWeights, gold_fp32: bool = False,
                  dequant_per_call: bool = False) -> Dict[str, torch.Tensor]:
    """Whole layer on CPU.  gold_fp32=False follows the reference module as
    shipped (bf16 experts); gold_fp32=True is the same module with fp32
    parameters and input, i.e. the fp32-accumulated output the tolerance is
    measured against.  Routing is fp32 in both.

    dequant_per_call=True (FP8 layers): every expert call first de-quantises its three
    matrices from W.q_* as the reference's Expert_Wrapper does on each forward
    (moe_gen/models/Wrapper.py:481-491) instead of reading the bf16 copies in W.w_*;
    the values are the same, only the work is."""
    T, H = x.shape
    logits = gate_logits(x, W.gate_w, bf16_out=(spec.gating == GATE_SOFTMAX_TOPK_RENORM))
    idx, w = route(spec, logits, W.bias)
    counts, offsets, order, src = permute_plan(idx, spec.n_experts)
    cd = torch.float32 if gold_fp32 else torch.bfloat16
    xs = x.to(cd)[src]                                                      # sorted_tokens
    outs = torch.empty(xs.shape[0], H, dtype=cd, device=x.device)
    for e in range(spec.n_experts):                                         # v3:675-691
        a, b = int(offsets[e]), int(offsets[e + 1])
        if b > a:
            if dequant_per_call and W.q_gate is not None:
                wg, wu, wd = (dequantize_fp8_block128(*W.q_gate[e]), dequantize_fp8_block128(*W.q_up[e]),
                              dequantize_fp8_block128(*W.q_down[e]))
            else:
                wg, wu, wd = W.w_gate[e], W.w_up[e], W.w_down[e]
            outs[a:b] = swiglu_mlp(xs[a:b], wg.to(cd), wu.to(cd), wd.to(cd))
    back = torch.empty_like(outs)
    back[order] = outs                                                      # new_x[idxs] = outs
    rows = back.view(T, spec.top_k, H)
    if gold_fp32:
        y = (rows * w.unsqueeze(-1)).sum(dim=1)
    else:
        y = combine(spec, rows, idx, w)
    if W.shared is not None:
        y = y + swiglu_mlp(x.to(cd), W.shared[0].to(cd), W.shared[1].to(cd), W.shared[2].to(cd))
    return {"y": y, "logits": logits, "topk_idx": idx, "topk_w": w, "counts": counts,
            "offsets": offsets, "order": order, "src_token": src}


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """DeepseekV3RMSNorm.forward (modeling_deepseek_v3.py:125-150; V2 has the same class):
    fp32 statistics, the normalised value cast back to the input dtype, then multiplied by
    the weight (bf16 in a model moved to bfloat16, so the product rounds to bf16 once more)."""
    h = x.to(torch.float32)
    variance = h.pow(2).mean(-1, keepdim=True)
    h = h * torch.rsqrt(variance + eps)
    return weight * h.to(x.dtype)


def block_forward(spec: LayerSpec, hidden: torch.Tensor, norm_w: torch.Tensor, eps: float, W: LayerWeights,
                  gold_fp32: bool = False) -> Dict[str, torch.Tensor]:
    """The decoder layer's second half (modeling_deepseek_v3.py:1361-1365): residual = h;
    h = post_attention_layernorm(h); h = mlp(h); h = residual + h.  gold_fp32 as in layer_forward
    (fp32 parameters and input, the normalisation included)."""
    if gold_fp32:
        xn = rmsnorm(hidden.float(), norm_w.float(), eps)
        out = layer_forward(spec, xn, W, gold_fp32=True)
        return {"y": hidden.float() + out["y"], "x_norm": xn, "moe": out}
    xn = rmsnorm(hidden, norm_w, eps)
    out = layer_forward(spec, xn, W)
    return {"y": hidden + out["y"], "x_norm": xn, "moe": out}


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double(); b = b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
