"""Generate the golden fixtures in this folder from the reference itself.

Run where the MoE-Gen reference tree is available; its root is passed with --reference
(or the MOEGEN_REFERENCE environment variable):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <MoE-Gen checkout>

What it does, per case:
  1. draws the seeded synthetic inputs (oracle.moe_oracle.make_inputs);
  2. loads them into the reference's own modules (DeepseekV2MoE / DeepseekV3MoE /
     MoEGate imported from the reference tree, run on CPU) and runs them;
  3. checks the oracle restatement against the reference output
     (routing sets exact, moe_infer bit-exact given the reference's own routing,
     layer output within a tight bound) and aborts on any mismatch;
  4. stores the reference's outputs (not the inputs: those are re-drawn from the
     seed; a digest of the inputs guards against generator drift) as .npz.

The fixtures are replayed by tests/test_oracle_golden.py (CPU) and by the GPU
parity tests.  Nothing here runs at test time.
"""
from __future__ import annotations

import argparse
import ast
import hashlib
import importlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import moe_oracle as O  # noqa: E402


def load_reference(ref_root: str):
    sys.path.insert(0, ref_root)
    import transformers.utils.import_utils as iu
    if not hasattr(iu, "is_torch_fx_available"):
        iu.is_torch_fx_available = lambda: False
    v2 = importlib.import_module("moe_gen.models.deepseek.deepseekv2.modeling_deepseek_v2")
    v3 = importlib.import_module("moe_gen.models.deepseek.deepseekv3.modeling_deepseek_v3")
    c2 = importlib.import_module("moe_gen.models.deepseek.deepseekv2.configuration_deepseek_v2")
    c3 = importlib.import_module("moe_gen.models.deepseek.deepseekv3.configuration_deepseek_v3")
    # the de-quantisation routine lives in Wrapper.py, whose module import pulls in
    # the native engine; evaluate just that one function from its source text
    src = open(os.path.join(ref_root, "moe_gen/models/Wrapper.py")).read()
    tree = ast.parse(src)
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "deepseek_v3_dequantization"][0]
    ns = {"torch": torch, "math": __import__("math")}
    exec(compile(ast.Module([fn], []), "Wrapper.py", "exec"), ns)
    return v2, v3, c2.DeepseekV2Config, c3.DeepseekV3Config, ns["deepseek_v3_dequantization"]


def digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().astype(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()


CASES = {
    # name: (spec, T, seed)
    "v2_greedy_small": (O.LayerSpec(256, 128, 64, 6, 256, 1, 1, O.GATE_SOFTMAX_GREEDY, False, 1.0,
                                    O.WEIGHT_BF16, O.COMBINE_BF16_PROD), 333, 10),
    "v2_group_small": (O.LayerSpec(256, 128, 160, 6, 256, 8, 3, O.GATE_SOFTMAX_GROUP_MAX, False, 16.0,
                                   O.WEIGHT_BF16, O.COMBINE_BF16_PROD), 200, 11),
    "v2_norm_small": (O.LayerSpec(256, 128, 32, 4, 0, 4, 2, O.GATE_SOFTMAX_GROUP_MAX, True, 3.0,
                                  O.WEIGHT_BF16, O.COMBINE_BF16_PROD), 129, 12),
    "v3_noaux_small_fp8": (O.LayerSpec(256, 128, 256, 8, 128, 8, 4, O.GATE_SIGMOID_NOAUX_TC, True, 2.5,
                                       O.WEIGHT_FP8_BLOCK128, O.COMBINE_FP32), 257, 13),
    "v3_noaux_small_bf16": (O.LayerSpec(512, 256, 64, 4, 256, 4, 2, O.GATE_SIGMOID_NOAUX_TC, True, 2.5,
                                        O.WEIGHT_BF16, O.COMBINE_FP32), 96, 14),
}

# whole-layer cases at the full size of a named configuration: the full routing and histogram are
# stored, of the outputs only SAMPLE_ROWS evenly spaced token rows (the fixture stays small)
FULL_CASES = {
    "v2lite_full": ("v2lite", 2048, 0),      # DeepSeek-V2-Lite layer exactly as the benchmark names it
}
SAMPLE_ROWS = 128

GATE_CASES = {
    # full-size gate shapes of the named configs, T=512
    "gate_v2lite": ("v2lite", 512, 0),
    "gate_v2_236b": ("v2_236b", 512, 2),
    "gate_v3": ("v3", 512, 3),
}


def build_ref_module(spec: O.LayerSpec, W: O.LayerWeights, v2, v3, C2, C3):
    common = dict(hidden_size=spec.hidden, moe_intermediate_size=spec.inter,
                  n_routed_experts=spec.n_experts, num_experts_per_tok=spec.top_k,
                  n_shared_experts=(spec.inter_shared // spec.inter) if spec.inter_shared else None,
                  n_group=spec.n_group, topk_group=spec.topk_group,
                  norm_topk_prob=spec.norm_topk_prob, routed_scaling_factor=spec.routed_scale)
    if spec.gating == O.GATE_SIGMOID_NOAUX_TC:
        m = v3.DeepseekV3MoE(C3(topk_method="noaux_tc", scoring_func="sigmoid", **common)).eval()
    else:
        tm = "greedy" if spec.gating == O.GATE_SOFTMAX_GREEDY else "group_limited_greedy"
        m = v2.DeepseekV2MoE(C2(topk_method=tm, **common)).eval()
    m.gate.weight.data = W.gate_w.clone()
    if W.bias is not None:
        m.gate.e_score_correction_bias.data = W.bias.clone()
    for e, ex in enumerate(m.experts):
        ex.gate_proj.weight.data = W.w_gate[e].clone()
        ex.up_proj.weight.data = W.w_up[e].clone()
        ex.down_proj.weight.data = W.w_down[e].clone()
    if W.shared is not None:
        m.shared_experts.gate_proj.weight.data = W.shared[0].clone()
        m.shared_experts.up_proj.weight.data = W.shared[1].clone()
        m.shared_experts.down_proj.weight.data = W.shared[2].clone()
    return m


def write_full_cases(v2, v3, C2, C3):
    for name, (cfg, T, seed) in FULL_CASES.items():
        spec = O.named_spec(cfg)
        x, W = O.make_inputs(spec, T, seed)
        m = build_ref_module(spec, W, v2, v3, C2, C3)
        with torch.no_grad():
            xin = x.view(1, T, spec.hidden)
            gout = m.gate(xin)
            ridx, rw = gout[0], gout[1]
            y_ref = m(xin).view(T, spec.hidden)
            m32 = build_ref_module(spec, W, v2, v3, C2, C3).float()
            if W.bias is not None:
                m32.gate.e_score_correction_bias.data = W.bias.clone()
            y_gold = m32(xin.float()).view(T, spec.hidden)
        out = O.layer_forward(spec, x, W)
        gold = O.layer_forward(spec, x, W, gold_fp32=True)
        ri, rwc = O.canonical_sets(ridx, rw)
        oi, owc = O.canonical_sets(out["topk_idx"], out["topk_w"])
        assert torch.equal(ri, oi), f"{name}: routing sets differ"
        assert (rwc - owc).abs().max() <= 2e-7 * max(1.0, spec.routed_scale), f"{name}: weights differ"
        cnt = torch.bincount(ridx.view(-1), minlength=spec.n_experts)
        assert torch.equal(cnt, out["counts"])
        r_bf = O.rel_l2(out["y"].float(), y_ref.float())
        r_gd = O.rel_l2(gold["y"], y_gold)
        assert r_bf < 2e-3 and r_gd < 1e-5, (name, r_bf, r_gd)
        rows = torch.linspace(0, T - 1, SAMPLE_ROWS).round().long()
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            T=T, seed=seed, input_digest=digest(x, W.gate_w, W.w_gate[0], W.w_down[-1]),
            topk_idx=ri.numpy().astype(np.int16), topk_w=rwc.numpy(), counts=cnt.numpy().astype(np.int32),
            rows=rows.numpy().astype(np.int32), y_ref_bf16_rows=bits(y_ref[rows]),
            y_gold_fp32_rows=y_gold[rows].numpy().astype(np.float32),
            ref_bf16_vs_gold=np.float64(O.rel_l2(y_ref.float(), y_gold)))
        print(f"{name}: ok  rel(oracle,ref)={r_bf:.2e} rel(oracle_gold,ref_gold)={r_gd:.2e} "
              f"ref_bf16_vs_gold={O.rel_l2(y_ref.float(), y_gold):.2e}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MOEGEN_REFERENCE"), required="MOEGEN_REFERENCE" not in os.environ)
    ap.add_argument("--only", default="", help="'block': write only the decoder-layer-glue fixture; "
                    "'full': only the full-size whole-layer fixtures")
    args = ap.parse_args()
    v2, v3, C2, C3, ref_dequant = load_reference(args.reference)
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    if args.only == "full":
        write_full_cases(v2, v3, C2, C3)
        return

    # ---- decoder-layer glue: the reference's RMSNorm in front of its V3 block, residual added after
    #      (modeling_deepseek_v3.py:1361-1365), on the inputs of the small bf16 V3 case
    spec, T, seed = CASES["v3_noaux_small_bf16"]
    hidden, W = O.make_inputs(spec, T, seed)
    g = torch.Generator().manual_seed(seed + 1000)
    norm_w = (1.0 + 0.1 * torch.randn(spec.hidden, generator=g)).to(torch.bfloat16)
    eps = 1e-6
    norm = v3.DeepseekV3RMSNorm(spec.hidden, eps=eps)
    norm.weight.data = norm_w.clone()
    m = build_ref_module(spec, W, v2, v3, C2, C3)
    with torch.no_grad():
        xn_ref = norm(hidden)
        y_blk = hidden + m(xn_ref.view(1, T, spec.hidden)).view(T, spec.hidden)
        m32 = build_ref_module(spec, W, v2, v3, C2, C3).float()
        m32.gate.e_score_correction_bias.data = W.bias.clone()
        norm32 = v3.DeepseekV3RMSNorm(spec.hidden, eps=eps)
        norm32.weight.data = norm_w.float()
        y_blk_gold = hidden.float() + m32(norm32(hidden.float()).view(1, T, spec.hidden)).view(T, spec.hidden)
    ob = O.block_forward(spec, hidden, norm_w, eps, W)
    assert xn_ref.dtype == torch.bfloat16 and torch.equal(ob["x_norm"], xn_ref), "rmsnorm restatement not bit-exact"
    r_blk = O.rel_l2(ob["y"].float(), y_blk.float())
    r_blk_gold = O.rel_l2(O.block_forward(spec, hidden, norm_w, eps, W, gold_fp32=True)["y"], y_blk_gold)
    assert r_blk < 2e-3 and r_blk_gold < 1e-5, (r_blk, r_blk_gold)
    np.savez_compressed(os.path.join(HERE, "block_v3_small.npz"), T=T, seed=seed, eps=eps,
                        input_digest=digest(hidden, norm_w, W.gate_w), norm_w=bits(norm_w),
                        x_norm_bf16=bits(xn_ref), y_block_bf16=bits(y_blk),
                        y_block_gold_fp32=y_blk_gold.numpy().astype(np.float32))
    print(f"block_v3_small: ok  rel(oracle,ref)={r_blk:.2e} rel(oracle_gold,ref_gold)={r_blk_gold:.2e}")
    if args.only == "block":
        return

    # ---- whole-layer cases -------------------------------------------------
    for name, (spec, T, seed) in CASES.items():
        x, W = O.make_inputs(spec, T, seed)
        if spec.weight_format == O.WEIGHT_FP8_BLOCK128:
            # the oracle's de-quantisation must equal the reference's bit for bit
            for qs, ws in ((W.q_gate, W.w_gate), (W.q_up, W.w_up), (W.q_down, W.w_down)):
                for (q, s), w in zip(qs, ws):
                    assert torch.equal(ref_dequant(q, s), w), f"{name}: dequant differs"
        m = build_ref_module(spec, W, v2, v3, C2, C3)
        with torch.no_grad():
            xin = x.view(1, T, spec.hidden)
            gout = m.gate(xin)
            ridx, rw = gout[0], gout[1]
            y_ref = m(xin).view(T, spec.hidden)
            y_infer = m.moe_infer(x, ridx, rw)
            # fp32 gold: same module, fp32 parameters and input
            m32 = build_ref_module(spec, W, v2, v3, C2, C3).float()
            if W.bias is not None:
                m32.gate.e_score_correction_bias.data = W.bias.clone()
            y_gold = m32(xin.float()).view(T, spec.hidden)
        out = O.layer_forward(spec, x, W)
        gold = O.layer_forward(spec, x, W, gold_fp32=True)
        # 1. routing sets identical, weights equal to fp32 rounding
        ri, rwc = O.canonical_sets(ridx, rw)
        oi, owc = O.canonical_sets(out["topk_idx"], out["topk_w"])
        assert torch.equal(ri, oi), f"{name}: routing sets differ"
        assert (rwc - owc).abs().max() <= 2e-7 * max(1.0, spec.routed_scale), f"{name}: weights differ"
        # 2. histogram identical
        cnt = torch.bincount(ridx.view(-1), minlength=spec.n_experts)
        assert torch.equal(cnt, out["counts"])
        # 3. moe_infer given the reference's routing: bit-exact
        order = ridx.view(-1).argsort(stable=True)
        src = order // spec.top_k
        outs = torch.empty(order.numel(), spec.hidden, dtype=torch.bfloat16)
        off = out["offsets"]
        for e in range(spec.n_experts):
            a, b = int(off[e]), int(off[e + 1])
            if b > a:
                outs[a:b] = O.swiglu_mlp(x[src[a:b]], W.w_gate[e], W.w_up[e], W.w_down[e])
        back = torch.empty_like(outs)
        back[order] = outs
        y2 = O.combine(spec, back.view(T, spec.top_k, spec.hidden), ridx, rw)
        assert torch.equal(y2, y_infer), f"{name}: moe_infer restatement not bit-exact"
        # 4. whole layer (oracle slot order differs from torch.topk's -> summation
        #    order of the k products may differ by an fp32 ulp before rounding)
        r_bf = O.rel_l2(out["y"].float(), y_ref.float())
        r_gd = O.rel_l2(gold["y"], y_gold)
        assert r_bf < 2e-3 and r_gd < 1e-5, (name, r_bf, r_gd)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            T=T, seed=seed, input_digest=digest(x, W.gate_w, W.w_gate[0], W.w_down[-1]),
            topk_idx=ri.numpy().astype(np.int16), topk_w=rwc.numpy(),
            counts=cnt.numpy().astype(np.int32),
            y_ref_bf16=bits(y_ref), y_gold_fp32=y_gold.numpy().astype(np.float32),
            ref_bf16_vs_gold=np.float64(O.rel_l2(y_ref.float(), y_gold)))
        print(f"{name}: ok  rel(oracle,ref)={r_bf:.2e} rel(oracle_gold,ref_gold)={r_gd:.2e} "
              f"ref_bf16_vs_gold={O.rel_l2(y_ref.float(), y_gold):.2e}")

    write_full_cases(v2, v3, C2, C3)

    # ---- gate-only cases at full gate shapes ---------------------------------
    for name, (cfg, T, seed) in GATE_CASES.items():
        spec = O.named_spec(cfg)
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(T, spec.hidden, generator=g).to(torch.bfloat16)
        gw = (torch.randn(spec.n_experts, spec.hidden, generator=g) * 0.02).to(torch.bfloat16)
        bias = torch.randn(spec.n_experts, generator=g) * 0.01 if spec.gating == O.GATE_SIGMOID_NOAUX_TC else None
        common = dict(hidden_size=spec.hidden, n_routed_experts=spec.n_experts,
                      num_experts_per_tok=spec.top_k, n_group=spec.n_group, topk_group=spec.topk_group,
                      norm_topk_prob=spec.norm_topk_prob, routed_scaling_factor=spec.routed_scale)
        if bias is not None:
            gate = v3.MoEGate(C3(**common)).eval()
            gate.e_score_correction_bias.data = bias.clone()
        else:
            tm = "greedy" if spec.gating == O.GATE_SOFTMAX_GREEDY else "group_limited_greedy"
            gate = v2.MoEGate(C2(topk_method=tm, **common)).eval()
        gate.weight.data = gw.clone()
        with torch.no_grad():
            gout = gate(x.view(1, T, -1))
        ri, rwc = O.canonical_sets(gout[0], gout[1])
        logits = O.gate_logits(x, gw)
        oi, owc = O.canonical_sets(*O.route(spec, logits, bias))
        assert torch.equal(ri, oi), f"{name}: routing sets differ"
        assert (rwc - owc).abs().max() <= 2e-7 * max(1.0, spec.routed_scale)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), T=T, seed=seed,
                            input_digest=digest(x, gw), topk_idx=ri.numpy().astype(np.int16),
                            topk_w=rwc.numpy())
        print(f"{name}: ok")


if __name__ == "__main__":
    main()
