"""Drop-in replacement of the MoE module forwards.

`patch_moe_module(module)` takes an existing instance of the reference's
DeepseekV2MoE (moe_gen/models/deepseek/deepseekv2/modeling_deepseek_v2.py:592-668),
DeepseekV3MoE (.../deepseekv3/modeling_deepseek_v3.py:564-626) or of transformers'
MixtralSparseMoeBlock (referenced at moe_gen/models/mixtral/Mixtral_Initializer.py:31-35),
copies its weights once into the packed device buffer and replaces `module.forward`
by a function that calls the native library.  Input and output keep the module's
contract: hidden_states [B,S,H] bf16 on the layer's CUDA device -> same shape.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import lib as L
from .layer import MoELayer


def _unwrap(expert):
    # Expert_Wrapper keeps the nn.Module under `.module` (moe_gen/models/Wrapper.py:449)
    return getattr(expert, "module", expert)


def _lin_weight(lin):
    w = lin.weight
    s = getattr(lin, "weight_scale_inv", None)
    return w, s


def layer_from_deepseek(module, device=None, ep_rank: int = 0, ep_size: int = 1) -> MoELayer:
    cfg = module.config
    gate = module.gate
    scoring = getattr(cfg, "scoring_func", "softmax")
    method = getattr(cfg, "topk_method", "greedy")
    if scoring == "sigmoid" and method == "noaux_tc":
        gating, combine = L.GATE_SIGMOID_NOAUX_TC, L.COMBINE_FP32
    elif scoring == "softmax" and method == "greedy":
        gating, combine = L.GATE_SOFTMAX_GREEDY, L.COMBINE_BF16_PROD
    elif scoring == "softmax" and method == "group_limited_greedy":
        gating, combine = L.GATE_SOFTMAX_GROUP_MAX, L.COMBINE_BF16_PROD
    else:
        # same failure as the reference gate (modeling_deepseek_v3.py:548-551)
        raise NotImplementedError(f"insupportable TopK function for MoE gating: {scoring}/{method}")
    n_shared = getattr(cfg, "n_shared_experts", None) or 0
    experts = [_unwrap(e) for e in module.experts]
    first = next(e for e in experts if e is not None)
    fp8 = first.gate_proj.weight.dtype == torch.float8_e4m3fn
    dev = device if device is not None else first.gate_proj.weight.device
    layer = MoELayer(hidden=cfg.hidden_size, inter=cfg.moe_intermediate_size, n_experts=cfg.n_routed_experts,
                     top_k=cfg.num_experts_per_tok, inter_shared=n_shared * cfg.moe_intermediate_size,
                     n_group=getattr(cfg, "n_group", 1) or 1, topk_group=getattr(cfg, "topk_group", 1) or 1,
                     gating=gating, norm_topk_prob=bool(cfg.norm_topk_prob),
                     routed_scale=float(cfg.routed_scaling_factor),
                     weight_format=L.WEIGHT_FP8_BLOCK128 if fp8 else L.WEIGHT_BF16, combine_mode=combine,
                     ep_rank=ep_rank, ep_size=ep_size, device=dev)
    layer.set_router(gate.weight, getattr(gate, "e_score_correction_bias", None))
    for i in range(layer.e_local):
        ex = experts[layer.expert_lo + i]
        (g, gs), (u, us), (d, ds) = _lin_weight(ex.gate_proj), _lin_weight(ex.up_proj), _lin_weight(ex.down_proj)
        layer.load_expert(i, g, u, d, (gs, us, ds) if fp8 else None)
    if n_shared:
        sh = _unwrap(module.shared_experts)
        mats = []
        for lin in (sh.gate_proj, sh.up_proj, sh.down_proj):
            w, s = _lin_weight(lin)
            mats.append(layer.dequant_fp8(w, s) if w.dtype == torch.float8_e4m3fn else w)
        layer.load_shared(*mats)
    return layer


def layer_from_mixtral(module, device=None) -> MoELayer:
    gate_w = module.gate.weight
    E, H = gate_w.shape
    top_k = getattr(module, "top_k", None) or getattr(module.gate, "top_k", 2)
    experts = module.experts
    if hasattr(experts, "gate_up_proj"):           # fused layout of newer transformers releases
        gu, dn = experts.gate_up_proj, experts.down_proj
        I = dn.shape[2]
        mats = [(gu[e, :I], gu[e, I:], dn[e]) for e in range(E)]
    else:                                          # transformers 4.42: per-expert w1, w3, w2
        mats = [(ex.w1.weight, ex.w3.weight, ex.w2.weight) for ex in (_unwrap(e) for e in experts)]
        I = mats[0][0].shape[0]
    dev = device if device is not None else gate_w.device
    layer = MoELayer(hidden=H, inter=I, n_experts=E, top_k=top_k, gating=L.GATE_SOFTMAX_TOPK_RENORM,
                     norm_topk_prob=True, routed_scale=1.0, combine_mode=L.COMBINE_BF16_SEQ, device=dev)
    layer.set_router(gate_w)
    for e, (g, u, d) in enumerate(mats):
        layer.load_expert(e, g.to(torch.bfloat16), u.to(torch.bfloat16), d.to(torch.bfloat16))
    return layer


def patch_moe_module(module, device=None, return_router_logits: Optional[bool] = None):
    """Replaces module.forward in place and returns the MoELayer that now serves it."""
    name = type(module).__name__
    if name in ("DeepseekV2MoE", "DeepseekV3MoE"):
        layer = layer_from_deepseek(module, device)

        def forward(hidden_states):
            if module.training:
                raise RuntimeError("moe_gen_b200 implements the inference path (moe_infer) only")
            return layer.forward(hidden_states.contiguous())
    elif name == "MixtralSparseMoeBlock":
        layer = layer_from_mixtral(module, device)
        tuple_out = True if return_router_logits is None else return_router_logits

        def forward(hidden_states):
            hs = hidden_states.contiguous()
            y = layer.forward(hs)
            if not tuple_out:
                return y
            # transformers 4.42 returns (hidden_states, router_logits[T,E])
            return y, layer.gate_logits(hs.view(-1, layer.H)).to(hs.dtype)
    else:
        raise TypeError(f"unsupported module type {name}")
    module.forward = forward
    module._moegen_b200_layer = layer
    return layer


def patch_decoder_layer(decoder_layer, device=None) -> MoELayer:
    """Replaces the forward of a reference DeepseekV2/V3DecoderLayer whose `.mlp` is a MoE block
    (modeling_deepseek_v3.py:1302-1375).  Attention and its residual add stay as they are; the three
    steps behind them - post_attention_layernorm, mlp, residual add - become one call,
    `MoELayer.block_forward`, which normalises, runs the block and adds the residual inside the
    combine kernel, updating the hidden states in place.  Same arguments and return tuple as the
    reference's forward."""
    layer = patch_moe_module(decoder_layer.mlp, device)
    norm = decoder_layer.post_attention_layernorm
    eps = float(getattr(norm, "variance_epsilon", getattr(norm, "eps", 1e-6)))

    def forward(hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                output_attentions=False, use_cache=False, **kwargs):
        residual = hidden_states
        hidden_states = decoder_layer.input_layernorm(hidden_states)
        hidden_states, self_attn_weights, present_key_value = decoder_layer.self_attn(
            hidden_states=hidden_states, attention_mask=attention_mask, position_ids=position_ids,
            past_key_value=past_key_value, output_attentions=output_attentions, use_cache=use_cache, **kwargs)
        hidden_states = (residual + hidden_states).contiguous()
        w = norm.weight
        if w.dtype != torch.bfloat16 or w.device != hidden_states.device:
            w = w.detach().to(hidden_states.device, torch.bfloat16)
        hidden_states = layer.block_forward(hidden_states, w, eps, out=hidden_states)
        outputs = (hidden_states,)
        if output_attentions:
            outputs += (self_attn_weights,)
        if use_cache:
            outputs += (present_key_value,)
        return outputs

    decoder_layer.forward = forward
    return layer
