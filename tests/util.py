"""Helpers shared by the tests: build a native layer from the oracle's synthetic inputs."""
import os

import numpy as np
import torch

from oracle import moe_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def make_layer(spec: O.LayerSpec, W: O.LayerWeights, device="cuda:0", ep_rank=0, ep_size=1):
    from moe_gen_b200 import MoELayer
    layer = MoELayer(hidden=spec.hidden, inter=spec.inter, n_experts=spec.n_experts, top_k=spec.top_k,
                     inter_shared=spec.inter_shared, n_group=spec.n_group, topk_group=spec.topk_group,
                     gating=spec.gating, norm_topk_prob=spec.norm_topk_prob, routed_scale=spec.routed_scale,
                     weight_format=spec.weight_format, combine_mode=spec.combine_mode,
                     ep_rank=ep_rank, ep_size=ep_size, device=device)
    layer.set_router(W.gate_w, W.bias)
    fp8 = spec.weight_format == O.WEIGHT_FP8_BLOCK128
    for i in range(layer.e_local if W.w_gate else 0):   # router-only tests carry no expert weights
        e = layer.expert_lo + i
        if fp8:
            (g, gs), (u, us), (d, ds) = W.q_gate[e], W.q_up[e], W.q_down[e]
            layer.load_expert(i, g, u, d, (gs, us, ds))
        else:
            layer.load_expert(i, W.w_gate[e], W.w_up[e], W.w_down[e])
    if W.shared is not None:
        layer.load_shared(*W.shared)
    return layer


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)
