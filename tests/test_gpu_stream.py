"""GPU: the layer whose expert weights are streamed from pinned host memory through a few group-sized
slots gives the same bits as the layer that keeps all experts resident."""
import pytest
import torch

from oracle import moe_oracle as O
from tests.util import make_layer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _streamed(spec, W, group, slots, routing_aware=False):
    from moe_gen_b200.stream import StreamedMoELayer
    lay = StreamedMoELayer(group_experts=group, slots=slots, routing_aware=routing_aware, device=DEV,
                           hidden=spec.hidden, inter=spec.inter, n_experts=spec.n_experts, top_k=spec.top_k,
                           inter_shared=spec.inter_shared, n_group=spec.n_group, topk_group=spec.topk_group,
                           gating=spec.gating, norm_topk_prob=spec.norm_topk_prob, routed_scale=spec.routed_scale,
                           weight_format=spec.weight_format, combine_mode=spec.combine_mode)
    lay.set_router(W.gate_w, W.bias)
    if W.shared is not None:
        lay.load_shared(*W.shared)
    fp8 = spec.weight_format == O.WEIGHT_FP8_BLOCK128
    for e in range(spec.n_experts):
        if fp8:
            (g, gs), (u, us), (d, ds) = W.q_gate[e], W.q_up[e], W.q_down[e]
            lay.load_expert(e, g, u, d, (gs, us, ds))
        else:
            lay.load_expert(e, W.w_gate[e], W.w_up[e], W.w_down[e])
    return lay


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("group,slots", [(4, 2), (2, 3), (16, 2)])
def test_streamed_layer_equals_resident_layer(built_lib, fp8, group, slots):
    spec = O.LayerSpec(256, 128, 16, 4, 128, 4, 2, O.GATE_SIGMOID_NOAUX_TC, True, 2.5,
                       O.WEIGHT_FP8_BLOCK128 if fp8 else O.WEIGHT_BF16, O.COMBINE_FP32)
    x, W = O.make_inputs(spec, 300, 23)
    want = make_layer(spec, W, DEV)
    got = _streamed(spec, W, group, slots)
    xd = x.to(DEV)
    y0 = want.forward(xd)
    for _ in range(2):                                   # twice: the slots are reused across forwards
        y1 = got.forward(xd)
        assert torch.equal(y0.view(torch.int16), y1.view(torch.int16))
    # and against the CPU oracle, not only against the resident layer
    assert O.rel_l2(y1.cpu().float(), O.layer_forward(spec, x, W, gold_fp32=True)["y"]) <= 1e-2
    assert got.layer.device_status() == (0, 0)
    assert got.last_groups_moved == spec.n_experts // group
    assert got.forward(xd[:0]).shape == (0, spec.hidden)


def test_routing_aware_streaming_skips_groups_without_rows(built_lib):
    spec = O.LayerSpec(256, 128, 16, 2, 0, combine_mode=O.COMBINE_FP32)
    x, W = O.make_inputs(spec, 3, 29)                    # 3 tokens x 2 picks reach at most 6 of 16 experts
    want = make_layer(spec, W, DEV)
    got = _streamed(spec, W, 2, 2, routing_aware=True)
    xd = x.to(DEV)
    assert torch.equal(want.forward(xd).view(torch.int16), got.forward(xd).view(torch.int16))
    idx, _ = want.gate_route(xd)[:2]
    groups_hit = len(set((idx.cpu().view(-1) // 2).tolist()))
    assert got.last_groups_moved == groups_hit < 8


def test_routing_aware_streaming_orders_the_copies_by_routed_rows(built_lib):
    """The groups travel in the order of their routed row counts (largest first, ties by group id), as read
    from the device-side plan; the result still equals the resident layer and the oracle."""
    spec = O.LayerSpec(256, 128, 16, 4, 128, 4, 2, O.GATE_SIGMOID_NOAUX_TC, True, 2.5, O.WEIGHT_FP8_BLOCK128,
                       O.COMBINE_FP32)
    x, W = O.make_inputs(spec, 500, 31, zipf_alpha=1.2)  # skewed routing: the groups differ in size
    want = make_layer(spec, W, DEV)
    got = _streamed(spec, W, 4, 2, routing_aware=True)
    xd = x.to(DEV)
    y0 = want.forward(xd)
    for _ in range(2):
        y1 = got.forward(xd)
        assert torch.equal(y0.view(torch.int16), y1.view(torch.int16))
    assert O.rel_l2(y1.cpu().float(), O.layer_forward(spec, x, W, gold_fp32=True)["y"]) <= 1e-2
    idx, _ = want.gate_route(xd)[:2]
    per_group = torch.bincount(idx.cpu().view(-1).long() // 4, minlength=4).tolist()
    expect = sorted((g for g in range(4) if per_group[g] > 0), key=lambda g: (-per_group[g], g))
    assert got.last_group_order == expect
    assert len(set(per_group)) > 1
    assert got.layer.device_status() == (0, 0)
