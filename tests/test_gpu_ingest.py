"""GPU: a checkpoint written in the Hugging Face naming, ingested shard -> packed buffer, gives the
same packed bytes and the same forward as loading the experts one by one."""
import pytest
import torch

from moe_gen_b200 import ingest
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("ep", [(0, 1), (1, 2)])
def test_ingested_layer_equals_directly_loaded_layer(built_lib, tmp_path, fp8, ep):
    rank, world = ep
    spec = O.LayerSpec(256, 128, 8, 2, 128, 4, 2, O.GATE_SIGMOID_NOAUX_TC, True, 2.5,
                       O.WEIGHT_FP8_BLOCK128 if fp8 else O.WEIGHT_BF16, O.COMBINE_FP32)
    x, W = O.make_inputs(spec, 200, 17)
    if fp8:
        experts = [(W.q_gate[e], W.q_up[e], W.q_down[e]) for e in range(spec.n_experts)]
    else:
        experts = [(W.w_gate[e], W.w_up[e], W.w_down[e]) for e in range(spec.n_experts)]
    # two shards: router + first experts + shared expert, then the other experts
    ingest.export_moe_layer(str(tmp_path / "model-00001-of-00002.safetensors"), 5, W.gate_w, W.bias, experts[:3],
                            shared=W.shared)
    gate_n, bias_n, exp_n, mats, shared_n = ingest.NAMING["deepseek"]
    rest = {}
    for e in range(3, spec.n_experts):
        for m, w in zip(mats, experts[e]):
            n = exp_n.format(p="model.layers.5", e=e, m=m)
            if fp8:
                rest[n + ".weight"], rest[n + ".weight_scale_inv"] = w
            else:
                rest[n + ".weight"] = w
    ingest.write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), rest)

    from moe_gen_b200 import MoELayer

    def blank():
        lay = MoELayer(hidden=spec.hidden, inter=spec.inter, n_experts=spec.n_experts, top_k=spec.top_k,
                       inter_shared=spec.inter_shared, n_group=spec.n_group, topk_group=spec.topk_group,
                       gating=spec.gating, norm_topk_prob=spec.norm_topk_prob, routed_scale=spec.routed_scale,
                       weight_format=spec.weight_format, combine_mode=spec.combine_mode, ep_rank=rank,
                       ep_size=world, device=DEV)
        lay.packed.zero_()                     # alignment gaps between the packed sections are never written
        return lay

    want, got = blank(), blank()
    want.set_router(W.gate_w, W.bias)
    for i in range(want.e_local):
        e = want.expert_lo + i
        if fp8:
            (g, gs), (u, us), (d, ds) = experts[e]
            want.load_expert(i, g, u, d, (gs, us, ds))
        else:
            want.load_expert(i, *experts[e])
    want.load_shared(*W.shared)
    ck = ingest.Checkpoint(str(tmp_path))
    stats = ingest.load_moe_layer(got, ck, 5, n_threads=2)
    ck.close()
    assert stats["experts"] == spec.n_experts // world and stats["bytes"] > 0
    assert torch.equal(got.gate_w, want.gate_w) and torch.equal(got.bias, want.bias)
    assert torch.equal(got.packed, want.packed)
    if world == 1:
        xd = x.to(DEV)
        assert torch.equal(got.forward(xd).view(torch.int16), want.forward(xd).view(torch.int16))


def test_wrong_storage_format_is_refused(built_lib, tmp_path):
    spec = O.LayerSpec(256, 128, 4, 2, 0, combine_mode=O.COMBINE_FP32)
    _, W = O.make_inputs(spec, 4, 2)
    ingest.export_moe_layer(str(tmp_path / "m.safetensors"), 0, W.gate_w, None,
                            [(W.w_gate[e], W.w_up[e], W.w_down[e]) for e in range(4)])
    from moe_gen_b200 import MoELayer
    fp8_layer = MoELayer(hidden=256, inter=128, n_experts=4, top_k=2, weight_format=O.WEIGHT_FP8_BLOCK128, device=DEV)
    ck = ingest.Checkpoint(str(tmp_path / "m.safetensors"))
    with pytest.raises((ValueError, KeyError)):
        ingest.load_moe_layer(fp8_layer, ck, 0)
    ck.close()
