"""GPU: the benchmark's full-size DeepSeek-V3 layer (T=65536, 256 FP8 experts) checked through
size-independent properties, plus a handful of tokens recomputed with the CPU oracle."""
import pytest
import torch

import bench
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def v3_layer(built_lib):
    if torch.cuda.mem_get_info(0)[0] < 90e9:
        pytest.skip("needs ~80 GB of free device memory")
    layer = bench.build_layer("v3", torch.device(DEV))
    x = bench.make_tokens("v3", 65536, torch.device(DEV))
    yield layer, x
    layer.close()


def test_fullsize_routing_and_permutation_properties(v3_layer):
    layer, x = v3_layer
    T, k, E = x.shape[0], layer.k, layer.E
    idx, w = layer.route_topk(layer.gate_logits(x))
    # every token picks k distinct experts from at most topk_group groups; weights sum to the scale
    srt = idx.sort(dim=1).values
    assert bool((srt[:, 1:] != srt[:, :-1]).all())
    groups = (idx // (E // 8)).long()
    n_groups = torch.zeros(T, 8, dtype=torch.bool, device=DEV).scatter_(1, groups, True).sum(1)
    assert int(n_groups.max()) <= 4
    assert torch.allclose(w.sum(1), torch.full((T,), 2.5, device=DEV), rtol=1e-5)
    counts, offsets, pad, dst = layer.permute_plan(idx)
    assert int(counts.sum()) == T * k and int(offsets[-1]) == T * k
    assert torch.equal(counts.long(), torch.bincount(idx.view(-1).long(), minlength=E))
    assert torch.equal(pad[1:] - pad[:-1], (counts + 127) // 128 * 128)
    # the placement is a bijection onto the experts' segments, tokens ascending inside a segment
    flat = dst.view(-1).long()
    assert torch.unique(flat).numel() == T * k
    seg = torch.searchsorted(pad[1:].long().contiguous(), flat, right=True)
    assert torch.equal(seg, idx.view(-1).long())
    assert bool((flat - pad.long()[seg] < counts.long()[seg]).all())
    order = torch.argsort(flat)
    tok = (order // k)
    same_seg = seg[order][1:] == seg[order][:-1]
    assert bool((tok[1:][same_seg] > tok[:-1][same_seg]).all())
    # checksum of checksums: the scattered rows carry exactly k copies of every token's bits
    rows = layer.padded_rows(T * k)
    perm = layer.permute_rows(x, dst, rows)
    live = torch.zeros(rows, dtype=torch.bool, device=DEV)
    live[flat] = True
    s_perm = perm.view(torch.int16)[live].to(torch.int64).sum()
    assert int(s_perm) == k * int(x.view(torch.int16).to(torch.int64).sum())
    del perm
    assert layer.device_status() == (0, 0)


def test_fullsize_layer_is_deterministic_and_matches_oracle_on_sampled_tokens(v3_layer):
    layer, x = v3_layer
    y1 = layer.forward(x).clone()
    y2 = layer.forward(x)
    torch.cuda.synchronize()
    assert layer.device_status() == (0, 0)
    assert torch.equal(y1.view(torch.int16), y2.view(torch.int16))
    assert bool(torch.isfinite(y1.float()).all())
    # recompute 4 tokens on the CPU from the same seeded weights
    H, I, Is, seed = layer.H, layer.I, layer.Is, bench.WORKLOADS["v3"][13]
    sample = [0, 12345, 40000, 65535]
    idx, w = layer.route_topk(layer.gate_logits(x))
    ge = torch.Generator(device=DEV)

    def expert_weights(e):
        ge.manual_seed(seed * 100003 + e)
        mats = [(torch.randn(r, c, generator=ge, device=DEV) * 0.02).to(torch.bfloat16)
                for r, c in ((I, H), (I, H), (H, I))]
        return [layer.dequant_fp8(*bench.quantize_fp8_block128_gpu(m)).float().cpu() for m in mats]

    ge.manual_seed(seed * 100003 + 99991)
    shared = [(torch.randn(r, c, generator=ge, device=DEV) * 0.02).to(torch.bfloat16).float().cpu()
              for r, c in ((Is, H), (Is, H), (H, Is))]
    for t in sample:
        xt = x[t:t + 1].float().cpu()
        ref = O.swiglu_mlp(xt, *shared)
        for j in range(layer.k):
            ref = ref + float(w[t, j]) * O.swiglu_mlp(xt, *expert_weights(int(idx[t, j])))
        assert O.rel_l2(y1[t:t + 1].float().cpu(), ref) <= 1e-2
