"""GPU parity tests: every stage and the whole layer, through the C ABI, against the CPU
oracle on identical seeded inputs and against the fixtures recorded from the reference.

Bars: routing indices, histogram and permutation bit-exact (tokens whose k-th / (k+1)-th
selection scores are closer than the fp32 noise of the logits are exempt, counted and
bounded); routing weights <= 1e-6 relative; de-quantisation and row copies bit-exact;
layer output <= 1e-2 relative L2 of the fp32-accumulated reference output."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.golden.make_golden import CASES, GATE_CASES
from tests.util import bf16_from_bits, load_golden, make_layer

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL_LAYER = 1e-2          # relative L2 vs the fp32-accumulated reference output
TOL_WEIGHT = 1e-6         # routing weights, relative, on identical logits
TOL_WEIGHT_FUSED = 1e-4   # same, when the logits come from the tensor-core router product, whose
                          # fp32 accumulation differs from a scalar fp32 sum by up to ~1e-5 absolute
NEAR_TIE = 1e-4           # relative gap below which that difference may decide a pick


def _status_ok(layer):
    torch.cuda.synchronize()
    assert layer.device_status() == (0, 0)


def _route_equal(spec, idx_gpu, w_gpu, idx_ref, w_ref, logits_ref, bias, exact_logits):
    """Compares per-token sets; returns number of exempted near-tie tokens."""
    gi, gw = O.canonical_sets(idx_gpu.cpu().long(), w_gpu.cpu())
    ri, rw = O.canonical_sets(idx_ref.long(), w_ref)
    same = (gi == ri).all(dim=1)
    if exact_logits:
        assert bool(same.all()), f"{int((~same).sum())} tokens differ on identical logits"
    else:
        gap = O.kth_gap(spec, logits_ref, bias)
        bad = ~same
        assert bool((gap[bad] < NEAR_TIE).all()), "a token with a clear score gap was routed differently"
        assert int(bad.sum()) <= max(2, idx_ref.shape[0] // 500), f"{int(bad.sum())} near-tie flips"
    rel = ((gw - rw).abs() / rw.abs().clamp_min(1e-12))[same]
    if rel.numel():
        assert float(rel.max()) <= (TOL_WEIGHT if exact_logits else TOL_WEIGHT_FUSED), float(rel.max())
    return int((~same).sum())


# --------------------------------------------------------------------------- routing
def test_fixup_recomputes_whole_rows_where_groups_are_not_runs_of_lanes(built_lib):
    """96 experts in 4 groups of 24: a group is six lanes of four experts, not a power-of-two run, so a
    token whose group selection is close gets its whole logits row recomputed; the selection still equals
    that of the exactly rounded logits for every token."""
    spec = O.LayerSpec(256, 128, 96, 4, 0, 4, 2, O.GATE_SIGMOID_NOAUX_TC, True, 2.5, O.WEIGHT_BF16, O.COMBINE_FP32)
    T = 60000
    gen = torch.Generator().manual_seed(77)
    x = torch.randn(T, spec.hidden, generator=gen).to(torch.bfloat16)
    gw = (torch.randn(spec.n_experts, spec.hidden, generator=gen) * 0.1).to(torch.bfloat16)
    bias = torch.randn(spec.n_experts, generator=gen) * 0.01
    layer = make_layer(spec, O.LayerWeights(gw, bias), DEV)
    idx, w, logits, fix = layer.gate_route(x.to(DEV))
    exact = (x.double() @ gw.double().t()).float()
    eidx, ew = O.route(spec, exact, bias)
    gi, _ = O.canonical_sets(idx.cpu().long(), w.cpu())
    ei, _ = O.canonical_sets(eidx, ew)
    assert torch.equal(gi, ei), f"{int((gi != ei).any(1).sum())} of {T} tokens differ from exact-logit routing"
    n_fix, n_rows, n_pairs = (int(v) for v in fix[:3])
    assert 0 < n_rows <= n_fix and n_pairs > 0
    rows = fix[4 + T:4 + T + n_rows].cpu().long()
    ulp = torch.finfo(torch.float32).eps * exact[rows].abs().clamp_min(2.0 ** -126)
    assert bool(((logits.cpu()[rows] - exact[rows]).abs() <= ulp).all())
    raw = layer.gate_logits(x.to(DEV)).cpu()
    bound = (6.0e-9 * spec.hidden + 4.0e-6) * exact.abs().amax(1, keepdim=True).clamp_min(1.0)
    assert float(((raw - exact).abs() / bound).max()) <= 0.5
    _status_ok(layer)


@pytest.mark.parametrize("name", sorted(GATE_CASES))
def test_topk_on_identical_logits_is_exact_at_full_gate_shapes(built_lib, name):
    cfg, T, seed = GATE_CASES[name]
    spec = O.named_spec(cfg)
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(T, spec.hidden, generator=gen).to(torch.bfloat16)
    gw = (torch.randn(spec.n_experts, spec.hidden, generator=gen) * 0.02).to(torch.bfloat16)
    bias = torch.randn(spec.n_experts, generator=gen) * 0.01 if spec.gating == O.GATE_SIGMOID_NOAUX_TC else None
    W = O.LayerWeights(gw, bias)
    layer = make_layer(O.LayerSpec(**{**spec.__dict__, "inter_shared": 0, "weight_format": 0}), W, DEV, 0, spec.n_experts)
    logits = O.gate_logits(x, gw)
    idx, w = layer.route_topk(logits.to(DEV))
    ridx, rw = O.route(spec, logits, bias)
    # slot order too: score descending, ties to the lower id
    assert torch.equal(idx.cpu().long(), ridx)
    _route_equal(spec, idx, w, ridx, rw, logits, bias, exact_logits=True)
    # and against what the reference's own gate produced (recorded fixture)
    g = load_golden(name)
    gi, gwt = O.canonical_sets(idx.cpu().long(), w.cpu())
    assert np.array_equal(gi.numpy().astype(np.int16), g["topk_idx"])
    assert np.abs(gwt.numpy() - g["topk_w"]).max() <= 2e-6 * max(1.0, spec.routed_scale)
    # fused path: logits from the tensor-core router GEMM, near-tie tokens re-routed from recomputed logits
    idx2, w2, logits2, fix = layer.gate_route(x.to(DEV))
    _route_equal(spec, idx2, w2, ridx, rw, logits, bias, exact_logits=False)
    # ... which is the routing of the correctly rounded logits (fp64 product rounded once), token for token
    exact = (x.double() @ gw.double().t()).float()
    eidx, ew = O.route(spec, exact, bias)
    gi, _ = O.canonical_sets(idx2.cpu().long(), w2.cpu())
    ei, _ = O.canonical_sets(eidx, ew)
    assert torch.equal(gi, ei), f"{int((gi != ei).any(1).sum())} of {T} tokens differ from exact-logit routing"
    n_fix, n_rows, n_pairs = (int(v) for v in fix[:3])
    again = fix[4:4 + n_fix].cpu().long()
    assert 0 < n_fix <= T // 10 and again.unique().numel() == n_fix
    assert n_rows == 0 and 0 < n_pairs <= 8 * T + 64                # groups are lane runs here, the pairs fit
    pairs = fix[4 + 2 * T:4 + 2 * T + 2 * n_pairs].cpu().long().view(-1, 2)
    assert set(pairs[:, 0].tolist()) == set(again.tolist())
    raw = layer.gate_logits(x.to(DEV)).cpu()
    bound = (6.0e-9 * spec.hidden + 4.0e-6) * exact.abs().amax(1, keepdim=True).clamp_min(1.0)
    assert float(((raw - exact).abs() / bound).max()) <= 0.5       # the error the flagging assumes, with 2x to spare
    # the recomputed entries are the exact product to the last bit or the one next to it
    got, want = logits2.cpu()[pairs[:, 0], pairs[:, 1]], exact[pairs[:, 0], pairs[:, 1]]
    assert bool(((got - want).abs() <= torch.finfo(torch.float32).eps * want.abs().clamp_min(2.0 ** -126)).all())
    # without the fix-up the staged calls give the raw tensor-core routing
    idx3, w3 = layer.route_topk(layer.gate_logits(x.to(DEV)))
    _route_equal(spec, idx3, w3, ridx, rw, logits, bias, exact_logits=False)
    # ... and so does the fused call with the fix-up switched off
    from moe_gen_b200 import lib as L
    layer.set_option(L.OPT_ROUTE_FIXUP, 0)
    idx4, w4, _, fix4 = layer.gate_route(x.to(DEV))
    assert torch.equal(idx4, idx3) and torch.equal(w4, w3) and int(fix4[0]) == 0
    layer.set_option(L.OPT_ROUTE_FIXUP, 1)
    _status_ok(layer)


def test_ties_break_toward_lower_expert_id(built_lib):
    spec = O.LayerSpec(256, 128, 16, 4, gating=O.GATE_SOFTMAX_GREEDY)
    W = O.LayerWeights(torch.zeros(16, 256, dtype=torch.bfloat16), None)
    layer = make_layer(spec, W, DEV, 0, 16)
    logits = torch.zeros(3, 16)
    logits[1, 5] = 1.0
    logits[2, 8:] = 2.0
    idx, w = layer.route_topk(logits.to(DEV))
    assert idx.cpu().tolist() == [[0, 1, 2, 3], [5, 0, 1, 2], [8, 9, 10, 11]]
    ridx, rw = O.route(spec, logits)
    assert torch.allclose(w.cpu(), rw, rtol=1e-6, atol=0)


def test_masked_groups_compete_as_zero(built_lib):
    spec = O.LayerSpec(256, 128, 8, 3, n_group=4, topk_group=1, gating=O.GATE_SIGMOID_NOAUX_TC,
                       norm_topk_prob=True, routed_scale=1.0)
    bias = torch.full((8,), -0.5)
    bias[2:4] = -0.1
    W = O.LayerWeights(torch.zeros(8, 256, dtype=torch.bfloat16), bias)
    layer = make_layer(spec, W, DEV, 0, 8)
    logits = torch.full((1, 8), -20.0)
    idx, w = layer.route_topk(logits.to(DEV))
    ridx, rw = O.route(spec, logits, bias)
    assert idx.cpu().tolist() == ridx.tolist() == [[0, 1, 4]]
    assert torch.allclose(w.cpu(), rw, rtol=1e-5, atol=1e-12)


@pytest.mark.parametrize("E,k,G,keep,gating", [
    (8, 2, 1, 1, O.GATE_SOFTMAX_TOPK_RENORM), (64, 6, 1, 1, O.GATE_SOFTMAX_GREEDY),
    (160, 6, 8, 3, O.GATE_SOFTMAX_GROUP_MAX), (256, 8, 8, 4, O.GATE_SIGMOID_NOAUX_TC),
    (32, 1, 4, 2, O.GATE_SIGMOID_NOAUX_TC), (128, 8, 16, 5, O.GATE_SOFTMAX_GROUP_MAX),
    (384, 8, 8, 4, O.GATE_SIGMOID_NOAUX_TC),
])
@pytest.mark.parametrize("T", [1, 2, 3, 127, 128, 129, 1000])
def test_topk_exhaustive_small_shapes(built_lib, E, k, G, keep, gating, T):
    spec = O.LayerSpec(256, 128, E, k, n_group=G, topk_group=keep, gating=gating, norm_topk_prob=(E % 3 == 0),
                       routed_scale=2.5)
    gen = torch.Generator().manual_seed(E * 1000 + T)
    bias = torch.randn(E, generator=gen) * 0.01 if gating == O.GATE_SIGMOID_NOAUX_TC else None
    W = O.LayerWeights(torch.zeros(E, 256, dtype=torch.bfloat16), bias)
    layer = make_layer(spec, W, DEV, 0, E)
    logits = torch.randn(T, E, generator=gen) * 1.7
    idx, w = layer.route_topk(logits.to(DEV))
    ridx, rw = O.route(spec, logits, bias)
    _route_equal(spec, idx, w, ridx, rw, logits, bias, exact_logits=True)


# --------------------------------------------------------------------------- permute
@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (3, 64, 6), (127, 64, 6), (128, 160, 6), (129, 256, 8), (5000, 256, 8),
                                   (4096, 8, 2)])
def test_permute_plan_and_rows_are_exact(built_lib, T, E, k):
    spec = O.LayerSpec(512, 128, E, k)
    W = O.LayerWeights(torch.zeros(E, 512, dtype=torch.bfloat16), None)
    layer = make_layer(spec, W, DEV)
    gen = torch.Generator().manual_seed(T + E)
    # distinct experts per token, skewed so that some experts stay empty
    scores = torch.rand(T, E, generator=gen)
    scores[:, E // 2:] *= 0.2
    scores[:, 1] = -1.0                      # expert 1 never chosen
    idx = scores.topk(k, dim=-1).indices.to(torch.int32)
    counts, offsets, pad, dst = layer.permute_plan(idx.to(DEV))
    rc, roff, order, src = O.permute_plan(idx.long(), E)
    assert torch.equal(counts.cpu().long(), rc)
    assert torch.equal(offsets.cpu().long(), roff)
    padc = pad.cpu().long()
    assert torch.equal(padc[1:] - padc[:-1], (rc + 127) // 128 * 128)
    # stable placement: the r-th row of expert e is the r-th pick of e in flattened order
    flat_dst = dst.cpu().long().view(-1)
    expert_of_sorted = torch.repeat_interleave(torch.arange(E), rc)
    rank = torch.arange(order.numel()) - roff[expert_of_sorted]
    assert torch.equal(flat_dst[order], padc[expert_of_sorted] + rank)
    x = torch.randn(T, 512, generator=gen).to(torch.bfloat16)
    rows = layer.padded_rows(T * k)
    assert int(padc[-1]) <= rows
    perm = layer.permute_rows(x.to(DEV), dst, rows).cpu()
    assert torch.equal(perm[flat_dst].view(torch.int16), x[torch.arange(T * k) // k].view(torch.int16))
    _status_ok(layer)


def test_permute_plan_expert_range_skips_foreign_picks(built_lib):
    spec = O.LayerSpec(256, 128, 64, 6)
    W = O.LayerWeights(torch.zeros(64, 256, dtype=torch.bfloat16), None)
    layer = make_layer(spec, W, DEV, 0, 64)
    gen = torch.Generator().manual_seed(5)
    idx = torch.rand(777, 64, generator=gen).topk(6, dim=-1).indices.to(torch.int32)
    counts, offsets, pad, dst = layer.permute_plan(idx.to(DEV), expert_lo=16, n_plan=16)
    local = (idx >= 16) & (idx < 32)
    assert torch.equal(counts.cpu().long(), torch.bincount(idx[local].long() - 16, minlength=16))
    assert bool((dst.cpu()[~local] == -1).all()) and bool((dst.cpu()[local] >= 0).all())


# --------------------------------------------------------------------------- de-quantisation
def test_fp8_dequant_is_bit_exact(built_lib):
    spec = O.LayerSpec(256, 128, 8, 2)
    layer = make_layer(spec, O.LayerWeights(torch.zeros(8, 256, dtype=torch.bfloat16), None), DEV, 0, 8)
    gen = torch.Generator().manual_seed(3)
    for shape in [(128, 256), (384, 512), (2048, 7168)]:
        w = (torch.randn(*shape, generator=gen) * 0.02).to(torch.bfloat16)
        q, s = O.quantize_fp8_block128(w)
        out = layer.dequant_fp8(q, s).cpu()
        assert torch.equal(out.view(torch.int16), O.dequantize_fp8_block128(q, s).view(torch.int16))


# --------------------------------------------------------------------------- experts
def _check_expert_rows(spec, W, x, layer, idx):
    counts, offsets, pad, dst = layer.permute_plan(idx)
    rows = layer.padded_rows(x.shape[0] * spec.top_k)
    perm = layer.permute_rows(x, dst, rows)
    hbuf, out = layer.expert_ffn(perm, pad, counts)
    _status_ok(layer)
    padc, cc, permc, outc = pad.cpu().long(), counts.cpu().long(), perm.cpu(), out.cpu()
    worst = 0.0
    for e in range(spec.n_experts):
        n, r0 = int(cc[e]), int(padc[e])
        if n == 0:
            continue
        ref = O.swiglu_mlp(permc[r0:r0 + n].float(), W.w_gate[e].float(), W.w_up[e].float(), W.w_down[e].float())
        worst = max(worst, O.rel_l2(outc[r0:r0 + n].float(), ref))
    return worst, (counts, offsets, pad, dst, out)


@pytest.mark.parametrize("T", [1, 5, 128, 700])
def test_grouped_swiglu_matches_fp32_oracle_with_ragged_and_empty_experts(built_lib, T):
    spec = O.LayerSpec(512, 256, 16, 4, combine_mode=O.COMBINE_FP32)
    x, W = O.make_inputs(spec, T, 40 + T)
    layer = make_layer(spec, W, DEV)
    gen = torch.Generator().manual_seed(T)
    scores = torch.rand(T, 16, generator=gen)
    scores[:, 3] = -1.0                       # empty expert
    scores[:, 7] += 0.6                       # heavy expert
    idx = scores.topk(4, dim=-1).indices.to(torch.int32).to(DEV)
    worst, _ = _check_expert_rows(spec, W, x.to(DEV), layer, idx)
    assert worst < 5e-3, worst


def test_all_tokens_to_one_expert(built_lib):
    spec = O.LayerSpec(256, 128, 8, 1, combine_mode=O.COMBINE_FP32)
    x, W = O.make_inputs(spec, 1000, 77)
    layer = make_layer(spec, W, DEV)
    idx = torch.full((1000, 1), 5, dtype=torch.int32, device=DEV)
    worst, (counts, *_rest) = _check_expert_rows(spec, W, x.to(DEV), layer, idx)
    assert counts.cpu().tolist() == [0, 0, 0, 0, 0, 1000, 0, 0]
    assert worst < 5e-3


@pytest.mark.parametrize("H,I", [(512, 256), (1024, 512)])
def test_fp8_weights_converted_in_the_gemm_equal_dequantise_first(built_lib, H, I):
    """W8A16: converting FP8 tiles inside the grouped GEMM gives the same bits as de-quantising
    the matrices first (the reference's order, Wrapper.py:481-491) and running the bf16 kernel.
    The two shapes take the two de-quantisation kernels of the packed stacks (rows of a multiple of
    512 bytes stream through the row kernel, others through the generic one)."""
    spec = O.LayerSpec(H, I, 16, 4, 256, 4, 2, O.GATE_SIGMOID_NOAUX_TC, True, 2.5, O.WEIGHT_FP8_BLOCK128,
                       O.COMBINE_FP32)
    x, W = O.make_inputs(spec, 900, 51)
    layer = make_layer(spec, W, DEV)
    xd = x.to(DEV)
    idx, w = layer.gate_route(xd)[:2]
    counts, offsets, pad, dst = layer.permute_plan(idx)
    perm = layer.permute_rows(xd, dst, layer.padded_rows(900 * 4))
    h1, o1 = layer.expert_ffn(perm, pad, counts, predequant=False)
    live = torch.zeros(perm.shape[0], dtype=torch.bool)
    live[dst.cpu().long().view(-1)] = True
    # scratch-based modes: the bf16 copy written by a separate pass (1), the L2-resident ring filled by
    # the GEMM kernel itself (3), the latter also with a ring of two slots that every expert reuses
    for mode, ring_mib in ((1, 56), (3, 56), (3, 1)):
        layer.set_option(1, mode)
        layer.set_option(7, ring_mib)
        for _ in range(2):
            h2, o2 = layer.expert_ffn(perm, pad, counts, predequant=True)
            _status_ok(layer)
            assert torch.equal(h1.cpu()[live].view(torch.int16), h2.cpu()[live].view(torch.int16)), (mode, ring_mib)
            assert torch.equal(o1.cpu()[live].view(torch.int16), o2.cpu()[live].view(torch.int16)), (mode, ring_mib)
    layer.set_option(7, 56)
    layer.set_option(1, 0)
    for tall in (0, 2, 1):                             # 128-row tiles, 256-row tiles, by expert size
        layer.set_option(4, tall)
        h4, o4 = layer.expert_ffn(perm, pad, counts, predequant=False)
        _status_ok(layer)
        assert torch.equal(h1.cpu()[live].view(torch.int16), h4.cpu()[live].view(torch.int16))
        assert torch.equal(o1.cpu()[live].view(torch.int16), o4.cpu()[live].view(torch.int16))
    worst, _ = _check_expert_rows(spec, W, xd, layer, idx)
    assert worst < 5e-3
    ys = []
    for pair in (0, 1):                                # one CTA per SM / SM pairs
        layer.set_option(2, pair)
        for mode in (0, 1, 2, 3, 1):                   # auto, pre-dequantise, in-kernel, ring, again
            layer.set_option(1, mode)
            ys.append(layer.forward(xd).cpu())
            _status_ok(layer)
        h3, o3 = layer.expert_ffn(perm, pad, counts, predequant=False)
        _status_ok(layer)
        assert torch.equal(h1.cpu()[live].view(torch.int16), h3.cpu()[live].view(torch.int16))
        assert torch.equal(o1.cpu()[live].view(torch.int16), o3.cpu()[live].view(torch.int16))
    for y in ys[1:]:
        assert torch.equal(ys[0].view(torch.int16), y.view(torch.int16))


@pytest.mark.parametrize("T", [3, 130, 700, 3000])
def test_sm_pair_gemm_equals_single_cta_gemm(built_lib, T):
    """The 2-CTA (cta_group::2) kernel computes the same sums in the same order as the 1-CTA one."""
    spec = O.LayerSpec(512, 256, 16, 4, 256, combine_mode=O.COMBINE_FP32)
    x, W = O.make_inputs(spec, T, 60 + T)
    layer = make_layer(spec, W, DEV)
    xd = x.to(DEV)
    gen = torch.Generator().manual_seed(T)
    scores = torch.rand(T, 16, generator=gen)
    scores[:, 3] = -1.0
    scores[:, 7] += 0.6
    idx = scores.topk(4, dim=-1).indices.to(torch.int32).to(DEV)
    counts, offsets, pad, dst = layer.permute_plan(idx)
    perm = layer.permute_rows(xd, dst, layer.padded_rows(T * 4))
    h1, o1 = layer.expert_ffn(perm, pad, counts)
    s1 = layer.shared_ffn(xd)
    layer.set_option(2, 1)
    h2, o2 = layer.expert_ffn(perm, pad, counts)
    s2 = layer.shared_ffn(xd)
    _status_ok(layer)
    live = torch.zeros(perm.shape[0], dtype=torch.bool)
    live[dst.cpu().long().view(-1)] = True
    assert torch.equal(h1.cpu()[live].view(torch.int16), h2.cpu()[live].view(torch.int16))
    assert torch.equal(o1.cpu()[live].view(torch.int16), o2.cpu()[live].view(torch.int16))
    assert torch.equal(s1.cpu().view(torch.int16), s2.cpu().view(torch.int16))
    worst, _ = _check_expert_rows(spec, W, xd, layer, idx)
    assert worst < 5e-3


# --------------------------------------------------------------------------- combine
@pytest.mark.parametrize("mode", [O.COMBINE_FP32, O.COMBINE_BF16_PROD, O.COMBINE_BF16_SEQ])
@pytest.mark.parametrize("with_shared", [False, True])
def test_combine_matches_oracle(built_lib, mode, with_shared):
    T, E, k, H = 300, 32, 4, 512
    spec = O.LayerSpec(H, 128, E, k, combine_mode=mode)
    layer = make_layer(spec, O.LayerWeights(torch.zeros(E, H, dtype=torch.bfloat16), None), DEV)
    gen = torch.Generator().manual_seed(mode * 2 + with_shared)
    idx = torch.rand(T, E, generator=gen).topk(k, dim=-1).indices.to(torch.int32)
    w = torch.rand(T, k, generator=gen) * 2.5
    counts, offsets, pad, dst = layer.permute_plan(idx.to(DEV))
    rows = layer.padded_rows(T * k)
    out_rows = torch.randn(rows, H, generator=gen).to(torch.bfloat16)
    shared = torch.randn(T, H, generator=gen).to(torch.bfloat16) if with_shared else None
    y = layer.combine(out_rows.to(DEV), dst, idx.to(DEV), w.to(DEV), None if shared is None else shared.to(DEV))
    by_slot = out_rows[dst.cpu().long().view(-1)].view(T, k, H)
    ref = O.combine(spec, by_slot, idx.long(), w)
    if shared is not None:
        ref = ref + shared
    diff = (y.cpu().float() - ref.float()).abs()
    # same arithmetic, same rounding points: at most a last-place difference from the order of
    # the k fp32 additions on a handful of elements
    assert float((diff > 0).float().mean()) < 2e-3
    assert O.rel_l2(y.cpu().float(), ref.float()) < 2e-4


# --------------------------------------------------------------------------- whole layer
@pytest.mark.parametrize("name", sorted(CASES))
def test_layer_against_reference_fixture(built_lib, name):
    spec, T, seed = CASES[name]
    g = load_golden(name)
    x, W = O.make_inputs(spec, T, seed)
    layer = make_layer(spec, W, DEV)
    xd = x.to(DEV)
    y = layer.forward(xd)
    _status_ok(layer)
    # routing as the layer computed it (read back from its workspace through the staged calls)
    logits = O.gate_logits(x, W.gate_w)
    idx, w = layer.gate_route(xd)[:2]
    ridx = torch.from_numpy(g["topk_idx"].astype(np.int64))
    rw = torch.from_numpy(g["topk_w"])
    flips = _route_equal(spec, idx, w, ridx, rw, logits, W.bias, exact_logits=False)
    counts, *_ = layer.permute_plan(idx)
    if flips == 0:
        assert np.array_equal(counts.cpu().numpy(), g["counts"])
    y_gold = torch.from_numpy(g["y_gold_fp32"])
    err = O.rel_l2(y.cpu().float(), y_gold)
    assert err <= TOL_LAYER, err
    # for information: distance to the reference's own bf16 output is of the same size as the
    # reference's bf16-vs-fp32 distance
    assert O.rel_l2(y.cpu().float(), bf16_from_bits(g["y_ref_bf16"]).float()) < 1.5e-2


# --------------------------------------------------------------------------- decoder-layer glue
def _bf16_ulps(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in bf16 steps between two bf16 tensors of the same sign pattern (monotone integer map)."""
    def key(t):
        i = t.view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return (key(a) - key(b)).abs()


@pytest.mark.parametrize("T,H", [(1, 256), (77, 2048), (300, 7168), (5, 16384)])
def test_rmsnorm_matches_oracle(built_lib, T, H):
    """fp32 statistics summed in a different order than torch's: a value may land on the neighbouring
    bf16 when its fp32 product sits on a rounding boundary; nothing further than one step."""
    from moe_gen_b200 import MoELayer
    layer = MoELayer(hidden=H, inter=128, n_experts=8, top_k=2, device=DEV)     # no weights needed
    g = torch.Generator().manual_seed(T + H)
    x = (torch.randn(T, H, generator=g) * 3.0).to(torch.bfloat16)
    x[0, : H // 2] = 0                                            # zeros stay zeros
    w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    ref = O.rmsnorm(x, w, 1e-6)
    got = layer.rmsnorm(x.to(DEV), w.to(DEV), 1e-6).cpu()
    _status_ok(layer)
    d = _bf16_ulps(got, ref)
    assert int(d.max()) <= 1
    assert float((d > 0).float().mean()) < 2e-3


def test_block_forward_against_reference_fixture(built_lib):
    """hidden + moe(rmsnorm(hidden)) against the output recorded from the reference's RMSNorm and V3
    block (fp32 gold: 1e-2 relative L2, as for the block alone), out of place and in place."""
    spec, T, seed = CASES["v3_noaux_small_bf16"]
    g = load_golden("block_v3_small")
    hidden, W = O.make_inputs(spec, T, seed)
    norm_w = bf16_from_bits(g["norm_w"])
    eps = float(g["eps"])
    layer = make_layer(spec, W, DEV)
    hd, wd = hidden.to(DEV), norm_w.to(DEV)
    xn = layer.rmsnorm(hd, wd, eps)
    d = _bf16_ulps(xn.cpu(), bf16_from_bits(g["x_norm_bf16"]))
    assert int(d.max()) <= 1 and float((d > 0).float().mean()) < 2e-3
    y = layer.block_forward(hd, wd, eps)
    _status_ok(layer)
    assert O.rel_l2(y.cpu().float(), torch.from_numpy(g["y_block_gold_fp32"])) <= TOL_LAYER
    assert O.rel_l2(y.cpu().float(), bf16_from_bits(g["y_block_bf16"]).float()) < 1.5e-2
    # the same sums in the same order as forward() on the normalised rows plus one bf16 add
    y2 = (hd.float() + layer.forward(xn).float()).to(torch.bfloat16)
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
    inplace = hd.clone()
    layer.block_forward(inplace, wd, eps, out=inplace)
    _status_ok(layer)
    assert torch.equal(inplace.view(torch.int16), y.view(torch.int16))
    assert layer.block_forward(hd[:0], wd, eps).shape == (0, spec.hidden)


def test_shared_expert_beside_the_routing_kernels_equals_after_the_experts(built_lib):
    """MG_OPT_SHARED_EARLY only moves the shared expert's GEMMs to another stream."""
    spec, T, seed = CASES["v3_noaux_small_bf16"]
    x, W = O.make_inputs(spec, T, seed)
    layer = make_layer(spec, W, DEV)
    xd = x.to(DEV)
    ys = []
    for mode in (0, 1, 2, 0):
        layer.set_option(6, mode)
        for _ in range(2):
            ys.append(layer.forward(xd).clone())
        _status_ok(layer)
    for y in ys[1:]:
        assert torch.equal(ys[0].view(torch.int16), y.view(torch.int16))


@pytest.mark.parametrize("T", [0, 1, 127, 129])
def test_layer_edge_token_counts(built_lib, T):
    spec = O.LayerSpec(256, 128, 64, 6, 256, 1, 1, O.GATE_SOFTMAX_GREEDY, False, 1.0, O.WEIGHT_BF16,
                       O.COMBINE_BF16_PROD)
    x, W = O.make_inputs(spec, max(T, 1), 90 + T)
    x = x[:T]
    layer = make_layer(spec, W, DEV)
    y = layer.forward(x.to(DEV))
    _status_ok(layer)
    assert y.shape == (T, 256)
    if T:
        gold = O.layer_forward(spec, x, W, gold_fp32=True)
        assert O.rel_l2(y.cpu().float(), gold["y"]) <= TOL_LAYER


def test_mixtral_layer(built_lib):
    spec = O.LayerSpec(512, 1024, 8, 2, gating=O.GATE_SOFTMAX_TOPK_RENORM, norm_topk_prob=True,
                       combine_mode=O.COMBINE_BF16_SEQ)
    x, W = O.make_inputs(spec, 900, 17)
    layer = make_layer(spec, W, DEV)
    y = layer.forward(x.to(DEV))
    _status_ok(layer)
    gold = O.layer_forward(spec, x, W, gold_fp32=True)
    ref = O.layer_forward(spec, x, W)
    # the bf16 router output makes exact ties common; both sides resolve them to the lower id,
    # but a logit that rounds differently can still flip a token: compare only agreeing tokens
    idx, w = layer.gate_route(x.to(DEV))[:2]
    same = (O.canonical_sets(idx.cpu().long(), w.cpu())[0] == O.canonical_sets(ref["topk_idx"], ref["topk_w"])[0]).all(1)
    assert float(same.float().mean()) > 0.995
    assert O.rel_l2(y.cpu().float()[same], gold["y"][same]) <= TOL_LAYER


@pytest.mark.parametrize("fp8", [False, True])
def test_forward_host_equals_forward(built_lib, fp8):
    spec = O.LayerSpec(256, 128, 64, 6, 256, 1, 1, O.GATE_SOFTMAX_GREEDY, False, 1.0,
                       O.WEIGHT_FP8_BLOCK128 if fp8 else O.WEIGHT_BF16, O.COMBINE_BF16_PROD)
    x, W = O.make_inputs(spec, 1000, 33)
    layer = make_layer(spec, W, DEV)
    if fp8:
        layer.set_option(1, 1)        # pre-dequantise: the chunks of one host forward share the bf16 copy
    y = layer.forward(x.to(DEV)).cpu()
    for _ in range(2):
        yh = layer.forward_host(x.pin_memory(), chunk_tokens=256)
        assert torch.equal(y.view(torch.int16), yh.view(torch.int16))
    # re-packing an expert must invalidate the kept copy
    if fp8:
        (g, gs), (u, us), (d, ds) = W.q_gate[5], W.q_up[5], W.q_down[5]
        layer.load_expert(0, g, u, d, (gs, us, ds))
        y2 = layer.forward(x.to(DEV)).cpu()
        yh2 = layer.forward_host(x.pin_memory(), chunk_tokens=256)
        assert torch.equal(y2.view(torch.int16), yh2.view(torch.int16))
        assert not torch.equal(y2.view(torch.int16), y.view(torch.int16))
    _status_ok(layer)


def test_patched_reference_style_module(built_lib):
    """The patcher reads the attributes the reference modules expose (config, gate,
    experts[i].{gate,up,down}_proj, shared_experts) and serves forward([B,S,H])."""
    import types
    import torch.nn as nn
    from moe_gen_b200 import patch_moe_module
    spec = O.LayerSpec(256, 128, 32, 4, 128, 4, 2, O.GATE_SIGMOID_NOAUX_TC, True, 2.5, O.WEIGHT_BF16, O.COMBINE_FP32)
    x, W = O.make_inputs(spec, 64, 3)

    def mlp(g, u, d):
        m = nn.Module()
        for n, w in (("gate_proj", g), ("up_proj", u), ("down_proj", d)):
            lin = nn.Linear(w.shape[1], w.shape[0], bias=False, dtype=torch.bfloat16)
            lin.weight.data = w.clone()
            setattr(m, n, lin)
        return m

    class DeepseekV3MoE(nn.Module):
        pass
    mod = DeepseekV3MoE().eval()
    mod.config = types.SimpleNamespace(hidden_size=256, moe_intermediate_size=128, n_routed_experts=32,
                                       num_experts_per_tok=4, n_shared_experts=1, n_group=4, topk_group=2,
                                       topk_method="noaux_tc", scoring_func="sigmoid", norm_topk_prob=True,
                                       routed_scaling_factor=2.5)
    mod.gate = nn.Module()
    mod.gate.weight = nn.Parameter(W.gate_w.clone())
    mod.gate.e_score_correction_bias = nn.Parameter(W.bias.clone())
    mod.experts = nn.ModuleList([mlp(W.w_gate[e], W.w_up[e], W.w_down[e]) for e in range(32)])
    mod.shared_experts = mlp(*W.shared)
    patch_moe_module(mod, device=DEV)
    y = mod(x.view(2, 32, 256).to(DEV))
    assert y.shape == (2, 32, 256)
    gold = O.layer_forward(spec, x, W, gold_fp32=True)
    assert O.rel_l2(y.view(64, 256).cpu().float(), gold["y"]) <= TOL_LAYER

    # the decoder layer around it: attention (a stand-in here) and its residual add stay, the
    # norm / block / residual add behind them become one fused call
    from moe_gen_b200 import patch_decoder_layer

    class Norm(nn.Module):
        def __init__(self, w):
            super().__init__()
            self.weight, self.variance_epsilon = nn.Parameter(w), 1e-6

        def forward(self, h):
            return O.rmsnorm(h.cpu(), self.weight.detach().cpu(), self.variance_epsilon).to(h.device)

    class Attn(nn.Module):
        def forward(self, hidden_states, **kw):
            return hidden_states * 0.5, None, None

    class DeepseekV3DecoderLayer(nn.Module):
        pass
    g = torch.Generator().manual_seed(8)
    dl = DeepseekV3DecoderLayer().eval()
    dl.input_layernorm = Norm((1.0 + 0.1 * torch.randn(256, generator=g)).to(torch.bfloat16))
    dl.post_attention_layernorm = Norm((1.0 + 0.1 * torch.randn(256, generator=g)).to(torch.bfloat16))
    dl.self_attn = Attn()
    mod2 = DeepseekV3MoE().eval()
    mod2.config, mod2.gate, mod2.experts, mod2.shared_experts = mod.config, mod.gate, mod.experts, mod.shared_experts
    dl.mlp = mod2
    patch_decoder_layer(dl, device=DEV)
    h0 = x.view(2, 32, 256).to(DEV)
    (out,) = dl(h0)
    h1 = (x + dl.input_layernorm(x) * 0.5)                        # what reaches the second half, on CPU
    want = O.block_forward(spec, h1, dl.post_attention_layernorm.weight.detach(), 1e-6, W, gold_fp32=True)["y"]
    assert out.shape == (2, 32, 256)
    assert O.rel_l2(out.view(64, 256).cpu().float(), want) <= TOL_LAYER


def test_bounded_wait_gives_up_and_reports(built_lib):
    """Failure detection without a fault: a wait that nothing satisfies runs out after its limit,
    the kernel returns, the status word says so, and the context keeps working."""
    import time
    spec = O.LayerSpec(256, 128, 8, 2)
    x, W = O.make_inputs(spec, 64, 1)
    layer = make_layer(spec, W, DEV)
    t0 = time.time()
    rc = layer.lib.mg_selftest_wait_timeout(layer._h, 50, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert 0.04 < time.time() - t0 < 5.0
    assert layer.device_status() == (1, 99)          # MG_DEV_WAIT_TIMEOUT, where = 99
    assert layer.device_status() == (0, 0)           # reading clears it
    y = layer.forward(x.to(DEV))                     # the context is intact
    torch.cuda.synchronize()
    assert layer.device_status() == (0, 0)
    assert O.rel_l2(y.cpu().float(), O.layer_forward(spec, x, W, gold_fp32=True)["y"]) <= TOL_LAYER


@pytest.mark.parametrize("push", [False, True, "copy"])
@pytest.mark.parametrize("dedup", [False, True])
@pytest.mark.parametrize("n_ranks", [2, 4])
def test_expert_parallel_ranks_emulated_on_one_gpu(built_lib, n_ranks, dedup, push):
    """The expert-parallel kernels (layout, peer scatter, peer gather) run for every rank in turn in
    one process, the 'peer' buffers being ordinary allocations of this GPU.  The result must equal
    the single-GPU forward bit for bit, and the layout must equal its host restatement."""
    import ctypes as C
    from moe_gen_b200 import lib as L
    from moe_gen_b200.ep import ep_layout_reference
    spec = O.LayerSpec(256, 128, 32, 4, 128, 4, 2, O.GATE_SIGMOID_NOAUX_TC, True, 2.5, O.WEIGHT_FP8_BLOCK128,
                       O.COMBINE_FP32)
    T = 120 * n_ranks
    x, W = O.make_inputs(spec, T, 71)
    xd = x.to(DEV)
    full = make_layer(spec, W, DEV)
    y_ref = full.forward(xd).cpu()
    Tl, E, El, k, H = T // n_ranks, 32, 32 // n_ranks, 4, 256
    ranks = [make_layer(spec, W, DEV, r, n_ranks) for r in range(n_ranks)]
    lib = ranks[0].lib
    st = torch.cuda.current_stream().cuda_stream
    cap = ((T * k + 127) // 128 + El) * 128
    recv = [torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(n_ranks)]
    outb = [torch.zeros(cap, H, dtype=torch.bfloat16, device=DEV) for _ in range(n_ranks)]
    peer_recv = (C.c_void_p * n_ranks)(*[t.data_ptr() for t in recv])
    peer_out = (C.c_void_p * n_ranks)(*[t.data_ptr() for t in outb])
    i32 = dict(dtype=torch.int32, device=DEV)
    dupt = [torch.zeros(cap, **i32) for _ in range(n_ranks)]
    peer_dup = (C.c_void_p * n_ranks)(*[t.data_ptr() for t in dupt])
    # pushed return: a return table per owner and a return buffer per token owner
    backt = [torch.full((cap,), -1, **i32) for _ in range(n_ranks)]
    rett = [torch.zeros(Tl * k, H, dtype=torch.bfloat16, device=DEV) for _ in range(n_ranks)]
    peer_back = (C.c_void_p * n_ranks)(*[t.data_ptr() for t in backt])
    peer_ret = (C.c_void_p * n_ranks)(*[t.data_ptr() for t in rett])
    for r, lay in enumerate(ranks):
        L.check(lib.mg_ep_clear_duplicates(lay._h, dupt[r].data_ptr(), cap, st))
    idx, w, counts, plan_ws = [], [], [], []
    for r, lay in enumerate(ranks):
        xs = xd[r * Tl:(r + 1) * Tl]
        i_, w_ = lay.gate_route(xs)[:2]
        nb = C.c_size_t()
        L.check(lib.mg_plan_ws_bytes(lay._h, Tl, C.byref(nb)))
        ws = torch.empty(nb.value, dtype=torch.uint8, device=DEV)
        c = torch.empty(E, **i32)
        L.check(lib.mg_ep_count(lay._h, i_.data_ptr(), Tl, c.data_ptr(), ws.data_ptr(), st))
        idx.append(i_); w.append(w_); counts.append(c); plan_ws.append(ws)
    counts_all = torch.stack(counts).contiguous()
    dst, rc, rp = [], [], []
    for r, lay in enumerate(ranks):
        d = torch.empty(Tl, k, **i32); c = torch.empty(El, **i32); p = torch.empty(El + 1, **i32)
        L.check(lib.mg_ep_place(lay._h, idx[r].data_ptr(), Tl, counts_all.data_ptr(), cap, plan_ws[r].data_ptr(),
                                c.data_ptr(), p.data_ptr(), d.data_ptr(), st))
        if push is True:
            L.check(lib.mg_ep_dispatch_back(lay._h, xd[r * Tl:(r + 1) * Tl].data_ptr(), d.data_ptr(), Tl, peer_recv,
                                            peer_dup if dedup else None, peer_back, st))
        elif dedup:
            L.check(lib.mg_ep_dispatch_dedup(lay._h, xd[r * Tl:(r + 1) * Tl].data_ptr(), d.data_ptr(), Tl, peer_recv,
                                             peer_dup, st))
        else:
            L.check(lib.mg_ep_dispatch(lay._h, xd[r * Tl:(r + 1) * Tl].data_ptr(), d.data_ptr(), Tl, peer_recv, st))
        dst.append(d); rc.append(c); rp.append(p)
        base, ref_c, ref_p, over = ep_layout_reference(counts_all.cpu().numpy(), r, El, cap)
        assert not over.any()
        assert np.array_equal(c.cpu().numpy(), ref_c) and np.array_equal(p.cpu().numpy(), ref_p)
        # first row of every expert's run on this rank equals the host layout
        flat_idx, flat_dst = idx[r].cpu().view(-1).long(), d.cpu().view(-1).long()
        for e in flat_idx.unique().tolist():
            assert int(flat_dst[flat_idx == e].min()) == int(base[e])
    if dedup:
        # with 4 picks on 2 or 4 ranks some picks must share a rank: the tables are in use
        assert sum(int((t >= 0).sum()) for t in dupt) > 0
        for r, lay in enumerate(ranks):
            L.check(lib.mg_ep_fill_duplicates(lay._h, recv[r].data_ptr(), dupt[r].data_ptr(), cap, st))
        # every live row of every receive buffer holds the hidden state of the token that picked it
        for r in range(n_ranks):
            got = recv[r].cpu()
            for s_ in range(n_ranks):
                d_ = dst[s_].cpu().long().view(-1)
                mine = (d_ >> 24) == r
                rows = d_[mine] & 0xFFFFFF
                toks = torch.arange(Tl).repeat_interleave(k)[mine] + s_ * Tl
                assert torch.equal(got[rows].view(torch.int16), x[toks].view(torch.int16))
    for r, lay in enumerate(ranks):
        hb = torch.zeros(cap, spec.inter, dtype=torch.bfloat16, device=DEV)
        if push == "copy":
            # the copy engines carry every (expert, source rank) segment home; sizes from the counts on the host
            counts_host = counts_all.cpu().contiguous()
            L.check(lib.mg_ep_expert_ffn_copy_return(lay._h, recv[r].data_ptr(), rp[r].data_ptr(), rc[r].data_ptr(), cap,
                                                     lay.packed.data_ptr(), hb.data_ptr(), outb[r].data_ptr(), None,
                                                     counts_host.data_ptr(), peer_ret, 3, st))
        elif push:
            L.check(lib.mg_ep_expert_ffn_return(lay._h, recv[r].data_ptr(), rp[r].data_ptr(), rc[r].data_ptr(), cap,
                                                lay.packed.data_ptr(), hb.data_ptr(), outb[r].data_ptr(), None,
                                                backt[r].data_ptr(), peer_ret, 3, st))
        else:
            L.check(lib.mg_expert_ffn(lay._h, recv[r].data_ptr(), rp[r].data_ptr(), rc[r].data_ptr(), cap,
                                      lay.packed.data_ptr(), hb.data_ptr(), outb[r].data_ptr(), None, st))
    ys = []
    for r, lay in enumerate(ranks):
        xs = xd[r * Tl:(r + 1) * Tl]
        sh = lay.shared_ffn(xs)
        y = torch.empty(Tl, H, dtype=torch.bfloat16, device=DEV)
        if push == "copy":
            torch.cuda.synchronize()            # every owner's copies have landed
            delta = torch.empty(E, **i32)
            L.check(lib.mg_ep_mirror_delta(lay._h, counts_all.data_ptr(), delta.data_ptr(), st))
            # the return buffer is this rank's rows in its own expert-sorted order: the single-GPU plan's offsets
            own = torch.cumsum(counts_all[r].cpu().long(), 0) - counts_all[r].cpu().long()
            base_r, *_ = ep_layout_reference(counts_all.cpu().numpy(), r, El, cap)
            assert np.array_equal(delta.cpu().numpy(), own.numpy() - (base_r & 0xFFFFFF))
            L.check(lib.mg_ep_combine_mirror(lay._h, rett[r].data_ptr(), dst[r].data_ptr(), delta.data_ptr(),
                                             idx[r].data_ptr(), w[r].data_ptr(), sh.data_ptr(), Tl, y.data_ptr(), st))
        elif push:
            torch.cuda.synchronize()            # every owner's pushes (on their return streams) have landed
            L.check(lib.mg_ep_combine_slots(lay._h, rett[r].data_ptr(), outb[r].data_ptr(), dst[r].data_ptr(), idx[r].data_ptr(),
                                            w[r].data_ptr(), sh.data_ptr(), Tl, y.data_ptr(), st))
        else:
            L.check(lib.mg_ep_combine(lay._h, peer_out, dst[r].data_ptr(), idx[r].data_ptr(), w[r].data_ptr(),
                                      sh.data_ptr(), Tl, y.data_ptr(), st))
        ys.append(y)
    torch.cuda.synchronize()
    for lay in ranks:
        assert lay.device_status() == (0, 0)
    assert torch.equal(torch.cat(ys).cpu().view(torch.int16), y_ref.view(torch.int16))
