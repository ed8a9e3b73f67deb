"""GPU: every named benchmark configuration at its full layer shape.

The CPU oracle cannot run these sizes in test time, so each case is checked through
  * routing on identical fp32 logits against oracle.route over ALL tokens (sets exact, no exemptions),
  * size-independent properties of the permutation (histogram, bijection, stable order, a checksum
    of checksums over the scattered rows),
  * at least 64 sampled tokens whose layer output is recomputed in fp32 with the oracle's expert
    function from the same seeded weights (1e-2 relative L2, the bound of the reference's
    fp32-accumulated output),
and the DeepSeek-V2-Lite configuration, which the reference itself runs on CPU, against the fixture
recorded from the reference's DeepseekV2MoE at the full size (tests/golden/v2lite_full.npz)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import bench
from oracle import moe_oracle as O
from tests.util import bf16_from_bits, load_golden, make_layer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_LAYER = 1e-2
N_SAMPLED = 64

# (workload, tokens, Zipf exponent of the router bias): configurations 1-5 of the benchmark
FULL_CASES = [("v2lite", 2048, 0.0), ("mixtral8x7b", 16384, 0.0), ("v2_236b", 32768, 0.0), ("v2_236b", 512, 0.0),
              ("v3", 65536, 0.0)] + [("v3", T, 1.2) for T in (64, 256, 1024, 4096, 16384)]


@pytest.fixture(scope="module")
def layers(built_lib):
    """One resident layer per workload, built on first use (the V3 layer holds 11 GB of weights)."""
    cache = {}

    def get(name):
        if name not in cache:
            if name == "v3" and torch.cuda.mem_get_info(0)[0] < 90e9:
                pytest.skip("needs ~80 GB of free device memory")
            cache[name] = bench.build_layer(name, torch.device(DEV))
        return cache[name]
    yield get
    for layer in cache.values():
        layer.close()


def _spec(name):
    H, I, E, k, Is, G, keep, gating, norm, scale, wfmt, comb = bench.WORKLOADS[name][:12]
    return O.LayerSpec(H, I, E, k, Is, G, keep, gating, norm, scale, wfmt, comb, name)


def _expert_fp32(name, layer, e):
    ws = bench.expert_tensors(name, torch.device(DEV), e)
    if isinstance(ws[0], tuple):
        ws = [layer.dequant_fp8(q, s) for q, s in ws]
    return [m.float() for m in ws]


def _sampled_reference(name, layer, x, idx, w, tokens):
    """fp32 layer output of the sampled tokens from the given routing: oracle.swiglu_mlp per expert,
    every needed expert's weights regenerated once from the seed."""
    spec = _spec(name)
    xs = x[tokens].float()
    ref = torch.zeros(len(tokens), spec.hidden, device=DEV)
    if spec.inter_shared:
        ref += O.swiglu_mlp(xs, *_expert_fp32(name, layer, -1))
    pick_e = idx[tokens].long()
    pick_w = w[tokens]
    for e in pick_e.unique().tolist():
        rows, slots = (pick_e == e).nonzero(as_tuple=True)
        out = O.swiglu_mlp(xs[rows], *_expert_fp32(name, layer, e))
        ref.index_add_(0, rows, out * pick_w[rows, slots].unsqueeze(1))
    return ref


def _permutation_properties(layer, x, idx):
    T, k, E = x.shape[0], layer.k, layer.E
    counts, offsets, pad, dst = layer.permute_plan(idx)
    assert int(counts.sum()) == T * k and int(offsets[-1]) == T * k
    assert torch.equal(counts.long(), torch.bincount(idx.view(-1).long(), minlength=E))
    assert torch.equal(offsets[1:] - offsets[:-1], counts)
    assert torch.equal(pad[1:] - pad[:-1], (counts + 127) // 128 * 128)
    # the placement is a bijection onto the experts' segments, tokens ascending inside a segment
    flat = dst.view(-1).long()
    assert torch.unique(flat).numel() == T * k
    seg = torch.searchsorted(pad[1:].long().contiguous(), flat, right=True)
    assert torch.equal(seg, idx.view(-1).long())
    assert bool((flat - pad.long()[seg] < counts.long()[seg]).all())
    order = torch.argsort(flat)
    tok = order // k
    same_seg = seg[order][1:] == seg[order][:-1]
    assert bool((tok[1:][same_seg] > tok[:-1][same_seg]).all())
    # checksum of checksums: the scattered rows carry exactly k copies of every token's bits
    rows = layer.padded_rows(T * k)
    perm = layer.permute_rows(x, dst, rows)
    live = torch.zeros(rows, dtype=torch.bool, device=DEV)
    live[flat] = True
    assert int(perm.view(torch.int16)[live].to(torch.int64).sum()) == k * int(x.view(torch.int16).to(torch.int64).sum())
    return counts


@pytest.mark.parametrize("name,T,zipf", FULL_CASES)
def test_named_configuration_at_full_shape(layers, name, T, zipf):
    layer = layers(name)
    spec = _spec(name)
    dev = torch.device(DEV)
    gate_w, bias = bench.router_tensors(name, dev, zipf)
    layer.set_router(gate_w, bias)
    x = bench.make_tokens(name, T, dev, 0, zipf)
    E, k = spec.n_experts, spec.top_k

    # ---- routing on identical fp32 logits: every token against the oracle, no exemptions
    if spec.gating == O.GATE_SOFTMAX_TOPK_RENORM:
        logits = F.linear(x, layer.gate_w).float().contiguous()        # the bf16 router of the Mixtral block
    else:
        logits = F.linear(x.float(), layer.gate_w.float()).contiguous()
    idx, w = layer.route_topk(logits)
    oi, ow = O.route(spec, logits.cpu(), None if layer.bias is None else layer.bias.cpu())
    gi, gw = O.canonical_sets(idx.cpu().long(), w.cpu())
    ri, rw = O.canonical_sets(oi, ow)
    assert torch.equal(gi, ri), f"{int((gi != ri).any(1).sum())} of {T} tokens routed differently on identical logits"
    assert float(((gw - rw).abs() / rw.abs().clamp_min(1e-12)).max()) <= 1e-6
    if spec.n_group > 1:
        groups = (idx // (E // spec.n_group)).long()
        used = torch.zeros(T, spec.n_group, dtype=torch.bool, device=DEV).scatter_(1, groups, True).sum(1)
        assert int(used.max()) <= spec.topk_group

    # ---- permutation properties, and the skew the Zipf cases are there for
    counts = _permutation_properties(layer, x, idx)
    if zipf > 0:
        mean = T * k / E
        assert int(counts.max()) > 10 * mean, "the skewed case has no hot expert"
        if T <= 1024:
            assert int((counts == 0).sum()) > 0, "the skewed case has no empty expert"

    # ---- whole layer on those logits: deterministic, finite, sampled tokens against the fp32 oracle
    y = layer.forward_from_logits(x, logits).clone()
    y2 = layer.forward_from_logits(x, logits)
    torch.cuda.synchronize()
    assert layer.device_status() == (0, 0)
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
    assert bool(torch.isfinite(y.float()).all())
    tokens = torch.linspace(0, T - 1, min(N_SAMPLED, T)).round().long().unique().to(DEV)
    ref = _sampled_reference(name, layer, x, idx, w, tokens)
    got = y[tokens].float()
    per_token = (got - ref).norm(dim=1) / ref.norm(dim=1).clamp_min(1e-30)
    assert float(per_token.max()) <= TOL_LAYER, float(per_token.max())
    assert O.rel_l2(got.cpu(), ref.cpu()) <= TOL_LAYER

    # ---- the default forward's routing (router product on the tensor cores + near-tie fix-up)
    idx_f, w_f, logits_f, fix = layer.gate_route(x)
    n_fix = int(fix[0])
    if spec.gating == O.GATE_SOFTMAX_TOPK_RENORM:
        # bf16-rounded logits tie exactly and both sides pick the lower id; a logit that rounds to the other
        # bf16 neighbour can still move a token
        assert n_fix == 0
        differ = (idx_f.sort(1).values != idx.sort(1).values).any(1)
        assert int(differ.sum()) <= max(2, T // 500)
    else:
        # equals the routing of the correctly rounded fp32 logits (fp64 product, rounded once): every
        # token, no exemptions
        exact = F.linear(x.double(), layer.gate_w.double()).float().contiguous()
        idx_e, w_e = layer.route_topk(exact)
        assert torch.equal(idx_f.sort(1).values, idx_e.sort(1).values), \
            f"{int((idx_f.sort(1).values != idx_e.sort(1).values).any(1).sum())} of {T} tokens differ from exact-logit routing"
        order_f, order_e = idx_f.argsort(1), idx_e.argsort(1)
        assert float(((w_f.gather(1, order_f) - w_e.gather(1, order_e)).abs() / w_e.gather(1, order_e).abs()).max()) <= 2e-4
        assert n_fix <= max(8, T // 10), f"{n_fix} of {T} tokens re-routed"
        # the error bound the flagging assumes holds with a factor of two to spare on this input
        raw = layer.gate_logits(x)
        bound = (6.0e-9 * spec.hidden + 4.0e-6) * exact.abs().amax(1, keepdim=True).clamp_min(1.0)
        assert float(((raw - exact).abs() / bound).max()) <= 0.5
        again = fix[4:4 + n_fix].long()
        assert again.unique().numel() == n_fix
        # the recomputed logits are the exact product to the last bit or the one next to it
        n_pairs = min(int(fix[2]), 8 * T + 64)
        pairs = fix[4 + 2 * T:4 + 2 * T + 2 * n_pairs].long().view(-1, 2)
        got, want = logits_f[pairs[:, 0], pairs[:, 1]], exact[pairs[:, 0], pairs[:, 1]]
        assert bool(((got - want).abs() <= torch.finfo(torch.float32).eps * want.abs().clamp_min(2.0 ** -126)).all())
        rows = fix[4 + T:4 + T + int(fix[1])].long()
        assert bool(((logits_f[rows] - exact[rows]).abs() <= torch.finfo(torch.float32).eps * exact[rows].abs().clamp_min(2.0 ** -126)).all())
        if T >= 16384:
            assert n_fix > 0
        differ = (idx_f.sort(1).values != idx.sort(1).values).any(1)     # against fp32 cuBLAS logits: near ties only
        gap = O.kth_gap(spec, logits.cpu(), None if layer.bias is None else layer.bias.cpu())
        assert int(differ.sum()) <= max(2, T // 500)
        assert bool((gap[differ.cpu()] < 1e-4).all()), "a token with a clear score gap was routed differently"
    yf = layer.forward(x)
    torch.cuda.synchronize()
    assert layer.device_status() == (0, 0)
    agree = ~differ[tokens]
    if bool(agree.any()):
        assert O.rel_l2(yf[tokens][agree].float().cpu(), ref[agree].cpu()) <= TOL_LAYER


def test_v2lite_full_size_against_the_reference_fixture(built_lib):
    """DeepSeek-V2-Lite layer exactly as the benchmark names it (T=2048, H=2048, 64 experts, top-6,
    I=1408, two shared experts, seed 0) against what the reference's DeepseekV2MoE produced on CPU:
    routing and histogram exact on the reference's logits, output rows within 1e-2 of its fp32 run."""
    spec = O.named_spec("v2lite")
    g = load_golden("v2lite_full")
    T, seed = int(g["T"]), int(g["seed"])
    x, W = O.make_inputs(spec, T, seed)
    layer = make_layer(spec, W, DEV)
    xd = x.to(DEV)
    logits = O.gate_logits(x, W.gate_w).to(DEV)         # the fp32 product the reference's gate computes
    idx, w = layer.route_topk(logits)
    gi, gw = O.canonical_sets(idx.cpu().long(), w.cpu())
    assert np.array_equal(gi.numpy().astype(np.int16), g["topk_idx"])       # zero exemptions
    assert float(np.abs(gw.numpy() - g["topk_w"]).max()) <= 2e-7
    counts, offsets, pad, dst = layer.permute_plan(idx)
    assert np.array_equal(counts.cpu().numpy(), g["counts"])
    rows = torch.from_numpy(g["rows"].astype(np.int64))
    gold = torch.from_numpy(g["y_gold_fp32_rows"])
    ref_bf16 = bf16_from_bits(g["y_ref_bf16_rows"]).float()
    y = layer.forward_from_logits(xd, logits)
    torch.cuda.synchronize()
    assert layer.device_status() == (0, 0)
    got = y.cpu().float()[rows]
    assert O.rel_l2(got, gold) <= TOL_LAYER
    assert float(((got - gold).norm(dim=1) / gold.norm(dim=1)).max()) <= TOL_LAYER
    assert O.rel_l2(got, ref_bf16) < 1.5e-2
    # the default forward (tensor-core router product) stays inside the same bound
    yf = layer.forward(xd).cpu().float()[rows]
    assert O.rel_l2(yf, gold) <= TOL_LAYER
