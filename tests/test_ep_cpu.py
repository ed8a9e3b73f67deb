"""CPU (gloo, world_size 2): the expert-parallel partition, layout and exchange logic."""
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from moe_gen_b200.ep import PEER_SHIFT, ep_copy_plan_reference, ep_layout_reference, ep_mirror_delta_reference
from oracle import moe_oracle as O
from tests import ep_worker


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("n,E", [(2, 8), (4, 64), (8, 256)])
def test_layout_tiles_every_owner_buffer_exactly(n, E):
    rng = np.random.default_rng(n * E)
    counts = rng.integers(0, 300, size=(n, E)).astype(np.int32)
    counts[:, 3] = 0                                         # an expert nobody picks
    El = E // n
    cap = 1 << 22
    per_rank = [ep_layout_reference(counts, r, El, cap) for r in range(n)]
    for d in range(n):
        _, recv_counts, recv_pad, over = per_rank[d]
        assert not over.any()
        assert np.array_equal(recv_counts, counts.sum(0)[d * El:(d + 1) * El])
        assert (recv_pad % 128 == 0).all()
        for j in range(El):
            e = d * El + j
            pos = recv_pad[j]
            for s in range(n):                                # source ranks in order, contiguous
                base = per_rank[s][0][e]
                assert base >> PEER_SHIFT == d
                assert (base & ((1 << PEER_SHIFT) - 1)) == pos
                pos += counts[s, e]
            assert pos == recv_pad[j] + recv_counts[j] <= recv_pad[j + 1]


@pytest.mark.parametrize("n,E,k", [(2, 8, 2), (4, 32, 4), (8, 64, 6)])
def test_copy_return_rebuilds_every_rank_own_expert_sorted_order(n, E, k):
    """The return through the copy engines, simulated on the host: every owner lays the picks it received out
    as ep_layout says (expert-major, source ranks in order, tokens ascending), copies one segment per (expert,
    source rank) as ep_copy_plan says, and every rank must end up with its own picks in stable expert-sorted
    order; the per-expert offset turns a row of the owner's layout into that row."""
    rng = np.random.default_rng(100 * n + E)
    Tl, El, cap = 37, E // n, 1 << 20
    idx = np.stack([np.stack([rng.choice(E, size=k, replace=False) for _ in range(Tl)]) for _ in range(n)])   # [n, Tl, k]
    counts = np.stack([np.bincount(idx[s].ravel(), minlength=E) for s in range(n)]).astype(np.int64)
    layouts = [ep_layout_reference(counts, s, El, cap) for s in range(n)]
    mask = (1 << PEER_SHIFT) - 1
    # dst[s][t, j]: owner << shift | row, ranks inside an expert's run in token order (the stable placement)
    dst = np.zeros((n, Tl, k), dtype=np.int64)
    out_rows = [dict() for _ in range(n)]                     # owner -> {row: (source rank, token, slot)}
    for s in range(n):
        seen = np.zeros(E, dtype=np.int64)
        for t in range(Tl):
            for j in range(k):
                e = idx[s, t, j]
                d = layouts[s][0][e] + seen[e]
                seen[e] += 1
                dst[s, t, j] = d
                out_rows[d >> PEER_SHIFT][d & mask] = (s, t, j)
    mirrors = [dict() for _ in range(n)]
    for owner in range(n):
        for dest, dest_row, src_row, rows in ep_copy_plan_reference(counts, owner, El, cap):
            for i in range(rows):
                assert dest_row + i not in mirrors[dest]
                mirrors[dest][dest_row + i] = out_rows[owner][src_row + i]
    for s in range(n):
        assert sorted(mirrors[s]) == list(range(Tl * k))      # every row of the return buffer written once
        order = sorted(((idx[s, t, j], t, j) for t in range(Tl) for j in range(k)))
        assert [mirrors[s][r] for r in range(Tl * k)] == [(s, t, j) for _, t, j in order]
        delta = ep_mirror_delta_reference(counts, s, El)
        for t in range(Tl):
            for j in range(k):
                assert mirrors[s][(dst[s, t, j] & mask) + delta[idx[s, t, j]]] == (s, t, j)
    # an owner whose buffer is too small copies nothing (its picks were dropped at the dispatch)
    assert ep_copy_plan_reference(counts, 0, El, 128) == []


def test_layout_flags_a_receive_buffer_that_is_too_small():
    counts = np.full((2, 8), 100, dtype=np.int32)
    counts[:, :4] = 1000                                     # rank 0's experts are hot
    base, rc, rp, over = ep_layout_reference(counts, 1, 4, 2048)
    assert over.tolist() == [True, False]
    assert (base[:4] < 0).all() and (base[4:] >= 0).all()


@pytest.mark.parametrize("spec,T", [
    (O.LayerSpec(64, 32, 16, 4, 32, 4, 2, O.GATE_SIGMOID_NOAUX_TC, True, 2.5, O.WEIGHT_BF16, O.COMBINE_FP32), 96),
    (O.LayerSpec(64, 32, 8, 2, 0, 1, 1, O.GATE_SOFTMAX_TOPK_RENORM, True, 1.0, O.WEIGHT_BF16, O.COMBINE_FP32), 50),
])
def test_expert_parallel_two_gloo_ranks_match_single_process_oracle(spec, T):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        result = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=ep_worker.cpu_ep_worker, args=(r, 2, port, spec, T, 7, result)) for r in range(2)]
        for p in procs:
            p.start()
        codes = ep_worker.join_all(procs, 240)
        assert all(c == 0 for c in codes), codes
        assert result["counts_ok"]
        assert result["rel_l2"] < 1e-5
