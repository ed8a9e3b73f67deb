"""CPU (gloo, world_size 2): the expert-parallel partition, layout and exchange logic."""
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from moe_gen_b200.ep import PEER_SHIFT, ep_layout_reference
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
