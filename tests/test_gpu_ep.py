"""GPU: expert-parallel forward over peer memory against the CPU oracle, as 2 ranks on 2 GPUs
(skipped on a single-GPU machine) and as a group of one rank, which runs the same host code,
collectives and kernels on one GPU."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

from oracle import moe_oracle as O
from tests import ep_worker

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("spec,T", [
    (O.LayerSpec(256, 128, 64, 4, 256, 4, 2, O.GATE_SIGMOID_NOAUX_TC, True, 2.5, O.WEIGHT_FP8_BLOCK128, O.COMBINE_FP32), 600),
    (O.LayerSpec(512, 256, 8, 2, 0, 1, 1, O.GATE_SOFTMAX_TOPK_RENORM, True, 1.0, O.WEIGHT_BF16, O.COMBINE_BF16_SEQ), 1000),
])
@pytest.mark.parametrize("world", [1, 2])
def test_expert_parallel_on_gpus(built_lib, spec, T, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        result = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=ep_worker.gpu_ep_worker, args=(r, world, port, spec, T, 9, result))
                 for r in range(world)]
        for p in procs:
            p.start()
        codes = ep_worker.join_all(procs, 300)
        assert all(c == 0 for c in codes), codes
        assert all(s == (0, 0) for s in result["status"]), result["status"]
        assert result["repeat_equal"]
        assert result["dedup_equal"]          # de-duplicated dispatch leaves the same rows as the plain one
        assert all(r in (None, True) for r in result["overflow_reported"]), result["overflow_reported"]
        assert result["routing_agree"] > 0.995
        assert result["rel_l2"] <= 1e-2
