"""GPU: the allocation-free permute plan (mg_permute_plan_static) gives exactly what
mg_permute_plan gives.

Some users of the library cannot allocate device memory when they call it: an engine that
claimed all free memory for its weight and KV buffers at start-up, or a decode loop that
cannot afford the device-wide stall of a cudaMalloc.  For them the plan's scratch sits in a
fixed array inside the library.  The array is shared by all calls and is never cleared, so
the check runs two calls in a row with different inputs: the second must not be disturbed by
what the first left behind.  This file sorts last on purpose, so a run that stops at the
first failure has already been through every other test."""
import ctypes as C

import pytest
import torch

from moe_gen_b200 import lib as L
from oracle import moe_oracle as O
from tests.util import make_layer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _plan_static(layer, idx, expert_lo=0, n_plan=None):
    n = layer.E if n_plan is None else n_plan
    T = idx.shape[0]
    counts = torch.full((n,), -7, dtype=torch.int32, device=DEV)
    offsets = torch.full((n + 1,), -7, dtype=torch.int32, device=DEV)
    pad = torch.full((n + 1,), -7, dtype=torch.int32, device=DEV)
    dst = torch.full((T, layer.k), -7, dtype=torch.int32, device=DEV)
    rc = layer.lib.mg_permute_plan_static(layer._h, idx.data_ptr(), T, expert_lo, n, counts.data_ptr(),
                                          offsets.data_ptr(), pad.data_ptr(), dst.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
    return rc, (counts, offsets, pad, dst)


def test_static_plan_equals_plan_on_two_calls_in_a_row(built_lib):
    spec = O.LayerSpec(256, 128, 256, 8)
    layer = make_layer(spec, O.LayerWeights(torch.zeros(256, 256, dtype=torch.bfloat16), None), DEV, 0, 256)
    gen = torch.Generator().manual_seed(123)
    cases = []
    for T in (5000, 777):                          # the second call is smaller: stale words stay behind it
        scores = torch.rand(T, 256, generator=gen)
        scores[:, 3] = -1.0
        cases.append(scores.topk(8, dim=-1).indices.to(torch.int32).to(DEV))
    torch.cuda.synchronize()
    results = []
    for i, idx in enumerate(cases):
        free_before = torch.cuda.mem_get_info()[0]
        rc, got = _plan_static(layer, idx)
        torch.cuda.synchronize()
        assert rc == 0, layer.lib.mg_last_error()
        if i == 1:                                 # nothing was allocated on the device by the call
            assert torch.cuda.mem_get_info()[0] == free_before
        results.append(got)
    for idx, got in zip(cases, results):
        want = layer.permute_plan(idx)
        torch.cuda.synchronize()
        for g, w in zip(got, want):
            assert torch.equal(g, w)
    # a sub-range of experts, as an expert-parallel rank would ask for
    rc, got = _plan_static(layer, cases[0], expert_lo=64, n_plan=32)
    assert rc == 0
    for g, w in zip(got, layer.permute_plan(cases[0], expert_lo=64, n_plan=32)):
        assert torch.equal(g, w)
    assert layer.device_status() == (0, 0)


def test_static_plan_rejects_sizes_beyond_its_scratch(built_lib):
    spec = O.LayerSpec(256, 128, 512, 8)
    layer = make_layer(spec, O.LayerWeights(torch.zeros(512, 256, dtype=torch.bfloat16), None), DEV, 0, 512)
    T = 65536 + 256                                # one block more than the array holds at 512 experts
    idx = torch.arange(8, dtype=torch.int32, device=DEV).repeat(T, 1).contiguous()
    rc, _ = _plan_static(layer, idx)
    assert rc == -7
    assert b"built-in scratch" in layer.lib.mg_last_error()
    rc, _ = _plan_static(layer, idx[:65536])       # exactly the maximum is accepted
    torch.cuda.synchronize()
    assert rc == 0
