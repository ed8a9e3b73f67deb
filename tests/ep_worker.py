"""Worker functions for the multi-process expert-parallel tests (spawned, one per rank)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import moe_oracle as O  # noqa: E402


def _init(rank, world, port, backend):
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    # finite: a rank that never joins or a stalled collective raises in the others instead of waiting forever
    dist.init_process_group(backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))


def join_all(procs, timeout):
    """Joins the spawned ranks; whatever is still alive after the timeout is ended (terminate, then
    kill) so that no rank keeps a GPU, an IPC mapping or a communicator.  Returns the exit codes."""
    for p in procs:
        p.join(timeout=timeout)
    for p in procs:
        if p.is_alive():
            p.terminate()
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    return [p.exitcode for p in procs]


def cpu_ep_worker(rank, world, port, spec, T_global, seed, result):
    """Expert-parallel layer on CPU ranks (gloo): routing, layout, exchange, experts, return.

    Rows are exchanged by gathering (destination, row) lists, which models 'every rank writes
    its rows into the owner's buffer'; the layout comes from ep_layout_reference, the host
    restatement of the device layout kernel."""
    from moe_gen_b200.ep import PEER_SHIFT, ep_layout_reference
    _init(rank, world, port, "gloo")
    torch.set_num_threads(2)
    x_all, W = O.make_inputs(spec, T_global, seed)
    Tl = T_global // world
    x = x_all[rank * Tl:(rank + 1) * Tl]
    E, El, k = spec.n_experts, spec.n_experts // world, spec.top_k
    logits = O.gate_logits(x, W.gate_w, bf16_out=(spec.gating == O.GATE_SOFTMAX_TOPK_RENORM))
    idx, w = O.route(spec, logits, W.bias)
    counts = torch.bincount(idx.reshape(-1), minlength=E).to(torch.int32)
    gathered = [torch.empty_like(counts) for _ in range(world)]
    dist.all_gather(gathered, counts)
    counts_all = torch.stack(gathered).numpy()
    cap = ((T_global * k + 127) // 128 + El) * 128
    send_base, recv_counts, recv_pad, over = ep_layout_reference(counts_all, rank, El, cap)
    assert not over.any()
    # stable placement of this rank's picks (tokens ascending inside an expert)
    flat = idx.reshape(-1)
    order = flat.argsort(stable=True)
    off = np.concatenate([[0], np.cumsum(counts.numpy())])
    dst = np.empty(Tl * k, dtype=np.int64)
    for pos, f in enumerate(order.tolist()):
        e = int(flat[f])
        dst[f] = send_base[e] + (pos - off[e])
    # dispatch: everybody learns every (dst, row); owners keep what is theirs
    mine = [(int(d), x[f // k]) for f, d in enumerate(dst.tolist())]
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    recv = torch.zeros(cap, spec.hidden, dtype=torch.float32)
    filled = np.zeros(cap, dtype=np.int32)
    for lst in everyone:
        for d, row in lst:
            if d >> PEER_SHIFT == rank:
                recv[d & ((1 << PEER_SHIFT) - 1)] = row.float()
                filled[d & ((1 << PEER_SHIFT) - 1)] += 1
    # every row of every local segment written exactly once, nothing outside the segments
    expect = np.zeros(cap, dtype=np.int32)
    for j in range(El):
        expect[recv_pad[j]:recv_pad[j] + recv_counts[j]] = 1
    assert np.array_equal(filled, expect)
    out = torch.zeros_like(recv)
    for j in range(El):
        a, n = int(recv_pad[j]), int(recv_counts[j])
        if n:
            e = rank * El + j
            out[a:a + n] = O.swiglu_mlp(recv[a:a + n], W.w_gate[e].float(), W.w_up[e].float(), W.w_down[e].float())
    outs = [None] * world
    dist.all_gather_object(outs, out)
    rows = torch.stack([outs[int(d) >> PEER_SHIFT][int(d) & ((1 << PEER_SHIFT) - 1)] for d in dst.tolist()])
    y = (rows.view(Tl, k, -1) * w.unsqueeze(-1)).sum(dim=1)
    if W.shared is not None:
        y = y + O.swiglu_mlp(x.float(), *[m.float() for m in W.shared])
    ys = [None] * world
    dist.all_gather_object(ys, y)
    if rank == 0:
        gold = O.layer_forward(spec, x_all, W, gold_fp32=True)
        result["rel_l2"] = O.rel_l2(torch.cat(ys), gold["y"])
        result["counts_ok"] = bool(np.array_equal(counts_all.sum(0), gold["counts"].numpy()))
    dist.barrier()
    dist.destroy_process_group()


def gpu_ep_worker(rank, world, port, spec, T_global, seed, result):
    """Expert-parallel layer on GPUs (NCCL + peer memory) against the CPU oracle."""
    from moe_gen_b200.ep import EPMoELayer
    from tests.util import make_layer
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    _init(rank, world, port, "nccl")
    x_all, W = O.make_inputs(spec, T_global, seed)
    Tl = T_global // world
    dev = f"cuda:{rank}"
    layer = make_layer(spec, W, dev, rank, world)
    ep = EPMoELayer(layer, push_return=True)             # owners push results home; the pulled return follows below
    x = x_all[rank * Tl:(rank + 1) * Tl].to(dev)
    ys = []
    for _ in range(2):                                   # twice: buffers are reused across forwards
        y = ep.forward(x)
        torch.cuda.synchronize()
        ys.append(y.cpu())
    ep.dedup = False                                     # one row per (token, expert) on the wire
    y_plain = ep.forward(x)
    torch.cuda.synchronize()
    same = bool(torch.equal(y_plain.cpu().view(torch.int16), ys[0].view(torch.int16)))
    ep.push_return = False                               # the combine gathers from the owners (no pushed return)
    for dd in (False, True):
        ep.dedup = dd
        y_pull = ep.forward(x)
        torch.cuda.synchronize()
        same = same and bool(torch.equal(y_pull.cpu().view(torch.int16), ys[0].view(torch.int16)))
    ep.copy_return = True                                # the copy engines carry the results home
    for dd in (False, True):
        ep.dedup = dd
        for _ in range(2):
            y_copy = ep.forward(x)
            torch.cuda.synchronize()
            same = same and bool(torch.equal(y_copy.cpu().view(torch.int16), ys[0].view(torch.int16)))
    yh_copy = ep.forward_host(x.cpu().pin_memory(), n_chunks=2)
    same = same and bool(torch.equal(yh_copy.view(torch.int16), ys[0].view(torch.int16)))
    ep.copy_return = False
    ep.push_return = True
    # host buffers in two parts per rank (last: it re-allocates the shared buffers for the part size)
    ep.dedup = True
    yh = ep.forward_host(x.cpu().pin_memory(), n_chunks=2)
    same = same and bool(torch.equal(yh.view(torch.int16), ys[0].view(torch.int16)))
    # two pipelined micro-batches, each with its own stream, buffers and process group
    ep_m = EPMoELayer(layer, n_micro=2)
    y_m = ep_m.forward(x)
    torch.cuda.synchronize()
    same = same and bool(torch.equal(y_m.cpu().view(torch.int16), ys[0].view(torch.int16)))
    ep_m.copy_return = True
    y_m = ep_m.forward(x)
    torch.cuda.synchronize()
    same = same and bool(torch.equal(y_m.cpu().view(torch.int16), ys[0].view(torch.int16)))
    status = layer.device_status()
    # a receive buffer that is too small must be reported, not silently produce a partial result
    overflow_reported = None
    if spec.n_experts <= 8:
        ep_s = EPMoELayer(layer, capacity_factor=0.3, min_headroom=0)
        ep_s.forward(x)
        try:
            ep_s.check_status(wait=True)
            overflow_reported = False
        except RuntimeError as e:
            overflow_reported = "overflowed" in str(e)
        ep_s.close()
        assert layer.device_status() == (0, 0)            # reading it cleared the word
    idx_l, w_l = layer.gate_route(x)[:2]
    gath = [None] * world
    dist.all_gather_object(gath, (ys[0], ys[1], status, same, idx_l.cpu(), w_l.cpu(), overflow_reported))
    if rank == 0:
        gold = O.layer_forward(spec, x_all, W, gold_fp32=True)
        y0 = torch.cat([g[0] for g in gath]).float()
        y1 = torch.cat([g[1] for g in gath]).float()
        # tokens whose routing agrees with the oracle's (a router logit that rounds differently can flip
        # a near-tie, above all with the Mixtral block's bf16 logits): the output bound applies to those
        idx_all = torch.cat([g[4] for g in gath]).long()
        w_all = torch.cat([g[5] for g in gath])
        agree = (O.canonical_sets(idx_all, w_all)[0] == O.canonical_sets(gold["topk_idx"], gold["topk_w"])[0]).all(1)
        result["routing_agree"] = float(agree.float().mean())
        result["rel_l2"] = O.rel_l2(y0[agree], gold["y"][agree])
        result["repeat_equal"] = bool(torch.equal(y0, y1))
        result["status"] = [g[2] for g in gath]
        result["dedup_equal"] = all(g[3] for g in gath)
        result["overflow_reported"] = [g[6] for g in gath]
    dist.barrier()
    ep_m.close()
    ep.close()
    dist.destroy_process_group()
