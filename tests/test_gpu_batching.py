"""GPU: the module-based batching driver on the native layer.  Tokens are independent in the layer, so
a micro-batch of padded sequences in one call must equal every sequence run on its own, bit for bit,
and stay within the layer's bound of the CPU oracle."""
import pytest
import torch

from moe_gen_b200 import ModuleBatchingConfig, MoEBatcher
from oracle import moe_oracle as O
from tests.util import make_layer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_batched_prefill_and_decoding_equal_per_sequence_forwards(built_lib):
    spec = O.LayerSpec(256, 128, 64, 4, 128, 4, 2, O.GATE_SIGMOID_NOAUX_TC, True, 2.5, O.WEIGHT_FP8_BLOCK128,
                       O.COMBINE_FP32)
    B, S = 11, 48
    x, W = O.make_inputs(spec, B * S, 77)
    layer = make_layer(spec, W, DEV)
    hidden = x.view(B, S, spec.hidden).to(DEV)
    mask = torch.ones(B, S, dtype=torch.bool, device=DEV)
    mask[:, :5] = False
    batcher = MoEBatcher(layer.forward, ModuleBatchingConfig(MoE_prefill_micro_batch_size=4, MoE_decoding_micro_batch_size=8))
    y = batcher.prefill(hidden, mask)
    torch.cuda.synchronize()
    assert layer.device_status() == (0, 0)
    assert batcher.log.tokens_per_call == [4 * S, 4 * S, 3 * S]
    assert batcher.log.padding_tokens_per_call == [20, 20, 15]
    for b in range(B):                                    # one sequence at a time: the same bits
        yb = layer.forward(hidden[b])
        assert torch.equal(yb.view(torch.int16), y[b].view(torch.int16))
    gold = O.layer_forward(spec, x, W, gold_fp32=True)["y"].view(B, S, spec.hidden)
    assert O.rel_l2(y.cpu().float(), gold) <= 1e-2
    # decoding: one token per sequence, the whole batch in micro-batches of 8
    step = hidden[:, -1:, :].contiguous()
    yd = batcher.decode_step(step)
    torch.cuda.synchronize()
    assert batcher.log.tokens_per_call[-2:] == [8, 3]
    assert torch.equal(yd.view(torch.int16), y[:, -1:, :].contiguous().view(torch.int16))
    # variable lengths: padded in front, cut back to each sequence's own tokens
    seqs = [hidden[b, S - n:] for b, n in enumerate((48, 7, 31))]
    outs = batcher.prefill_sequences(seqs, pad_to=S)
    for b, (o, s) in enumerate(zip(outs, seqs)):
        assert torch.equal(o.view(torch.int16), y[b, S - s.shape[0]:].view(torch.int16))
