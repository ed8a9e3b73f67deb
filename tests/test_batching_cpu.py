"""CPU: token accounting of the module-based batching driver (moe_gen_b200/batching.py) with a
stand-in layer; the micro-batch rule against the values the reference's initializer computes
(moe_gen/models/deepseek/deepseekv3/deepseekv3_initializer.py:864-900)."""
import torch

from moe_gen_b200.batching import ModuleBatchingConfig, MoEBatcher


def test_micro_batch_rule_follows_the_reference_initializer():
    # context <= 544: 20 sequences per MoE prefill micro-batch; decoding takes the global batch
    c = ModuleBatchingConfig.from_lengths(padding_length=512, max_decoding_length=32, num_queries=5000, num_host_slots=3000)
    assert (c.MoE_prefill_micro_batch_size, c.MoE_decoding_micro_batch_size, c.global_batch_size) == (20, 3000, 3000)
    # longer contexts scale the prefill micro-batch down by 544 / context
    c = ModuleBatchingConfig.from_lengths(padding_length=1024, max_decoding_length=64, num_queries=100)
    assert c.MoE_prefill_micro_batch_size == (20 * 544) // 1088 == 10
    assert c.global_batch_size == c.MoE_decoding_micro_batch_size == 100
    assert c.expert_prefill_batch_size_upper_bound == 2048


def test_prefill_cuts_the_batch_like_torch_split_and_counts_padding():
    calls = []

    def layer(x):                               # a token-wise map, so batching must not change results
        calls.append(x.shape)
        return x * 2 + 1
    cfg = ModuleBatchingConfig(MoE_prefill_micro_batch_size=20)
    b = MoEBatcher(layer, cfg)
    hidden = torch.randn(47, 512, 8)
    mask = torch.ones(47, 512, dtype=torch.bool)
    mask[:, :100] = False                       # 100 padding tokens in front of every sequence
    y = b.prefill(hidden, mask)
    assert torch.equal(y, hidden * 2 + 1)
    assert b.log.tokens_per_call == [20 * 512, 20 * 512, 7 * 512]          # T = sequences x padded length
    assert b.log.padding_tokens_per_call == [20 * 100, 20 * 100, 7 * 100]   # padding goes through the layer too
    assert [tuple(s) for s in calls] == [(10240, 8), (10240, 8), (3584, 8)]
    # the benchmark's T: 128 sequences of 512 tokens in one micro-batch
    b2 = MoEBatcher(layer, ModuleBatchingConfig(MoE_prefill_micro_batch_size=128))
    b2.prefill(torch.zeros(128, 512, 8))
    assert b2.log.tokens_per_call == [65536]


def test_variable_length_sequences_are_padded_in_front_and_cut_back():
    b = MoEBatcher(lambda x: x + 1, ModuleBatchingConfig(MoE_prefill_micro_batch_size=2))
    seqs = [torch.full((n, 4), float(n)) for n in (3, 7, 5)]
    outs = b.prefill_sequences(seqs, pad_to=6)
    assert [o.shape[0] for o in outs] == [3, 6, 5]          # the 7-token sequence is truncated to 6, from the front
    assert all(torch.equal(o, torch.full_like(o, float(n) + 1)) for o, n in zip(outs, (3, 7, 5)))
    assert b.log.tokens_per_call == [12, 6] and b.log.padding_tokens_per_call == [3, 1]


def test_decode_step_takes_the_global_batch_in_micro_batches():
    b = MoEBatcher(lambda x: -x, ModuleBatchingConfig(MoE_decoding_micro_batch_size=1000))
    h = torch.randn(2500, 1, 16)
    y = b.decode_step(h)
    assert y.shape == h.shape and torch.equal(y, -h)
    assert b.log.tokens_per_call == [1000, 1000, 500]
