"""Module-based batching for the MoE layer: the caller that makes T large.

MoE-Gen runs a model module by module over a large host-resident batch: the sequences are padded to
one length, cut into micro-batches of `MoE_prefill_micro_batch_size` sequences (prefill) or
`MoE_decoding_micro_batch_size` sequences of one token (decoding), and every micro-batch goes
through the layer in one call, padding tokens included (moe_gen/engine.py:485-491 pads every query
to max_input_length, :708-763 splits the batch with torch.split and runs one forward per
micro-batch; the micro-batch sizes come from
moe_gen/models/deepseek/deepseekv3/deepseekv3_initializer.py:864-900).  This file is that driver
for the MoE layer alone: it owns no model, only the cutting, the padding and the layer calls, so
that a MoELayer (or a patched reference module) sees the token counts the benchmark assumes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch


@dataclass
class ModuleBatchingConfig:
    """The fields of the reference's Module_Batching_Config that concern the MoE layer, with its own
    rule for their values (deepseekv3_initializer.py:864-900)."""
    MoE_prefill_micro_batch_size: int = 20
    MoE_decoding_micro_batch_size: int = 1
    expert_prefill_batch_size_upper_bound: int = 2048
    expert_decoding_batch_size_upper_bound: int = 2048
    global_batch_size: int = 1

    @classmethod
    def from_lengths(cls, padding_length: int, max_decoding_length: int, num_queries: int,
                     num_host_slots: Optional[int] = None) -> "ModuleBatchingConfig":
        """global batch = min(host KV slots, queries); sequences per MoE prefill micro-batch = 20, scaled
        down by 544 / context length for long contexts; decoding takes the whole global batch at once."""
        global_batch = min(num_host_slots if num_host_slots is not None else num_queries, num_queries)
        context_length = max_decoding_length + padding_length
        prefill = math.floor(20 * 544 / context_length) if context_length > 544 else 20
        return cls(MoE_prefill_micro_batch_size=max(1, prefill), MoE_decoding_micro_batch_size=max(1, global_batch),
                   global_batch_size=max(1, global_batch))


@dataclass
class BatchLog:
    """Token accounting of the calls a batcher made (for tests and reports)."""
    tokens_per_call: List[int] = field(default_factory=list)
    padding_tokens_per_call: List[int] = field(default_factory=list)

    @property
    def calls(self) -> int:
        return len(self.tokens_per_call)


class MoEBatcher:
    """Cuts a batch of sequences into MoE micro-batches and runs `layer` once per micro-batch.

    `layer` is anything that maps [T, H] -> [T, H] (MoELayer.forward, EPMoELayer.forward, a patched
    module's forward over [1, T, H]).  Tokens are independent in the layer, so the result equals
    running every sequence on its own, bit for bit."""

    def __init__(self, layer: Callable[[torch.Tensor], torch.Tensor], config: ModuleBatchingConfig):
        self.layer = layer
        self.config = config
        self.log = BatchLog()

    # ------------------------------------------------------------------ prefill
    def pad_sequences(self, sequences: Sequence[torch.Tensor], pad_to: int) -> (torch.Tensor, torch.Tensor):
        """[S_i, H] tensors -> ([B, pad_to, H], mask [B, pad_to]).  Padding goes in front (the reference's
        tokenizer pads on the left for generation) and is zero; longer sequences are cut from the front,
        as truncation to max_input_length does."""
        H = sequences[0].shape[-1]
        B = len(sequences)
        out = torch.zeros(B, pad_to, H, dtype=sequences[0].dtype, device=sequences[0].device)
        mask = torch.zeros(B, pad_to, dtype=torch.bool, device=sequences[0].device)
        for i, s in enumerate(sequences):
            s = s[-pad_to:]
            n = s.shape[0]
            out[i, pad_to - n:] = s
            mask[i, pad_to - n:] = True
        return out, mask

    def prefill(self, hidden: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """hidden [B, S, H] (already padded to one length) -> [B, S, H]: micro-batches of
        MoE_prefill_micro_batch_size sequences (torch.split, engine.py:708-720), every token of a
        micro-batch, padding included, in one layer call."""
        B, S, H = hidden.shape
        out = torch.empty_like(hidden)
        start = 0
        masks = None if attention_mask is None else torch.split(attention_mask, self.config.MoE_prefill_micro_batch_size)
        for i, part in enumerate(torch.split(hidden, self.config.MoE_prefill_micro_batch_size)):
            n = part.shape[0]
            y = self.layer(part.reshape(n * S, H))
            out[start:start + n] = y.reshape(n, S, H)
            start += n
            self.log.tokens_per_call.append(n * S)
            self.log.padding_tokens_per_call.append(0 if masks is None else int((~masks[i].bool()).sum()))
        return out

    def prefill_sequences(self, sequences: Sequence[torch.Tensor], pad_to: int) -> List[torch.Tensor]:
        """Variable-length sequences: padded to pad_to, batched, and cut back to their own tokens."""
        padded, mask = self.pad_sequences(sequences, pad_to)
        y = self.prefill(padded, mask)
        return [y[i, pad_to - min(s.shape[0], pad_to):] for i, s in enumerate(sequences)]

    # ------------------------------------------------------------------ decoding
    def decode_step(self, hidden: torch.Tensor) -> torch.Tensor:
        """hidden [B, 1, H] or [B, H] (one new token per sequence) -> same shape: micro-batches of
        MoE_decoding_micro_batch_size sequences, by default the whole global batch in one call."""
        shape = hidden.shape
        h2 = hidden.reshape(shape[0], shape[-1])
        out = torch.empty_like(h2)
        start = 0
        for part in torch.split(h2, self.config.MoE_decoding_micro_batch_size):
            n = part.shape[0]
            out[start:start + n] = self.layer(part.contiguous())
            start += n
            self.log.tokens_per_call.append(n)
            self.log.padding_tokens_per_call.append(0)
        return out.view(shape)
