"""moe_gen_b200: the MoE-layer hot path of MoE-Gen for NVIDIA B200 (sm_100a).

Python here is host code only; all arithmetic is in libmoegen_b200.so, reached through
the C ABI declared in include/moegen_b200.h."""
from .lib import (COMBINE_BF16_PROD, COMBINE_BF16_SEQ, COMBINE_FP32, GATE_SIGMOID_NOAUX_TC,  # noqa: F401
                  GATE_SOFTMAX_GREEDY, GATE_SOFTMAX_GROUP_MAX, GATE_SOFTMAX_TOPK_RENORM, WEIGHT_BF16,
                  WEIGHT_FP8_BLOCK128, MoeGenError, load)
from .layer import MoELayer  # noqa: F401
from .patch import layer_from_deepseek, layer_from_mixtral, patch_decoder_layer, patch_moe_module  # noqa: F401
from .batching import ModuleBatchingConfig, MoEBatcher  # noqa: F401
