"""(parity: inference/v2/modules/configs/unembed_config.py:12-39)"""
from typing import Optional

from ...inference_utils import DtypeEnum, NormTypeEnum
from ..ds_module import DSModuleConfig


class DSUnembedConfig(DSModuleConfig):
    dtype: DtypeEnum = DtypeEnum.fp16
    norm_type: Optional[NormTypeEnum] = None
    model_dim: int
    max_sequences: int
    vocab_size: int
    eps: float = 1e-5
    norm_weight_offset: float = 0.0  # the final norm multiplies by (weight + offset): 1.0 for zero-centred weights (applied as 1 + w)
    logit_softcap: float = 0.0  # > 0: logits <- cap * tanh(logits / cap)
    residual_fp32: bool = False  # the hidden states arrive as the fp32 residual stream; logits leave in fp32
    logit_scale: float = 1.0  # the logits are multiplied by this (folded into the final norm's weight: `transform_norm_param`)
    norm_groups: int = 1  # with residual_fp32: the final RMS norm works on this many equal consecutive parts of the row, each on its own
