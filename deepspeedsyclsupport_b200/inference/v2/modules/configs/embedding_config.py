"""(parity: inference/v2/modules/configs/embedding_config.py:14-70)"""
from typing import Optional

from ...inference_utils import DtypeEnum, NormTypeEnum
from ..ds_module import DSModuleConfig


class DSEmbeddingsConfig(DSModuleConfig):
    residual_dtype: DtypeEnum = DtypeEnum.fp16
    embedding_dim: int
    positional_embedding: bool = False
    positional_offset: int = 0  # OPT stores position p at row p + 2
    use_token_type: bool = False
    output_normalization: Optional[NormTypeEnum] = None
    # not None: a fixed sinusoidal position vector is added (entry 2i = sin(p base^(-2i/dim)), entry 2i+1 = cos of the same) and the
    # result is the fp32 start of the residual stream
    sinusoidal_base: Optional[float] = None
    # the embedding leaves as the fp32 start of a residual stream whatever the table's dtype (implied by sinusoidal_base)
    fp32_stream: bool = False
    # the table row is multiplied by this (in fp32) on its way into an fp32 stream
    embedding_scale: float = 1.0
