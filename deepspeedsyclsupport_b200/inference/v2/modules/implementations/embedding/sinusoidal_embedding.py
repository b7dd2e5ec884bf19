"""Token embedding (times an optional constant), optionally plus a fixed sinusoidal position vector, written as the fp32 start of the
residual stream.

Entry 2i of the position vector is sin(p * base^(-2i / dim)) and entry 2i + 1 the cosine of the same angle, p being the token's
position in its sequence.  The angles are formed in double precision on the device (a position in the thousands times a
frequency near one loses the low bits of a float), from a frequency table computed once on the host."""
from typing import Any, Dict, Optional

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum
from ...configs import DSEmbeddingsConfig
from ...interfaces import DSEmbeddingBase, DSEmbeddingRegistry


@DSEmbeddingRegistry.register_module
class DSSinusoidalEmbedding(DSEmbeddingBase):

    @staticmethod
    def name() -> str:
        return "sinusoidal_embedding"

    @staticmethod
    def supports_config(config: DSEmbeddingsConfig) -> bool:
        if DtypeEnum(config.residual_dtype) not in (DtypeEnum.bf16, DtypeEnum.fp32):
            return False
        return (config.sinusoidal_base is not None or config.fp32_stream) and not config.positional_embedding and not config.use_token_type

    def __init__(self, config: DSEmbeddingsConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        self._freq = None
        self._output = None

    def transform_param(self, embed_param: torch.Tensor) -> InferenceParameter:
        """The table stays in the activation dtype (`residual_dtype` of the config names the table here; the sum is fp32)."""
        return InferenceParameter.initialize(embed_param.to(DtypeEnum(self._config.residual_dtype).value).contiguous())

    @property
    def output(self) -> torch.Tensor:
        return self._output

    def forward(self, ragged_batch, word_embeddings: torch.Tensor, position_embeddings: Optional[torch.Tensor] = None,
                token_type_ids: Optional[torch.Tensor] = None, token_type_embeddings: Optional[torch.Tensor] = None) -> torch.Tensor:
        assert position_embeddings is None and token_type_ids is None
        if self._config.sinusoidal_base is not None and (self._freq is None or self._freq.device != word_embeddings.device):
            self._freq = K.sinusoid_frequencies(self._config.embedding_dim, self._config.sinusoidal_base, word_embeddings.device)
        self._output = K.embed_sinusoid(ragged_batch.input_ids(), word_embeddings, ragged_batch.tok_pos(), self._freq, scale=self._config.embedding_scale)
        return self._output
