"""RMS norm that sits BEHIND the residual sum, on an fp32 stream:

    x <- rms_norm(mult * x + sublayer(x) [+ bias]) * w

The norm's result IS the new stream (nothing un-normed is carried along), and the sublayers read the stream itself.  One pass over the
token's row forms the sum, the statistic and the new stream, and also writes the stream in the activation dtype for the sublayer that reads it
next (csrc/ragged/latent_ops.cu `post_sum_norm`).  Sum, statistic, weight and stream are fp32 whatever the activation dtype is."""
from typing import Optional, Tuple

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum, NormTypeEnum
from ...configs import DSNormConfig
from ...interfaces import DSPostNormBase, DSPostNormRegistry


@DSPostNormRegistry.register_module
class DSPostSumRMSNorm(DSPostNormBase):

    @staticmethod
    def name() -> str:
        return "cuda_post_sum_rms"

    @staticmethod
    def supports_config(config: DSNormConfig) -> bool:
        return (NormTypeEnum(config.type) == NormTypeEnum.RMSNorm and config.post_sum and DtypeEnum(config.residual_dtype) == DtypeEnum.fp32 and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32) and DtypeEnum(config.output_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32))

    def transform_param(self, param: torch.Tensor) -> InferenceParameter:
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())

    def emit(self, residual: torch.Tensor) -> torch.Tensor:
        """The stream in the activation dtype (the stream itself when that is fp32): what the first sublayer reads."""
        dt = DtypeEnum(self._config.output_dtype).value
        return residual if dt == torch.float32 else K.sandwich_norm(residual, out_dtype=dt, plain_out=True)

    def forward(self, residual: torch.Tensor, hidden_states: Optional[torch.Tensor], gamma: torch.Tensor, beta: Optional[torch.Tensor] = None,
                fp32_branch: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """residual: fp32 stream (replaced in place by the normed sum).  hidden_states: the sublayer's output in the activation dtype and / or
        fp32_branch: its output in fp32; bias (fp32 [channels]): what the sublayer's last projection still lacks.  Returns (stream, stream in
        the activation dtype)."""
        c = self._config
        assert beta is None, "RMS norms have no shift"
        h = K.post_sum_norm(residual, hidden_states, gamma, alpha=c.stream_mult, eps=c.eps, y32=fp32_branch, bias=bias,
                            out_dtype=DtypeEnum(c.output_dtype).value)
        return residual, h
