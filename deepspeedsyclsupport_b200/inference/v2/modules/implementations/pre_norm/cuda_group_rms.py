"""The norm of blocks whose sublayers all read ONE normed input and add their outputs to an fp32 residual stream:

    x <- x + (outputs of the previous layer's sublayers)        (a plain fp32 sum; the outputs arrive in the activation dtype or fp32)
    out = rms_norm_in_groups(x) * w                             (the input of every sublayer of this layer, in the activation dtype)

in one pass over the token's row (csrc/ragged/latent_ops.cu `stream_group_norm`).  The row is normed in `groups` equal consecutive parts,
each divided by its own sqrt(mean(part^2) + eps).  Statistics, weight and stream are fp32 whatever the activation dtype is."""
from typing import Any, Dict, Optional, Sequence

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum, NormTypeEnum
from ...configs import DSNormConfig
from ...interfaces import DSPreNormBase, DSPreNormRegistry


@DSPreNormRegistry.register_module
class DSGroupRMSNorm(DSPreNormBase):

    @staticmethod
    def name() -> str:
        return "cuda_group_rms"

    @staticmethod
    def supports_config(config: DSNormConfig) -> bool:
        return (NormTypeEnum(config.type) == NormTypeEnum.RMSNorm and config.shared_input and DtypeEnum(config.residual_dtype) == DtypeEnum.fp32 and
                config.groups >= 1 and config.channels % config.groups == 0 and config.weight_offset == 0.0 and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32) and DtypeEnum(config.output_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32))

    def transform_param(self, param: torch.Tensor) -> InferenceParameter:
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())

    def forward(self, residual: torch.Tensor, hidden_states: Optional[Sequence[torch.Tensor]], gamma: Optional[torch.Tensor],
                beta: Optional[torch.Tensor] = None, fp32_branch: Optional[torch.Tensor] = None, fp32_copy: bool = False):
        """residual: fp32 stream (updated in place).  hidden_states: the finished sublayers' outputs in the activation dtype (a tensor, up to
        two tensors, or None); fp32_branch: one more output that is already fp32 (an expert combine).  gamma: weight of the norm that feeds
        the next layer, None when only the sum is wanted.  Returns (residual, normed input or None); with `fp32_copy` a third value: the
        normed input before its rounding to the activation dtype (what an fp32 router decides on)."""
        c = self._config
        assert beta is None, "RMS norms have no shift"
        branches = () if hidden_states is None else ((hidden_states, ) if torch.is_tensor(hidden_states) else tuple(hidden_states))
        out = K.stream_group_norm(residual, branches, fp32_branch, gamma, c.groups, c.eps, out_dtype=DtypeEnum(c.output_dtype).value, fp32_copy=fp32_copy)
        if fp32_copy:
            return residual, out[0], out[1]
        return residual, out
