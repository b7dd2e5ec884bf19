"""Minimal gated recurrence: one number of state per channel and sequence, gates that read only the current token.

Per layer and step one scan over every sequence's new tokens (csrc/ragged/recurrent_ops.cu `mingru_scan`): it reads the gate, candidate and
output-gate pre-activations straight from the fused projection, adds the biases and forms sigmoid / candidate / silu in fp32, and writes
S_t silu(g_t) for the output projection.  The update S <- (1 - z) S + z c is an affine map of S, and affine maps compose: prompt portions are
cut into pieces whose composed maps are formed side by side, a short walk over the pieces leaves the state in front of each, and a second
pass writes the outputs -- decode steps and short portions take the plain walk, one thread per (sequence, channel).  The state lives in the
state manager's slots as fp32 and starts at zero (a sequence at position 0 ignores what its slot held)."""
from typing import Any, Dict, List, Type

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum
from ....ragged.state_slots import StateBufferSpec
from ...configs import DSMinGRUConfig
from ...interfaces import DSRecurrentMixerBase, DSRecurrentRegistry


@DSRecurrentRegistry.register_module
class DSMinGRU(DSRecurrentMixerBase):

    @staticmethod
    def name() -> str:
        return "min_gru"

    @staticmethod
    def config_class() -> Type[DSMinGRUConfig]:
        return DSMinGRUConfig

    @staticmethod
    def supports_config(config) -> bool:
        return (isinstance(config, DSMinGRUConfig) and config.input_dtype == config.output_dtype and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32) and config.width >= 1)

    def __init__(self, config: DSMinGRUConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        self._dtype = DtypeEnum(config.input_dtype).value

    def state_specs(self, prefix: str) -> List[StateBufferSpec]:
        return [StateBufferSpec(prefix + ".S", (self._config.width, ), torch.float32)]

    def transform_fp32_param(self, param: torch.Tensor) -> InferenceParameter:
        """The gate and candidate biases stay fp32."""
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())

    def forward(self, proj: torch.Tensor, cols, z_bias: torch.Tensor, x_bias: torch.Tensor, batch, state_manager, prefix: str,
                out: torch.Tensor, pieces=None) -> torch.Tensor:
        """proj [T, N]: the fused projection; cols = (gate, candidate, output gate) column offsets in it.  out: [T, width] view."""
        z0, x0, g0 = cols
        return K.mingru_scan(proj, z0, x0, g0, z_bias, x_bias, batch.tok_seq(), batch.seq_desc(), batch.current_sequences,
                             state_manager.get_state(prefix + ".S"), out, self._config.width, pieces=pieces)
