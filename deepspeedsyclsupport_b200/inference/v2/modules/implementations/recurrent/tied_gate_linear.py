"""Linear attention whose forget gate also decides what is written (one d x dv matrix per head and sequence, no key projection).

Per layer and step: the scan kernel walks every sequence's new tokens in order with the state in registers (prompt portions and decode
tokens alike; csrc/ragged/recurrent_ops.cu `tied_gate_scan`) -- it reads the query and gate pre-activations and the values straight from the
fused projection and forms silu / sigmoid / the gate's lower bound in fp32 while a chunk is staged -- then one pass applies the per-head RMS
norm with the weight the heads share (`head_norm_gate` without a gate).  Gates, state and read-out are fp32 whatever the activation dtype."""
from typing import Any, Dict, List, Type

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum
from ....ragged.state_slots import StateBufferSpec
from ...configs import DSTiedGateConfig
from ...interfaces import DSRecurrentMixerBase, DSRecurrentRegistry


@DSRecurrentRegistry.register_module
class DSTiedGateLinearAttention(DSRecurrentMixerBase):

    @staticmethod
    def name() -> str:
        return "tied_gate_linear"

    @staticmethod
    def config_class() -> Type[DSTiedGateConfig]:
        return DSTiedGateConfig

    @staticmethod
    def supports_config(config) -> bool:
        return (isinstance(config, DSTiedGateConfig) and config.input_dtype == config.output_dtype and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32) and min(config.n_heads, config.key_size, config.value_size) >= 1 and
                config.key_size <= 2048)

    def __init__(self, config: DSTiedGateConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        self._dtype = DtypeEnum(config.input_dtype).value

    def state_specs(self, prefix: str) -> List[StateBufferSpec]:
        c = self._config
        return [StateBufferSpec(prefix + ".S", (c.n_heads, K.scan_state_floats(c.key_size, c.value_size)), torch.float32)]

    def transform_fp32_param(self, param: torch.Tensor) -> InferenceParameter:
        """The gate's bias and lower bound and the read-out norm's weight stay fp32."""
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())

    def forward(self, proj: torch.Tensor, cols, f_bias: torch.Tensor, lower: torch.Tensor, norm_w: torch.Tensor, batch, state_manager, prefix: str,
                out: torch.Tensor) -> torch.Tensor:
        """proj [T, N]: the fused projection; cols = (query, gate, value) column offsets in it.  out: [T, heads * value_size] view that
        receives the normed read-out."""
        c = self._config
        q0, f0, v0 = cols
        o = K.tied_gate_scan(proj, q0, f0, v0, f_bias, lower, batch.seq_desc(), batch.current_sequences, state_manager.get_state(prefix + ".S"),
                             c.n_heads, c.key_size, c.value_size)
        return K.head_norm_gate(o, norm_w, None, out, c.n_heads, c.value_size, c.eps, mult=c.out_scale, shared_weight=True)
