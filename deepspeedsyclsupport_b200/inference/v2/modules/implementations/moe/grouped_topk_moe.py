"""Mixture-of-experts MLP with a configurable fp32 router and a gated activation.

Router (fp32): scores = softmax(W_r h) over all experts, or (`score_function` "sigmoid") the sigmoid of every logit on its own; the
SELECTION uses scores + correction (when the config has one), restricted to the `keep_groups` contiguous expert groups whose best
selection score is largest; the WEIGHTS are the plain scores of the chosen experts (optionally renormalised).  They multiply the
experts' outputs in the combine or, with `scale_input`, the experts' inputs in the scatter (out = sum_k expert_k(s_k h)).  `n_identity_experts`: the router has that many outputs more than there are
expert weights; a token that picks one of them gets its own input back, times the routing weight.  Experts: two
grouped GEMMs over the rows sorted by expert with the gated activation between them (clamped swish, or plain silu(g) * u for SiGLU); the
combine leaves in fp32 (it feeds an fp32 norm / residual).

The grouped GEMMs run on the persistent tcgen05 kernel (csrc/gemm/gemm_grouped.cu) when the operands are bf16 with
TMA-compatible shapes, else on the CUDA-core grouped GEMM of csrc/ragged/latent_ops.cu (any shape, bf16 or true fp32)."""
from typing import Any, Dict, Optional

import torch

from ......ops.gemm import dense_matmul, moe_gemm
from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import ActivationType, DtypeEnum
from ...configs import DSMoEConfig
from ...interfaces import DSMoEBase, DSMoERegistry


@DSMoERegistry.register_module
class DSGroupedTopKMoE(DSMoEBase):

    @staticmethod
    def name() -> str:
        return "grouped_topk_moe"

    @staticmethod
    def supports_config(config: DSMoEConfig) -> bool:
        if config.input_dtype != config.output_dtype or DtypeEnum(config.input_dtype) not in (DtypeEnum.bf16, DtypeEnum.fp32):
            return False
        if ActivationType(config.activation) not in (ActivationType.ClampedSwiGLU, ActivationType.SiGLU) or config.score_function not in ("softmax", "sigmoid"):
            return False
        g, k = config.n_groups, config.keep_groups
        routed = config.n_experts + config.n_identity_experts  # router outputs: experts with weights, then identity experts
        if config.n_identity_experts < 0 or (config.n_identity_experts and config.scale_input) or config.n_experts < 1:
            return False
        return (1 <= config.top_k <= min(routed, 32) and routed <= 2048 and g >= 1 and routed % g == 0 and 1 <= k <= g and k * (routed // g) >= config.top_k)

    def __init__(self, config: DSMoEConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        self._dtype = DtypeEnum(config.input_dtype).value
        self._output = None

    def transform_gate_param(self, param: torch.Tensor) -> InferenceParameter:
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())  # router weights and correction: fp32

    def transform_moe_mlp_1_param(self, param: torch.Tensor) -> InferenceParameter:
        return InferenceParameter.initialize(param.to(self._dtype).contiguous())

    def transform_moe_mlp_2_param(self, param: torch.Tensor) -> InferenceParameter:
        return InferenceParameter.initialize(param.to(self._dtype).contiguous())

    @property
    def output(self) -> torch.Tensor:
        return self._output

    def _grouped(self, x, w, cumsum):
        if x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and w.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0:
            return moe_gemm(x, w, cumsum)
        return K.moe_gemm_rows(x, w, cumsum)

    def forward(self, hidden_states: torch.Tensor, gate_w: torch.Tensor, mlp_1_w: torch.Tensor, mlp_2_w: torch.Tensor,
                mlp_1_b: Optional[torch.Tensor] = None, mlp_2_b: Optional[torch.Tensor] = None,
                correction: Optional[torch.Tensor] = None, router_input: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`router_input`: fp32 [tokens, model_dim], the hidden states before their rounding to the activation dtype (the norm in front
        can emit them in the same pass); without it the router reads the rounded hidden states."""
        c = self._config
        assert mlp_1_b is None and mlp_2_b is None, "these experts have no biases"
        assert (correction is not None) == c.use_correction
        logits = dense_matmul(router_input if router_input is not None else hidden_states.float(), gate_w)  # fp32 router logits
        counts, scores, assignments, offsets = K.grouped_topk_gating(logits, c.top_k, correction, c.n_groups, c.keep_groups, c.normalize_scores,
                                                                     sigmoid_scores=c.score_function == "sigmoid")
        moe_in, cumsum, slots = K.moe_scatter_rows(hidden_states, counts, assignments, offsets, row_scale=scores if c.scale_input else None)
        identity = None
        if c.n_identity_experts:  # their rows sit behind the last real expert's in the sorted order: the GEMMs never touch them, the combine
            cumsum = cumsum[:c.n_experts]  # reads the token's own (fp32) input instead
            identity = router_input if router_input is not None else hidden_states.float()
        gu = self._grouped(moe_in, mlp_1_w, cumsum)
        if ActivationType(c.activation) == ActivationType.SiGLU:  # silu(g) * u: the clamped form without its limit and shift
            act = K.clamped_swish_gate(gu, 1.0, float("inf"), 0.0)
        else:
            act = K.clamped_swish_gate(gu, c.act_alpha, c.act_limit, c.act_shift)
        out = self._grouped(act, mlp_2_w, cumsum)
        if identity is not None:
            self._output = K.moe_gather_rows(out, scores, slots, assignments=assignments, n_real=c.n_experts, identity_src=identity)
        else:
            self._output = K.moe_gather_rows(out, None if c.scale_input else scores, slots)
        return self._output
