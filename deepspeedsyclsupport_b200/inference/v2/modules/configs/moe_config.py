"""(parity: inference/v2/modules/configs/moe_config.py:12-56)"""
from ...inference_utils import ActivationType, DtypeEnum
from ..ds_module import DSModuleConfig


class DSMoEConfig(DSModuleConfig):
    model_dim: int
    intermediate_features: int
    n_experts: int
    top_k: int = 1
    input_dtype: DtypeEnum = DtypeEnum.fp16
    output_dtype: DtypeEnum = DtypeEnum.fp16
    activation: ActivationType = ActivationType.IDENTITY
    normalize_scores: bool = False
    # router with a selection bias and contiguous expert groups ("grouped_topk_moe"): experts form n_groups contiguous groups of equal size,
    # only the keep_groups groups with the largest best selection score stay selectable; use_correction adds a per-expert term to the
    # scores for the selection only (the combine weights stay the plain softmax scores)
    n_groups: int = 1
    keep_groups: int = 1
    use_correction: bool = False
    # how a router logit becomes a score: "softmax" over the experts, or "sigmoid" of every logit on its own
    score_function: str = "softmax"
    # True: the chosen expert's score multiplies the expert's INPUT (out = sum_k expert_k(s_k h)) instead of its output
    scale_input: bool = False
    # ActivationType.ClampedSwiGLU: min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + shift)
    act_alpha: float = 1.702
    act_limit: float = 7.0
    act_shift: float = 1.0
    # identity experts: the router has n_experts + n_identity_experts outputs; the last n_identity_experts of them have no weights and
    # return their input (times the routing weight)
    n_identity_experts: int = 0
    # the weighted sum of the experts' outputs leaves in fp32 (it joins an fp32 residual stream) whatever the activation dtype
    fp32_combine: bool = False
