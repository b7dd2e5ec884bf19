"""One place that decides which implementation serves each building block of a model (parity:
inference/v2/modules/heuristics.py:36-179).  Decisions here depend on the engine configuration, not on the model: the
quantisation mode selects the fp8 tensor-core linear; everything else currently has one B200 implementation."""
from ..config_v2 import RaggedInferenceEngineConfig
from ..inference_utils import ActivationType, NormTypeEnum
from . import implementations  # noqa: F401  (registers the implementations)
from .configs import (DSConvSinkAttentionConfig, DSDeltaRuleConfig, DSEmbeddingsConfig, DSLatentAttentionConfig, DSLinearConfig, DSMatrixMemoryConfig,
                      DSMinGRUConfig, DSMoEConfig, DSNormConfig, DSRotaryLatentAttentionConfig, DSSelfAttentionConfig, DSSinkAttentionConfig,
                      DSTiedGateConfig, DSUnembedConfig, DSWindowedAttentionConfig)
from .interfaces import (DSEmbeddingBase, DSEmbeddingRegistry, DSLinearBase, DSLinearRegistry, DSMoEBase, DSMoERegistry, DSPostNormBase,
                         DSPostNormRegistry, DSPreNormBase, DSPreNormRegistry, DSRecurrentMixerBase, DSRecurrentRegistry, DSSelfAttentionBase,
                         DSSelfAttentionRegistry, DSUnembedBase, DSUnembedRegistry)
from .module_registry import ConfigBundle


def _quant_mode(engine_config) -> str:
    q = getattr(engine_config, "quantization", None) if engine_config is not None else None
    return getattr(q, "quantization_mode", "") or ""


def instantiate_attention(attention_config, engine_config: RaggedInferenceEngineConfig = None) -> DSSelfAttentionBase:
    if isinstance(attention_config, DSLatentAttentionConfig):  # keys / values are up-projections of a cached latent
        return DSSelfAttentionRegistry.instantiate_config(ConfigBundle(name="latent_blocked_attention", config=attention_config))
    if isinstance(attention_config, DSRotaryLatentAttentionConfig):  # a cached latent with one rotated key part beside it, learned sinks
        return DSSelfAttentionRegistry.instantiate_config(ConfigBundle(name="rotary_latent_attention", config=attention_config))
    if isinstance(attention_config, DSConvSinkAttentionConfig):  # convolved q / k / v, distance term, mask by parts, learned sinks, value mixing
        return DSSelfAttentionRegistry.instantiate_config(ConfigBundle(name="conv_sink_attention", config=attention_config))
    if isinstance(attention_config, DSWindowedAttentionConfig):  # convolved q / k, values = keys, sliding window that keeps the first tokens
        return DSSelfAttentionRegistry.instantiate_config(ConfigBundle(name="windowed_conv_attention", config=attention_config))
    if isinstance(attention_config, DSSinkAttentionConfig):  # per-head q / k / v norms, soft-capped scores, a sink in the softmax
        return DSSelfAttentionRegistry.instantiate_config(ConfigBundle(name="sink_blocked_attention", config=attention_config))
    return DSSelfAttentionRegistry.instantiate_config(ConfigBundle(name="dense_blocked_attention", config=attention_config))


def instantiate_recurrent(mixer_config, engine_config: RaggedInferenceEngineConfig = None) -> DSRecurrentMixerBase:
    """Token mixers with a fixed-size state per sequence; the config class names the recurrence."""
    name = {DSMatrixMemoryConfig: "matrix_memory", DSDeltaRuleConfig: "channel_delta_rule", DSTiedGateConfig: "tied_gate_linear",
            DSMinGRUConfig: "min_gru"}[type(mixer_config)]
    return DSRecurrentRegistry.instantiate_config(ConfigBundle(name=name, config=mixer_config))


def instantiate_embed(embed_config: DSEmbeddingsConfig, engine_config: RaggedInferenceEngineConfig = None) -> DSEmbeddingBase:
    name = "sinusoidal_embedding" if (embed_config.sinusoidal_base is not None or embed_config.fp32_stream) else "ragged_embedding"
    return DSEmbeddingRegistry.instantiate_config(ConfigBundle(name=name, config=embed_config))


def instantiate_linear(linear_config: DSLinearConfig, engine_config: RaggedInferenceEngineConfig = None) -> DSLinearBase:
    name = "blas_fp_linear"
    mode = _quant_mode(engine_config)
    if mode == "wf8af8" and DSLinearRegistry.registry["fp8_linear"].supports_config(linear_config):
        name = "fp8_linear"
    elif mode == "wf8af8_block" and DSLinearRegistry.registry["fp8_block_linear"].supports_config(linear_config):
        name = "fp8_block_linear"
    elif mode == "wf8af8_mx" and DSLinearRegistry.registry["mxfp8_linear"].supports_config(linear_config):
        name = "mxfp8_linear"
    return DSLinearRegistry.instantiate_config(ConfigBundle(name=name, config=linear_config))


def instantiate_moe(moe_config: DSMoEConfig, engine_config: RaggedInferenceEngineConfig = None) -> DSMoEBase:
    if (moe_config.n_groups > 1 or moe_config.use_correction or ActivationType(moe_config.activation) == ActivationType.ClampedSwiGLU or
            moe_config.score_function != "softmax" or moe_config.scale_input or moe_config.n_identity_experts > 0 or moe_config.fp32_combine):
        return DSMoERegistry.instantiate_config(ConfigBundle(name="grouped_topk_moe", config=moe_config))
    bundle = ConfigBundle(name="cutlass_multi_gemm_moe", config=moe_config, implementation_config={"weight_dtype": moe_config.input_dtype})
    return DSMoERegistry.instantiate_config(bundle)


def instantiate_post_norm(norm_config: DSNormConfig, engine_config: RaggedInferenceEngineConfig = None) -> DSPostNormBase:
    name = "cuda_post_sum_rms" if (NormTypeEnum(norm_config.type) == NormTypeEnum.RMSNorm and norm_config.post_sum) else "cuda_post_ln"
    return DSPostNormRegistry.instantiate_config(ConfigBundle(name=name, config=norm_config))


def instantiate_pre_norm(norm_config: DSNormConfig, engine_config: RaggedInferenceEngineConfig = None) -> DSPreNormBase:
    kind = NormTypeEnum(norm_config.type)
    name = "cuda_pre_ln" if kind == NormTypeEnum.LayerNorm else ("cuda_sandwich_rms" if norm_config.sandwich else "cuda_pre_rms")
    if kind == NormTypeEnum.RMSNorm and norm_config.shared_input:
        name = "cuda_group_rms"
    return DSPreNormRegistry.instantiate_config(ConfigBundle(name=name, config=norm_config))


def instantiate_unembed(unembed_config: DSUnembedConfig, engine_config: RaggedInferenceEngineConfig = None) -> DSUnembedBase:
    return DSUnembedRegistry.instantiate_config(ConfigBundle(name="ragged_unembed", config=unembed_config))
