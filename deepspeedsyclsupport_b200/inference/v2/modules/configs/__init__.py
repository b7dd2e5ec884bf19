from .attention_configs import (DSConvSinkAttentionConfig, DSLatentAttentionConfig, DSRotaryLatentAttentionConfig, DSSelfAttentionConfig, DSSinkAttentionConfig, DSWindowedAttentionConfig, MaskingType,
                                PositionalEmbeddingType, RampRotaryScalingConfig, RotaryScalingConfig, RotateHalfConfig)
from .embedding_config import DSEmbeddingsConfig
from .linear_config import DSLinearConfig
from .moe_config import DSMoEConfig
from .norm_config import DSNormConfig
from .recurrent_configs import DSDeltaRuleConfig, DSMatrixMemoryConfig, DSMinGRUConfig, DSTiedGateConfig
from .unembed_config import DSUnembedConfig
