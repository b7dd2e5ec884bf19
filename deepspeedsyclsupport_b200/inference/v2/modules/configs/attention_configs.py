"""Configuration of the self-attention modules (parity: inference/v2/modules/configs/attention_configs.py:16-110)."""
from enum import Enum
from typing import Dict, Optional

from pydantic import model_validator

from .....runtime.config_utils import DeepSpeedConfigModel
from ...inference_utils import DtypeEnum
from ..ds_module import DSModuleConfig


class PositionalEmbeddingType(Enum):
    none = "none"
    rotate_half = "rotate_half"  # rotary, (x[:d/2], x[d/2:]) pairing (llama / neox style)
    rotate_every_other = "rotate_every_other"  # rotary, (x[2i], x[2i+1]) pairing (gpt-j style)
    alibi = "alibi"


class RotateHalfConfig(DeepSpeedConfigModel):
    use_trained_freqs: bool = False  # take `inv_freqs` from the caller instead of synthesising theta_base ** (-2i/d)
    theta_base: float = 10_000.0
    rotate_dim: Optional[int] = None  # number of rotated channels per head; None = all (no hidden doubling)


class MaskingType(Enum):
    none = "none"
    causal = "causal"
    local = "local"
    symmetric = "symmetric"
    asymmetric = "asymmetric"


class DSSelfAttentionConfig(DSModuleConfig):
    n_heads_q: int
    n_heads_kv: int
    head_size: int
    max_sequences: int
    scale_factor: float = 1.0
    input_dtype: DtypeEnum = DtypeEnum.fp16
    output_dtype: DtypeEnum = DtypeEnum.fp16
    masking_type: MaskingType = MaskingType.causal
    masking_args: Dict = {}
    positional_embedding_type: PositionalEmbeddingType = PositionalEmbeddingType.none
    positional_embedding_config: Optional[RotateHalfConfig] = None

    @model_validator(mode="after")
    def _consistent_heads(self):
        if self.n_heads_q <= 0 or self.n_heads_kv <= 0 or self.head_size <= 0:
            raise ValueError("head counts and head size must be positive")
        if self.n_heads_q % self.n_heads_kv != 0:
            raise ValueError(f"n_heads_q ({self.n_heads_q}) must be a multiple of n_heads_kv ({self.n_heads_kv})")
        rc = self.positional_embedding_config
        if rc is not None and rc.rotate_dim is not None and not (0 < rc.rotate_dim <= self.head_size and rc.rotate_dim % 2 == 0):
            raise ValueError(f"rotate_dim must be even and at most head_size ({self.head_size}), got {rc.rotate_dim}")
        return self

    @property
    def group_size(self) -> int:
        """query heads served by one key/value head"""
        return self.n_heads_q // self.n_heads_kv


class DSLatentAttentionConfig(DSModuleConfig):
    """Attention whose keys and values are up-projections of one cached low-rank latent per token (no positional rotation):
    c_q = rms(W_dq h), q = W_uq c_q;  c = rms(W_dkv h) is cached;  k = W_uk c, v = W_uv c per head; causal softmax."""
    n_heads: int
    qk_dim: int  # query / key size per head
    v_dim: int  # value size per head
    kv_rank: int  # size of the cached latent
    q_rank: int  # size of the query latent
    scale: float  # softmax scale (given, not derived from qk_dim)
    eps: float = 1e-6  # of the two latent norms
    max_sequences: int
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16

    @model_validator(mode="after")
    def _positive(self):
        for k in ("n_heads", "qk_dim", "v_dim", "kv_rank", "q_rank"):
            if getattr(self, k) <= 0:
                raise ValueError(f"{k} must be positive")
        if self.kv_rank > 1024:
            raise ValueError("the latent attention kernels hold a latent row of at most 1024 values")
        return self


class RotaryScalingConfig(DeepSpeedConfigModel):
    """Slows the long-wavelength rotary frequencies down: a frequency f with wavelength l = 2 pi / f is kept when l < original / high,
    divided by `factor` when l > original / low, and blended linearly in (original / l - low) / (high - low) in between."""
    factor: float
    low: float
    high: float
    original: float


class DSWindowedAttentionConfig(DSModuleConfig):
    """Attention whose queries and keys pass a short causal convolution over time, an RMS norm over the whole projection and an
    interleaved partial rotation, whose values ARE the convolved keys (no value projection), and whose mask is a sliding window that
    also keeps the first tokens of the sequence: query i sees key j <= i when i - j < window or j < keep_first."""
    n_heads_q: int
    n_heads_kv: int
    head_size: int
    conv_taps: int  # the last taps - 1 projected rows of a sequence are state
    window: int
    keep_first: int = 0
    scale: float  # softmax scale (given, not derived from the head size)
    rotate_dim: int = 0  # entries per head that are rotated (pairs (2i, 2i + 1)); 0 = no rotation
    theta_base: float = 10_000.0
    rotary_scaling: Optional[RotaryScalingConfig] = None
    eps: float = 1e-6  # of the query / key norms
    out_scale: float = 1.0  # the result is multiplied by this before it is rounded (mixers that are summed with weights)
    max_sequences: int
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16

    @model_validator(mode="after")
    def _consistent(self):
        if self.n_heads_q <= 0 or self.n_heads_kv <= 0 or self.n_heads_q % self.n_heads_kv != 0:
            raise ValueError(f"n_heads_q ({self.n_heads_q}) must be a positive multiple of n_heads_kv ({self.n_heads_kv})")
        if self.head_size <= 0:
            raise ValueError(f"head_size must be positive, got {self.head_size}")
        if not (0 <= self.rotate_dim <= self.head_size and self.rotate_dim % 2 == 0):
            raise ValueError(f"rotate_dim must be even and at most head_size ({self.head_size}), got {self.rotate_dim}")
        if self.conv_taps < 1 or self.window < 1 or self.keep_first < 0:
            raise ValueError("conv_taps and window must be at least 1, keep_first at least 0")
        return self

    @property
    def group_size(self) -> int:
        return self.n_heads_q // self.n_heads_kv


class RampRotaryScalingConfig(DeepSpeedConfigModel):
    """Frequency scaling with a linear ramp over the channel index: with c(t) = dims ln(original / (2 pi t)) / (2 ln base) the channel that
    makes t turns over `original` positions, lo = max(floor(c(fast)), 0), hi = min(ceil(c(slow)), dims - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), channel i turns at f_i / factor * ramp_i + f_i (1 - ramp_i); cosine and sine are
    multiplied by 0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float


class DSSinkAttentionConfig(DSModuleConfig):
    """Causal attention with per-head query / key RMS norms (one weight of head size shared by the heads, applied before the rotation), a
    rotate-half rotation of the first `rotate_dim` entries of a head, values divided by their own root mean square (no weight; cached so),
    scores scale * q . k soft-capped as softcap tanh(. / softcap), and a softmax whose denominator has `sink` added (1: one more entry of
    score 0 without a value).  Query / key heads have `head_size` entries, value heads `value_size`."""
    n_heads_q: int
    n_heads_kv: int
    head_size: int
    value_size: int
    scale: float  # softmax scale (given, not derived from the head size)
    softcap: float = 0.0  # 0 = no cap
    sink: float = 1.0
    qk_norm: bool = True
    v_norm: bool = True
    rotate_dim: int = 0
    theta_base: float = 10_000.0
    rotary_scaling: Optional[RampRotaryScalingConfig] = None
    eps: float = 1e-6
    max_sequences: int
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16

    @model_validator(mode="after")
    def _consistent(self):
        if self.n_heads_q <= 0 or self.n_heads_kv <= 0 or self.n_heads_q % self.n_heads_kv != 0:
            raise ValueError(f"n_heads_q ({self.n_heads_q}) must be a positive multiple of n_heads_kv ({self.n_heads_kv})")
        if self.head_size <= 0 or self.value_size <= 0:
            raise ValueError("head sizes must be positive")
        if not (0 <= self.rotate_dim <= self.head_size and self.rotate_dim % 2 == 0):
            raise ValueError(f"rotate_dim must be even and at most head_size ({self.head_size}), got {self.rotate_dim}")
        if self.softcap < 0 or self.sink < 0:
            raise ValueError("softcap and sink cannot be negative")
        return self

    @property
    def group_size(self) -> int:
        return self.n_heads_q // self.n_heads_kv


class DSRotaryLatentAttentionConfig(DSModuleConfig):
    """Attention whose keys and values are per-head up-projections of one cached, RMS-normed low-rank latent per token, with a rotated part
    beside it: a query head has `qk_dim` plain and `rot_dim` rotated entries; every token adds ONE rotated key part of `rot_dim` entries that
    all heads share, cached beside the latent.  score = scale (q_plain . W_uk c + q_rot . k_rot); rotate-half pairs over the first `rotate_dim`
    of the rot_dim entries; causal softmax, optionally with a learned sink per head (exp(sink_h) joins the denominator) and a sigmoid gate
    per token and head on the head's output."""
    n_heads: int
    qk_dim: int  # plain (unrotated) query / key entries per head
    rot_dim: int  # rotated entries per query head = size of the shared key part
    v_dim: int
    kv_rank: int
    scale: float
    rotate_dim: int  # entries of the rot_dim part that are rotated (pairs (i, i + rotate_dim / 2)); the rest pass unchanged
    theta_base: float = 10_000.0
    learned_sink: bool = False
    head_gate: bool = False
    eps: float = 1e-6  # of the latent's norm
    max_sequences: int
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16

    @model_validator(mode="after")
    def _consistent(self):
        for k in ("n_heads", "v_dim", "kv_rank"):
            if getattr(self, k) <= 0:
                raise ValueError(f"{k} must be positive")
        if self.qk_dim < 0 or self.rot_dim < 0 or self.qk_dim + self.rot_dim <= 0:
            raise ValueError("a query head needs at least one entry")
        if not (0 <= self.rotate_dim <= self.rot_dim and self.rotate_dim % 2 == 0):
            raise ValueError(f"rotate_dim must be even and at most rot_dim ({self.rot_dim}), got {self.rotate_dim}")
        if self.kv_rank + self.rot_dim > 4096:
            raise ValueError("the attention kernels hold a cached row of at most 4096 values")
        return self


class DSConvSinkAttentionConfig(DSModuleConfig):
    """Attention whose query, key and value projections (with biases) pass a short causal convolution over time, then per-head RMS norms of
    queries and keys (one weight of head size shared by the heads); no rotation.  score = scale q . k - r1_h ln(1 + r2_h (i - j)) when
    `distance_bias`; a query at position i sees the keys j <= i of its own part, floor(i / part_size) = floor(j / part_size) (0: all);
    `learned_sink`: exp(sink_h) joins the softmax denominator.  `value_mix`: "source" = the layer's convolved values are handed to later
    layers; "mix" = the cached value is (1 - m) v + m v_source with the source layer's values of the same token; "none"."""
    n_heads_q: int
    n_heads_kv: int
    head_size: int
    value_size: int
    conv_taps: int  # the last taps - 1 projected rows of a sequence are state
    scale: float
    part_size: int = 0
    distance_bias: bool = False
    learned_sink: bool = False
    value_mix: str = "none"
    eps: float = 1e-6
    max_sequences: int
    input_dtype: DtypeEnum = DtypeEnum.bf16
    output_dtype: DtypeEnum = DtypeEnum.bf16

    @model_validator(mode="after")
    def _consistent(self):
        if self.n_heads_q <= 0 or self.n_heads_kv <= 0 or self.n_heads_q % self.n_heads_kv != 0:
            raise ValueError(f"n_heads_q ({self.n_heads_q}) must be a positive multiple of n_heads_kv ({self.n_heads_kv})")
        if self.head_size <= 0 or self.value_size <= 0 or self.conv_taps < 1 or self.part_size < 0:
            raise ValueError("head sizes and conv_taps must be positive, part_size cannot be negative")
        if self.value_mix not in ("none", "source", "mix"):
            raise ValueError(f"value_mix must be none, source or mix, got {self.value_mix}")
        return self

    @property
    def group_size(self) -> int:
        return self.n_heads_q // self.n_heads_kv
