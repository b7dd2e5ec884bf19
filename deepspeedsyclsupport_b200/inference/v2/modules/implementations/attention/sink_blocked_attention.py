"""Causal attention over a paged cache with per-head query / key norms, a partial rotate-half rotation whose frequencies may be scaled with a
ramp over the channel index, weightless value norms, soft-capped scores and a softmax with a sink.

Per layer and step: `head_norm_rotary_append` (norms, rotation with angles formed in double precision, keys and normed values into the
cache), then the attention kernel.  Query / key heads and value heads may differ in size: with equal sizes the layer's cache is the usual
[blocks, 2, block_size, kv_heads, head_size] tensor, otherwise two single-plane tensors [blocks, block_size, kv_heads, size] that share the
block ids.  csrc/ragged/sink_attention_ops.cu.

Two attention kernels.  bf16 with head sizes up to 128: the tcgen05 paged flash kernels (csrc/attn/paged_flash.cu) with the soft cap and the
sink.  They want one head size of 64 or 128 for queries, keys and values, so every head is PADDED to that width with zeros (a zero entry of
a query / key adds nothing to a score; a zero column of the values gives a zero column of the output, which the output projection meets
with zero weights): the layer's cache is then one two-plane tensor of the padded width and `out_width` is heads x padded width.  Everything
else (fp32, head sizes above 128): `sink_attention`, a CUDA-core kernel with fp32 scores and accumulation that takes any sizes."""
import math
from typing import Any, Dict, Optional, Type

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum
from ...configs import DSSinkAttentionConfig
from ...interfaces import DSSelfAttentionBase, DSSelfAttentionRegistry


def ramp_scaled_frequencies(rotate_dim, theta_base, scaling=None):
    """(float64 [rotate_dim / 2] frequencies, factor on cosine and sine): f_i = theta_base^(-2i / rotate_dim), scaled as
    `RampRotaryScalingConfig` describes."""
    half = rotate_dim // 2
    f = [float(theta_base) ** (-2.0 * i / rotate_dim) for i in range(half)]
    if scaling is None or half == 0:
        return torch.tensor(f, dtype=torch.float64), 1.0

    def channel(turns):
        return rotate_dim * math.log(scaling.original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta_base))

    lo = max(math.floor(channel(scaling.fast)), 0)
    hi = min(math.ceil(channel(scaling.slow)), rotate_dim - 1)
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        f[i] = f[i] / scaling.factor * ramp + f[i] * (1.0 - ramp)
    return torch.tensor(f, dtype=torch.float64), 0.1 * math.log(scaling.factor) + 1.0


@DSSelfAttentionRegistry.register_module
class DSSinkBlockedAttention(DSSelfAttentionBase):

    @staticmethod
    def name() -> str:
        return "sink_blocked_attention"

    @staticmethod
    def config_class() -> Type[DSSinkAttentionConfig]:
        return DSSinkAttentionConfig

    @staticmethod
    def supports_config(config) -> bool:
        return (isinstance(config, DSSinkAttentionConfig) and config.input_dtype == config.output_dtype and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32))

    def __init__(self, config: DSSinkAttentionConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        self._dtype = DtypeEnum(config.input_dtype).value
        self._freq_host, self._mag = ramp_scaled_frequencies(config.rotate_dim, config.theta_base, config.rotary_scaling)
        self._freq = None
        # common width of all heads on the tensor-core path (None: every head keeps its own size)
        widest = max(config.head_size, config.value_size)
        self._pad = (64 if widest <= 64 else 128) if (self._dtype == torch.bfloat16 and widest <= 128) else None

    @property
    def kv_block_size(self) -> int:
        return 64

    @property
    def q_block_size(self) -> int:
        return 1

    def cache_shapes(self):
        """(planes, heads, width) of the cache tensors this layer needs, in the order `forward` takes them."""
        c = self._config
        if self._pad is not None:
            return [(2, c.n_heads_kv, self._pad)]
        if c.head_size == c.value_size:
            return [(2, c.n_heads_kv, c.head_size)]
        return [(1, c.n_heads_kv, c.head_size), (1, c.n_heads_kv, c.value_size)]

    @property
    def out_head_width(self) -> int:
        """Entries per head of the attention output (the value size, or the padded width)."""
        return self._pad if self._pad is not None else self._config.value_size

    @property
    def out_width(self) -> int:
        return self._config.n_heads_q * self.out_head_width

    def transform_fp32_param(self, param: torch.Tensor) -> InferenceParameter:
        """The norm weights stay fp32."""
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())

    def forward(self, proj: torch.Tensor, cols, k_cache: torch.Tensor, v_cache: Optional[torch.Tensor], batch, norm_q: Optional[torch.Tensor],
                norm_k: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        """proj [T, N]: the fused projection with queries, keys and values at the columns cols = (q, k, v).  k_cache / v_cache: the layer's
        cache tensor(s) as `cache_shapes` lists them (v_cache None for the two-plane tensor).  out: [T, out_width] view."""
        c = self._config
        q0, k0, v0 = cols
        H, G, d, dv = c.n_heads_q, c.n_heads_kv, c.head_size, c.value_size
        if c.rotate_dim and (self._freq is None or self._freq.device != proj.device):
            self._freq = self._freq_host.to(proj.device)
        kp, vp = K.cache_planes(k_cache, v_cache)
        bs = k_cache.shape[2] if v_cache is None else k_cache.shape[1]
        P = self._pad
        q = torch.empty(proj.shape[0], H * (P or d), dtype=proj.dtype, device=proj.device)
        K.head_norm_rotary_append(proj, q0, k0, v0, norm_q if c.qk_norm else None, norm_k if c.qk_norm else None, self._freq if c.rotate_dim else None,
                                  self._mag, batch.tok_seq(), batch.tok_pos(), batch.block_table(), bs, kp, vp, q, H, G, d, dv, c.rotate_dim, c.eps,
                                  norm_v=c.v_norm, row=P)
        if P is not None:
            d = dv = P  # from here on every head is P wide
        if v_cache is None and K.paged_flash_sink_ok(q, k_cache, out, H, G, d, dv):
            return K.paged_flash_sink(q, k_cache, batch.tok_seq(), batch.tok_pos(), batch.block_table(), out, H, G, d, c.scale, c.softcap, c.sink,
                                      decode=batch.current_tokens <= 2 * batch.current_sequences)
        return K.sink_attention(q, kp, vp, batch.tok_seq(), batch.tok_pos(), batch.block_table(), bs, out, H, G, d, dv, c.scale, c.softcap, c.sink)
