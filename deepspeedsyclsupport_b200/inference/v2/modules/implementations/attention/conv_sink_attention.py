"""Attention over a paged cache whose query, key and value projections pass a short causal convolution over time, with per-head query / key
norms, a logarithmic distance term on the scores, a mask by fixed parts of the sequence, a learned sink per head and values that can be mixed
with an earlier layer's values of the same token.

Per layer and step: `conv_head_norm_append` (biases, convolution from the batch rows and the sequence's state, norms, value mixing, keys and
values into the cache; one kernel), `conv_state_update` (the last taps - 1 projected rows of every sequence become its state), then the
attention kernel.  Query / key heads and value heads may differ in size: with equal sizes the layer's cache is one
[blocks, 2, block_size, kv_heads, head_size] tensor, otherwise two single-plane tensors that share the block ids.
csrc/ragged/sink_attention_ops.cu, csrc/ragged/recurrent_ops.cu.

Two attention kernels.  bf16 with head sizes up to 128: the tcgen05 paged flash kernels (csrc/attn/paged_flash.cu) with the distance term, the
part mask and per-head sinks; heads are padded with zeros to a common width of 64 / 128 (a zero entry of a query / key adds nothing to a
score; a zero column of the values gives a zero column of the output, which the output projection meets with zero weights).  Everything else
(fp32, head sizes above 128): `sink_attention_ex`, a CUDA-core kernel with fp32 scores and accumulation that takes any sizes."""
import os
from typing import Any, Dict, List, Optional, Type

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum
from ....ragged.state_slots import StateBufferSpec
from ...configs import DSConvSinkAttentionConfig
from ...interfaces import DSSelfAttentionBase, DSSelfAttentionRegistry


@DSSelfAttentionRegistry.register_module
class DSConvSinkAttention(DSSelfAttentionBase):

    @staticmethod
    def name() -> str:
        return "conv_sink_attention"

    @staticmethod
    def config_class() -> Type[DSConvSinkAttentionConfig]:
        return DSConvSinkAttentionConfig

    @staticmethod
    def supports_config(config) -> bool:
        return (isinstance(config, DSConvSinkAttentionConfig) and config.input_dtype == config.output_dtype and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32))

    def __init__(self, config: DSConvSinkAttentionConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        self._dtype = DtypeEnum(config.input_dtype).value
        widest = max(config.head_size, config.value_size)
        flash = self._dtype == torch.bfloat16 and widest <= 128 and os.environ.get("DSB200_CONV_ATTN_FLASH", "1") != "0"
        self._pad = (64 if widest <= 64 else 128) if flash else None  # common width of all heads on the tensor-core path

    @property
    def kv_block_size(self) -> int:
        return 64

    @property
    def q_block_size(self) -> int:
        return 1

    @property
    def conv_channels(self) -> int:
        c = self._config
        return (c.n_heads_q + c.n_heads_kv) * c.head_size + c.n_heads_kv * c.value_size

    def state_specs(self, prefix: str) -> List[StateBufferSpec]:
        c = self._config
        return [StateBufferSpec(prefix + ".conv", (c.conv_taps - 1, self.conv_channels), self._dtype)] if c.conv_taps > 1 else []

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
        """Biases, convolution taps, norm weights, the distance term's numbers, sinks and the mixing weight stay fp32."""
        return InferenceParameter.initialize(param.to(torch.float32).reshape(-1 if param.dim() == 0 else param.shape).contiguous())

    def forward(self, proj: torch.Tensor, col0: int, bias: Optional[torch.Tensor], conv_w: torch.Tensor, norm_q: torch.Tensor, norm_k: torch.Tensor,
                r1: Optional[torch.Tensor], r2: Optional[torch.Tensor], sink: Optional[torch.Tensor], k_cache: torch.Tensor,
                v_cache: Optional[torch.Tensor], batch, state_manager, prefix: str, out: torch.Tensor, v_source: Optional[torch.Tensor] = None,
                mix: Optional[torch.Tensor] = None):
        """proj [T, N]: the fused projection with (queries | keys | values) from column col0 (without their biases: `bias`, fp32, is added
        here); conv_w fp32 [taps, conv_channels].  k_cache / v_cache: the layer's cache tensor(s) as `cache_shapes` lists them (v_cache None for the two-plane tensor).  out:
        [T, out_width] view.  value_mix "mix": v_source = the source layer's values of these tokens, mix = the weight (fp32 [1]).  Returns
        (out, this layer's convolved values when value_mix is "source", else None)."""
        c = self._config
        H, G, d, dv = c.n_heads_q, c.n_heads_kv, c.head_size, c.value_size
        T = proj.shape[0]
        desc = batch.seq_desc()
        conv_state = state_manager.get_state(prefix + ".conv") if c.conv_taps > 1 else None
        kp, vp = K.cache_planes(k_cache, v_cache)
        bs = k_cache.shape[2] if v_cache is None else k_cache.shape[1]
        P = self._pad
        q = torch.empty(T, H * (P or d), dtype=proj.dtype, device=proj.device)
        v_own = torch.empty(T, G * dv, dtype=proj.dtype, device=proj.device) if c.value_mix == "source" else None
        mixing = c.value_mix == "mix"
        assert not mixing or (v_source is not None and mix is not None)
        K.conv_head_norm_append(proj, col0, bias, conv_w, norm_q, norm_k, conv_state, desc, batch.tok_seq(), batch.tok_pos(), batch.block_table(), bs,
                                kp, vp, q, H, G, d, dv, c.conv_taps, c.eps, v_other=v_source if mixing else None, mix=mix if mixing else None,
                                v_own=v_own, row=P)
        if conv_state is not None:
            K.conv_state_update(proj, col0, self.conv_channels, conv_state, 0, desc, batch.current_sequences, c.conv_taps)
        if P is not None:
            d = dv = P  # from here on every head is P wide
        r1, r2 = (r1, r2) if c.distance_bias else (None, None)
        sink = sink if c.learned_sink else None
        if P is not None and v_cache is None and K.paged_flash_sink_ok(q, k_cache, out, H, G, d, dv):
            K.paged_flash_sink(q, k_cache, batch.tok_seq(), batch.tok_pos(), batch.block_table(), out, H, G, d, c.scale, 0.0, 0.0, sink_logit=sink,
                               r1=r1, r2=r2, part=c.part_size, decode=batch.current_tokens <= 2 * batch.current_sequences)
        else:
            K.sink_attention_ex(q, d, kp, d, vp, dv, batch.tok_seq(), batch.tok_pos(), batch.block_table(), bs, out, dv, H, G, d, dv, c.scale,
                                sink_logit=sink, r1=r1, r2=r2, part=c.part_size)
        return out, v_own
