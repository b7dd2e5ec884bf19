"""Attention over a paged cache of low-rank latents with a rotated key part beside them: per token and layer ONE row (c | k_rot) of
kv_rank + rot_dim values is cached -- the RMS-normed latent c, of which every head's keys and values are up-projections, and one rotated
key part that all heads share.

With k_h = U_h c the score q_h . k_h + q_rot,h . k_rot equals (U_h^T q_h | q_rot,h) . (c | k_rot): the plain part of every query head is mapped
into the latent space once per token (a batched GEMM whose right operand also carries the rotated part through: [[U_h, 0], [0, I]]), all heads
of a token then share the cached rows as keys, their first kv_rank values as values, and the value up-projection is applied to the attended
latent.  Nothing but the row is cached or expanded, for prompt portions and decode steps alike.

Per layer: rotation of the query heads' rotated parts in place + latent norm + key rotation + cache append (one kernel), per-head map into the
latent space (batched GEMM), the attention kernel with a learned sink per head, per-head value up-projection (batched GEMM), head
concatenation + sigmoid gate per (token, head) in one pass.

Two attention kernels.  bf16 with kv_rank + rot_dim <= 128 and at most 128 heads: the tcgen05 paged flash kernels in their one-plane mode with
per-head sinks (rows zero-padded to 64 / 128 values, heads to a divisor of 128: neither changes a score or an output).  Everything else:
`sink_attention_ex`, a CUDA-core kernel with fp32 scores and accumulation that takes any size."""
import os
from typing import Any, Dict, Optional, Type

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum
from ...configs import DSRotaryLatentAttentionConfig
from ...interfaces import DSSelfAttentionBase, DSSelfAttentionRegistry
from .latent_blocked_attention import _bmm


@DSSelfAttentionRegistry.register_module
class DSRotaryLatentAttention(DSSelfAttentionBase):

    @staticmethod
    def name() -> str:
        return "rotary_latent_attention"

    @staticmethod
    def config_class() -> Type[DSRotaryLatentAttentionConfig]:
        return DSRotaryLatentAttentionConfig

    @staticmethod
    def supports_config(config) -> bool:
        return (isinstance(config, DSRotaryLatentAttentionConfig) and config.input_dtype == config.output_dtype and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32))

    def __init__(self, config: DSRotaryLatentAttentionConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        c = config
        self._dtype = DtypeEnum(c.input_dtype).value
        half = c.rotate_dim // 2
        self._freq_host = torch.tensor([float(c.theta_base)**(-2.0 * i / c.rotate_dim) for i in range(half)], dtype=torch.float64)
        self._freq = None
        used = c.kv_rank + c.rot_dim
        self._flash = (self._dtype == torch.bfloat16 and used <= 128 and c.n_heads <= 128 and os.environ.get("DSB200_ROTARY_LATENT_FLASH", "1") != "0")
        self._row = (64 if used <= 64 else 128) if self._flash else used  # width of a cached row
        self._heads_p = 1
        while self._heads_p < c.n_heads:
            self._heads_p *= 2

    @property
    def kv_block_size(self) -> int:
        return 64

    @property
    def q_block_size(self) -> int:
        return 1

    @property
    def cache_row(self) -> int:
        return self._row

    @property
    def attended_width(self) -> int:
        """Values per head the attention kernel returns: the whole (padded) row on the tensor cores, the latent alone otherwise."""
        return self._row if self._flash else self._config.kv_rank

    def cache_shapes(self):
        """(planes, heads, width) of the layer's cache tensor: one plane, one shared 'head', the row."""
        return [(1, 1, self._row)]

    # ---- parameter layouts
    def transform_fp32_param(self, param: torch.Tensor) -> InferenceParameter:
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())

    def transform_sink_param(self, param: torch.Tensor) -> InferenceParameter:
        """One sink score per head, fp32; padded to the heads the tensor-core kernel works on."""
        w = param.to(torch.float32).reshape(-1)
        if self._flash and self._heads_p > w.numel():
            w = torch.nn.functional.pad(w, (0, self._heads_p - w.numel()))
        return InferenceParameter.initialize(w.contiguous())

    def transform_key_up_param(self, param: torch.Tensor) -> InferenceParameter:
        """[heads * qk_dim, kv_rank] -> [heads, qk_dim + rot_dim, row]: right operand of the per-head map (q_h | q_rot,h) -> (U_h^T q_h | q_rot,h)."""
        c = self._config
        w = torch.zeros(c.n_heads, c.qk_dim + c.rot_dim, self._row, dtype=self._dtype)
        w[:, :c.qk_dim, :c.kv_rank] = param.to(self._dtype).reshape(c.n_heads, c.qk_dim, c.kv_rank)
        w[:, c.qk_dim:, c.kv_rank:c.kv_rank + c.rot_dim] = torch.eye(c.rot_dim, dtype=self._dtype)
        return InferenceParameter.initialize(w)

    def transform_value_up_param(self, param: torch.Tensor) -> InferenceParameter:
        """[heads * v_dim, kv_rank] -> [heads, attended width, v_dim]: right operand of the per-head value up-projection (zero rows meet what
        the attended row holds behind the latent)."""
        c = self._config
        w = torch.zeros(c.n_heads, self.attended_width, c.v_dim, dtype=self._dtype)
        w[:, :c.kv_rank] = param.to(self._dtype).reshape(c.n_heads, c.v_dim, c.kv_rank).transpose(1, 2)
        return InferenceParameter.initialize(w)

    # ---- forward
    def forward(self, proj: torch.Tensor, cols, kv_cache: torch.Tensor, batch, kv_norm_w: torch.Tensor, key_up_w: torch.Tensor,
                value_up_w: torch.Tensor, sink: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """proj [T, N]: the fused projection with the query heads (qk_dim plain | rot_dim to rotate, head by head) at column cols[0], the
        low-rank row (kv_rank | rot_dim) at cols[1] and, with `head_gate`, one gate pre-activation per head at cols[2]; the query heads'
        rotated parts are overwritten.  kv_cache [blocks, block_size, 1, row].  sink fp32 [heads].  Returns [T, heads * v_dim]."""
        c = self._config
        q0, kv0, g0 = cols
        T, H, R, dq = proj.shape[0], c.n_heads, self._row, c.qk_dim + c.rot_dim
        cache = kv_cache.view(kv_cache.shape[0], kv_cache.shape[1], R)
        tok_seq, tok_pos, bt = batch.tok_seq(), batch.tok_pos(), batch.block_table()
        if c.rotate_dim and (self._freq is None or self._freq.device != proj.device):
            self._freq = self._freq_host.to(proj.device)
        K.latent_rotary_append(proj, q0, kv0, kv_norm_w, self._freq if c.rotate_dim else None, tok_seq, tok_pos, bt, cache, H, c.qk_dim, c.rot_dim,
                               c.kv_rank, c.rotate_dim, c.eps)
        q = proj[:, q0:q0 + H * dq].view(T, H, dq).transpose(0, 1)  # [H, T, dq]
        bs = cache.shape[1]
        sink = sink if c.learned_sink else None
        if self._flash and bs >= 8 and 128 % bs == 0:
            qa = torch.bmm(q, key_up_w)  # [H, T, R]; the kernel reads it head-major through its TMA strides, missing heads as zeros
            att = K.paged_latent_flash(qa.transpose(0, 1), cache, tok_seq, tok_pos, bt, c.scale, heads=self._heads_p, sink_logit=sink,
                                       decode=batch.current_tokens <= 2 * batch.current_sequences)
            o = torch.bmm(att[:, :H].transpose(0, 1), value_up_w)  # [H, T, v_dim]
        else:
            qa = _bmm(q, key_up_w, self._dtype)  # [H, T, R]
            W = self.attended_width
            att = torch.empty(H, T, W, dtype=self._dtype, device=proj.device)
            plane = (cache, cache.stride(0))
            K.sink_attention_ex(qa.transpose(0, 1), qa.stride(0), plane, R, plane, R, tok_seq, tok_pos, bt, bs, att.transpose(0, 1), att.stride(0), H, 1,
                                R, W, c.scale, sink_logit=sink[:H] if sink is not None else None)
            o = _bmm(att, value_up_w, self._dtype)  # [H, T, v_dim]
        if c.head_gate:
            return K.gate_heads_scalar(o.contiguous(), proj[:, g0:g0 + H], out)  # heads side by side per token and the gate, one pass
        o = o.transpose(0, 1).reshape(T, H * c.v_dim)
        if out is not None:
            out.copy_(o)
            return out
        return o
