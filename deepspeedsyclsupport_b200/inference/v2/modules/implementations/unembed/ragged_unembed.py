"""(parity: inference/v2/modules/implementations/unembed/ragged_unembed.py:24-120: logits_gather + final norm + projection)"""
from typing import Any, Dict, Optional

import torch

from ......ops import fused_ops as FO
from ......ops.gemm import dense_matmul, gemm
from .... import kernels as K
from ....inference_utils import DtypeEnum, NormTypeEnum
from ...configs import DSUnembedConfig
from ...interfaces import DSUnembedBase, DSUnembedRegistry


@DSUnembedRegistry.register_module
class DSRaggedUnembed(DSUnembedBase):

    @staticmethod
    def name() -> str:
        return "ragged_unembed"

    @staticmethod
    def supports_config(config: DSUnembedConfig) -> bool:
        return DtypeEnum(config.dtype) in (DtypeEnum.fp16, DtypeEnum.bf16, DtypeEnum.fp32)

    def __init__(self, config: DSUnembedConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        self._norm = None if config.norm_type is None else NormTypeEnum(config.norm_type)
        self._output = None

    @property
    def output(self) -> torch.Tensor:
        return self._output

    def transform_norm_param(self, param: torch.Tensor) -> torch.Tensor:
        """Weight of the final norm in fp32, times `logit_scale`: scale * (W (n * w)) = W (n * (scale w)), so the constant costs no pass."""
        return param.to(torch.float32) * self._config.logit_scale if self._config.logit_scale != 1.0 else param.to(torch.float32)

    def forward(self, hidden_states: torch.Tensor, vocab_embedding: torch.Tensor, ragged_metadata, bias: Optional[torch.Tensor] = None,
                gamma: Optional[torch.Tensor] = None, beta: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, pending=None) -> torch.Tensor:
        """`residual` (optional): the residual stream the last hidden state still has to be added to -- only the gathered rows
        (one per sequence) are added and normalised, not the whole batch.  `pending` (fp32 stream only): ((outputs in the activation
        dtype, ...), fp32 output or None) of the last layer's sublayers that have not joined the stream yet; they are added to the
        gathered rows only."""
        last_tok = ragged_metadata.logit_rows()
        c = self._config
        if c.residual_fp32:
            return self._forward_fp32_residual(hidden_states, vocab_embedding, last_tok, gamma, pending)
        h = K.logits_gather(hidden_states, last_tok)
        r = K.logits_gather(residual, last_tok) if residual is not None else None
        if self._norm == NormTypeEnum.RMSNorm:
            h = FO.rms_norm(h, gamma, self._config.eps, r)
        elif self._norm == NormTypeEnum.LayerNorm:
            h = FO.layer_norm(h, gamma, beta, self._config.eps, r)
        elif r is not None:
            h = h + r
        if isinstance(h, tuple):
            h = h[0]
        if h.is_cuda and h.dtype == torch.bfloat16:
            logits = gemm(h, vocab_embedding)
        else:
            logits = torch.nn.functional.linear(h, vocab_embedding)
        if bias is not None:
            logits = logits + bias
        if c.logit_softcap > 0:
            logits = c.logit_softcap * torch.tanh(logits.float() / c.logit_softcap)
        self._output = logits
        return logits

    def _forward_fp32_residual(self, residual, vocab_embedding, rows, gamma, pending=None):
        """Gather + RMS norm of the wanted rows in one kernel (fp32 in, activation dtype out), projection with fp32 logits,
        soft cap in place."""
        c = self._config
        assert self._norm == NormTypeEnum.RMSNorm and residual.dtype == torch.float32
        act = DtypeEnum(c.dtype).value
        if rows.numel() == 0:
            return torch.empty(0, vocab_embedding.shape[0], dtype=torch.float32, device=residual.device)
        if c.norm_groups > 1 or pending is not None:  # the stream still lacks the last layer's outputs and / or is normed in parts
            assert c.norm_weight_offset == 0.0
            branches, fp32_branch = pending if pending is not None else ((), None)
            h = K.stream_group_norm(residual, branches, fp32_branch, gamma, c.norm_groups, c.eps, out_dtype=act, rows=rows)
        else:
            h = K.sandwich_norm(residual, w=gamma, o=c.norm_weight_offset, eps=c.eps, out_dtype=act, rows=rows)
        logits = dense_matmul(h, vocab_embedding, out_dtype=torch.float32)
        if not logits.is_contiguous():
            logits = logits.contiguous()
        if c.logit_softcap > 0:
            K.softcap_(logits, c.logit_softcap)
        self._output = logits
        return logits
