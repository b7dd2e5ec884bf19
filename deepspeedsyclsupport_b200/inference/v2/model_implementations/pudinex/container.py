"""Containers of the Pudinex family: tensor names of its checkpoints -> parameters of the inference model.

Every layer has `l<i>.norm1` and a mixer under `l<i>.mix.`: `{q, f, f.b, lower, v, norm, o}` for a 'hgrn2' layer, `{q, k, v, q.norm, k.norm,
o}` for an 'attention' layer.  A dense feed-forward is `l<i>.mlp.{gate, up, down}`; a mixture of experts `l<i>.mlp.{router, correction,
e<j>.gate, e<j>.up, e<j>.down}` and, with a shared expert, `l<i>.mlp.shared.{gate, up, down}`.  Outside the layers: `embed`, `final.norm`,
`head`.  Linear weights have shape [out, in]."""
from typing import Optional

import torch

from ..common_parameters import (EmbeddingParameter, MoEGatingWeightParameter, NormParameter, UnembedParameter, UnfusedMoEGatedMLPParameter,
                                 UnfusedMoEMLP2Parameter)
from ..layer_container_base import LayerContainer
from ..parameter_base import ParameterBase


class DenseParameter(ParameterBase):
    """A linear weight in the activation dtype."""
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(self.params)


class Fp32Parameter(ParameterBase):
    """Small tensors that enter norms, gates or routers: kept fp32."""
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_fp32_param(self.params)


class TiedGateInputParameter(ParameterBase):
    """(query | forget gate | value) projections of a tied-gate linear attention mixer, stacked."""
    q: torch.Tensor
    f: torch.Tensor
    v: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(torch.cat([self.q, self.f, self.v], dim=0))


class AttentionInputParameter(ParameterBase):
    """(query | key | value) projections of an attention mixer, stacked."""
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(torch.cat([self.q, self.k, self.v], dim=0))


class GatedPairParameter(ParameterBase):
    """(gate | up) projections of a gated feed-forward, stacked."""
    gate: torch.Tensor
    up: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(torch.cat([self.gate, self.up], dim=0))


class _PudinexLayerContainer(LayerContainer):
    norm1_w: NormParameter
    o_w: DenseParameter
    ff_in_w: Optional[GatedPairParameter]
    ff_down_w: Optional[DenseParameter]
    router_w: Optional[MoEGatingWeightParameter]
    correction: Optional[Fp32Parameter]
    experts_gu: Optional[UnfusedMoEGatedMLPParameter]
    experts_dn: Optional[UnfusedMoEMLP2Parameter]
    shared_in_w: Optional[GatedPairParameter]
    shared_down_w: Optional[DenseParameter]

    PARAM_MAPPING = {
        "norm1": "norm1_w.params",
        "mix.o": "o_w.params",
        "mlp.gate": "ff_in_w.gate",
        "mlp.up": "ff_in_w.up",
        "mlp.down": "ff_down_w.params",
        "mlp.router": "router_w.params",
        "mlp.correction": "correction.params",
        "mlp.e*.gate": "experts_gu.gating_experts",
        "mlp.e*.up": "experts_gu.up_experts",
        "mlp.e*.down": "experts_dn.experts",
        "mlp.shared.gate": "shared_in_w.gate",
        "mlp.shared.up": "shared_in_w.up",
        "mlp.shared.down": "shared_down_w.params",
    }

    def __init__(self, model, layer_index: int) -> None:
        self.layer_index = layer_index
        model._loading_layer = layer_index  # the expert lists are sized per layer
        super().__init__(model)
        for p in self._params.values():
            p.layer_index = layer_index


class PudinexTiedGateContainer(_PudinexLayerContainer):
    mix_in_w: TiedGateInputParameter
    f_bias: Fp32Parameter
    lower: Fp32Parameter
    mix_norm: Fp32Parameter

    PARAM_MAPPING = {
        "mix.q": "mix_in_w.q",
        "mix.f": "mix_in_w.f",
        "mix.v": "mix_in_w.v",
        "mix.f.b": "f_bias.params",
        "mix.lower": "lower.params",
        "mix.norm": "mix_norm.params",
    }


class PudinexAttentionContainer(_PudinexLayerContainer):
    mix_in_w: AttentionInputParameter
    norm_q: Fp32Parameter
    norm_k: Fp32Parameter

    PARAM_MAPPING = {
        "mix.q": "mix_in_w.q",
        "mix.k": "mix_in_w.k",
        "mix.v": "mix_in_w.v",
        "mix.q.norm": "norm_q.params",
        "mix.k.norm": "norm_k.params",
    }


class PudinexNonTransformerContainer(LayerContainer):
    embed: EmbeddingParameter
    final_norm_w: NormParameter
    lm_head: UnembedParameter

    PARAM_MAPPING = {"embed": "embed.params", "final.norm": "final_norm_w.params", "head": "lm_head.params"}
