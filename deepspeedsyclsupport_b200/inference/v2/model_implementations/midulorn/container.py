"""Containers of the Midulorn family: tensor names of its checkpoints -> parameters of the inference model.

Every layer has `l<i>.norm1` (and `l<i>.norm2` with a feed-forward) and a mixer under `l<i>.mix.`:
  latent_attention  {q, dkv, dkv.norm, uk, uv, sink, g, o}
  mingru            {z, z.b, x, x.b, g, o}
  attention         {q, k, v, o} with biases `<name>.b`, {q, k, v}.conv, {q, k}.norm, vmix, r1, r2, sink
A dense feed-forward is `l<i>.mlp.{up, down, act}`; a mixture of experts `l<i>.mlp.{router, e<j>.gate, e<j>.up, e<j>.down}`.  Outside the
layers: `embed` (also the output projection) and `final.norm`.  Linear weights have shape [out, in]."""
from typing import Optional

import torch

from ..common_parameters import EmbeddingParameter, MoEGatingWeightParameter, NormParameter, UnfusedMoEGatedMLPParameter, UnfusedMoEMLP2Parameter
from ..layer_container_base import LayerContainer
from ..parameter_base import ParameterBase


class DenseParameter(ParameterBase):
    """A linear weight in the activation dtype."""
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(self.params)


class Fp32Parameter(ParameterBase):
    """Small tensors that enter norms, gates, scores or routers: kept fp32 (a single number becomes a tensor of one entry)."""
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_fp32_param(self.params.reshape(-1) if self.params.dim() == 0 else self.params)


class ActivationPairParameter(ParameterBase):
    """The two numbers (p, q) of an xIELU activation -> the pair of coefficients its kernel reads."""
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_xielu_param(self.params)


class FinalNormParameter(ParameterBase):
    """Weight of the norm in front of the output projection (the logit constant is folded into it)."""
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_final_norm_param(self.params)


class LatentInputParameter(ParameterBase):
    """(queries | low-rank row | head gates) projections of a latent-attention mixer, stacked."""
    q: torch.Tensor
    dkv: torch.Tensor
    g: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(torch.cat([self.q, self.dkv, self.g], dim=0))


class KeyUpParameter(ParameterBase):
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_key_up_param(self.params, self.layer_index)


class HeadSinkParameter(ParameterBase):
    """One sink score per head of a latent-attention mixer (padded to the heads its kernel works on)."""
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_head_sink_param(self.params, self.layer_index)


class ValueUpParameter(ParameterBase):
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_value_up_param(self.params, self.layer_index)


class GatedUnitInputParameter(ParameterBase):
    """(gate | candidate | output gate) projections of a minimal gated recurrence, stacked."""
    z: torch.Tensor
    x: torch.Tensor
    g: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(torch.cat([self.z, self.x, self.g], dim=0))


class AttentionInputParameter(ParameterBase):
    """(query | key | value) projections of an attention mixer, stacked."""
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(torch.cat([self.q, self.k, self.v], dim=0))


class StackedFp32Parameter(ParameterBase):
    """Per-channel fp32 tensors of the query, key and value projections (their biases), stacked."""
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_fp32_param(torch.cat([self.q, self.k, self.v], dim=0))


class ConvTapsParameter(ParameterBase):
    """Convolution taps [channels, taps] of the query, key and value projections -> one fp32 tensor [taps, all channels]: the layout the
    prepare kernel reads (the lanes of a warp read neighbouring channels of one tap)."""
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_fp32_param(torch.cat([self.q, self.k, self.v], dim=0).t())


class _MidulornLayerContainer(LayerContainer):
    norm1_w: NormParameter
    norm2_w: Optional[NormParameter]
    o_w: DenseParameter
    ff_up_w: Optional[DenseParameter]
    ff_down_w: Optional[DenseParameter]
    ff_act: Optional[ActivationPairParameter]
    router_w: Optional[MoEGatingWeightParameter]
    experts_gu: Optional[UnfusedMoEGatedMLPParameter]
    experts_dn: Optional[UnfusedMoEMLP2Parameter]

    PARAM_MAPPING = {
        "norm1": "norm1_w.params",
        "norm2": "norm2_w.params",
        "mix.o": "o_w.params",
        "mlp.up": "ff_up_w.params",
        "mlp.down": "ff_down_w.params",
        "mlp.act": "ff_act.params",
        "mlp.router": "router_w.params",
        "mlp.e*.gate": "experts_gu.gating_experts",
        "mlp.e*.up": "experts_gu.up_experts",
        "mlp.e*.down": "experts_dn.experts",
    }

    def __init__(self, model, layer_index: int) -> None:
        self.layer_index = layer_index
        model._loading_layer = layer_index  # the expert lists are sized per layer
        super().__init__(model)
        for p in self._params.values():
            p.layer_index = layer_index


class MidulornLatentContainer(_MidulornLayerContainer):
    in_w: LatentInputParameter
    kv_norm: Fp32Parameter
    key_up: KeyUpParameter
    value_up: ValueUpParameter
    sink: HeadSinkParameter

    PARAM_MAPPING = {
        "mix.q": "in_w.q",
        "mix.dkv": "in_w.dkv",
        "mix.g": "in_w.g",
        "mix.dkv.norm": "kv_norm.params",
        "mix.uk": "key_up.params",
        "mix.uv": "value_up.params",
        "mix.sink": "sink.params",
    }


class MidulornGatedUnitContainer(_MidulornLayerContainer):
    in_w: GatedUnitInputParameter
    z_bias: Fp32Parameter
    x_bias: Fp32Parameter

    PARAM_MAPPING = {
        "mix.z": "in_w.z",
        "mix.x": "in_w.x",
        "mix.g": "in_w.g",
        "mix.z.b": "z_bias.params",
        "mix.x.b": "x_bias.params",
    }


class MidulornAttentionContainer(_MidulornLayerContainer):
    in_w: AttentionInputParameter
    in_bias: StackedFp32Parameter
    conv_w: ConvTapsParameter
    norm_q: Fp32Parameter
    norm_k: Fp32Parameter
    vmix: Optional[Fp32Parameter]
    r1: Fp32Parameter
    r2: Fp32Parameter
    sink: Fp32Parameter
    o_bias: Fp32Parameter

    PARAM_MAPPING = {
        "mix.q": "in_w.q",
        "mix.k": "in_w.k",
        "mix.v": "in_w.v",
        "mix.q.b": "in_bias.q",
        "mix.k.b": "in_bias.k",
        "mix.v.b": "in_bias.v",
        "mix.q.conv": "conv_w.q",
        "mix.k.conv": "conv_w.k",
        "mix.v.conv": "conv_w.v",
        "mix.q.norm": "norm_q.params",
        "mix.k.norm": "norm_k.params",
        "mix.vmix": "vmix.params",
        "mix.r1": "r1.params",
        "mix.r2": "r2.params",
        "mix.sink": "sink.params",
        "mix.o.b": "o_bias.params",
    }


class MidulornNonTransformerContainer(LayerContainer):
    embed: EmbeddingParameter
    final_norm_w: FinalNormParameter

    PARAM_MAPPING = {"embed": "embed.params", "final.norm": "final_norm_w.params"}
