"""Midulorn: a decoder-only family built from
  * an fp32 residual stream that starts as the token embedding times a constant,
  * layers whose norms sit BEHIND the sums: x <- norm1(alpha x + mixer(x)), x <- norm2(alpha x + ff(x)); the sublayers read the stream itself,
  * 'latent_attention' mixers: keys and values are per-head up-projections of one cached, normed low-rank latent per token; beside it one
    rotated key part that all heads share (rotate-half pairs); a learned sink per head in the softmax; a sigmoid gate per token and head,
  * 'mingru' mixers: a minimal gated recurrence with one number of state per channel whose gates read only the current token,
  * 'attention' mixers: projections with biases behind a short causal convolution, per-head query / key norms, no rotation, a logarithmic
    distance term on the scores, a mask by fixed parts of the sequence, a learned sink per head, values mixed with the first such layer's,
  * feed-forwards that are absent, dense (xIELU) or a mixture of experts (softmax router, weights not renormalised, silu-gated experts),
  * a final norm and the embedding table as output projection, times a constant.
Every size may differ from layer to layer; all of them, the order of layers and the constants come from config.json.

The class reuses the ragged engine's plumbing from `RaggedTransformer` (containers and streamed loading, decode-step CUDA graphs, the state
manager's paged cache and block tables) and replaces the module set and the layer loop.  Attention layers of both kinds get their cache
tensors, all sharing a sequence's block ids; recurrent states and convolution tails live in the state manager's per-sequence slots,
described by `state_config`.

Fused steps: all projections that read a mixer's input are ONE GEMM; sum + norm + the activation-dtype copy of the new stream are one kernel
(the attention's output bias joins there, in fp32); rotation + latent norm + cache append are one kernel, as are bias + convolution + head
norms + value mixing + cache append; the recurrence forms its gates itself; gather of the wanted rows + final norm is one kernel."""
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ...inference_utils import ActivationType, DtypeEnum, NormTypeEnum
from ...modules import heuristics
from ...modules.configs import (DSConvSinkAttentionConfig, DSEmbeddingsConfig, DSLinearConfig, DSMinGRUConfig, DSMoEConfig, DSNormConfig,
                                DSRotaryLatentAttentionConfig, DSUnembedConfig)
from ...ragged.manager_configs import KVCacheConfig
from ... import kernels as K
from ..inference_model_base import DSInferenceModelBase
from ..ragged_transformer import RaggedTransformer


@dataclass
class MidulornLatentSpec:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float


@dataclass
class MidulornGatedUnitSpec:
    width: int


@dataclass
class MidulornAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    part: int
    value_mix: str  # "none" | "source" (the first layer that mixes values: it hands its own on) | "mix"


@dataclass
class MidulornFeedForwardSpec:
    kind: str  # "dense" | "moe"
    ff: int = 0  # dense: hidden size; moe: hidden size of an expert
    experts: int = 0
    top: int = 0


@dataclass
class MidulornLayerSpec:
    kind: str  # "latent_attention" | "mingru" | "attention"
    latent: Optional[MidulornLatentSpec] = None
    unit: Optional[MidulornGatedUnitSpec] = None
    attn: Optional[MidulornAttentionSpec] = None
    mlp: Optional[MidulornFeedForwardSpec] = None


@dataclass
class MidulornSpec:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    stream_mult: float
    embedding_scale: float
    logit_scale: float
    layers: List[MidulornLayerSpec] = field(default_factory=list)
    family: str = "midulorn"

    @property
    def num_layers(self):
        return len(self.layers)

    @classmethod
    def from_config(cls, c: dict) -> "MidulornSpec":
        layers, mixes_values = [], None
        for i, lc in enumerate(c["layers"]):
            m = lc["mixer"]
            mlp = None
            f = lc.get("mlp")
            if f is not None:
                if f.get("kind") == "dense":
                    mlp = MidulornFeedForwardSpec("dense", ff=int(f["ff"]))
                elif f.get("kind") == "moe":
                    mlp = MidulornFeedForwardSpec("moe", ff=int(f["expert"]["ff"]), experts=int(f["router"]["experts"]), top=int(f["router"]["top"]))
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind '{f.get('kind')}'")
            if lc["type"] == "latent_attention":
                rot = m.get("rot") or {}
                spec = MidulornLatentSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]), kv_rank=int(m["kv_rank"]),
                                          scale=float(m["scale"]), rot_dims=int(rot.get("dims", m["rot_dim"])), rot_base=float(rot.get("base", 10000.0)))
                layers.append(MidulornLayerSpec("latent_attention", latent=spec, mlp=mlp))
            elif lc["type"] == "mingru":
                layers.append(MidulornLayerSpec("mingru", unit=MidulornGatedUnitSpec(width=int(m["width"])), mlp=mlp))
            elif lc["type"] == "attention":
                heads = int(m["heads"])
                spec = MidulornAttentionSpec(heads=heads, kv_heads=int(m.get("kv_heads", heads)), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                             conv=int(m.get("conv", 1)), scale=float(m["scale"]), part=int((m.get("mask") or {}).get("size", 0)),
                                             value_mix="none")
                if m.get("v_mix"):
                    if mixes_values is None:
                        spec.value_mix, mixes_values = "source", spec
                    else:
                        spec.value_mix = "mix"
                        if spec.kv_heads * spec.vdim != mixes_values.kv_heads * mixes_values.vdim:
                            raise ValueError(f"layer {i}: its values ({spec.kv_heads} x {spec.vdim}) cannot be mixed with the first mixing layer's "
                                             f"({mixes_values.kv_heads} x {mixes_values.vdim})")
                layers.append(MidulornLayerSpec("attention", attn=spec, mlp=mlp))
            else:
                raise ValueError(f"layer {i}: unknown mixer type '{lc['type']}'")
        return cls(vocab_size=int(c["vocab"]), hidden_size=int(c["width"]), norm_eps=float(c["norm"]["eps"]), stream_mult=float(c.get("postln_alpha", 1.0)),
                   embedding_scale=float((c.get("embedding") or {}).get("scale", 1.0)), logit_scale=float(c.get("logit_scale", 1.0)), layers=layers)


class MidulornInferenceModel(RaggedTransformer, DSInferenceModelBase):
    describes_own_cache = True  # the engine builds its paged cache from `kv_cache_config` below

    def __init__(self, spec: MidulornSpec, tp_group=None, dtype=torch.bfloat16, device=None, engine_config=None, quantization_mode=""):
        from .container import MidulornAttentionContainer, MidulornGatedUnitContainer, MidulornLatentContainer, MidulornNonTransformerContainer
        assert dtype in (torch.bfloat16, torch.float32), "Midulorn runs with bf16 or fp32 activations"
        assert not quantization_mode, "Midulorn has no quantised linears"
        self._loading_layer = 0
        self._init_plumbing(spec, tp_group, dtype, device, engine_config)
        assert self.tp == 1, "Midulorn is served on one GPU per replica (its recurrent mixers are not sharded for tensor parallelism)"
        self.hq = self.hkv = 0
        self.vocab_padded = spec.vocab_size
        self._build_modules()
        kinds = {"latent_attention": MidulornLatentContainer, "mingru": MidulornGatedUnitContainer, "attention": MidulornAttentionContainer}
        self.layers = [kinds[L.kind](self, i) for i, L in enumerate(spec.layers)]
        self.non_transformer = MidulornNonTransformerContainer(self)
        # cache tensors of every attention layer of either kind (the recurrent layers have none)
        self._cache_index, n = {}, 0
        for i, L in enumerate(spec.layers):
            if self.attn_mods[i] is not None:
                k = len(self.attn_mods[i].cache_shapes())
                self._cache_index[i] = tuple(range(n, n + k))
                n += k
        self._layer_hook = None  # debugging aid: called as hook(layer index, fp32 residual) after every layer

    # ---- facts the parameter classes ask for
    @property
    def n_experts(self):
        mlp = self.spec.layers[self._loading_layer].mlp
        return mlp.experts if mlp is not None else 0

    # ---- cache and state
    def kv_cache_config(self, block_size: int = 64):
        name = {torch.bfloat16: "bf16", torch.float32: "fp32"}[self.dtype]
        shapes = [s for m in self.attn_mods if m is not None for s in m.cache_shapes()]
        if not shapes:
            shapes = [(1, 1, 1)]  # a model without attention layers caches nothing per token; the block bookkeeping stays uniform
        return KVCacheConfig(block_size=block_size, cache_shape=(len(shapes), max(s[1] for s in shapes), max(s[2] for s in shapes)),
                             cache_dtype=name, layer_shapes=shapes)

    def state_config(self):
        """What a sequence carries between steps besides its cache blocks: `l<i>.mix.S` (the recurrent layers' state) and `l<i>.mix.conv`
        (the last projected rows in front of an attention layer's convolution)."""
        specs = []
        for i, L in enumerate(self.spec.layers):
            if L.kind == "mingru":
                specs += self.unit_mods[i].state_specs(f"l{i}.mix")
            elif L.kind == "attention":
                specs += self.attn_mods[i].state_specs(f"l{i}.mix")
        return specs

    # ---- building blocks
    def _build_modules(self):
        s, ec, dt = self.spec, self.engine_config, DtypeEnum(self.dtype)
        sm = getattr(ec, "state_manager", None)
        max_tokens = getattr(sm, "max_ragged_batch_size", 768)
        max_seqs = getattr(sm, "max_ragged_sequence_count", 512)
        D = s.hidden_size
        common = dict(max_tokens=max_tokens, input_dtype=dt, output_dtype=dt)
        self.embed_mod = heuristics.instantiate_embed(DSEmbeddingsConfig(max_tokens=max_tokens, residual_dtype=dt, embedding_dim=D, fp32_stream=True,
                                                                         embedding_scale=s.embedding_scale), ec)
        self.norm_mod = heuristics.instantiate_post_norm(DSNormConfig(type=NormTypeEnum.RMSNorm, channels=D, residual_dtype=DtypeEnum.fp32, eps=s.norm_eps,
                                                                       post_sum=True, stream_mult=s.stream_mult, **common), ec)
        self.lin_mod = heuristics.instantiate_linear(DSLinearConfig(in_channels=D, out_channels=D, **common), None)
        self.attn_mods, self.unit_mods, self.moe_mods = [], [], []
        for L in s.layers:
            attn = unit = None
            if L.kind == "latent_attention":
                a = L.latent
                attn = heuristics.instantiate_attention(DSRotaryLatentAttentionConfig(
                    n_heads=a.heads, qk_dim=a.dim, rot_dim=a.rot_dim, v_dim=a.vdim, kv_rank=a.kv_rank, scale=a.scale, rotate_dim=a.rot_dims,
                    theta_base=a.rot_base, learned_sink=True, head_gate=True, eps=s.norm_eps, max_sequences=max_seqs, **common), ec)
            elif L.kind == "attention":
                a = L.attn
                attn = heuristics.instantiate_attention(DSConvSinkAttentionConfig(
                    n_heads_q=a.heads, n_heads_kv=a.kv_heads, head_size=a.dim, value_size=a.vdim, conv_taps=a.conv, scale=a.scale, part_size=a.part,
                    distance_bias=True, learned_sink=True, value_mix=a.value_mix, eps=s.norm_eps, max_sequences=max_seqs, **common), ec)
            else:
                unit = heuristics.instantiate_recurrent(DSMinGRUConfig(width=L.unit.width, max_sequences=max_seqs, **common), ec)
            self.attn_mods.append(attn)
            self.unit_mods.append(unit)
            f = L.mlp
            self.moe_mods.append(None if f is None or f.kind != "moe" else heuristics.instantiate_moe(
                DSMoEConfig(model_dim=D, intermediate_features=f.ff, n_experts=f.experts, top_k=f.top, activation=ActivationType.SiGLU,
                            normalize_scores=False, fp32_combine=True, **common), ec))
        self.unembed_mod = heuristics.instantiate_unembed(DSUnembedConfig(max_tokens=max_tokens, dtype=dt, norm_type=NormTypeEnum.RMSNorm, model_dim=D,
                                                                          max_sequences=max_seqs, vocab_size=s.vocab_size, eps=s.norm_eps,
                                                                          logit_scale=s.logit_scale, residual_fp32=True), ec)

    # ---- parameter transforms
    def transform_embedding_param(self, param):
        return self._dev(self.embed_mod.transform_param(param))  # the table in the activation dtype: also the output projection

    def transform_norm_param(self, param):
        return self._dev(self.norm_mod.transform_param(param))

    def transform_final_norm_param(self, param):
        return self._dev(self.unembed_mod.transform_norm_param(param).contiguous())

    def transform_dense_param(self, param):
        return self._dev(self.lin_mod.transform_param(param))

    def transform_fp32_param(self, param):
        return self._dev(param.to(torch.float32).contiguous())

    def transform_xielu_param(self, param):
        p, q = (float(v) for v in param.to(torch.float32).reshape(-1))
        return self._dev(K.xielu_coefficients(p, q))

    def transform_key_up_param(self, param, layer_index):
        return self._dev(self.attn_mods[layer_index].transform_key_up_param(param))

    def transform_value_up_param(self, param, layer_index):
        return self._dev(self.attn_mods[layer_index].transform_value_up_param(param))

    def transform_head_sink_param(self, param, layer_index):
        return self._dev(self.attn_mods[layer_index].transform_sink_param(param))

    def _any_moe(self):
        mods = [m for m in self.moe_mods if m is not None]
        assert mods, "an expert tensor arrived for a model without mixture-of-experts layers"
        return mods[0]

    def transform_moe_gate_param(self, param):
        return self._dev(self._any_moe().transform_gate_param(param))

    def transform_moe_mlp_1_param(self, param, gated=True):
        return self._dev(self._any_moe().transform_moe_mlp_1_param(param))

    def transform_moe_mlp_2_param(self, param):
        return self._dev(self._any_moe().transform_moe_mlp_2_param(param))

    def load_canonical(self, sd):
        """State dict with the family's own tensor names."""
        import re
        rx = re.compile(r"^l(\d+)\.(.*)$")
        for name, tensor in sd.items():
            m = rx.match(name)
            ok = self.layers[int(m.group(1))].set_dependency(m.group(2), tensor) if m else self.non_transformer.set_dependency(name, tensor)
            if not ok:
                raise KeyError(f"unexpected parameter '{name}' for family midulorn")
        self.check_populated()

    def check_populated(self):
        super().check_populated()
        for i, (L, c) in enumerate(zip(self.spec.layers, self.layers)):
            f = L.mlp
            need = []
            if f is not None:
                need = ["norm2_w"] + (["ff_up_w", "ff_down_w", "ff_act"] if f.kind == "dense" else ["router_w", "experts_gu", "experts_dn"])
            if L.kind == "attention" and L.attn.value_mix == "mix":
                need.append("vmix")
            if any(k not in c for k in need):
                raise RuntimeError(f"layer {i}: tensors are missing ({[k for k in need if k not in c]})")

    # ---- forward
    def _latent_mixer(self, li, L, W, h, batch, state_manager):
        a = L.latent
        nq, nkv = a.heads * (a.dim + a.rot_dim), a.kv_rank + a.rot_dim
        proj = self.lin_mod(h, W["in_w"])  # (queries | low-rank row | head gates)
        o = self.attn_mods[li](proj, (0, nq, nq + nkv), state_manager.get_cache(self._cache_index[li][0]), batch, W["kv_norm"], W["key_up"],
                               W["value_up"], W["sink"])
        return self.lin_mod(o, W["o_w"]), None

    def _unit_mixer(self, li, L, W, h, batch, state_manager):
        n = L.unit.width
        proj = self.lin_mod(h, W["in_w"])  # (gate | candidate | output gate)
        o = torch.empty(h.shape[0], n, dtype=h.dtype, device=h.device)
        self.unit_mods[li](proj, (0, n, 2 * n), W["z_bias"], W["x_bias"], batch, state_manager, f"l{li}.mix", o)
        return self.lin_mod(o, W["o_w"]), None

    def _attention_mixer(self, li, L, W, h, batch, state_manager, shared):
        a, mod = L.attn, self.attn_mods[li]
        proj = self.lin_mod(h, W["in_w"])  # (queries | keys | values); their biases join in front of the convolution
        caches = [state_manager.get_cache(ci) for ci in self._cache_index[li]]
        o = torch.empty(h.shape[0], -(-mod.out_width // 8) * 8, dtype=h.dtype, device=h.device)[:, :mod.out_width]
        _, v_own = mod(proj, 0, W["in_bias"], W["conv_w"], W["norm_q"], W["norm_k"], W["r1"], W["r2"], W["sink"], caches[0],
                       caches[1] if len(caches) > 1 else None, batch, state_manager, f"l{li}.mix", o, v_source=shared.get("v"),
                       mix=W["vmix"] if a.value_mix == "mix" else None)
        if v_own is not None:
            shared["v"] = v_own
        return self.lin_mod(o, self._out_weight(li, L, W)), W["o_bias"]

    def _out_weight(self, li, L, W):
        """The attention's output weight; on the tensor-core path with zero columns where the heads' padding sits."""
        mod, a = self.attn_mods[li], L.attn
        if mod.out_head_width == a.vdim:
            return W["o_w"]
        cached = getattr(self, "_padded_out", None)
        if cached is None:
            cached = self._padded_out = {}
        if li not in cached:
            w, P = W["o_w"], mod.out_head_width
            cached[li] = torch.nn.functional.pad(w.view(w.shape[0], a.heads, a.vdim), (0, P - a.vdim)).reshape(w.shape[0], a.heads * P).contiguous()
        return cached[li]

    def forward(self, batch, state_manager):
        """batch: finalized RaggedBatchWrapper.  Returns fp32 logits [batch.n_logit_rows, vocab]."""
        s, nt = self.spec, self.non_transformer
        x = self.embed_mod(batch, nt.embed)  # fp32 residual stream [T, width]
        h = self.norm_mod.emit(x)  # the stream in the activation dtype: what the sublayers read
        shared = {}  # what later layers read of earlier ones within a step: the first mixing layer's values
        for li, L in enumerate(s.layers):
            W = self.layers[li]
            if L.kind == "latent_attention":
                y, bias = self._latent_mixer(li, L, W, h, batch, state_manager)
            elif L.kind == "mingru":
                y, bias = self._unit_mixer(li, L, W, h, batch, state_manager)
            else:
                y, bias = self._attention_mixer(li, L, W, h, batch, state_manager, shared)
            x, h = self.norm_mod(x, y, W["norm1_w"], bias=bias)
            f = L.mlp
            if f is not None and f.kind == "dense":
                y = self.lin_mod(K.xielu(self.lin_mod(h, W["ff_up_w"]), W["ff_act"]), W["ff_down_w"])
                x, h = self.norm_mod(x, y, W["norm2_w"])
            elif f is not None:
                y32 = self.moe_mods[li](h, W["router_w"], W["experts_gu"], W["experts_dn"], router_input=x)  # the router reads the fp32 stream
                x, h = self.norm_mod(x, None, W["norm2_w"], fp32_branch=y32)
            elif "norm2_w" in W:  # no feed-forward, yet a second norm was stored: it norms the scaled stream alone
                x, h = self.norm_mod(x, None, W["norm2_w"])
            if self._layer_hook is not None:
                self._layer_hook(li, x)
        return self.unembed_mod(x, nt.embed, batch, gamma=nt.final_norm_w)
