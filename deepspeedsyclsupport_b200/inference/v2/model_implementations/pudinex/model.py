"""Pudinex: a decoder-only family built from
  * an fp32 residual stream that starts as the token embedding times a constant,
  * layers with ONE norm whose output every sublayer reads -- x += mixer(h) + ff(h), h = norm(x) -- where the norm is an RMS norm over equal
    consecutive parts of the row, each part on its own,
  * 'attention' mixers: per-head RMS norms of queries and keys (one weight shared by the heads), a rotate-half rotation of the first entries
    of a head with ramp-scaled frequencies, values divided by their own root mean square, scores with a tanh soft cap, a softmax with one
    more, valueless entry of score 0; query / key and value heads may differ in size,
  * 'hgrn2' mixers: linear attention whose forget gate (with a learned lower bound per channel) also decides what is written; the read-out
    gets a per-head RMS norm,
  * feed-forwards that are absent, dense (clamped gate times (up + 1)), or a mixture of experts with a softmax router over experts plus
    weightless identity experts, a selection bias, renormalised weights and an optional shared expert,
  * a final norm of the same kind and the unembedding.
Every size may differ from layer to layer; all of them, the order of layers and the constants come from config.json.

The class reuses the ragged engine's plumbing from `RaggedTransformer` (containers and streamed loading, decode-step CUDA graphs, the state
manager's paged cache and block tables) and replaces the module set and the layer loop.  Attention layers get their cache tensors (one
two-plane tensor -- in bf16 of heads padded to a width the tensor-core kernels take -- or a key and a value tensor when the head sizes
differ), all sharing a sequence's block ids; the recurrent mixers' matrices
live in the state manager's per-sequence state slots, described by `state_config`.

Fused steps: all projections that read a layer's normed input are ONE GEMM (mixer inputs | dense or shared-expert gate and up); the mixer's
output projection and the dense / shared-expert down projection are ONE GEMM over the concatenated [mixer output | activated hidden] rows,
which also forms their sum before any rounding; the sublayers' outputs join the fp32 stream inside the next layer's norm kernel (the last
layer's inside the final norm, for the wanted rows only)."""
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ...inference_utils import ActivationType, DtypeEnum, NormTypeEnum
from ...modules import heuristics
from ...modules.configs import (DSEmbeddingsConfig, DSLinearConfig, DSMoEConfig, DSNormConfig, DSSinkAttentionConfig, DSTiedGateConfig,
                                DSUnembedConfig, RampRotaryScalingConfig)
from ...ragged.manager_configs import KVCacheConfig
from ... import kernels as K
from ..inference_model_base import DSInferenceModelBase
from ..ragged_transformer import RaggedTransformer

DENSE_ACT_ALPHA = 1.702  # the dense feed-forward's gate is g sigmoid(1.702 g) ...
DENSE_ACT_SHIFT = 1.0  # ... times (up + 1)
SOFTMAX_SINK = 1.0  # the attention softmax has one more entry of score 0: exp(0) joins the denominator


@dataclass
class PudinexAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[dict]


@dataclass
class PudinexTiedGateSpec:
    heads: int
    dim: int
    vdim: int


@dataclass
class PudinexFeedForwardSpec:
    kind: str  # "dense" | "moe"
    ff: int = 0  # dense: hidden size; moe: hidden size of an expert
    limit: float = 0.0  # dense: clamp of gate and up
    experts: int = 0
    identity: int = 0
    top: int = 0
    shared_ff: int = 0  # 0 = no shared expert


@dataclass
class PudinexLayerSpec:
    kind: str  # "attention" | "hgrn2"
    attn: Optional[PudinexAttentionSpec] = None
    gate: Optional[PudinexTiedGateSpec] = None
    mlp: Optional[PudinexFeedForwardSpec] = None


@dataclass
class PudinexSpec:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    norm_groups: int
    embedding_scale: float
    layers: List[PudinexLayerSpec] = field(default_factory=list)
    family: str = "pudinex"

    @property
    def num_layers(self):
        return len(self.layers)

    @classmethod
    def from_config(cls, c: dict) -> "PudinexSpec":
        layers = []
        for i, lc in enumerate(c["layers"]):
            m = lc["mixer"]
            mlp = None
            f = lc.get("mlp")
            if f is not None:
                if f.get("kind") == "dense":
                    mlp = PudinexFeedForwardSpec("dense", ff=int(f["ff"]), limit=float(f["limit"]))
                elif f.get("kind") == "moe":
                    r, sh = f["router"], f.get("shared")
                    mlp = PudinexFeedForwardSpec("moe", ff=int(f["expert"]["ff"]), experts=int(r["experts"]), identity=int(r.get("identity", 0)),
                                                 top=int(r["top"]), shared_ff=int(sh["ff"]) if sh else 0)
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind '{f.get('kind')}'")
            if lc["type"] == "attention":
                rot = m.get("rot") or {}
                attn = PudinexAttentionSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                            scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0), rot_dims=int(rot.get("dims", 0)),
                                            rot_base=float(rot.get("base", 10000.0)), rot_scaling=dict(rot["scaling"]) if rot.get("scaling") else None)
                layers.append(PudinexLayerSpec("attention", attn=attn, mlp=mlp))
            elif lc["type"] == "hgrn2":
                layers.append(PudinexLayerSpec("hgrn2", gate=PudinexTiedGateSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"])), mlp=mlp))
            else:
                raise ValueError(f"layer {i}: unknown mixer type '{lc['type']}'")
        return cls(vocab_size=int(c["vocab"]), hidden_size=int(c["width"]), norm_eps=float(c["norm"]["eps"]), norm_groups=int(c["norm"].get("groups", 1)),
                   embedding_scale=float((c.get("embedding") or {}).get("scale", 1.0)), layers=layers)


class PudinexInferenceModel(RaggedTransformer, DSInferenceModelBase):
    describes_own_cache = True  # the engine builds its paged cache from `kv_cache_config` below

    def __init__(self, spec: PudinexSpec, tp_group=None, dtype=torch.bfloat16, device=None, engine_config=None, quantization_mode=""):
        from .container import PudinexAttentionContainer, PudinexNonTransformerContainer, PudinexTiedGateContainer
        assert dtype in (torch.bfloat16, torch.float32), "Pudinex runs with bf16 or fp32 activations"
        assert not quantization_mode, "Pudinex has no quantised linears"
        self._loading_layer = 0
        self._init_plumbing(spec, tp_group, dtype, device, engine_config)
        assert self.tp == 1, "Pudinex is served on one GPU per replica (its recurrent mixers are not sharded for tensor parallelism)"
        self.hq = self.hkv = 0
        self.vocab_padded = spec.vocab_size
        self._build_modules()
        self.layers = [(PudinexAttentionContainer if L.kind == "attention" else PudinexTiedGateContainer)(self, i) for i, L in enumerate(spec.layers)]
        self.non_transformer = PudinexNonTransformerContainer(self)
        # cache tensors of every attention layer (the recurrent layers have none): one two-plane tensor or a (key, value) pair
        self._cache_index, n = {}, 0
        for i, L in enumerate(spec.layers):
            if L.kind == "attention":
                k = len(self.attn_mods[i].cache_shapes())
                self._cache_index[i] = tuple(range(n, n + k))
                n += k
        self._fused = [None] * len(spec.layers)  # per layer, after loading: (input weight, output weight)
        self._layer_hook = None  # debugging aid: called as hook(layer index, fp32 residual) after every layer

    # ---- facts the parameter classes ask for
    @property
    def n_experts(self):
        mlp = self.spec.layers[self._loading_layer].mlp
        return mlp.experts if mlp is not None else 0

    # ---- cache and state
    def kv_cache_config(self, block_size: int = 64):
        name = {torch.bfloat16: "bf16", torch.float32: "fp32"}[self.dtype]
        shapes = [s for i, L in enumerate(self.spec.layers) if L.kind == "attention" for s in self.attn_mods[i].cache_shapes()]
        if not shapes:
            shapes = [(1, 1, 1)]  # a model without attention layers caches nothing per token; the block bookkeeping stays uniform
        return KVCacheConfig(block_size=block_size, cache_shape=(len(shapes), max(s[1] for s in shapes), max(s[2] for s in shapes)),
                             cache_dtype=name, layer_shapes=shapes)

    def state_config(self):
        """What a sequence carries between steps besides its cache blocks: `l<i>.mix.S`, the matrices of every recurrent layer."""
        specs = []
        for i, L in enumerate(self.spec.layers):
            if L.kind == "hgrn2":
                specs += self.gate_mods[i].state_specs(f"l{i}.mix")
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
        self.norm_mod = heuristics.instantiate_pre_norm(DSNormConfig(type=NormTypeEnum.RMSNorm, channels=D, residual_dtype=DtypeEnum.fp32, eps=s.norm_eps,
                                                                      shared_input=True, groups=s.norm_groups, **common), ec)
        self.lin_mod = heuristics.instantiate_linear(DSLinearConfig(in_channels=D, out_channels=D, **common), None)
        self.attn_mods, self.gate_mods, self.moe_mods = [], [], []
        for L in s.layers:
            attn = gate = None
            if L.kind == "attention":
                a = L.attn
                attn = heuristics.instantiate_attention(DSSinkAttentionConfig(
                    n_heads_q=a.heads, n_heads_kv=a.kv_heads, head_size=a.dim, value_size=a.vdim, scale=a.scale, softcap=a.softcap, sink=SOFTMAX_SINK,
                    rotate_dim=a.rot_dims, theta_base=a.rot_base,
                    rotary_scaling=RampRotaryScalingConfig(**a.rot_scaling) if a.rot_scaling else None, eps=s.norm_eps, max_sequences=max_seqs,
                    **common), ec)
            else:
                g = L.gate
                gate = heuristics.instantiate_recurrent(DSTiedGateConfig(n_heads=g.heads, key_size=g.dim, value_size=g.vdim, eps=s.norm_eps,
                                                                         max_sequences=max_seqs, **common), ec)
            self.attn_mods.append(attn)
            self.gate_mods.append(gate)
            f = L.mlp
            self.moe_mods.append(None if f is None or f.kind != "moe" else heuristics.instantiate_moe(
                DSMoEConfig(model_dim=D, intermediate_features=f.ff, n_experts=f.experts, n_identity_experts=f.identity, top_k=f.top,
                            activation=ActivationType.SiGLU, normalize_scores=True, use_correction=True, **common), ec))
        self.unembed_mod = heuristics.instantiate_unembed(DSUnembedConfig(max_tokens=max_tokens, dtype=dt, norm_type=NormTypeEnum.RMSNorm, model_dim=D,
                                                                          max_sequences=max_seqs, vocab_size=s.vocab_size, eps=s.norm_eps,
                                                                          norm_groups=s.norm_groups, residual_fp32=True), ec)

    # ---- parameter transforms
    def transform_embedding_param(self, param):
        return self._dev(self.embed_mod.transform_param(param))

    def transform_norm_param(self, param):
        return self._dev(self.norm_mod.transform_param(param))

    def transform_dense_param(self, param):
        return self._dev(self.lin_mod.transform_param(param))

    def transform_fp32_param(self, param):
        return self._dev(param.to(torch.float32).contiguous())

    def transform_unembed_param(self, param):
        return self._dev(param.to(self.dtype).contiguous())

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
                raise KeyError(f"unexpected parameter '{name}' for family pudinex")
        self.finish_loading()

    def check_populated(self):
        super().check_populated()
        for i, (L, c) in enumerate(zip(self.spec.layers, self.layers)):
            f = L.mlp
            need = []
            if f is not None and f.kind == "dense":
                need = ["ff_in_w", "ff_down_w"]
            elif f is not None:
                need = ["router_w", "correction", "experts_gu", "experts_dn"] + (["shared_in_w", "shared_down_w"] if f.shared_ff else [])
            if any(k not in c for k in need):
                raise RuntimeError(f"layer {i}: feed-forward tensors are missing ({[k for k in need if k not in c]})")

    def finish_loading(self):
        """All tensors have arrived: check every layer and form its fused weights -- the input weight (mixer projections | dense or shared
        gate and up) and the output weight (mixer output | dense or shared down, side by side along the input axis)."""
        self.check_populated()
        for i, (L, c) in enumerate(zip(self.spec.layers, self.layers)):
            f = L.mlp
            side_in = side_out = None
            if f is not None and f.kind == "dense":
                side_in, side_out = c["ff_in_w"], c["ff_down_w"]
            elif f is not None and f.shared_ff:
                side_in, side_out = c["shared_in_w"], c["shared_down_w"]
            o_w = c["o_w"]
            if L.kind == "attention" and self.attn_mods[i].out_head_width != L.attn.vdim:
                # the attention kernels work on heads padded to a common width: zero weights meet the (zero) padding columns of their output
                P = self.attn_mods[i].out_head_width
                o_w = torch.nn.functional.pad(o_w.view(o_w.shape[0], L.attn.heads, L.attn.vdim), (0, P - L.attn.vdim)).reshape(o_w.shape[0], L.attn.heads * P)
            if side_in is None:
                self._fused[i] = (c["mix_in_w"], o_w.contiguous())
            else:
                self._fused[i] = (torch.cat([c["mix_in_w"], side_in], dim=0).contiguous(), torch.cat([o_w, side_out], dim=1).contiguous())

    # ---- forward
    def _side_hidden(self, L):
        """Hidden size of the feed-forward part that shares the layer's two fused GEMMs (dense, or the shared expert); 0 = none."""
        f = L.mlp
        if f is None:
            return 0
        return f.ff if f.kind == "dense" else f.shared_ff

    def forward(self, batch, state_manager):
        """batch: finalized RaggedBatchWrapper.  Returns fp32 logits [batch.n_logit_rows, vocab]."""
        s, nt = self.spec, self.non_transformer
        x = self.embed_mod(batch, nt.embed)  # fp32 residual stream [T, width]
        pending = None  # outputs of the previous layer's sublayers that have not joined the stream yet: ((activation dtype, ...), fp32 or None)
        for li, L in enumerate(s.layers):
            W = self.layers[li]
            w_in, w_out = self._fused[li]
            moe = self.moe_mods[li]
            branches, fp32_branch = pending if pending is not None else (None, None)
            if moe is not None:
                _, h, h32 = self.norm_mod(x, branches, W["norm1_w"], fp32_branch=fp32_branch, fp32_copy=True)
            else:
                _, h = self.norm_mod(x, branches, W["norm1_w"], fp32_branch=fp32_branch)
            proj = self.lin_mod(h, w_in)
            side = self._side_hidden(L)
            if L.kind == "attention":
                a = L.attn
                n_mix_in, n_mix_out = (a.heads + a.kv_heads) * a.dim + a.kv_heads * a.vdim, self.attn_mods[li].out_width
            else:
                g = L.gate
                n_mix_in, n_mix_out = g.heads * (2 * g.dim + g.vdim), g.heads * g.vdim
            # [mixer output | activated hidden]; rows start 16 bytes apart at least (what the tensor-core attention's stores want) whatever the sizes
            mixed = torch.empty(h.shape[0], -(-(n_mix_out + side) // 8) * 8, dtype=h.dtype, device=h.device)[:, :n_mix_out + side]
            if L.kind == "attention":
                caches = [state_manager.get_cache(ci) for ci in self._cache_index[li]]
                self.attn_mods[li](proj, (0, a.heads * a.dim, (a.heads + a.kv_heads) * a.dim), caches[0], caches[1] if len(caches) > 1 else None, batch,
                                   W["norm_q"], W["norm_k"], mixed[:, :n_mix_out])
            else:
                self.gate_mods[li](proj, (0, g.heads * g.dim, 2 * g.heads * g.dim), W["f_bias"], W["lower"], W["mix_norm"], batch, state_manager,
                                   f"l{li}.mix", mixed[:, :n_mix_out])
            if side:
                f = L.mlp
                if f.kind == "dense":
                    K.clamped_swish_gate_cols(proj, n_mix_in, n_mix_in + side, side, mixed[:, n_mix_out:], DENSE_ACT_ALPHA, f.limit, DENSE_ACT_SHIFT)
                else:  # the shared expert: silu(gate) * up
                    K.clamped_swish_gate_cols(proj, n_mix_in, n_mix_in + side, side, mixed[:, n_mix_out:], 1.0, float("inf"), 0.0)
            y = self.lin_mod(mixed, w_out)  # mixer output projection + dense / shared down projection, summed inside the GEMM
            y32 = None
            if moe is not None:
                y32 = moe(h, W["router_w"], W["experts_gu"], W["experts_dn"], correction=W["correction"], router_input=h32)
            pending = ((y, ), y32)
            if self._layer_hook is not None:
                self.norm_mod(x, pending[0], None, fp32_branch=pending[1])
                pending = None
                self._layer_hook(li, x)
        return self.unembed_mod(x, nt.lm_head, batch, gamma=nt.final_norm_w, pending=pending)
