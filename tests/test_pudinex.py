"""Pudinex on the ragged engine against the plain float64 oracle of tests/pudinex_oracle.py: every mechanism alone (kernels of
csrc/ragged/sink_attention_ops.cu, the tied-gate scan of csrc/ragged/recurrent_ops.cu, the grouped norm / identity-expert extensions of
csrc/ragged/latent_ops.cu), then whole models of several small random configurations through the engine factory, the paged cache, the state
slots, the scheduler and the decode-step graphs."""
import copy
import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import pudinex_oracle as O  # noqa: E402

F64 = torch.float64
SCALING = {"factor": 6.0, "original": 48, "fast": 6.0, "slow": 1.0}


# ------------------------------------------------------------------------------------------------------------------ CPU: plumbing
def test_spec_reads_every_size_from_the_config():
    from deepspeedsyclsupport_b200.inference.v2.model_implementations.pudinex import PudinexSpec
    cfg = O.make_config([O.attention_layer(6, 3, 10, 14, scale=0.3, softcap=9.0, rot_dims=4, base=500.0, scaling=SCALING, mlp=O.moe(5, 2, 3, 12, shared_ff=7)),
                         O.hgrn2_layer(5, 6, 9, mlp=O.dense(22, limit=0.7)), O.hgrn2_layer(2, 4, 4)], vocab=77, width=40, eps=3e-5, groups=5, embedding_scale=1.5)
    s = PudinexSpec.from_config(cfg)
    assert (s.vocab_size, s.hidden_size, s.norm_eps, s.norm_groups, s.embedding_scale, s.num_layers) == (77, 40, 3e-5, 5, 1.5, 3)
    a, f = s.layers[0].attn, s.layers[0].mlp
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.softcap, a.rot_dims, a.rot_base, a.rot_scaling) == (6, 3, 10, 14, 0.3, 9.0, 4, 500.0, SCALING)
    assert (f.kind, f.experts, f.identity, f.top, f.ff, f.shared_ff) == ("moe", 5, 2, 3, 12, 7)
    g, d = s.layers[1].gate, s.layers[1].mlp
    assert (g.heads, g.dim, g.vdim) == (5, 6, 9) and (d.kind, d.ff, d.limit) == ("dense", 22, 0.7) and s.layers[2].mlp is None
    with pytest.raises(ValueError):
        PudinexSpec.from_config(dict(cfg, layers=[dict(cfg["layers"][0], type="other")]))
    with pytest.raises(ValueError):
        PudinexSpec.from_config(dict(cfg, layers=[dict(cfg["layers"][1], mlp={"kind": "other"})]))


def test_family_is_registered_and_chosen_by_the_config():
    from deepspeedsyclsupport_b200.inference.v2.engine_factory import model_type_of
    from deepspeedsyclsupport_b200.inference.v2.model_implementations import PudinexPolicy, policy_for
    assert model_type_of({"architecture": "Pudinex"}) == "pudinex" and policy_for("pudinex") is PudinexPolicy


def test_ramp_scaled_frequencies():
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import RampRotaryScalingConfig
    from deepspeedsyclsupport_b200.inference.v2.modules.implementations.attention.sink_blocked_attention import ramp_scaled_frequencies
    for dims, base, sc in ((16, 10000.0, None), (40, 5e5, {"factor": 3.0, "original": 256, "fast": 16.0, "slow": 2.0}), (24, 300.0, SCALING), (2, 7.0, SCALING),
                           (8, 100.0, {"factor": 2.0, "original": 4, "fast": 1000.0, "slow": 900.0})):
        got, mag = ramp_scaled_frequencies(dims, base, RampRotaryScalingConfig(**sc) if sc else None)
        want, wmag = O.yarn_frequencies(dims, base, sc)
        assert torch.allclose(got, want, rtol=1e-14, atol=0) and abs(mag - wmag) < 1e-15
    f, mag = O.yarn_frequencies(24, 300.0, SCALING)  # fast channels kept, slow ones divided, a ramp between them
    ratio = (f / O.yarn_frequencies(24, 300.0)[0]).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 6) < 1e-12 and any(1 / 6 + 1e-9 < r < 1 - 1e-9 for r in ratio) and abs(mag - (0.1 * math.log(6.0) + 1)) < 1e-15


def test_cache_state_and_fused_weights_of_a_model():
    from deepspeedsyclsupport_b200.inference.v2.checkpoint import InMemoryModelEngine
    from deepspeedsyclsupport_b200.inference.v2.engine_factory import build_model_from_checkpoint
    cfg = O.make_config([O.hgrn2_layer(2, 8, 6, mlp=O.dense(20)), O.attention_layer(4, 2, 6, 10, rot_dims=4, mlp=O.moe(3, 2, 2, 10, shared_ff=12)),
                         O.attention_layer(2, 1, 12, 12), O.hgrn2_layer(3, 4, 4, mlp=O.moe(2, 0, 1, 6))], width=24)
    w = O.random_weights(cfg)
    m = build_model_from_checkpoint("pudinex", cfg, InMemoryModelEngine(w), None, device=torch.device("cpu"), dtype=torch.float32)
    kc = m.kv_cache_config(block_size=32)
    # unequal key / value head sizes: a key tensor and a value tensor; equal: one two-plane tensor; recurrent layers cache nothing per token
    assert kc.layer_shapes == [(1, 2, 6), (1, 2, 10), (2, 1, 12)] and kc.cache_dtype == "fp32" and m._cache_index == {1: (0, 1), 2: (2, )}
    w_in, w_out = m._fused[0]
    assert w_in.shape == (2 * (8 + 8 + 6) + 2 * 20, 24) and w_out.shape == (24, 2 * 6 + 20)  # (q | f | v | gate | up), (o | down)
    w_in, w_out = m._fused[1]
    assert w_in.shape == (4 * 6 + 2 * 6 + 2 * 10 + 2 * 12, 24) and w_out.shape == (24, 4 * 10 + 12)  # the shared expert rides along
    assert m._fused[2][0].shape == (2 * 12 + 12 + 12, 24) and m._fused[3][1].shape == (24, 12)
    assert m.layers[1]["experts_gu"].shape == (3, 20, 24) and m.layers[1]["router_w"].shape == (5, 24) and m.layers[1]["router_w"].dtype == torch.float32
    assert m.layers[0].get("experts_gu") is None and m.layers[0]["lower"].dtype == torch.float32
    for missing in ("l1.mlp.correction", "l1.mlp.shared.up", "l0.mlp.down", "l3.mix.lower"):
        with pytest.raises(Exception):  # a missing tensor is reported, not ignored
            w2 = dict(w)
            w2.pop(missing)
            build_model_from_checkpoint("pudinex", cfg, InMemoryModelEngine(w2), None, device=torch.device("cpu"), dtype=torch.float32)


def test_bf16_attention_heads_are_padded_to_a_tensor_core_width():
    """bf16: keys and values of any sizes up to 128 share one two-plane cache tensor of width 64 / 128 and the output projection gets zero
    columns for the padding; fp32 and wider heads keep their own sizes."""
    from deepspeedsyclsupport_b200.inference.v2.checkpoint import InMemoryModelEngine
    from deepspeedsyclsupport_b200.inference.v2.engine_factory import build_model_from_checkpoint
    cfg = O.make_config([O.attention_layer(4, 2, 6, 10, mlp=O.dense(8)), O.attention_layer(2, 1, 96, 40), O.attention_layer(2, 2, 64, 64), O.attention_layer(1, 1, 130, 20)],
                        width=24)
    w = O.random_weights(cfg)
    m = build_model_from_checkpoint("pudinex", cfg, InMemoryModelEngine(w), None, device=torch.device("cpu"), dtype=torch.bfloat16)
    assert m.kv_cache_config(block_size=16).layer_shapes == [(2, 2, 64), (2, 1, 128), (2, 2, 64), (1, 1, 130), (1, 1, 20)]
    assert [a.out_head_width for a in m.attn_mods] == [64, 128, 64, 20]
    w_out = m._fused[0][1]
    assert w_out.shape == (24, 4 * 64 + 8)
    per_head = w_out[:, :4 * 64].view(24, 4, 64)
    assert torch.equal(per_head[:, :, :10].reshape(24, 40), w["l0.mix.o"]) and float(per_head[:, :, 10:].abs().max()) == 0
    assert torch.equal(w_out[:, 4 * 64:], w["l0.mlp.down"])


def test_router_with_identity_experts_is_served_by_the_grouped_router():
    from deepspeedsyclsupport_b200.inference.v2.inference_utils import ActivationType, DtypeEnum
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSMoEConfig
    kw = dict(max_tokens=8, model_dim=8, intermediate_features=4, activation=ActivationType.SiGLU, normalize_scores=True, use_correction=True,
              input_dtype=DtypeEnum.bf16, output_dtype=DtypeEnum.bf16)
    assert heuristics.instantiate_moe(DSMoEConfig(n_experts=3, n_identity_experts=2, top_k=5, **kw), None).name() == "grouped_topk_moe"
    with pytest.raises(Exception):  # more picks than router outputs
        heuristics.instantiate_moe(DSMoEConfig(n_experts=3, n_identity_experts=2, top_k=6, **kw), None)


# ------------------------------------------------------------------------------------------------------------- GPU: mechanisms
gpu = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def _K():
    from deepspeedsyclsupport_b200.inference.v2 import kernels
    return kernels


class _Batch:
    """Ragged metadata of a step, built by hand: seqs = [(slot, seen, new tokens, block ids)]."""

    def __init__(self, seqs, block, max_blocks=16):
        tok_seq, tok_pos, desc, at = [], [], [], 0
        bt = torch.zeros(len(seqs), max_blocks, dtype=torch.int32)
        for i, (slot, seen, n, blocks) in enumerate(seqs):
            tok_seq += [i] * n
            tok_pos += list(range(seen, seen + n))
            desc.append([at, n, seen, slot])
            bt[i, :len(blocks)] = torch.tensor(blocks, dtype=torch.int32)
            at += n
        self.current_sequences, self.current_tokens = len(seqs), at
        self._ts, self._tp = torch.tensor(tok_seq, dtype=torch.int32).cuda(), torch.tensor(tok_pos, dtype=torch.int32).cuda()
        self._bt, self._desc = bt.cuda(), torch.tensor(desc, dtype=torch.int32).cuda()

    def tok_seq(self):
        return self._ts

    def tok_pos(self):
        return self._tp

    def block_table(self):
        return self._bt

    def seq_desc(self):
        return self._desc


class _State:
    """Stand-in for the state manager: named per-slot buffers (filled with garbage: a sequence at position 0 must not read them)."""

    def __init__(self, specs, slots):
        self.buf = {s.name: torch.full((slots, ) + tuple(s.shape), 7.5, dtype=s.dtype, device="cuda") for s in specs}

    def get_state(self, name):
        return self.buf[name]


def _rel(got, want):
    return float((got.cpu().double() - want).norm() / want.norm())


def _cuts(total, sizes):
    out, at = [], 0
    for n in sizes:
        out.append((at, min(n, total - at)))
        at += n
        if at >= total:
            break
    if at < total:
        out.append((at, total - at))
    return out


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("dim,groups", [(6, 3), (40, 5), (42, 1), (384, 3), (512, 4), (1024, 1), (320, 2)])
def test_grouped_norm_sums_the_branches_into_the_stream(dim, groups, dt):
    """Part sizes that take the 16-byte path (multiples of 128) and ones that do not; zero to three branches; a row gather that adds the
    branches to the gathered rows only and leaves the stream alone; the unrounded copy."""
    K = _K()
    g = torch.Generator().manual_seed(dim)
    x0 = (torch.randn(9, dim, generator=g) * 3).cuda()
    ya, yb = ((torch.randn(9, dim, generator=g) * 2).to(dt).cuda() for _ in range(2))
    yc = torch.randn(9, dim, generator=g).cuda()
    w = (1 + 0.3 * torch.randn(dim, generator=g)).cuda()
    # one part much larger than the others: a norm over the whole row would flatten every other part
    x0[:, :dim // groups] *= 50
    tol = dict(rtol=1e-5, atol=1e-5) if dt == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    for branches, extra in (((), None), ((ya, ), None), ((ya, yb), yc), ((), yc)):
        total = x0.cpu().double() + sum(b.cpu().double() for b in branches) + (extra.cpu().double() if extra is not None else 0)
        want = O.group_rms_norm(total, w.cpu(), groups, 1e-5)
        x = x0.clone()
        out, out32 = K.stream_group_norm(x, branches, extra, w, groups, 1e-5, out_dtype=dt, fp32_copy=True)
        assert torch.allclose(x.cpu().double(), total, rtol=1e-6, atol=1e-5)
        assert out.dtype == dt and out32.dtype == torch.float32 and torch.allclose(out.cpu().double(), want, **tol)
        assert torch.allclose(out32.cpu().double(), want, rtol=1e-5, atol=1e-5) and torch.equal(out32.to(dt), out)
        x = x0.clone()
        assert K.stream_group_norm(x, branches, extra, None, groups, 1e-5) is None and torch.allclose(x.cpu().double(), total, rtol=1e-6, atol=1e-5)
        rows = torch.tensor([7, 0, 7, 3], dtype=torch.int32).cuda()
        x = x0.clone()
        got = K.stream_group_norm(x, branches, extra, w, groups, 1e-5, out_dtype=dt, rows=rows)
        assert torch.equal(x, x0) and torch.allclose(got.cpu().double(), want[[7, 0, 7, 3]], **tol)


@gpu
def test_embedding_times_a_constant():
    K = _K()
    table = torch.randn(11, 20).bfloat16().cuda()
    ids = torch.tensor([3, 0, 10, 3]).cuda()
    got = K.embed_sinusoid(ids, table, None, None, scale=2.75)
    assert got.dtype == torch.float32 and torch.equal(got, table[ids].float() * 2.75)  # the product is formed in fp32, not rounded to the table's dtype


def _attention_module(m, dt, eps=1e-5):
    from deepspeedsyclsupport_b200.inference.v2.inference_utils import DtypeEnum
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSSinkAttentionConfig, RampRotaryScalingConfig
    rot = m.get("rot") or {}
    return heuristics.instantiate_attention(DSSinkAttentionConfig(
        max_tokens=512, n_heads_q=m["heads"], n_heads_kv=m["kv_heads"], head_size=m["dim"], value_size=m["vdim"], scale=m["scale"], softcap=m.get("softcap") or 0.0,
        rotate_dim=rot.get("dims", 0), theta_base=rot.get("base", 10000.0), rotary_scaling=RampRotaryScalingConfig(**rot["scaling"]) if rot.get("scaling") else None,
        eps=eps, max_sequences=8, input_dtype=DtypeEnum(dt), output_dtype=DtypeEnum(dt)), None)


def _caches(mod, blocks, block, dt):
    return [torch.full((blocks, ) + ((p, ) if p != 1 else ()) + (block, h, d), 3.0, dtype=dt, device="cuda") for p, h, d in mod.cache_shapes()]


ATTENTION_CASES = [
    dict(heads=6, kv_heads=2, dim=10, vdim=6, softcap=4.0, rot=dict(dims=6, base=300.0, scaling=SCALING)),  # grouped heads, unequal sizes, partial rotation
    dict(heads=2, kv_heads=2, dim=8, vdim=8, softcap=0.0, rot=dict(dims=8, base=50.0)),  # equal sizes (two-plane cache), every entry rotated, no cap
    dict(heads=3, kv_heads=1, dim=14, vdim=20, softcap=25.0),  # one key / value head, no rotation, values wider than keys
    dict(heads=4, kv_heads=4, dim=64, vdim=32, softcap=10.0, rot=dict(dims=32, base=1e5, scaling={"factor": 3.0, "original": 64, "fast": 8.0, "slow": 2.0})),
    dict(heads=1, kv_heads=1, dim=5, vdim=3, softcap=1.0, rot=dict(dims=2, base=10.0)),  # one head, a tight cap
    dict(heads=2, kv_heads=2, dim=32, vdim=96, softcap=15.0, rot=dict(dims=16, base=1000.0)),  # values wider than keys, padded to 128 in bf16
    dict(heads=2, kv_heads=1, dim=136, vdim=40, softcap=8.0, rot=dict(dims=136, base=1e4)),  # heads above 128: the CUDA-core kernel in bf16 too
]


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("case", range(len(ATTENTION_CASES)))
@pytest.mark.parametrize("sizes", [[70], [40] + [1] * 30, [2, 5, 1, 25, 2, 9, 14]])
def test_attention_mixer(case, sizes, dt):
    """Whole, a prompt followed by single tokens, and portions cut inside pages (block 16), on shuffled pages that held something else."""
    m = dict(ATTENTION_CASES[case])
    m["scale"] = 1.7 * m["dim"] ** -0.5
    D, T, H, G, d, dv = 24, 70, m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    cfg = O.make_config([dict(type="attention", mixer=m, mlp=None)], width=D)
    w = O.sub(O.random_weights(cfg, seed=case), "l0.mix.")
    w["o"] = torch.eye(H * dv).bfloat16()
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(5)).bfloat16().double()
    want, _ = O.attention_mixer(h, w, m, 1e-5)
    mod = _attention_module(m, dt)
    caches = _caches(mod, 8, 16, dt)
    Win = torch.cat([w["q"], w["k"], w["v"]]).double()
    pages = [5, 2, 7, 0, 3]
    outs = []
    for at, n in _cuts(T, sizes):
        proj = (h[at:at + n] @ Win.T).to(dt).cuda()
        out = torch.empty(n, mod.out_width, dtype=dt, device="cuda")
        mod(proj, (0, H * d, (H + G) * d), caches[0], caches[1] if len(caches) > 1 else None, _Batch([(0, at, n, pages)], 16),
            w["q.norm"].float().cuda(), w["k.norm"].float().cuda(), out)
        per_head = out.view(n, H, mod.out_head_width)
        if mod.out_head_width > dv:  # the padding columns of a head stay empty (a masked key of a garbage page may leave ~1e-37 there)
            assert float(per_head[:, :, dv:].abs().max()) < 1e-30
        outs.append(per_head[:, :, :dv].reshape(n, H * dv))
    assert _rel(torch.cat(outs), want) < (2e-5 if dt == torch.float32 else 2.5e-2)


@gpu
@pytest.mark.parametrize("d,dv,G", [(16, 24, 1), (64, 64, 2)])
@pytest.mark.parametrize("far", [0, 3, 15, 16, 255, 256, 300, 511])
def test_a_far_key_a_sink_and_the_causal_limit_show_in_the_output(far, d, dv, G):
    """Hundreds of weak keys and ONE strong key at `far` (the first and last rows of a page, chunk borders of the kernel, far away): the
    queries at and behind it must find it, the query just before it must not; where no key is strong the sink takes most of the weight."""
    K = _K()
    H, T, block = 2 * G, 520, 16
    g = torch.Generator().manual_seed(far + d)
    q = torch.randn(T, H, d, generator=g, dtype=F64) * 0.3
    k = torch.randn(T, G, d, generator=g, dtype=F64) * 0.3
    v = torch.randn(T, G, dv, generator=g, dtype=F64)
    u = torch.randn(d, generator=g, dtype=F64)
    u = u / u.norm()
    q[:] = q - (q @ u)[..., None] * u + 2.0 * u  # every query has the same component along u ...
    k[:] = k - (k @ u)[..., None] * u - 3.0 * u  # ... which every key opposes (weights far below the sink's) ...
    k[far] += 9.0 * u  # ... except one
    scale, cap = 1.5, 20.0
    want = O.sink_attention(q, k, v, scale, cap, 1.0)
    perm = torch.randperm(40, generator=g)[:T // block + 1].tolist()
    kc = torch.zeros(40, block, G, d, device="cuda")
    vc = torch.zeros(40, block, G, dv, device="cuda")
    for j in range(T):
        kc[perm[j // block], j % block] = k[j].float().cuda()
        vc[perm[j // block], j % block] = v[j].float().cuda()
    planes = K.cache_planes(kc, vc)
    # the last 120 positions as a prompt portion and the ones around the strong key as single tokens of a step each
    checks = [list(range(T - 120, T))] + [[p] for p in (far - 1, far, far + 1, far + 17) if 0 <= p < T]
    for rows in checks:
        b = _Batch([(0, rows[0], len(rows), perm)], block, max_blocks=40)
        out = torch.empty(len(rows), H * dv, device="cuda")
        K.sink_attention(q[rows].reshape(len(rows), H * d).float().cuda(), planes[0], planes[1], b.tok_seq(), b.tok_pos(), b.block_table(), block, out, H, G, d, dv,
                         scale, cap, 1.0)
        got = out.cpu().double().view(len(rows), H, dv)
        assert torch.allclose(got, want[rows], rtol=1e-4, atol=1e-5), rows[0]
    if far >= 1:
        assert float(want[far - 1].abs().max()) < 0.05 * float(want[far].abs().max())  # the sink held the weight until the strong key came


@gpu
@pytest.mark.parametrize("d,G,group", [(64, 2, 2), (128, 1, 4), (128, 2, 1)])
@pytest.mark.parametrize("cap,sink", [(12.0, 1.0), (0.0, 1.0), (30.0, 0.0)])
@pytest.mark.parametrize("far", [5, 127, 128, 300])
def test_tensor_core_kernels_agree_with_the_oracle(far, cap, sink, d, G, group):
    """bf16, equal head sizes of 64 / 128 in a two-plane cache: the prefill and the small-atom decode kernel (with and without splits along
    the keys) against the float64 formula, with ONE strong key among hundreds of opposed ones at a page's last / first row and far away --
    found by the queries at and behind it, not by the one before it -- with and without cap and sink."""
    K = _K()
    H, T, block = G * group, 400, 16
    g = torch.Generator().manual_seed(far + d)
    q = torch.randn(T, H, d, generator=g, dtype=F64) * 0.3
    k = torch.randn(T, G, d, generator=g, dtype=F64) * 0.3
    v = torch.randn(T, G, d, generator=g, dtype=F64)
    u = torch.randn(d, generator=g, dtype=F64)
    u = u / u.norm()
    q[:] = q - (q @ u)[..., None] * u + 2.0 * u
    k[:] = k - (k @ u)[..., None] * u - 2.0 * u
    k[far] += 6.0 * u
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    scale = 1.3
    want = O.sink_attention(q.double(), k.double(), v.double(), scale, cap, sink)
    perm = torch.randperm(40, generator=g)[:T // block + 1].tolist()
    cache = torch.zeros(40, 2, block, G, d, dtype=torch.bfloat16, device="cuda")
    for j in range(T):
        cache[perm[j // block], 0, j % block] = k[j].cuda()
        cache[perm[j // block], 1, j % block] = v[j].cuda()
    cases = [(list(range(T - 150, T)), False, None), (list(range(max(far - 40, 0), min(far + 60, T))), False, 3)]
    cases += [([p], dec, sp) for p in (far - 1, far, far + 1, T - 1) if 0 <= p < T for dec in (False, True) for sp in (None, 2)]
    for rows, decode, splits in cases:
        b = _Batch([(0, rows[0], len(rows), perm)], block, max_blocks=40)
        wide = torch.zeros(len(rows), H * d + 8, dtype=torch.bfloat16, device="cuda")
        qq = q[rows].reshape(len(rows), H * d).cuda()
        assert K.paged_flash_sink_ok(qq, cache, wide[:, :H * d], H, G, d, d)
        K.paged_flash_sink(qq, cache, b.tok_seq(), b.tok_pos(), b.block_table(), wide[:, :H * d], H, G, d, scale, cap, sink, decode=decode, n_splits=splits)
        got = wide[:, :H * d].cpu().double().view(len(rows), H, d)
        assert float(wide[:, H * d:].abs().max()) == 0
        err = (got - want[rows]).abs().max() / want[rows].abs().max()
        assert float(err) < 2e-2, (rows[0], decode, splits, float(err))
    if sink > 0 and far >= 1:
        assert float(want[far - 1].abs().max()) < 0.2 * float(want[far].abs().max())  # the sink held the weight until the strong key came


def _gate_module(m, dt):
    from deepspeedsyclsupport_b200.inference.v2.inference_utils import DtypeEnum
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSTiedGateConfig
    return heuristics.instantiate_recurrent(DSTiedGateConfig(max_tokens=512, n_heads=m["heads"], key_size=m["dim"], value_size=m["vdim"], eps=1e-5, max_sequences=8,
                                                             input_dtype=DtypeEnum(dt), output_dtype=DtypeEnum(dt)), None)


def _gate_weights(m, D, seed):
    cfg = O.make_config([O.hgrn2_layer(m["heads"], m["dim"], m["vdim"])], width=D)
    w = O.sub(O.random_weights(cfg, seed=seed), "l0.mix.")
    w["o"] = torch.eye(m["heads"] * m["vdim"]).bfloat16()
    return w


def _run_gate(mod, w, m, h, cuts, dt, state, slot):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    Win = torch.cat([w["q"], w["f"], w["v"]]).double()
    outs = []
    for at, n in cuts:
        proj = (h[at:at + n] @ Win.T).to(dt).cuda()
        out = torch.empty(n, H * dv, dtype=dt, device="cuda")
        mod(proj, (0, H * d, 2 * H * d), w["f.b"].float().cuda(), w["lower"].float().cuda(), w["norm"].float().cuda(), _Batch([(slot, at, n, [])], 16), state, "r", out)
        outs.append(out)
    return torch.cat(outs)


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim", [(3, 8, 16), (1, 5, 3), (2, 32, 48), (2, 72, 40), (1, 130, 300), (2, 128, 128)])
@pytest.mark.parametrize("sizes", [[90], [1] * 60, [2, 5, 1, 33, 2, 9]])
def test_tied_gate_mixer(heads, dim, vdim, sizes, dt):
    """Whole, token by token and in portions, with the state carried in a slot that held something else before; sizes that are not powers
    of two, one head, more rows than a thread group holds at once, several column tiles."""
    m = {"heads": heads, "dim": dim, "vdim": vdim}
    D, T = 24, 60
    w = _gate_weights(m, D, heads * dim)
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(5)).bfloat16().double()
    want, _ = O.hgrn2_mixer(h, w, m, 1e-5)
    mod = _gate_module(m, dt)
    got = _run_gate(mod, w, m, h, _cuts(T, sizes), dt, _State(mod.state_specs("r"), 3), 2)
    assert _rel(got, want) < (2e-5 if dt == torch.float32 else 2.5e-2)


@gpu
def test_slow_channels_remember_the_first_tokens_through_long_decoding():
    """Lower bounds close to 1 keep a channel's memory for hundreds of tokens, a lower bound of 0 with a negative bias forgets at once: after
    400 single-token steps the read-out still equals the oracle's (a state that is lost, reset or mixed up between steps would not)."""
    m = {"heads": 2, "dim": 12, "vdim": 20}
    w = _gate_weights(m, 24, 9)
    low = torch.zeros(24)
    low[::2] = 0.995
    w["lower"] = low.bfloat16()
    w["f.b"] = torch.where(low > 0, torch.tensor(2.0), torch.tensor(-6.0)).bfloat16()
    h = torch.randn(430, 24, generator=torch.Generator().manual_seed(1)).bfloat16().double()
    h[:3] *= 4  # what the slow channels should still carry at the end
    want, S = O.hgrn2_mixer(h, w, m, 1e-5)
    mod = _gate_module(m, torch.float32)
    got = _run_gate(mod, w, m, h, _cuts(430, [30] + [1] * 400), torch.float32, _State(mod.state_specs("r"), 2), 1)
    assert _rel(got[-50:], want[-50:]) < 2e-5
    forgot, _ = O.hgrn2_mixer(h[3:], w, m, 1e-5)  # the same tokens without the first three give another read-out: they are remembered
    assert _rel(forgot[-50:], want[-50:]) > 1e-2


@gpu
def test_sequences_of_a_batch_keep_their_own_state():
    """Three sequences advance side by side with unequal portions; each equals the sequence run alone, and a new sequence that takes over a
    used slot starts from nothing."""
    m = {"heads": 2, "dim": 8, "vdim": 16}
    D = 24
    w = _gate_weights(m, D, 3)
    mod = _gate_module(m, torch.float32)
    state = _State(mod.state_specs("r"), 4)
    Win = torch.cat([w["q"], w["f"], w["v"]]).double()
    hs = {u: torch.randn(n, D, generator=torch.Generator().manual_seed(u)).bfloat16().double() for u, n in ((0, 30), (1, 7), (2, 19), (3, 12))}
    want = {u: O.hgrn2_mixer(h, w, m, 1e-5)[0] for u, h in hs.items()}
    slot = {0: 3, 1: 0, 2: 2, 3: 0}  # sequence 3 reuses the slot of sequence 1
    steps = [[(0, 10), (1, 6), (2, 1)], [(0, 1), (1, 1), (2, 17)], [(0, 19), (2, 1), (3, 5)], [(3, 7)]]
    at, got = {u: 0 for u in hs}, {u: [] for u in hs}
    for step in steps:
        hcat = torch.cat([hs[u][at[u]:at[u] + n] for u, n in step])
        proj = (hcat @ Win.T).float().cuda()
        out = torch.empty(hcat.shape[0], 32, dtype=torch.float32, device="cuda")
        mod(proj, (0, 16, 32), w["f.b"].float().cuda(), w["lower"].float().cuda(), w["norm"].float().cuda(), _Batch([(slot[u], at[u], n, []) for u, n in step], 16),
            state, "r", out)
        r = 0
        for u, n in step:
            got[u].append(out[r:r + n])
            r += n
            at[u] += n
    for u in hs:
        assert at[u] == hs[u].shape[0] and _rel(torch.cat(got[u]), want[u]) < 2e-5, u


def _moe_module(f, D, dt):
    from deepspeedsyclsupport_b200.inference.v2.inference_utils import ActivationType, DtypeEnum
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSMoEConfig
    r = f["router"]
    return heuristics.instantiate_moe(DSMoEConfig(max_tokens=512, model_dim=D, intermediate_features=f["expert"]["ff"], n_experts=r["experts"],
                                                  n_identity_experts=r.get("identity", 0), top_k=r["top"], activation=ActivationType.SiGLU, normalize_scores=True,
                                                  use_correction=True, input_dtype=DtypeEnum(dt), output_dtype=DtypeEnum(dt)), None)


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("experts,identity,top,ff,D", [(5, 2, 3, 12, 24), (4, 0, 1, 8, 40), (3, 3, 6, 16, 64), (8, 1, 2, 32, 128), (2, 5, 2, 10, 24)])
def test_router_with_identity_experts(experts, identity, top, ff, D, dt):
    """The selection adds the correction, the weights do not; identity experts hand the token's input back; the weights of the chosen sum to
    one.  A correction that lifts the otherwise weakest outputs makes the two differ for every token."""
    f = O.moe(experts, identity, top, ff)
    cfg = O.make_config([O.hgrn2_layer(1, 4, 4, mlp=f)], width=D)
    w = O.sub(O.random_weights(cfg, seed=experts * 7 + identity, router_gain=5.0), "l0.mlp.")
    corr = torch.zeros(experts + identity)
    corr[-1], corr[0] = 0.9, 0.6  # the last output (an identity expert when there is one) and the first are picked whatever their scores
    w["correction"] = corr.bfloat16()
    h = torch.randn(50, D, generator=torch.Generator().manual_seed(2)).to(dt)
    idx, wt = O.route(h, w, experts, identity, top)
    assert top < 2 or bool((idx == experts + identity - 1).any(-1).all())
    assert abs(float(wt.sum(-1).mean()) - 1) < 1e-9
    plain = torch.softmax(h.double() @ w["router"].double().T, -1).topk(top, dim=-1).indices
    assert not torch.equal(plain.sort(-1).values, idx.sort(-1).values) or top == experts + identity
    want = O.moe_ff(h, w, f)
    mod = _moe_module(f, D, dt)
    gu = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(experts)]).to(dt).cuda()
    dn = torch.stack([w[f"e{e}.down"] for e in range(experts)]).to(dt).cuda()
    got = mod(h.cuda(), w["router"].float().cuda(), gu, dn, correction=w["correction"].float().cuda(), router_input=h.float().cuda())
    assert got.dtype == torch.float32 and _rel(got, want) < (2e-5 if dt == torch.float32 else 1.5e-2)


@gpu
@pytest.mark.parametrize("dt", DTYPES)
def test_clamped_gate_on_column_ranges(dt):
    """Gate and up as column ranges of a wider projection, the result into a column range of a wider buffer; limits that cut both; odd offsets
    (one value per thread) and offsets / sizes that are multiples of four (four values per thread)."""
    K = _K()
    g = torch.Generator().manual_seed(4)
    for c0, F, pad, lead in ((7, 18, 3, 5), (8, 20, 4, 4)):
        proj = (torch.randn(13, c0 + 2 * F + pad, generator=g) * 2).to(dt).cuda()
        wide = torch.zeros(13, lead + F, dtype=dt, device="cuda")
        for alpha, limit, shift in ((1.702, 0.8, 1.0), (1.0, float("inf"), 0.0)):
            K.clamped_swish_gate_cols(proj, c0, c0 + F, F, wide[:, lead:], alpha, limit, shift)
            gt, up = proj[:, c0:c0 + F].cpu().double(), proj[:, c0 + F:c0 + 2 * F].cpu().double()
            gt, up = gt.clamp(max=limit), up.clamp(-limit, limit)
            want = gt * torch.sigmoid(alpha * gt) * (up + shift)
            assert torch.allclose(wide[:, lead:].cpu().double(), want, rtol=1e-5 if dt == torch.float32 else 1e-2, atol=1e-5 if dt == torch.float32 else 1e-2)
            assert float(wide[:, :lead].abs().max()) == 0


# ------------------------------------------------------------------------------------------------------------ GPU: whole models
CONFIGS = {
    # odd sizes that differ per layer; three norm parts; grouped and single key / value heads; unequal and equal head sizes; rotation of some,
    # all and no entries; with and without a cap; every kind of feed-forward including none, no identity expert, no shared expert, top 1
    "odd": O.make_config([
        O.hgrn2_layer(3, 6, 10, mlp=O.dense(20, limit=0.8)),
        O.attention_layer(6, 2, 10, 6, scale=0.5, softcap=5.0, rot_dims=6, base=300.0, scaling=SCALING, mlp=O.moe(5, 2, 3, 18, shared_ff=10)),
        O.hgrn2_layer(1, 12, 5),
        O.attention_layer(2, 2, 8, 8, scale=0.4, softcap=0.0, rot_dims=8, base=40.0, mlp=O.moe(3, 0, 1, 9)),
        O.attention_layer(3, 1, 14, 20, scale=0.3, softcap=50.0, mlp=O.dense(30, limit=3.0)),
        O.hgrn2_layer(2, 4, 4, mlp=O.moe(4, 1, 2, 6)),
    ], vocab=61, width=42, eps=1e-5, groups=3, embedding_scale=1.7),
    # aligned sizes (tensor-core GEMMs in bf16, 16-byte norm path), head sizes 64 and 128, one norm part
    "aligned": O.make_config([
        O.hgrn2_layer(4, 32, 32, mlp=O.moe(8, 2, 2, 32, shared_ff=32)),
        O.attention_layer(4, 2, 64, 64, softcap=30.0, rot_dims=32, base=1e5, scaling={"factor": 5.0, "original": 128, "fast": 16.0, "slow": 2.0}, mlp=O.moe(8, 2, 2, 32)),
        O.attention_layer(2, 1, 128, 128, softcap=20.0, rot_dims=128, mlp=O.dense(256, limit=2.0)),
        O.hgrn2_layer(2, 64, 128, mlp=O.dense(128, limit=1.0)),
    ], vocab=96, width=256, eps=1e-6, groups=1, embedding_scale=1.0),
    # no attention layer at all: nothing is cached per token, everything lives in the state slots
    "recurrent": O.make_config([O.hgrn2_layer(2, 8, 8, mlp=O.dense(16)), O.hgrn2_layer(2, 4, 12, mlp=O.moe(2, 1, 1, 8, shared_ff=8))], vocab=40, width=24, groups=2),
    # no recurrent layer at all: no state slots
    "attention": O.make_config([O.attention_layer(2, 1, 8, 12, rot_dims=4, mlp=O.dense(16)), O.attention_layer(4, 4, 6, 6, softcap=0.0, mlp=O.moe(3, 1, 2, 8))],
                               vocab=40, width=24, groups=4),
}
_MODELS = {}


def _model(name, tmp_path_factory, dt=torch.float32):
    """fp32 runs keep the configured top-k (every selection is compared tightly).  bf16 runs let every token use ALL router outputs of a
    layer, weighted by their scores: a top-k choice between two close scores flips under rounding and the flipped token then colours the
    rest of its sequence through the recurrent state, which says nothing about the engine (the selection itself is checked on equal inputs
    in test_router_with_identity_experts)."""
    every = dt == torch.bfloat16
    if (name, every) not in _MODELS:
        cfg = copy.deepcopy(CONFIGS[name])
        if every:
            for L in cfg["layers"]:
                if L["mlp"] is not None and L["mlp"]["kind"] == "moe":
                    L["mlp"]["router"]["top"] = L["mlp"]["router"]["experts"] + L["mlp"]["router"]["identity"]
        w = O.random_weights(cfg, seed=len(name))
        _MODELS[(name, every)] = (cfg, w, O.write_model(str(tmp_path_factory.mktemp(name)), cfg, w))
    return _MODELS[(name, every)]


def _engine(path, dt, pool_tokens=256, block=16, max_seqs=4):
    from deepspeedsyclsupport_b200.inference.v2.config_v2 import RaggedInferenceEngineConfig
    from deepspeedsyclsupport_b200.inference.v2.engine_factory import build_hf_engine
    from deepspeedsyclsupport_b200.inference.v2.ragged.manager_configs import AllocationMode, DSStateManagerConfig, MemoryConfig
    mgr = DSStateManagerConfig(max_tracked_sequences=max_seqs, max_ragged_sequence_count=max_seqs, max_ragged_batch_size=pool_tokens, max_context=pool_tokens,
                               memory_config=MemoryConfig(mode=AllocationMode.ALLOCATE, size=pool_tokens // block), kv_block_size=block)
    return build_hf_engine(path, RaggedInferenceEngineConfig(state_manager=mgr), dtype=dt)


def _close(got, want, dt):
    """Every logit row agrees up to a per-row shift, relative to the spread of the logits.  fp32: tightly.  bf16: within a few times what
    rounding of the matrix products does to these small random models, far below what a wrong key, a lost state or a wrong expert causes
    (order 1)."""
    d = got.cpu().double() - want
    d = d - d.mean(-1, keepdim=True)
    err = d.pow(2).mean(-1).sqrt() / want.std()
    if dt == torch.float32:
        return float(err.max()) < 5e-5, float(err.max())
    return float(err.max()) < 0.2 and float(err.median()) < 0.05, (float(err.median()), float(err.max()))


def _tokens(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n, ), generator=torch.Generator().manual_seed(seed))


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_every_layer(name, dt, tmp_path_factory):
    cfg, w, path = _model(name, tmp_path_factory, dt)
    eng = _engine(path, dt)
    toks = _tokens(cfg, 75, 1)
    want, res = O.run(cfg, w, toks.tolist(), collect_layers=True)
    got_res = []
    eng.model()._layer_hook = lambda li, x: got_res.append(x.clone())
    got = eng.put([7], [toks], logit_positions=[list(range(75))])
    assert got.shape == (75, cfg["vocab"]) and len(got_res) == len(res)
    for r, (a, b) in enumerate(zip(got_res, res)):
        if dt == torch.float32:
            assert torch.allclose(a.cpu().double(), b, rtol=1e-4, atol=1e-4), f"layer {r}"
        else:
            row = (a.cpu().double() - b).norm(dim=-1) / b.norm(dim=-1)
            assert float(row.max()) < 0.2 and float(row.median()) < 0.04, f"layer {r}"
    ok, err = _close(got, want, dt)
    assert ok, err
    eng.model()._layer_hook = None  # the same without the per-layer sums: the last layer's outputs join the stream inside the final norm
    eng.flush(7)
    again = eng.put([8], [toks], logit_positions=[[3, 74]])
    assert _close(again, want[[3, 74]], dt)[0]


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("name,cuts", [("odd", [1] * 60), ("odd", [2, 2, 15, 1, 17, 3, 2, 18]), ("aligned", [16, 16, 1, 1, 6, 2, 30]), ("aligned", [31, 2, 7, 32]),
                                       ("recurrent", [3, 33, 2, 2, 1, 1, 9]), ("attention", [2, 14, 1, 1, 17, 2, 20])])
def test_portions_and_token_by_token_equal_the_whole_prompt(name, cuts, dt, tmp_path_factory):
    """Prefill against decoding token by token, and portions cut inside pages (block 16), down to two tokens."""
    cfg, w, path = _model(name, tmp_path_factory, dt)
    eng = _engine(path, dt)
    toks = _tokens(cfg, sum(cuts), 2)
    want = O.run(cfg, w, toks.tolist())
    rows, at = [], 0
    for n in cuts:
        rows.append(eng.put([3], [toks[at:at + n]], logit_positions=[list(range(n))]))
        at += n
    ok, err = _close(torch.cat(rows), want, dt)
    assert ok, err


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("name", ["odd", "aligned"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(name, dt, tmp_path_factory):
    """Four requests of unequal length share steps (portions beside single tokens), one pauses for a step, they finish at different
    times, and two more take over their state slots and pages: every logit row equals the request run alone."""
    cfg, w, path = _model(name, tmp_path_factory, dt)
    eng = _engine(path, dt, pool_tokens=160, block=16)
    prompts = {u: _tokens(cfg, n, 10 + u) for u, n in ((0, 50), (1, 17), (2, 33), (3, 1), (4, 48), (5, 31))}
    want = {u: O.run(cfg, w, p.tolist()) for u, p in prompts.items()}
    schedule = [[(0, 20), (1, 16), (3, 1)], [(0, 1), (2, 30)], [(0, 1), (1, 1), (2, 1)], [(0, 28), (2, 1)], [(2, 1), (4, 15)], [(4, 33), (5, 2)], [(5, 29)]]
    at, got = {u: 0 for u in prompts}, {u: [] for u in prompts}
    free0 = eng.free_blocks
    for step in schedule:
        uids = [u for u, _ in step]
        out = eng.put(uids, [prompts[u][at[u]:at[u] + n] for u, n in step], logit_positions=[list(range(n)) for _, n in step])
        r = 0
        for u, n in step:
            got[u].append(out[r:r + n])
            r += n
            at[u] += n
            if at[u] == len(prompts[u]):
                eng.flush(u)
    assert eng.free_blocks == free0 and all(at[u] == len(p) for u, p in prompts.items())
    assert eng._state_manager.state_slots.free_slots == 4
    for u in prompts:
        ok, err = _close(torch.cat(got[u]), want[u], dt)
        assert ok, (u, err)


@gpu
@pytest.mark.parametrize("name", ["aligned", "odd"])
def test_long_decoding_through_the_step_graphs(name, tmp_path_factory):
    """A prompt, then 150 single-token steps (the steady-state ones replay a captured graph) across page borders; some steps ask for no
    logits."""
    cfg, w, path = _model(name, tmp_path_factory)
    eng = _engine(path, torch.float32, pool_tokens=256, block=16)
    toks = _tokens(cfg, 200, 5)
    want = O.run(cfg, w, toks.tolist())
    got = [eng.put([1], [toks[:50]], logit_positions=[[49]])]
    keep = [49]
    for i in range(50, 200):
        wanted = i % 7 != 0
        out = eng.put([1], [toks[i:i + 1]], logit_positions=[[0] if wanted else []])
        assert out.shape[0] == int(wanted)
        if wanted:
            got.append(out)
            keep.append(i)
    ok, err = _close(torch.cat(got), want[keep], torch.float32)
    assert ok, err
    graphs = eng.model()._graphs
    assert 1 in graphs and (1, 0) in graphs, list(graphs)


@gpu
def test_greedy_generation_through_the_scheduler(tmp_path_factory):
    from deepspeedsyclsupport_b200.inference.v2.scheduler import SplitFuseScheduler
    cfg, w, path = _model("odd", tmp_path_factory)
    eng = _engine(path, torch.float32, pool_tokens=192, block=16)
    sched = SplitFuseScheduler(eng, token_budget=24)  # prompts are split into portions and fused with running decodes
    prompts = {0: _tokens(cfg, 37, 20), 1: _tokens(cfg, 5, 21), 2: _tokens(cfg, 21, 22)}
    for u, p in prompts.items():
        sched.add_request(u, p, max_new_tokens=6)
    done = sched.run_to_completion()
    for u, p in prompts.items():
        assert done[u] == O.greedy(cfg, w, p.tolist(), 6), u


@gpu
def test_trace_runner_replays_steps(tmp_path_factory):
    """bin/trace_run as a process: portions of three requests beside single tokens, a request that pauses for a step, wanted positions
    anywhere in a portion, requests ending at different steps with their pages and slots reused by a later one (pool of 3 pages)."""
    import json
    import subprocess
    cfg, w, path = _model("odd", tmp_path_factory)
    out_dir = str(tmp_path_factory.mktemp("trace_out"))
    reqs = {"a": _tokens(cfg, 70, 31).tolist(), "b": _tokens(cfg, 9, 32).tolist(), "c": _tokens(cfg, 64, 33).tolist(), "d": _tokens(cfg, 100, 34).tolist()}
    want = {k: O.run(cfg, w, v) for k, v in reqs.items()}
    plan = [[("a", 30, [0, 29]), ("b", 8, [3])], [("a", 2, [1]), ("c", 64, [63])], [("a", 37, [36]), ("b", 1, [0])], [("a", 1, [0]), ("d", 64, [])],
            [("d", 2, [0, 1])], [("d", 1, [])], [("d", 33, [32])]]
    at = {k: 0 for k in reqs}
    lines, expect = [], []
    for n, step in enumerate(plan):
        entries, end, rows = [], [], []
        for k, cnt, wanted in step:
            entries.append({"id": k, "tokens": reqs[k][at[k]:at[k] + cnt], "want": wanted})
            rows += [want[k][at[k] + p] for p in wanted]
            at[k] += cnt
            if at[k] == len(reqs[k]):
                end.append(k)
        lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
        expect.append(torch.stack(rows) if rows else None)
    assert all(at[k] == len(v) for k, v in reqs.items())
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", out_dir, "--max-tokens", "192"],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {n}" for n in range(len(plan))]
    for n, e in enumerate(expect):
        f = os.path.join(out_dir, f"{n}.f32")
        if e is None:
            assert not os.path.exists(f)
            continue
        got = torch.frombuffer(bytearray(open(f, "rb").read()), dtype=torch.float32).view(len(e), cfg["vocab"])
        ok, err = _close(got, e, torch.float32)
        assert ok, (n, err)
