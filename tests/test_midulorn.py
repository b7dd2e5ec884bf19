"""Midulorn on the ragged engine against the plain float64 oracle of tests/midulorn_oracle.py: every mechanism alone (the norm behind the sum,
xIELU and the scalar head gates of csrc/ragged/latent_ops.cu; the minimal gated recurrence of csrc/ragged/recurrent_ops.cu; the two attention
mixers on the CUDA-core kernels of csrc/ragged/sink_attention_ops.cu and on the tcgen05 kernels of csrc/attn/paged_flash.cu), then whole models
of several small random configurations through the engine factory, the paged cache, the state slots, the scheduler and the step graphs."""
import copy
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import midulorn_oracle as O  # noqa: E402

F64 = torch.float64
gpu = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


# ------------------------------------------------------------------------------------------------------------------ CPU: plumbing
def test_spec_reads_every_size_from_the_config():
    from deepspeedsyclsupport_b200.inference.v2.model_implementations.midulorn import MidulornSpec
    cfg = O.make_config([O.latent_layer(3, 6, 4, 5, 10, scale=0.3, base=500.0, mlp=O.dense(20)), O.mingru_layer(7, mlp=O.moe(5, 2, 6)),
                         O.attention_layer(6, 2, 10, 6, conv=4, part=24, scale=0.2), O.attention_layer(6, 2, 10, 6, v_mix=True),
                         O.attention_layer(2, 1, 8, 12, conv=1, part=5, v_mix=True, mlp=O.dense(9)), O.attention_layer(3, 3, 4, 4, v_mix=True)],
                        vocab=61, width=42, eps=3e-5, alpha=1.25, embedding_scale=1.7, logit_scale=0.4)
    s = MidulornSpec.from_config(cfg)
    assert (s.vocab_size, s.hidden_size, s.norm_eps, s.stream_mult, s.embedding_scale, s.logit_scale) == (61, 42, 3e-5, 1.25, 1.7, 0.4)
    a = s.layers[0].latent
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.scale, a.rot_dims, a.rot_base) == (3, 6, 4, 5, 10, 0.3, 4, 500.0)
    assert s.layers[0].mlp.kind == "dense" and s.layers[0].mlp.ff == 20
    assert s.layers[1].unit.width == 7 and (s.layers[1].mlp.experts, s.layers[1].mlp.top, s.layers[1].mlp.ff) == (5, 2, 6)
    b = s.layers[2].attn
    assert (b.heads, b.kv_heads, b.dim, b.vdim, b.conv, b.part, b.scale, b.value_mix) == (6, 2, 10, 6, 4, 24, 0.2, "none") and s.layers[2].mlp is None
    # the first layer that mixes values hands its own on, the later ones mix with them
    assert [L.attn.value_mix for L in s.layers[3:]] == ["source", "mix", "mix"]
    bad = copy.deepcopy(cfg)
    bad["layers"][5]["mixer"]["vdim"] = 5
    with pytest.raises(ValueError):
        MidulornSpec.from_config(bad)
    bad = copy.deepcopy(cfg)
    bad["layers"][1]["type"] = "gru"
    with pytest.raises(ValueError):
        MidulornSpec.from_config(bad)


def test_family_is_registered_and_its_modules_are_chosen_by_their_configs():
    from deepspeedsyclsupport_b200.inference.v2.engine_factory import model_type_of
    from deepspeedsyclsupport_b200.inference.v2.inference_utils import ActivationType, NormTypeEnum
    from deepspeedsyclsupport_b200.inference.v2.model_implementations import FAMILIES, policy_for
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import (DSConvSinkAttentionConfig, DSMinGRUConfig, DSMoEConfig, DSNormConfig,
                                                                        DSRotaryLatentAttentionConfig)
    assert "midulorn" in FAMILIES and model_type_of({"architecture": "Midulorn"}) == "midulorn"
    assert policy_for("midulorn").__name__ == "MidulornPolicy"
    norm = heuristics.instantiate_post_norm(DSNormConfig(max_tokens=64, type=NormTypeEnum.RMSNorm, channels=8, residual_dtype="fp32", input_dtype="bf16", output_dtype="bf16",
                                                         post_sum=True, stream_mult=2.0))
    assert norm.name() == "cuda_post_sum_rms"
    assert heuristics.instantiate_recurrent(DSMinGRUConfig(max_tokens=64, width=5, max_sequences=2)).name() == "min_gru"
    a = heuristics.instantiate_attention(DSRotaryLatentAttentionConfig(max_tokens=64, n_heads=3, qk_dim=6, rot_dim=4, v_dim=5, kv_rank=10, scale=0.3, rotate_dim=4,
                                                                       learned_sink=True, head_gate=True, max_sequences=2))
    assert a.name() == "rotary_latent_attention"
    b = heuristics.instantiate_attention(DSConvSinkAttentionConfig(max_tokens=64, n_heads_q=4, n_heads_kv=2, head_size=8, value_size=6, conv_taps=3, scale=0.3, part_size=16,
                                                                   distance_bias=True, learned_sink=True, max_sequences=2))
    assert b.name() == "conv_sink_attention"
    moe = heuristics.instantiate_moe(DSMoEConfig(max_tokens=64, model_dim=16, intermediate_features=8, n_experts=4, top_k=2, input_dtype="bf16", output_dtype="bf16",
                                                 activation=ActivationType.SiGLU, fp32_combine=True))
    assert moe.name() == "grouped_topk_moe"
    with pytest.raises(ValueError):
        DSRotaryLatentAttentionConfig(max_tokens=64, n_heads=3, qk_dim=6, rot_dim=4, v_dim=5, kv_rank=10, scale=0.3, rotate_dim=6, max_sequences=2)
    with pytest.raises(ValueError):
        DSConvSinkAttentionConfig(max_tokens=64, n_heads_q=3, n_heads_kv=2, head_size=8, value_size=6, conv_taps=3, scale=0.3, max_sequences=2)


def test_cache_rows_and_state_of_the_mixers():
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSConvSinkAttentionConfig, DSMinGRUConfig, DSRotaryLatentAttentionConfig

    def latent(dt, rank, rot, heads=3):
        return heuristics.instantiate_attention(DSRotaryLatentAttentionConfig(max_tokens=64, n_heads=heads, qk_dim=6, rot_dim=rot, v_dim=5, kv_rank=rank, scale=0.3, rotate_dim=rot,
                                                                              max_sequences=2, input_dtype=dt, output_dtype=dt))

    # fp32: the row is latent + rotated key part; bf16: padded to what the tensor-core kernels take, or left alone when it is too wide
    assert latent("fp32", 10, 4).cache_shapes() == [(1, 1, 14)] and latent("fp32", 10, 4).attended_width == 10
    assert latent("bf16", 10, 4).cache_shapes() == [(1, 1, 64)] and latent("bf16", 60, 8).cache_shapes() == [(1, 1, 128)]
    assert latent("bf16", 200, 8).cache_shapes() == [(1, 1, 208)]
    m = latent("bf16", 10, 4)
    up = m.transform_key_up_param(torch.arange(3 * 6 * 10, dtype=torch.float32).view(18, 10) / 100)
    assert up.shape == (3, 10, 64) and float(up[1, 6:, 10:14].float().trace()) == 4.0 and float(up[:, :6, 10:].abs().sum()) == 0 and float(up[:, 6:, :10].abs().sum()) == 0
    assert m.transform_value_up_param(torch.ones(15, 10)).shape == (3, 64, 5) and m.transform_sink_param(torch.ones(3)).shape == (4, )

    def conv(dt, d, dv, taps=3, G=2):
        return heuristics.instantiate_attention(DSConvSinkAttentionConfig(max_tokens=64, n_heads_q=4, n_heads_kv=G, head_size=d, value_size=dv, conv_taps=taps, scale=0.3,
                                                                          max_sequences=2, input_dtype=dt, output_dtype=dt))

    assert conv("fp32", 10, 6).cache_shapes() == [(1, 2, 10), (1, 2, 6)] and conv("fp32", 8, 8).cache_shapes() == [(2, 2, 8)]
    assert conv("bf16", 10, 6).cache_shapes() == [(2, 2, 64)] and conv("bf16", 72, 40).out_width == 4 * 128 and conv("bf16", 160, 8).cache_shapes() == [(1, 2, 160), (1, 2, 8)]
    s = conv("fp32", 10, 6).state_specs("l3.mix")
    assert [(x.name, tuple(x.shape), x.dtype) for x in s] == [("l3.mix.conv", (2, 4 * 10 + 2 * 10 + 2 * 6), torch.float32)] and conv("fp32", 10, 6, taps=1).state_specs("p") == []
    g = heuristics.instantiate_recurrent(DSMinGRUConfig(max_tokens=64, width=5, max_sequences=2)).state_specs("l1.mix")
    assert [(x.name, tuple(x.shape), x.dtype) for x in g] == [("l1.mix.S", (5, ), torch.float32)]


# ------------------------------------------------------------------------------------------------------------ GPU: mechanisms alone
def _K():
    from deepspeedsyclsupport_b200.inference.v2 import kernels
    return kernels


class _Batch:
    """Ragged metadata of a step, built by hand: seqs = [(slot, seen, new tokens, block ids)]."""

    def __init__(self, seqs, block, max_blocks=40):
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


def _tol(dt):
    return 2e-5 if dt == torch.float32 else 2.5e-2


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("dim", [6, 40, 42, 384, 1024, 4104])
def test_norm_behind_the_sum(dim, dt):
    """x <- rms(alpha x + branch + fp32 branch + bias) * w, and its copy in the activation dtype; one row 50x larger than the others."""
    K = _K()
    g = torch.Generator().manual_seed(dim)
    x = torch.randn(9, dim, generator=g)
    x[4] *= 50
    y, y32, bias, w = torch.randn(9, dim, generator=g).to(dt), torch.randn(9, dim, generator=g), torch.randn(dim, generator=g), 1 + 0.3 * torch.randn(dim, generator=g)
    for use_y, use_32, use_b in ((1, 0, 0), (0, 1, 0), (1, 1, 1), (0, 0, 0)):
        want = O.join(x.double(), (y.double() if use_y else 0) + (y32.double() if use_32 else 0) + (bias.double() if use_b else 0), w, 1.75, 1e-5)
        xs = x.cuda().clone()
        h = K.post_sum_norm(xs, y.cuda() if use_y else None, w.cuda(), alpha=1.75, eps=1e-5, y32=y32.cuda() if use_32 else None, bias=bias.cuda() if use_b else None,
                            out_dtype=dt)
        assert torch.allclose(xs.cpu().double(), want, rtol=1e-5, atol=1e-5)
        assert h.dtype == dt and torch.allclose(h.cpu().double(), want, rtol=1e-5 if dt == torch.float32 else 1e-2, atol=1e-5 if dt == torch.float32 else 1e-2)


@gpu
@pytest.mark.parametrize("dt", DTYPES)
def test_xielu_and_scalar_head_gates(dt):
    K = _K()
    g = torch.Generator().manual_seed(3)
    for rows, F in ((7, 13), (5, 64)):
        wide = (3 * torch.randn(rows, F + 3, generator=g)).to(dt)
        for p, q in ((0.4, -0.3), (-2.0, 1.5)):
            want = O.xielu(wide[:, :F].double(), p, q)
            for u in (wide.cuda()[:, :F], wide[:, :F].contiguous().cuda()):  # a column range of a wider tensor, and rows that lie back to back
                got = K.xielu(u, K.xielu_coefficients(p, q).cuda())
                assert torch.allclose(got.cpu().double(), want, rtol=1e-5 if dt == torch.float32 else 1e-2, atol=1e-5 if dt == torch.float32 else 1e-2)
    a, gate = torch.randn(3, 6, 5, generator=g).to(dt), torch.randn(6, 4, generator=g).to(dt)
    out = torch.zeros(6, 16, dtype=dt, device="cuda")
    K.gate_heads_scalar(a.cuda(), gate.cuda()[:, :3], out[:, :15])
    want = (a.double() * torch.sigmoid(gate[:, :3].double()).T.unsqueeze(-1)).transpose(0, 1).reshape(6, 15)
    assert torch.allclose(out[:, :15].cpu().double(), want, rtol=1e-5 if dt == torch.float32 else 1e-2, atol=1e-5 if dt == torch.float32 else 1e-2)
    assert float(out[:, 15].abs().max()) == 0


# ---- minimal gated recurrence
def _unit(width, dt):
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSMinGRUConfig
    name = {torch.float32: "fp32", torch.bfloat16: "bf16"}[dt]
    return heuristics.instantiate_recurrent(DSMinGRUConfig(max_tokens=64, width=width, max_sequences=4, input_dtype=name, output_dtype=name))


def _unit_weights(width, D, seed, slow=False):
    g = torch.Generator().manual_seed(seed)
    P = {"mix.z": (torch.randn(width, D, generator=g) * 2 * D**-0.5).bfloat16(), "mix.x": (torch.randn(width, D, generator=g) * 2 * D**-0.5).bfloat16(),
         "mix.g": (torch.randn(width, D, generator=g) * 2 * D**-0.5).bfloat16(), "mix.z.b": (torch.randn(width, generator=g) * 2 - 1).bfloat16(),
         "mix.x.b": (0.3 * torch.randn(width, generator=g)).bfloat16(), "mix.o": torch.eye(width).bfloat16()}
    if slow:  # half of the channels forget slowly (z around 0.003): what the first tokens wrote is still there after hundreds of steps
        P["mix.z.b"][::2] = -6.0
    return P


def _run_unit(mod, P, h, cuts, dt, state, slot, pieces=None):
    W = P["mix.z"].shape[0]
    w_in = torch.cat([P["mix.z"], P["mix.x"], P["mix.g"]]).to(dt).cuda()
    zb, xb = P["mix.z.b"].float().cuda(), P["mix.x.b"].float().cuda()
    rows = []
    for at, n in cuts:
        proj = (h[at:at + n].to(dt).cuda() @ w_in.T).contiguous()
        out = torch.empty(n, W, dtype=dt, device="cuda")
        mod(proj, (0, W, 2 * W), zb, xb, _Batch([(slot, at, n, [])], 16), state, "u", out, pieces=pieces)
        rows.append(out)
    return torch.cat(rows)


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("width", [5, 130, 328])
@pytest.mark.parametrize("sizes,pieces", [([90], None), ([90], False), ([90], True), ([1] * 60, None), ([2, 5, 1, 33, 2, 9], True), ([2, 5, 1, 70, 2, 9], None)])
def test_minimal_gated_recurrence(width, sizes, pieces, dt):
    """Whole, token by token and in portions down to two tokens, as one walk and cut into pieces, in a slot that held garbage."""
    D = 24
    P = _unit_weights(width, D, width)
    h = torch.randn(90, D, generator=torch.Generator().manual_seed(7)).to(dt).double()
    want = O.mingru(h, P, {"width": width})
    mod = _unit(width, dt)
    state = _State(mod.state_specs("u"), 3)
    got = _run_unit(mod, P, h, _cuts(90, sizes), dt, state, 2, pieces)
    assert _rel(got, want) < _tol(dt)
    assert float((state.get_state("u.S")[0] - 7.5).abs().max()) == 0  # other slots are left alone


@gpu
def test_slow_channels_remember_the_first_tokens_through_long_decoding():
    """400 single-token steps after a short prompt: channels that forget slowly still hold what the first tokens wrote (fp32 state), and the
    read-out differs from a run whose first tokens were different."""
    width, D, T = 16, 12, 420
    P = _unit_weights(width, D, 5, slow=True)
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(8)).double()
    want = O.mingru(h, P, {"width": width})
    other = h.clone()
    other[:3] = 4 * torch.randn(3, D, generator=torch.Generator().manual_seed(9)).double()
    assert float((O.mingru(other, P, {"width": width})[-1] - want[-1]).abs().max()) > 1e-2  # the first tokens still show at the end
    mod = _unit(width, torch.float32)
    state = _State(mod.state_specs("u"), 1)
    got = _run_unit(mod, P, h, _cuts(T, [20] + [1] * 400), torch.float32, state, 0)
    assert torch.allclose(got.cpu().double(), want, rtol=1e-4, atol=1e-5)


@gpu
@pytest.mark.parametrize("pieces", [False, True])
def test_sequences_of_a_batch_keep_their_own_state(pieces):
    """Three sequences side by side in every step (a portion, a single token, a new one whose slot another sequence used before): pieces of
    the walk hold the end of one sequence and the start of the next."""
    K = _K()
    width, D = 40, 16
    P = _unit_weights(width, D, 11)
    hs = [torch.randn(n, D, generator=torch.Generator().manual_seed(20 + i)).double() for i, n in enumerate((75, 9, 50, 41))]
    want = [O.mingru(h, P, {"width": width}) for h in hs]
    mod = _unit(width, torch.float32)
    state = _State(mod.state_specs("u"), 3)
    w_in = torch.cat([P["mix.z"], P["mix.x"], P["mix.g"]]).float().cuda()
    zb, xb = P["mix.z.b"].float().cuda(), P["mix.x.b"].float().cuda()
    # (sequence, slot, first, count) per step; sequence 3 takes over slot 1 after sequence 1 has ended
    steps = [[(0, 0, 0, 40), (1, 1, 0, 8), (2, 2, 0, 3)], [(0, 0, 40, 1), (1, 1, 8, 1), (2, 2, 3, 45)], [(0, 0, 41, 34), (3, 1, 0, 41), (2, 2, 48, 2)]]
    got = {i: [] for i in range(4)}
    for step in steps:
        proj = (torch.cat([hs[s][a:a + n] for s, _, a, n in step]).float().cuda() @ w_in.T).contiguous()
        out = torch.empty(proj.shape[0], width, device="cuda")
        b = _Batch([(slot, a, n, []) for _, slot, a, n in step], 16)
        K.mingru_scan(proj, 0, width, 2 * width, zb, xb, b.tok_seq(), b.seq_desc(), len(step), state.get_state("u.S"), out, width, pieces=pieces)
        at = 0
        for s, _, _, n in step:
            got[s].append(out[at:at + n])
            at += n
    for i in range(4):
        assert torch.allclose(torch.cat(got[i]).cpu().double(), want[i], rtol=1e-4, atol=1e-5), i


# ---- attention with a cached latent and a shared rotated key part
def _latent_module(m, dt, eps=1e-5):
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSRotaryLatentAttentionConfig
    name = {torch.float32: "fp32", torch.bfloat16: "bf16"}[dt]
    return heuristics.instantiate_attention(DSRotaryLatentAttentionConfig(max_tokens=64, 
        n_heads=m["heads"], qk_dim=m["dim"], rot_dim=m["rot_dim"], v_dim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"], rotate_dim=m["rot"]["dims"],
        theta_base=m["rot"]["base"], learned_sink=True, head_gate=True, eps=eps, max_sequences=4, input_dtype=name, output_dtype=name))


def _mixer_weights(layer, D, seed):
    cfg = O.make_config([layer], width=D)
    return O.layer_params(O.random_weights(cfg, seed), 0)


def _run_latent(mod, P, m, h, cuts, dt, blocks, block=16):
    w_in = torch.cat([P["mix.q"], P["mix.dkv"], P["mix.g"]]).to(dt).cuda()
    nq, nkv = m["heads"] * (m["dim"] + m["rot_dim"]), m["kv_rank"] + m["rot_dim"]
    args = (P["mix.dkv.norm"].float().cuda(), mod.transform_key_up_param(P["mix.uk"]).cuda(), mod.transform_value_up_param(P["mix.uv"]).cuda(),
            mod.transform_sink_param(P["mix.sink"]).cuda())
    cache = torch.full((max(blocks) + 1, block, 1, mod.cache_row), 3.0, dtype=dt, device="cuda")  # pages that held something else before
    rows = []
    for at, n in cuts:
        proj = (h[at:at + n].to(dt).cuda() @ w_in.T).contiguous()
        o = mod(proj, (0, nq, nq + nkv), cache, _Batch([(0, at, n, blocks)], block), *args)
        rows.append((o @ P["mix.o"].to(dt).cuda().T).clone())
    return torch.cat(rows)


LATENT_CASES = [
    O.latent_layer(3, 6, 4, 5, 10, scale=0.4, base=300.0)["mixer"],              # odd sizes
    O.latent_layer(2, 8, 8, 8, 24, scale=0.3, rot_dims=4, base=50.0)["mixer"],     # only some of the rotated part's entries are rotated
    O.latent_layer(4, 16, 16, 24, 40, scale=0.25)["mixer"],                       # bf16: row padded to 64, on the tensor cores
    O.latent_layer(5, 32, 32, 16, 96, scale=0.15, base=5e5)["mixer"],             # bf16: a full row of 128, heads padded to 8
    O.latent_layer(2, 24, 16, 32, 160, scale=0.2)["mixer"],                       # too wide for the tensor-core kernels: CUDA cores in bf16 too
]


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("case", range(len(LATENT_CASES)))
@pytest.mark.parametrize("sizes", [[70], [40] + [1] * 30, [2, 5, 1, 25, 2, 9, 14]])
def test_latent_attention_mixer(case, sizes, dt):
    """Whole, prompt + single tokens, portions cut inside pages; shuffled pages that held garbage."""
    m, D = LATENT_CASES[case], 48
    P = _mixer_weights({"type": "latent_attention", "mixer": m, "mlp": None}, D, 30 + case)
    h = torch.randn(70, D, generator=torch.Generator().manual_seed(case)).to(dt).double()
    want = O.latent_attention(h, P, m, 1e-5)
    got = _run_latent(_latent_module(m, dt), P, m, h, _cuts(70, sizes), dt, [5, 2, 7, 0, 3])
    assert _rel(got, want) < _tol(dt), _rel(got, want)


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("case", [0, 3])
@pytest.mark.parametrize("far", [0, 15, 16, 127, 128, 300])
def test_a_far_key_shows_in_latent_attention(far, case, dt):
    """ONE token among hundreds gets a rotated key part 40 times larger (that part is not normed): the queries behind it find it or shun it,
    whatever page row it lies in -- the outputs with and without it differ by order 1, and the engine's follow the oracle's; in the prompt
    and for single decoded tokens (CUDA-core kernel in fp32, both tcgen05 kernels in bf16)."""
    m, D, T = LATENT_CASES[case], 32, 420
    P = _mixer_weights({"type": "latent_attention", "mixer": m, "mlp": None}, D, 40 + case)
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(far)).to(dt).double()
    plain = O.latent_attention(h, P, m, 1e-5)
    h[far] *= 40
    want = O.latent_attention(h, P, m, 1e-5)
    assert float((want[far + 1:] - plain[far + 1:]).norm() / plain[far + 1:].norm()) > 0.1
    got = _run_latent(_latent_module(m, dt), P, m, h, _cuts(T, [400] + [1] * 20), dt, list(range(27, 0, -1)))
    assert _rel(got[:far], want[:far]) < _tol(dt) if far else True
    assert _rel(got, want) < _tol(dt), _rel(got, want)


# ---- attention behind a short convolution
def _conv_module(m, dt, value_mix="none", eps=1e-5):
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSConvSinkAttentionConfig
    name = {torch.float32: "fp32", torch.bfloat16: "bf16"}[dt]
    return heuristics.instantiate_attention(DSConvSinkAttentionConfig(max_tokens=64, 
        n_heads_q=m["heads"], n_heads_kv=m["kv_heads"], head_size=m["dim"], value_size=m["vdim"], conv_taps=m["conv"], scale=m["scale"],
        part_size=m["mask"]["size"], distance_bias=True, learned_sink=True, value_mix=value_mix, eps=eps, max_sequences=4, input_dtype=name, output_dtype=name))


def _conv_caches(mod, blocks, block, dt):
    return [torch.full((blocks, ) + ((2, ) if p == 2 else ()) + (block, g, w), 3.0, dtype=dt, device="cuda") for p, g, w in mod.cache_shapes()]


def _conv_args(P, dt):
    f = lambda t: t.float().reshape(-1 if t.dim() == 0 else t.shape).cuda()  # noqa: E731
    return dict(w_in=torch.cat([P["mix.q"], P["mix.k"], P["mix.v"]]).to(dt).cuda(), bias=f(torch.cat([P["mix.q.b"], P["mix.k.b"], P["mix.v.b"]])),
                conv=f(torch.cat([P["mix.q.conv"], P["mix.k.conv"], P["mix.v.conv"]]).t().contiguous()), nq=f(P["mix.q.norm"]), nk=f(P["mix.k.norm"]), r1=f(P["mix.r1"]),
                r2=f(P["mix.r2"]), sink=f(P["mix.sink"]), mix=f(P["mix.vmix"]))


def _run_conv(mod, P, m, h, cuts, dt, blocks, block=16, state=None, v_source=None, slot=1):
    """-> (mixer output before its bias, the layer's own values when it is a source)."""
    A = _conv_args(P, dt)
    caches = _conv_caches(mod, max(blocks) + 1, block, dt)
    state = state or _State(mod.state_specs("a"), 3)
    o_w = P["mix.o"].to(dt).cuda()
    if mod.out_head_width != m["vdim"]:
        o_w = torch.nn.functional.pad(o_w.view(-1, m["heads"], m["vdim"]), (0, mod.out_head_width - m["vdim"])).reshape(o_w.shape[0], -1)
    rows, own = [], []
    for at, n in cuts:
        proj = (h[at:at + n].to(dt).cuda() @ A["w_in"].T).contiguous()
        out = torch.empty(n, mod.out_width, dtype=dt, device="cuda")
        _, v = mod(proj, 0, A["bias"], A["conv"], A["nq"], A["nk"], A["r1"], A["r2"], A["sink"], caches[0], caches[1] if len(caches) > 1 else None,
                   _Batch([(slot, at, n, blocks)], block), state, "a", out, v_source=None if v_source is None else v_source[at:at + n].contiguous(), mix=A["mix"])
        rows.append(out @ o_w.T)
        own.append(v)
    return torch.cat(rows), (torch.cat(own) if own[0] is not None else None)


CONV_CASES = [
    O.attention_layer(6, 2, 10, 6, conv=3, part=16, scale=0.5)["mixer"],      # odd sizes, grouped heads, unequal key and value heads
    O.attention_layer(4, 4, 8, 8, conv=1, part=1000, scale=0.6)["mixer"],     # one tap (no state), one part for the whole sequence
    O.attention_layer(2, 1, 64, 64, conv=4, part=24, scale=0.2)["mixer"],     # bf16: head size 64 on the tensor cores; parts that cut pages
    O.attention_layer(4, 2, 128, 128, conv=2, part=50, scale=0.12)["mixer"],  # bf16: head size 128, also the small-atom kernel
    O.attention_layer(4, 1, 72, 40, conv=3, part=32, scale=0.15)["mixer"],    # bf16: heads padded to 128
    O.attention_layer(2, 2, 6, 12, conv=5, part=7, scale=0.7)["mixer"],       # more taps than some portions have tokens, short parts
]


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("case", range(len(CONV_CASES)))
@pytest.mark.parametrize("sizes", [[70], [40] + [1] * 30, [2, 5, 1, 25, 2, 9, 1, 1, 14]])
def test_convolved_attention_mixer(case, sizes, dt):
    """Whole, prompt + single tokens, portions cut inside pages, parts and the convolution's reach; shuffled pages that held garbage."""
    m, D = CONV_CASES[case], 48
    P = _mixer_weights({"type": "attention", "mixer": m, "mlp": None}, D, 50 + case)
    h = torch.randn(70, D, generator=torch.Generator().manual_seed(case)).to(dt).double()
    want = O.conv_attention(h, P, m, 1e-5)[0] - P["mix.o.b"].double()
    got, _ = _run_conv(_conv_module(m, dt), P, m, h, _cuts(70, sizes), dt, [5, 2, 7, 0, 3])
    assert _rel(got, want) < _tol(dt), _rel(got, want)


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("sizes", [[60], [2, 30, 1, 1, 26]])
def test_values_are_mixed_with_the_first_mixing_layers(sizes, dt):
    """The source layer hands on its convolved values; the mixing layer caches (1 - m) v + m v_source, also for tokens decoded later."""
    m, D = CONV_CASES[0], 40
    P0 = _mixer_weights({"type": "attention", "mixer": m, "mlp": None}, D, 61)
    P1 = _mixer_weights({"type": "attention", "mixer": m, "mlp": None}, D, 62)
    h = torch.randn(60, D, generator=torch.Generator().manual_seed(1)).to(dt).double()
    want0, v0 = O.conv_attention(h, P0, m, 1e-5)
    want1, _ = O.conv_attention(h, P1, m, 1e-5, v_first=v0)
    plain1, _ = O.conv_attention(h, P1, m, 1e-5)
    assert _rel(plain1, want1) > 0.05  # the mixing shows
    got0, own = _run_conv(_conv_module(m, dt, "source"), P0, m, h, _cuts(60, sizes), dt, [4, 1, 6, 2])
    assert _rel(own, v0) < _tol(dt) and _rel(got0, want0 - P0["mix.o.b"].double()) < _tol(dt)
    got1, none = _run_conv(_conv_module(m, dt, "mix"), P1, m, h, _cuts(60, sizes), dt, [3, 0, 5, 2], v_source=own)
    assert none is None and _rel(got1, want1 - P1["mix.o.b"].double()) < _tol(dt)


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("case,T", [(0, 200), (2, 200), (3, 420), (4, 300)])
@pytest.mark.parametrize("where", ["first of a part", "last of a part", "middle", "page border"])
def test_a_huge_value_shows_exactly_inside_its_part(where, case, T, dt):
    """ONE token's input is made 200 times larger, so its value dwarfs all others (values are not normed): every query of the same part behind
    it feels it, the last query of the part before and the first query of the next part do not -- in the prompt and for single decoded tokens,
    with parts that cut pages (CUDA-core kernel in fp32, both tcgen05 kernels in bf16)."""
    m, D = CONV_CASES[case], 32
    part, taps = m["mask"]["size"], m["conv"]
    base = (T - 60) // part * part  # a part in the region that is decoded token by token below, or just before it
    far = {"first of a part": base, "last of a part": base + part - 1, "middle": base + part // 2, "page border": (base // 16 + 1) * 16}[where]
    P = _mixer_weights({"type": "attention", "mixer": m, "mlp": None}, D, 70 + case)
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(far)).to(dt).double()
    plain = O.conv_attention(h, P, m, 1e-5)[0]
    h[far] *= 200
    want = O.conv_attention(h, P, m, 1e-5)[0]
    end = (far // part + 1) * part  # first position of the next part
    felt = (want - plain).norm(dim=-1) / plain.norm(dim=-1).mean()
    assert float(felt[far:min(end, T)].min()) > 0.02  # every query of the part from `far` on
    assert float(felt[:far].max()) < 1e-9
    if far + taps - 1 < end and end < T:  # (the convolution carries the token into the next taps - 1 positions: they must lie in the same part)
        assert float(felt[end:].max()) < 1e-9
    want = want - P["mix.o.b"].double()
    got, _ = _run_conv(_conv_module(m, dt), P, m, h, _cuts(T, [T - 45] + [1] * 45), dt, list(range(27, 0, -1)))
    err = (got.cpu().double() - want).norm(dim=-1) / want.norm(dim=-1)
    assert float(err.max()) < (1e-4 if dt == torch.float32 else 6e-2), (float(err.max()), int(err.argmax()))


@gpu
def test_both_attention_kernels_agree_on_a_mixed_batch():
    """A portion beside single tokens of other sequences in ONE step, bf16: the tcgen05 kernels (prompt and small-atom form, with and without
    key splits) against the CUDA-core kernel on the same cache."""
    K = _K()
    H, G, d, block = 4, 2, 128, 16
    g = torch.Generator().manual_seed(4)
    cache = (0.5 * torch.randn(40, 2, block, G, d, generator=g)).bfloat16().cuda()
    seqs = [(0, 300, 70, list(range(0, 24))), (1, 210, 1, list(range(24, 38))), (2, 0, 3, [38]), (3, 31, 1, [39, 5])]
    r1, r2, sink = (0.5 + torch.rand(H, generator=g)).cuda(), (0.1 + torch.rand(H, generator=g)).cuda(), torch.randn(H, generator=g).cuda()
    kp, vp = K.cache_planes(cache)
    for part in (0, 48, 200):
        for decode in (False, True):
            ss = seqs if not decode else [(s, seen + n - 1, 1, b) for s, seen, n, b in seqs]
            b = _Batch(ss, block)
            q = (0.3 * torch.randn(b.current_tokens, H * d, generator=g)).bfloat16().cuda()
            ref = torch.empty_like(q)
            K.sink_attention_ex(q, d, kp, d, vp, d, b.tok_seq(), b.tok_pos(), b.block_table(), block, ref, d, H, G, d, d, 0.09, sink_logit=sink, r1=r1, r2=r2, part=part)
            for splits in (1, 3):
                out = torch.empty_like(q)
                K.paged_flash_sink(q, cache, b.tok_seq(), b.tok_pos(), b.block_table(), out, H, G, d, 0.09, 0.0, 0.0, decode=decode, n_splits=splits,
                                   sink_logit=sink, r1=r1, r2=r2, part=part)
                assert _rel(out.float(), ref.double().cpu()) < 1.5e-2, (part, decode, splits)


# ---- router
@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("experts,top,ff,D", [(5, 2, 12, 24), (4, 1, 8, 40), (3, 3, 16, 64), (8, 2, 32, 128)])
def test_softmax_router_without_renormalisation(experts, top, ff, D, dt):
    from deepspeedsyclsupport_b200.inference.v2.inference_utils import ActivationType
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSMoEConfig
    name = {torch.float32: "fp32", torch.bfloat16: "bf16"}[dt]
    f = O.moe(experts, top, ff)
    P = O.layer_params(O.random_weights(O.make_config([O.mingru_layer(4, mlp=f)], width=D), 3, router_gain=6.0), 0)
    mod = heuristics.instantiate_moe(DSMoEConfig(max_tokens=64, model_dim=D, intermediate_features=ff, n_experts=experts, top_k=top, activation=ActivationType.SiGLU,
                                                 normalize_scores=False, fp32_combine=True, input_dtype=name, output_dtype=name))
    h = torch.randn(33, D, generator=torch.Generator().manual_seed(experts)).to(dt)
    want = O.moe_ff(h.double(), P, f)
    gu = torch.stack([torch.cat([P[f"mlp.e{e}.gate"], P[f"mlp.e{e}.up"]]) for e in range(experts)]).to(dt).cuda()
    dn = torch.stack([P[f"mlp.e{e}.down"] for e in range(experts)]).to(dt).cuda()
    got = mod(h.cuda(), P["mlp.router"].float().cuda(), gu, dn, router_input=h.float().cuda())
    assert got.dtype == torch.float32 and _rel(got, want) < _tol(dt)
    idx, wts = O.route(h.double(), P, top)
    assert float(wts.sum(-1).max()) < 1.0 or top == experts  # the weights are the plain scores: they do not sum to one


# ------------------------------------------------------------------------------------------------------------ GPU: whole models
CONFIGS = {
    # odd sizes that differ per layer; every mixer and every kind of feed-forward, also none; grouped and single key / value heads; one tap; a
    # source of values and two layers that mix with it; top 1
    "odd": O.make_config([
        O.latent_layer(3, 6, 4, 5, 10, scale=0.4, base=300.0, mlp=O.dense(20)),
        O.mingru_layer(7, mlp=O.moe(5, 2, 6)),
        O.attention_layer(6, 2, 10, 6, conv=3, part=16, scale=0.5, v_mix=True),
        O.mingru_layer(50),
        O.attention_layer(3, 1, 8, 12, conv=1, part=5, v_mix=True, mlp=O.moe(3, 1, 9)),
        O.attention_layer(2, 2, 14, 6, conv=4, part=40, v_mix=True, mlp=O.dense(30)),
        O.latent_layer(2, 8, 8, 8, 24, scale=0.3, rot_dims=4, base=50.0, mlp=O.moe(4, 2, 6)),
    ], vocab=61, width=42, eps=1e-5, alpha=1.5, embedding_scale=1.7, logit_scale=0.6),
    # aligned sizes (tensor-core GEMMs and attention in bf16, 16-byte norm path), head sizes 64 and 128, latent rows of 64 and 128
    "aligned": O.make_config([
        O.attention_layer(4, 2, 64, 64, conv=3, part=24, scale=0.2, mlp=O.moe(8, 2, 32)),
        O.latent_layer(4, 16, 16, 32, 40, scale=0.25, mlp=O.dense(256)),
        O.mingru_layer(384, mlp=O.moe(8, 2, 32)),
        O.attention_layer(2, 1, 128, 128, conv=2, part=48, scale=0.12, v_mix=True, mlp=O.dense(128)),
        O.latent_layer(8, 32, 32, 32, 96, scale=0.15, base=5e5),
        O.attention_layer(4, 1, 72, 128, conv=3, part=32, scale=0.15, v_mix=True, mlp=O.dense(64)),
    ], vocab=96, width=256, eps=1e-6, alpha=2.0, embedding_scale=3.0, logit_scale=0.4),
    # no attention layer at all: nothing is cached per token, everything lives in the state slots
    "recurrent": O.make_config([O.mingru_layer(24, mlp=O.dense(16)), O.mingru_layer(9, mlp=O.moe(2, 1, 8))], vocab=40, width=24, alpha=1.0, logit_scale=1.0),
    # no recurrent layer and one tap everywhere: no state slots
    "attention": O.make_config([O.attention_layer(2, 1, 8, 12, conv=1, part=9, mlp=O.dense(16)), O.latent_layer(4, 6, 6, 6, 12, mlp=O.moe(3, 2, 8))],
                               vocab=40, width=24, alpha=3.0, embedding_scale=1.0),
}
_MODELS = {}


def _model(name, tmp_path_factory, dt=torch.float32):
    """fp32 runs keep the configured top-k (every selection is compared tightly).  bf16 runs let every token use ALL experts of a layer,
    weighted by their scores: a top-k choice between two close scores flips under rounding and the flipped token then colours the rest of its
    sequence through the recurrent state, which says nothing about the engine (the selection itself is checked on equal inputs in
    test_softmax_router_without_renormalisation); their routers are also kept soft, since a sharp softmax over the experts turns a 1 % change
    of the stream into a much larger change of the weights, layer after layer."""
    every = dt == torch.bfloat16
    if (name, every) not in _MODELS:
        cfg = copy.deepcopy(CONFIGS[name])
        if every:
            for L in cfg["layers"]:
                if L["mlp"] is not None and L["mlp"]["kind"] == "moe":
                    L["mlp"]["router"]["top"] = L["mlp"]["router"]["experts"]
        w = O.random_weights(cfg, seed=len(name), router_gain=1.0 if every else 4.0)
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
    eng.model()._layer_hook = None
    eng.flush(7)
    again = eng.put([8], [toks], logit_positions=[[3, 74]])
    assert _close(again, want[[3, 74]], dt)[0]


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("name,cuts", [("odd", [1] * 60), ("odd", [2, 2, 15, 1, 17, 3, 2, 18]), ("aligned", [16, 16, 1, 1, 6, 2, 30]), ("aligned", [31, 2, 7, 32]),
                                       ("recurrent", [3, 33, 2, 2, 1, 1, 9]), ("attention", [2, 14, 1, 1, 17, 2, 20])])
def test_portions_and_token_by_token_equal_the_whole_prompt(name, cuts, dt, tmp_path_factory):
    """Prefill against decoding token by token, and portions cut inside pages (block 16), parts and convolutions, down to two tokens."""
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
    """A prompt, then 150 single-token steps (the steady-state ones replay a captured graph) across page borders and from part to part; some
    steps ask for no logits."""
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
def test_long_decoding_in_bf16_on_the_tensor_core_kernels(tmp_path_factory):
    cfg, w, path = _model("aligned", tmp_path_factory, torch.bfloat16)
    eng = _engine(path, torch.bfloat16, pool_tokens=256, block=16)
    toks = _tokens(cfg, 150, 6)
    want = O.run(cfg, w, toks.tolist())
    got = [eng.put([1], [toks[:40]], logit_positions=[list(range(40))])] + [eng.put([1], [toks[i:i + 1]], logit_positions=[[0]]) for i in range(40, 150)]
    ok, err = _close(torch.cat(got), want, torch.bfloat16)
    assert ok, err


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
