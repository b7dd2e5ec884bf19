"""Plain float64 restatement of the Pudinex family, one function per mechanism, token by token where the mechanism is sequential.
Shares no code with the engine: the tests compare the engine's kernels and whole models against these functions.

Tensor names follow the family's checkpoints (`l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`, `embed`, `final.norm`, `head`); a model is a
(config dict, {name: tensor}) pair."""
import math

import torch

F64 = torch.float64


def group_rms_norm(x, w, groups, eps):
    """x [..., D] split into `groups` consecutive parts, each divided by its own sqrt(mean(part^2) + eps); the whole times w."""
    D = x.shape[-1]
    parts = x.to(F64).reshape(*x.shape[:-1], groups, D // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    y = parts.reshape(x.shape)
    return y * w.to(F64) if w is not None else y


def yarn_frequencies(dims, base, scaling=None):
    """([dims / 2] frequencies, magnitude of cos / sin).  Channel i turns at base^(-2i/dims); with scaling the slow channels are
    divided by `factor`, the fast ones kept, and a linear ramp between two channel indices blends the two."""
    half = dims // 2
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def channel_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(channel_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(channel_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(float(f[i]) / factor * ramp + float(f[i]) * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate_half_partial(x, pos, freq, mag):
    """x [T, heads, d]; the first 2 * len(freq) entries of a head are rotated, entry i paired with entry i + len(freq)."""
    half = freq.numel()
    ang = pos.to(F64)[:, None] * freq[None, :]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], dim=-1)


def sink_attention(q, k, v, scale, cap, sink, pos0=0):
    """q [T, H, d] at positions pos0 .. pos0 + T - 1; k [N, G, d], v [N, G, dv] at positions 0 .. N - 1.  Query i sees the keys j <= i; its
    weights are exp(s_j) / (sink + sum_j exp(s_j)) with s_j = scale q . k_j, capped as cap tanh(s_j / cap) when cap > 0."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        n = pos0 + t + 1
        for hh in range(H):
            g = hh // (H // G)
            s = (k[:n, g].to(F64) @ q[t, hh].to(F64)) * scale
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            e = torch.exp(s)
            out[t, hh] = (e / (sink + e.sum())) @ v[:n, g].to(F64)
    return out


def attention_mixer(h, W, m, eps, pos0=0, past=None):
    """h [T, D] of ONE sequence whose first row sits at position pos0; past = (keys, values) of the earlier positions or None.
    Returns (output [T, D], (keys, values) including the new rows)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = h.to(F64)
    q = (h @ W["q"].to(F64).T).reshape(T, H, d)
    k = (h @ W["k"].to(F64).T).reshape(T, G, d)
    v = (h @ W["v"].to(F64).T).reshape(T, G, dv)
    q = group_rms_norm(q, W["q.norm"], 1, eps)
    k = group_rms_norm(k, W["k.norm"], 1, eps)
    rot = m.get("rot")
    if rot and rot.get("dims", 0):
        freq, mag = yarn_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        pos = torch.arange(pos0, pos0 + T)
        q, k = rotate_half_partial(q, pos, freq, mag), rotate_half_partial(k, pos, freq, mag)
    v = group_rms_norm(v, None, 1, eps)
    if past is not None:
        k, v = torch.cat([past[0], k]), torch.cat([past[1], v])
    out = sink_attention(q, k, v, float(m["scale"]), float(m.get("softcap") or 0.0), 1.0, pos0)
    return out.reshape(T, H * dv) @ W["o"].to(F64).T, (k, v)


def hgrn2_mixer(h, W, m, eps, state=None):
    """h [T, D] of ONE sequence; state [heads, d, dv] or None (zeros).  Returns (output [T, D], state after the last row)."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    h = h.to(F64)
    q = torch.nn.functional.silu(h @ W["q"].to(F64).T).reshape(T, H, d)
    v = (h @ W["v"].to(F64).T).reshape(T, H, dv)
    low = W["lower"].to(F64)
    f = (low + (1.0 - low) * torch.sigmoid(h @ W["f"].to(F64).T + W["f.b"].to(F64))).reshape(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = group_rms_norm(o, W["norm"], 1, eps)
    return o.reshape(T, H * dv) @ W["o"].to(F64).T, S


def dense_ff(h, W, limit):
    h = h.to(F64)
    g = torch.clamp(h @ W["gate"].to(F64).T, max=limit)
    u = torch.clamp(h @ W["up"].to(F64).T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W["down"].to(F64).T


def silu_ff(h, W):
    h = h.to(F64)
    return (torch.nn.functional.silu(h @ W["gate"].to(F64).T) * (h @ W["up"].to(F64).T)) @ W["down"].to(F64).T


def route(h, W, n_real, n_identity, top):
    """(chosen expert ids [T, top], their weights [T, top]); ids >= n_real name identity experts."""
    z = h.to(F64) @ W["router"].to(F64).T
    assert z.shape[1] == n_real + n_identity
    s = torch.softmax(z, -1)
    choice = s + W["correction"].to(F64) if "correction" in W else s
    idx = choice.topk(top, dim=-1).indices
    w = s.gather(1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20)


def moe_ff(h, W, f):
    r = f["router"]
    E, I, top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
    idx, w = route(h, W, E, I, top)
    h64 = h.to(F64)
    out = torch.zeros_like(h64)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            y = h64[t] if e >= E else silu_ff(h64[t:t + 1], {n: W[f"e{e}.{n}"] for n in ("gate", "up", "down")})[0]
            out[t] += w[t, j] * y
    if f.get("shared"):
        out += silu_ff(h64, {n: W[f"shared.{n}"] for n in ("gate", "up", "down")})
    return out


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens, carry=None, hook=None):
    """One sequence's next tokens; carry = per-layer state of the earlier tokens (None at the start).  Returns (logits [T, vocab], carry)."""
    eps, groups = float(config["norm"]["eps"]), int(config["norm"]["groups"])
    n_layers = len(config["layers"])
    carry = carry or {"pos": 0, "layers": [None] * n_layers}
    pos0 = carry["pos"]
    x = weights["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)] * float(config["embedding"]["scale"])
    new = []
    for i, L in enumerate(config["layers"]):
        h = group_rms_norm(x, weights[f"l{i}.norm1"], groups, eps)
        Wm = sub(weights, f"l{i}.mix.")
        if L["type"] == "attention":
            y, st = attention_mixer(h, Wm, L["mixer"], eps, pos0, carry["layers"][i])
        elif L["type"] == "hgrn2":
            y, st = hgrn2_mixer(h, Wm, L["mixer"], eps, carry["layers"][i])
        else:
            raise ValueError(L["type"])
        new.append(st)
        f = L.get("mlp")
        if f is not None:
            Wf = sub(weights, f"l{i}.mlp.")
            y = y + (dense_ff(h, Wf, float(f["limit"])) if f["kind"] == "dense" else moe_ff(h, Wf, f))
        x = x + y
        if hook is not None:
            hook(i, x)
    h = group_rms_norm(x, weights["final.norm"], groups, eps)
    return h @ weights["head"].to(F64).T, {"pos": pos0 + len(tokens), "layers": new}


# ------------------------------------------------------------------------------------------------ small models for the tests
def attention_layer(heads, kv_heads, dim, vdim, scale=None, softcap=30.0, rot_dims=0, base=10000.0, scaling=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5, "softcap": softcap}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
        if scaling:
            m["rot"]["scaling"] = dict(scaling)
    return {"type": "attention", "mixer": m, "mlp": mlp}


def hgrn2_layer(heads, dim, vdim, mlp=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}


def dense(ff, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, identity, top, ff, shared_ff=0):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared_ff:
        f["shared"] = {"ff": shared_ff}
    return f


def make_config(layers, vocab=64, width=32, eps=1e-5, groups=2, embedding_scale=2.0):
    return {"architecture": "Pudinex", "embedding": {"scale": embedding_scale}, "layers": layers, "norm": {"eps": eps, "groups": groups}, "vocab": vocab,
            "width": width}


def random_weights(cfg, seed=0, router_gain=4.0):
    """bf16 tensors under the family's names.  Projections ~ N(0, 1 / fan_in) so that activations stay O(1); norm weights around 1; gate
    biases and lower bounds spread so that slow and fast channels both occur; router rows scaled up so that selections are decided."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]

    def lin(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * gain * i ** -0.5).bfloat16()

    def around_one(n):
        return (1.0 + 0.2 * torch.randn(n, generator=g)).bfloat16()

    w = {"embed": (torch.randn(cfg["vocab"], D, generator=g) * 0.5).bfloat16(), "final.norm": around_one(D), "head": lin(cfg["vocab"], D, 2.0)}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}."
        w[p + "norm1"] = around_one(D)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w.update({p + "mix.q": lin(H * d, D, 2.0), p + "mix.k": lin(G * d, D, 2.0), p + "mix.v": lin(G * dv, D), p + "mix.q.norm": around_one(d),
                      p + "mix.k.norm": around_one(d), p + "mix.o": lin(D, H * dv)})
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            w.update({p + "mix.q": lin(H * d, D), p + "mix.f": lin(H * d, D, 2.0), p + "mix.f.b": (torch.randn(H * d, generator=g) * 1.5 + 1.0).bfloat16(),
                      p + "mix.lower": torch.rand(H * d, generator=g).mul(0.9).bfloat16(), p + "mix.v": lin(H * dv, D), p + "mix.norm": around_one(dv),
                      p + "mix.o": lin(D, H * dv)})
        f = L.get("mlp")
        if f is None:
            continue
        if f["kind"] == "dense":
            w.update({p + "mlp.gate": lin(f["ff"], D, 2.0), p + "mlp.up": lin(f["ff"], D, 2.0), p + "mlp.down": lin(D, f["ff"])})
            continue
        r = f["router"]
        n_out = r["experts"] + r.get("identity", 0)
        w[p + "mlp.router"] = lin(n_out, D, router_gain)
        w[p + "mlp.correction"] = (torch.randn(n_out, generator=g) * 0.05).bfloat16()
        for e in range(r["experts"]):
            w.update({p + f"mlp.e{e}.gate": lin(f["expert"]["ff"], D), p + f"mlp.e{e}.up": lin(f["expert"]["ff"], D), p + f"mlp.e{e}.down": lin(D, f["expert"]["ff"])})
        if f.get("shared"):
            sf = f["shared"]["ff"]
            w.update({p + "mlp.shared.gate": lin(sf, D), p + "mlp.shared.up": lin(sf, D), p + "mlp.shared.down": lin(D, sf)})
    return w


def run(cfg, w, tokens, collect_layers=False):
    """Logits of every position of one sequence (float64 [T, vocab]); with collect_layers also the residual after every layer."""
    res = []
    logits, _ = forward(cfg, w, tokens, hook=(lambda i, x: res.append(x.clone())) if collect_layers else None)
    return (logits, res) if collect_layers else logits


def greedy(cfg, w, prompt, n_new):
    """Greedy continuation, recomputing the whole sequence for every new token."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(run(cfg, w, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out


def write_model(folder, cfg, w):
    """config.json + model.safetensors (8-byte little-endian header length, JSON header, raw little-endian data) -> folder."""
    import json
    import os
    import struct
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    names = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32"}
    header, blobs, at = {}, [], 0
    for k, t in w.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[k] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as fh:
        fh.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    return folder
