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
    cap = float(m.get("softcap") or 0.0)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        n = pos0 + t + 1
        for hh in range(H):
            g = hh // (H // G)
            s = (k[:n, g] @ q[t, hh]) * float(m["scale"])
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            e = torch.exp(s)
            out[t, hh] = (e / (1.0 + e.sum())) @ v[:n, g]
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
