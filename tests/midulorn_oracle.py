"""Plain float64 statement of the Midulorn family, one function per mechanism, for the tests.  Nothing here is shared with the engine:
whole sequences, dense matrices, Python loops over tokens where the definition has a recurrence.

Notation: h [T, D] is what a sublayer reads (the residual stream itself), P a dict of the layer's tensors by their checkpoint names
without the `l<i>.` prefix, m the layer's `mixer` dict of config.json."""
import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w.to(F64)


def join(x, y, w, alpha, eps):
    """The norm sits behind the sum: the new stream is norm(alpha x + y)."""
    return rms_norm(alpha * x + y, w, eps)


def rotate_half(v, pos, dims, base):
    """v [T, ..., n]: entry i < dims / 2 pairs with entry i + dims / 2; angle = position * base^(-2 i / dims).  Entries from `dims` on pass."""
    half = dims // 2
    out = v.clone()
    f = torch.tensor([base**(-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = pos.to(F64).view(-1, *([1] * (v.dim() - 1))) * f
    u, w = v[..., :half], v[..., half:dims]
    out[..., :half] = u * torch.cos(a) - w * torch.sin(a)
    out[..., half:dims] = w * torch.cos(a) + u * torch.sin(a)
    return out


def softmax_with_sink(scores, visible, sink):
    """scores [T, T] of one head, visible [T, T] bool, sink a number: weights exp(s_j) / (exp(sink) + sum_visible exp(s))."""
    s = scores.masked_fill(~visible, -math.inf)
    top = torch.maximum(s.max(dim=-1, keepdim=True).values, torch.as_tensor(float(sink), dtype=F64))
    e = torch.exp(s - top)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink.to(F64) - top))


def latent_attention(h, P, m, eps):
    T = h.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ P["mix.q"].to(F64).T).view(T, H, d + dr)
    low = h @ P["mix.dkv"].to(F64).T
    c = rms_norm(low[:, :R], P["mix.dkv.norm"], eps)
    k_rot = rotate_half(low[:, R:], pos, m["rot"]["dims"], m["rot"]["base"])  # one rotated key part for all heads
    q_rot = rotate_half(q[..., d:], pos, m["rot"]["dims"], m["rot"]["base"])
    k = (c @ P["mix.uk"].to(F64).T).view(T, H, d)
    v = (c @ P["mix.uv"].to(F64).T).view(T, H, dv)
    gate = torch.sigmoid(h @ P["mix.g"].to(F64).T)  # [T, H]
    visible = pos.view(-1, 1) >= pos.view(1, -1)
    out = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        s = (q[:, a, :d] @ k[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        out[:, a] = softmax_with_sink(s, visible, P["mix.sink"][a]) @ v[:, a] * gate[:, a:a + 1]
    return out.reshape(T, H * dv) @ P["mix.o"].to(F64).T


def mingru(h, P, m):
    z = torch.sigmoid(h @ P["mix.z"].to(F64).T + P["mix.z.b"].to(F64))
    u = h @ P["mix.x"].to(F64).T + P["mix.x.b"].to(F64)
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = h @ P["mix.g"].to(F64).T
    S = torch.zeros(m["width"], dtype=F64)
    rows = []
    for t in range(h.shape[0]):
        S = (1 - z[t]) * S + z[t] * cand[t]
        rows.append(S * g[t] * torch.sigmoid(g[t]))
    return torch.stack(rows) @ P["mix.o"].to(F64).T


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=F64), u])
    return sum(padded[j:j + u.shape[0]] * w[:, j].to(F64) for j in range(taps))


def conv_attention_values(h, P):
    return short_conv(h @ P["mix.v"].to(F64).T + P["mix.v.b"].to(F64), P["mix.v.conv"])


def conv_attention(h, P, m, eps, v_first=None):
    """Returns (mixer output, this layer's own values before any mixing).  `v_first`: the values of the first value-mixing layer, or None
    when this layer does not mix (or is that first layer)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(h @ P["mix.q"].to(F64).T + P["mix.q.b"].to(F64), P["mix.q.conv"]).view(T, H, d)
    k = short_conv(h @ P["mix.k"].to(F64).T + P["mix.k.b"].to(F64), P["mix.k.conv"]).view(T, G, d)
    v_own = conv_attention_values(h, P)
    v = v_own
    if v_first is not None:
        lam = P["mix.vmix"].to(F64)
        v = (1 - lam) * v_own + lam * v_first
    v = v.view(T, G, dv)
    q = rms_norm(q, P["mix.q.norm"], eps)
    k = rms_norm(k, P["mix.k.norm"], eps)
    pos = torch.arange(T)
    dist = (pos.view(-1, 1) - pos.view(1, -1)).clamp(min=0).to(F64)
    size = m["mask"]["size"]
    visible = (pos.view(-1, 1) >= pos.view(1, -1)) & ((pos.view(-1, 1) // size) == (pos.view(1, -1) // size))
    out = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        s = q[:, a] @ k[:, g].T * m["scale"] - P["mix.r1"][a].to(F64) * torch.log1p(P["mix.r2"][a].to(F64) * dist)
        out[:, a] = softmax_with_sink(s, visible, P["mix.sink"][a]) @ v[:, g]
    return out.reshape(T, H * dv) @ P["mix.o"].to(F64).T + P["mix.o.b"].to(F64), v_own


def softplus(x):
    return math.log1p(math.exp(x))


def xielu(z, p, q):
    pos = softplus(p) * z * z + z / 2
    neg = (0.5 + softplus(q)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + z / 2
    return torch.where(z > 0, pos, neg)


def dense_ff(h, P):
    p, q = (float(x) for x in P["mlp.act"])
    return xielu(h @ P["mlp.up"].to(F64).T, p, q) @ P["mlp.down"].to(F64).T


def route(h, P, top):
    """(chosen experts [T, top], their weights [T, top]): plain softmax scores over all experts, the largest `top`, not renormalised."""
    s = torch.softmax(h @ P["mlp.router"].to(F64).T, dim=-1)
    w, idx = torch.topk(s, top, dim=-1)
    return idx, w


def moe_ff(h, P, f):
    idx, w = route(h, P, f["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(idx[t].tolist(), w[t]):
            g = h[t] @ P[f"mlp.e{e}.gate"].to(F64).T
            u = h[t] @ P[f"mlp.e{e}.up"].to(F64).T
            out[t] += wt * ((g * torch.sigmoid(g) * u) @ P[f"mlp.e{e}.down"].to(F64).T)
    return out


def layer_params(sd, i):
    pre = f"l{i}."
    return {k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)}


def forward(tokens, sd, cfg):
    """tokens: list of ids of ONE sequence.  Returns (logits [T, vocab], residual stream after every layer [L, T, D]), float64."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = sd["embed"].to(F64)[torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    v_first, streams = None, []
    for i, L in enumerate(cfg["layers"]):
        P, m = layer_params(sd, i), L["mixer"]
        if L["type"] == "latent_attention":
            y = latent_attention(x, P, m, eps)
        elif L["type"] == "mingru":
            y = mingru(x, P, m)
        elif L["type"] == "attention":
            mixes = bool(m.get("v_mix"))
            y, v_own = conv_attention(x, P, m, eps, v_first if mixes else None)
            if mixes and v_first is None:
                v_first = v_own
        else:
            raise ValueError(L["type"])
        x = join(x, y, P["norm1"], alpha, eps)
        f = L.get("mlp")
        if f is not None:
            y = dense_ff(x, P) if f["kind"] == "dense" else moe_ff(x, P, f)
            x = join(x, y, P["norm2"], alpha, eps)
        streams.append(x)
    logits = rms_norm(x, sd["final.norm"], eps) @ sd["embed"].to(F64).T * cfg["logit_scale"]
    return logits, torch.stack(streams)
