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


# ------------------------------------------------------------------------------------------------ small models for the tests
def latent_layer(heads, dim, rot_dim, vdim, kv_rank, scale=None, rot_dims=None, base=10000.0, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale if scale is not None else (dim + rot_dim)**-0.5,
         "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def mingru_layer(width, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def attention_layer(heads, kv_heads, dim, vdim, conv=3, part=16, scale=None, v_mix=False, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "mask": {"size": part}, "scale": scale if scale is not None else dim**-0.5,
         "v_mix": v_mix}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def make_config(layers, vocab=64, width=32, eps=1e-5, alpha=1.5, embedding_scale=2.0, logit_scale=0.7):
    return {"architecture": "Midulorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha,
            "embedding": {"scale": embedding_scale}, "logit_scale": logit_scale, "layers": layers}


def random_weights(cfg, seed=0, router_gain=4.0):
    """bf16 tensors under the family's names.  Projections ~ N(0, 1 / fan_in) so that activations stay O(1); norm weights around 1; gate
    biases spread so that slow and fast channels both occur; router rows scaled up so that selections are decided."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]

    def lin(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * gain * i**-0.5).bfloat16()

    def around_one(n):
        return (1.0 + 0.2 * torch.randn(n, generator=g)).bfloat16()

    def small(*shape, gain=0.3):
        return (gain * torch.randn(*shape, generator=g)).bfloat16()

    w = {"embed": (torch.randn(cfg["vocab"], D, generator=g) * 0.5).bfloat16(), "final.norm": around_one(D)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"] = around_one(D)
        if L["type"] == "latent_attention":
            H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w.update({p + "mix.q": lin(H * (d + dr), D, 2.0), p + "mix.dkv": lin(R + dr, D, 2.0), p + "mix.dkv.norm": around_one(R), p + "mix.uk": lin(H * d, R, 2.0),
                      p + "mix.uv": lin(H * dv, R), p + "mix.sink": small(H, gain=1.0), p + "mix.g": lin(H, D, 2.0), p + "mix.o": lin(D, H * dv)})
        elif L["type"] == "mingru":
            n = m["width"]
            w.update({p + "mix.z": lin(n, D, 2.0), p + "mix.z.b": (torch.randn(n, generator=g) * 2.0 - 1.0).bfloat16(), p + "mix.x": lin(n, D, 2.0),
                      p + "mix.x.b": small(n), p + "mix.g": lin(n, D, 2.0), p + "mix.o": lin(D, n)})
        else:
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for name, n in (("q", H * d), ("k", G * d), ("v", G * dv)):
                w[p + f"mix.{name}"] = lin(n, D, 2.0)
                w[p + f"mix.{name}.b"] = small(n)
                w[p + f"mix.{name}.conv"] = (torch.randn(n, taps, generator=g) * taps**-0.5 + (torch.arange(taps) == taps - 1) * 0.5).bfloat16()
            w.update({p + "mix.q.norm": around_one(d), p + "mix.k.norm": around_one(d), p + "mix.vmix": torch.tensor(0.35).bfloat16(),
                      p + "mix.r1": (0.5 + torch.rand(H, generator=g)).bfloat16(), p + "mix.r2": (0.1 + torch.rand(H, generator=g)).bfloat16(),
                      p + "mix.sink": small(H, gain=1.0), p + "mix.o": lin(D, H * dv), p + "mix.o.b": small(D)})
        f = L["mlp"]
        if f is None:
            continue
        w[p + "norm2"] = around_one(D)
        if f["kind"] == "dense":
            w.update({p + "mlp.up": lin(f["ff"], D, 2.0), p + "mlp.down": lin(D, f["ff"]), p + "mlp.act": torch.tensor([0.4, -0.3]).bfloat16()})
        else:
            w[p + "mlp.router"] = lin(f["router"]["experts"], D, router_gain)
            for e in range(f["router"]["experts"]):
                w.update({p + f"mlp.e{e}.gate": lin(f["expert"]["ff"], D, 2.0), p + f"mlp.e{e}.up": lin(f["expert"]["ff"], D, 2.0),
                          p + f"mlp.e{e}.down": lin(D, f["expert"]["ff"])})
    return w


def run(cfg, w, tokens, collect_layers=False):
    logits, streams = forward(tokens, w, cfg)
    return (logits, list(streams)) if collect_layers else logits


def greedy(cfg, w, prompt, n_new):
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(toks, w, cfg)[0][-1].argmax())
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
        raw = t.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[k] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as fh:
        fh.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    return folder
