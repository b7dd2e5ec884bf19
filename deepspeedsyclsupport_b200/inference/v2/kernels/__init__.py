"""Python wrappers of the ragged device ops (csrc/ragged/ragged_ops.cu) with PyTorch oracles for CPU / tests."""
import math
import os

import torch

from ....ops import native

native.register_sigs({
    "dsb200_kv_rotary_append": "pppppp iiiiiii p",
    "dsb200_paged_attention": "pppppp iiiiii f p",
    "dsb200_paged_flash_attention": "pppppp iiiiiii f ii p p i p",
    "dsb200_paged_flash_decode": "pppppp iiiiiii f ii p p i p",
    "dsb200_paged_flash_scratch_bytes": "iiiii",
    "dsb200_ragged_embed": "ppppp iii p",
    "dsb200_logits_gather": "ppp ii p",
    "dsb200_top_k_gating": "ppppp iiii p",
    "dsb200_moe_scatter": "ppppppp iiii p",
    "dsb200_moe_gather": "pppp iii p",
}, restype_long=("dsb200_paged_flash_scratch_bytes", ))


def kv_rotary_append(qkv, kv_cache, tok_seq, tok_pos, block_table, inv_freq, hq, hkv, d, rot_dim=None):
    """In place: RoPE on q,k heads of qkv [T, (hq+2hkv)*d]; k,v rows appended to kv_cache [blocks,2,bs,hkv,d]."""
    T = qkv.shape[0]
    bs = kv_cache.shape[2]
    rot_dim = d if rot_dim is None else rot_dim
    if qkv.is_cuda:
        rc = native.lib().dsb200_kv_rotary_append(native.ptr(qkv), native.ptr(kv_cache), native.ptr(tok_seq), native.ptr(tok_pos),
                                                  native.ptr(block_table), native.ptr(inv_freq), T, hq, hkv, d, bs,
                                                  block_table.shape[1], int(rot_dim), native.stream_ptr())
        native.check(rc)
        return qkv
    from ....ops.fused_ops import rope_ref
    if rot_dim == d:
        qkv.copy_(rope_ref(qkv, inv_freq, tok_pos, 0, hq + hkv, d))
    elif rot_dim > 0:
        xv = qkv.view(T, hq + 2 * hkv, d)
        rot = rope_ref(xv[:, :hq + hkv, :rot_dim].reshape(T, -1).contiguous(), inv_freq, tok_pos, 0, hq + hkv, rot_dim)
        xv[:, :hq + hkv, :rot_dim] = rot.view(T, hq + hkv, rot_dim)
    x = qkv.view(T, hq + 2 * hkv, d)
    for t in range(T):
        pos, seq = int(tok_pos[t]), int(tok_seq[t])
        blk = int(block_table[seq, pos // bs])
        kv_cache[blk, 0, pos % bs] = x[t, hq:hq + hkv]
        kv_cache[blk, 1, pos % bs] = x[t, hq + hkv:]
    return qkv


def paged_attention_ref(qkv, kv_cache, tok_seq, tok_pos, block_table, hq, hkv, d, scale, alibi_slopes=None, window=0):
    T = qkv.shape[0]
    bs = kv_cache.shape[2]
    out = torch.empty(T, hq * d, dtype=qkv.dtype, device=qkv.device)
    q = qkv.view(T, hq + 2 * hkv, d)[:, :hq].float()
    for t in range(T):
        n = int(tok_pos[t]) + 1
        seq = int(tok_seq[t])
        blocks = block_table[seq, :-(-n // bs)].long()
        k = kv_cache[blocks, 0].reshape(-1, hkv, d)[:n].float().repeat_interleave(hq // hkv, 1)
        v = kv_cache[blocks, 1].reshape(-1, hkv, d)[:n].float().repeat_interleave(hq // hkv, 1)
        s = torch.einsum("hd,nhd->hn", q[t], k) * scale
        if alibi_slopes is not None:
            s = s + alibi_slopes.float().to(s.device)[:, None] * torch.arange(n, device=s.device, dtype=torch.float32)[None, :]
        if window and n > window:
            s[:, :n - window] = float("-inf")
        out[t] = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), v).reshape(-1).to(qkv.dtype)
    return out


def paged_flash_supported(qkv, kv_cache, hq, hkv, d):
    """The tcgen05 kernel covers bf16, head_dim 64 / 128, q:kv head ratios and KV block sizes that divide 128."""
    group = hq // max(hkv, 1)
    return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and kv_cache.dtype == torch.bfloat16 and d in (64, 128) and hq % hkv == 0 and
            128 % group == 0 and kv_cache.shape[2] >= 8 and 128 % kv_cache.shape[2] == 0 and os.environ.get("DSB200_PAGED_FLASH", "1") != "0")


def _pick_splits(T, hq, d, ctas, pages, page_us=0.7):
    """KV splits per (atom, kv head): more splits fill the 148 SMs when the batch is small, but every split writes an fp32
    partial per (token, head) that the merge kernel reads back.  Cost model in microseconds: waves of CTAs x (5 us of set-up + pages per CTA at
    ~0.7 us a page), plus the partial traffic at HBM speed and the merge launch."""
    best, best_cost = 1, None
    for n in range(1, min(16, pages) + 1):
        waves = -(-ctas * n // 148)
        cost = (5.0 + -(-pages // n) * page_us) * waves
        if n > 1:
            cost += 2.0 * T * hq * (d + 2) * 4 * n / 6.0e6 + 3.0
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = n, cost
    return best


def paged_flash_attention(qkv, kv_cache, tok_seq, tok_pos, block_table, hq, hkv, d, scale=None, max_context=None, n_splits=None,
                          decode=None, alibi_slopes=None, window=0):
    """Attention of every ragged token over its sequence's paged KV history on the tensor cores (csrc/attn/paged_flash.cu):
    atoms of up to 128/group tokens x kv head, KV pages fetched by TMA through the block table, prefill chunks and decode steps
    alike; small batches over long contexts are split along the KV axis (`n_splits`, chosen here unless given) and merged.
    `decode`: the batch is (almost) one token per sequence -- use the transposed small-atom kernel (keys on the MMA M axis,
    16 q rows per atom).  Default: when the batch has no more tokens than the block table has sequences and d == 128.
    `alibi_slopes`: optional [hq] fp32 device tensor; adds slope[head] * key position to the scores (BLOOM-style ALiBi).
    `window` > 0: local attention over the last `window` keys (GPT-Neo's local layers)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    T = qkv.shape[0]
    bs, group = kv_cache.shape[2], hq // hkv
    if decode is None:
        decode = T <= block_table.shape[0]
    decode = bool(decode) and d == 128 and 16 % group == 0 and os.environ.get("DSB200_PAGED_DECODE", "1") != "0"
    nt = (16 if decode else 128) // group
    max_atoms = max(1, min(T, (T + nt - 1) // nt + block_table.shape[0]))
    if n_splits is None:
        pages = -(-(max_context if max_context is not None else block_table.shape[1] * bs) // 128)
        n_splits = _pick_splits(T, hq, d, max_atoms * hkv, pages, page_us=0.45 if decode else 0.7)
    out = torch.empty(T, hq * d, dtype=qkv.dtype, device=qkv.device)
    nbytes = native.lib().dsb200_paged_flash_scratch_bytes(T, hq, d, max_atoms, n_splits)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=qkv.device)
    fn = native.lib().dsb200_paged_flash_decode if decode else native.lib().dsb200_paged_flash_attention
    rc = fn(native.ptr(qkv), native.ptr(kv_cache), native.ptr(out), native.ptr(tok_seq), native.ptr(tok_pos), native.ptr(block_table), T, hq,
            hkv, d, bs, block_table.shape[1], kv_cache.shape[0], float(scale), max_atoms, n_splits, native.ptr(scratch),
            native.ptr(alibi_slopes), int(window), native.stream_ptr())
    native.check(rc)
    return out


def paged_attention(qkv, kv_cache, tok_seq, tok_pos, block_table, hq, hkv, d, scale=None, max_context=None, decode=None, alibi_slopes=None,
                    window=0):
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if not qkv.is_cuda:
        return paged_attention_ref(qkv, kv_cache, tok_seq, tok_pos, block_table, hq, hkv, d, scale, alibi_slopes, window)
    if paged_flash_supported(qkv, kv_cache, hq, hkv, d):
        return paged_flash_attention(qkv, kv_cache, tok_seq, tok_pos, block_table, hq, hkv, d, scale, max_context=max_context, decode=decode,
                                     alibi_slopes=alibi_slopes, window=window)
    assert alibi_slopes is None and not window, "ALiBi / local attention need the tensor-core kernel (bf16, head size 64 / 128)"
    # head sizes the tensor-core kernel does not cover (96, 256): CUDA-core kernel, one CTA per (token, kv head)
    T = qkv.shape[0]
    out = torch.empty(T, hq * d, dtype=qkv.dtype, device=qkv.device)
    rc = native.lib().dsb200_paged_attention(native.ptr(qkv), native.ptr(kv_cache), native.ptr(out), native.ptr(tok_seq),
                                             native.ptr(tok_pos), native.ptr(block_table), T, hq, hkv, d, kv_cache.shape[2],
                                             block_table.shape[1], float(scale), native.stream_ptr())
    native.check(rc)
    return out


def ragged_embed(ids, wte, wpe=None, tok_pos=None, pos_offset=0):
    if not wte.is_cuda or wte.dtype != torch.bfloat16:
        x = wte[ids]
        if wpe is not None:
            x = x + wpe[tok_pos.long() + pos_offset]
        return x
    T, dim = ids.numel(), wte.shape[1]
    out = torch.empty(T, dim, dtype=wte.dtype, device=wte.device)
    rc = native.lib().dsb200_ragged_embed(native.ptr(ids), native.ptr(wte), native.ptr(wpe), native.ptr(tok_pos if wpe is not None else None),
                                          native.ptr(out), T, dim, pos_offset, native.stream_ptr())
    native.check(rc)
    return out


def logits_gather(hidden, last_tok):
    if not hidden.is_cuda or hidden.dtype != torch.bfloat16:
        return hidden[last_tok.long()]
    out = torch.empty(last_tok.numel(), hidden.shape[1], dtype=hidden.dtype, device=hidden.device)
    rc = native.lib().dsb200_logits_gather(native.ptr(hidden), native.ptr(last_tok), native.ptr(out), last_tok.numel(), hidden.shape[1],
                                           native.stream_ptr())
    native.check(rc)
    return out


def top_k_gating(logits, k, normalize=True):
    """logits [T, E] fp32 -> (expert_counts [E] int32, scores [T,k] fp32, assignments [T,k] int32, offsets [T,k] int32)."""
    T, E = logits.shape
    if not logits.is_cuda:
        probs = torch.softmax(logits.float(), -1)
        sc, asg = probs.topk(k, dim=-1)
        if normalize:
            sc = sc / sc.sum(-1, keepdim=True)
        counts = torch.zeros(E, dtype=torch.int32)
        offsets = torch.zeros(T, k, dtype=torch.int32)
        for t in range(T):
            for j in range(k):
                e = int(asg[t, j])
                offsets[t, j] = counts[e]
                counts[e] += 1
        return counts, sc, asg.int(), offsets
    counts = torch.zeros(E, dtype=torch.int32, device=logits.device)
    scores = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    asg = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    off = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    rc = native.lib().dsb200_top_k_gating(native.ptr(logits.contiguous()), native.ptr(counts), native.ptr(scores), native.ptr(asg),
                                          native.ptr(off), T, E, k, int(normalize), native.stream_ptr())
    native.check(rc)
    return counts, scores, asg, off


def moe_scatter(x, counts, assignments, offsets):
    """rows of x copied into expert-sorted order.  returns (moe_in [T*k, dim], expert_cumsum [E] int64, mapped_slots [T,k])."""
    T, dim = x.shape
    k = assignments.shape[1]
    E = counts.numel()
    if not x.is_cuda or x.dtype != torch.bfloat16:
        cumsum = counts.long().cumsum(0)
        start = torch.cat([cumsum.new_zeros(1), cumsum[:-1]])
        slots = (start[assignments.long()] + offsets.long()).int()
        moe_in = x.new_zeros(T * k, dim)
        for j in range(k):
            moe_in[slots[:, j].long()] = x
        return moe_in, cumsum, slots
    moe_in = torch.empty(T * k, dim, dtype=x.dtype, device=x.device)
    cumsum = torch.empty(E, dtype=torch.int64, device=x.device)
    slots = torch.empty(T, k, dtype=torch.int32, device=x.device)
    rc = native.lib().dsb200_moe_scatter(native.ptr(x), native.ptr(counts), native.ptr(assignments), native.ptr(offsets),
                                         native.ptr(cumsum), native.ptr(moe_in), native.ptr(slots), T, E, dim, k, native.stream_ptr())
    native.check(rc, 2)
    return moe_in, cumsum, slots


def moe_gather(moe_out, scores, mapped_slots):
    T, k = mapped_slots.shape
    dim = moe_out.shape[1]
    if not moe_out.is_cuda or moe_out.dtype != torch.bfloat16:
        return (moe_out[mapped_slots.long()].float() * scores[..., None]).sum(1).to(moe_out.dtype)
    out = torch.empty(T, dim, dtype=moe_out.dtype, device=moe_out.device)
    rc = native.lib().dsb200_moe_gather(native.ptr(moe_out), native.ptr(scores), native.ptr(mapped_slots), native.ptr(out), T, dim, k,
                                        native.stream_ptr())
    native.check(rc)
    return out


# ---- kernels of csrc/ragged/latent_ops.cu: fp32 residual stream, latent-cache attention, grouped top-k router, expert MLP pieces
# for any width in bf16 or fp32.  Device only: these ops have no host form (their oracles live with the tests).
native.register_sigs({
    "dsb200_embed_sinusoid": "pp i pp p ii f p",
    "dsb200_stream_group_norm": "ppp i pp p i pp iii f p",
    "dsb200_sandwich_norm": "pp i p ff p f p i pp ii f i p",
    "dsb200_latent_norm_append": "p i pp pp ppp iiii ii f i p",
    "dsb200_paged_flash_latent": "p i ll pp ppp iiiiii f ii p i p",
    "dsb200_paged_flash_latent_sink": "p i ll pp ppp iiiiii f p ii p i p",
    "dsb200_gate_heads": "pp l p iii i p",
    "dsb200_latent_attention_scratch_floats": "iiii",
    "dsb200_latent_attention": "p i ll p i p ll p ppp ii iii f i p",
    "dsb200_sigmoid_gate_mul": "p l p l l i i p",
    "dsb200_clamped_swish_gate": "pp l i fff i p",
    "dsb200_clamped_swish_gate_cols": "p l ii p l l i fff i p",
    "dsb200_softcap": "p l l i f p",
    "dsb200_grouped_topk_gating": "pppppp iiiiiii p",
    "dsb200_moe_scatter_rows": "ppppppp iiii i p p",
    "dsb200_moe_gather_rows": "pppp iii i p i p p",
    "dsb200_moe_gemm_rows": "pppp iiii i p",
}, restype_long=("dsb200_latent_attention_scratch_floats", ))

_DT = {torch.bfloat16: 0, torch.float32: 1}


def _dt(t):
    if not t.is_cuda or t.dtype not in _DT:
        raise native.NativeError(f"this op runs on CUDA tensors of bf16 or fp32 (got {t.dtype} on {t.device})")
    return _DT[t.dtype]


def sinusoid_frequencies(dim, base=10000.0, device=None):
    """f_i = base ** (-2 i / dim), i < ceil(dim / 2), in float64 (positions times these are taken in double on the device)."""
    i = torch.arange((dim + 1) // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dim).to(device)


def embed_sinusoid(ids, table, tok_pos, freq, scale=1.0):
    """fp32 [T, dim]: scale * table[ids] + (sin(p f_0), cos(p f_0), sin(p f_1), ...); `freq` None: the scaled table rows alone."""
    T, dim = ids.numel(), table.shape[1]
    out = torch.empty(T, dim, dtype=torch.float32, device=table.device)
    native.check(native.lib().dsb200_embed_sinusoid(native.ptr(ids), native.ptr(table), _dt(table), native.ptr(tok_pos), native.ptr(freq),
                                                    native.ptr(out), T, dim, float(scale), native.stream_ptr()))
    return out


def stream_group_norm(x, branches=(), branch_fp32=None, w=None, groups=1, eps=1e-6, out_dtype=torch.bfloat16, rows=None, fp32_copy=False):
    """On the fp32 residual x [T, dim], in place: x += every tensor of `branches` (at most two, in one activation dtype) + branch_fp32
    (fp32).  With w: returns x normed in `groups` equal consecutive parts (each divided by its own root mean square, eps inside the root)
    times w, in `out_dtype`; with `fp32_copy` -> (out, the same values before rounding).  `rows` (int32 indices): only those rows are summed
    and normed, the result has one row per index and x itself is left as it was."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.is_cuda and len(branches) <= 2
    ys = [y if y.is_contiguous() else y.contiguous() for y in branches]
    assert all(y.shape == x.shape and y.dtype == ys[0].dtype for y in ys)
    assert branch_fp32 is None or (branch_fp32.shape == x.shape and branch_fp32.dtype == torch.float32 and branch_fp32.is_contiguous())
    n = x.shape[0] if rows is None else rows.numel()
    out = torch.empty(n, x.shape[1], dtype=out_dtype, device=x.device) if w is not None else None
    out32 = torch.empty(n, x.shape[1], dtype=torch.float32, device=x.device) if (fp32_copy and w is not None and out_dtype != torch.float32) else None
    ys += [None] * (2 - len(ys))
    native.check(native.lib().dsb200_stream_group_norm(native.ptr(x), native.ptr(ys[0]), native.ptr(ys[1]), _dt(ys[0]) if ys[0] is not None else 0,
                                                       native.ptr(branch_fp32), native.ptr(w), native.ptr(out), _DT[out_dtype], native.ptr(out32),
                                                       native.ptr(rows), n, x.shape[1], int(groups), float(eps), native.stream_ptr()))
    if fp32_copy:
        return out, (out32 if out32 is not None else out)
    return out


def sandwich_norm(x, y=None, wb=None, ob=0.0, w=None, o=0.0, eps=1e-6, out_dtype=torch.bfloat16, rows=None, fp32_copy=False, y_mult=1.0,
                  plain_out=False):
    """On the fp32 residual x [T, dim], in place: x += y_mult * rms_norm(y) * (wb + ob) when a branch output y is given; returns
    rms_norm(x) * (w + o) in `out_dtype` when w is given, the stream itself in `out_dtype` when `plain_out` (blocks whose sublayers
    read the stream unnormed), else None.  `rows` (int32 indices): normalise only those rows of x (no branch then); the result has
    one row per index.  `fp32_copy`: also return the normed values before their rounding to `out_dtype` -> (out, out_fp32); for an
    fp32 `out_dtype` both are the same tensor."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.is_cuda
    assert not (plain_out and (w is not None or fp32_copy))
    n = x.shape[0] if rows is None else rows.numel()
    out = torch.empty(n, x.shape[1], dtype=out_dtype, device=x.device) if (w is not None or plain_out) else None
    out32 = torch.empty(n, x.shape[1], dtype=torch.float32, device=x.device) if (fp32_copy and w is not None and out_dtype != torch.float32) else None
    if y is not None:
        assert y.shape == x.shape
        y = y if y.is_contiguous() else y.contiguous()  # a GEMM output whose rows were padded to the TMA stride (odd widths only)
    native.check(native.lib().dsb200_sandwich_norm(native.ptr(x), native.ptr(y), _dt(y) if y is not None else 0, native.ptr(wb), float(ob),
                                                   float(y_mult), native.ptr(w), float(o), native.ptr(out), _DT[out_dtype], native.ptr(out32),
                                                   native.ptr(rows), n, x.shape[1], float(eps), int(plain_out), native.stream_ptr()))
    if fp32_copy:
        return out, (out32 if out32 is not None else out)
    return out


def latent_norm_append(lat, wq, wkv, cache, tok_seq, tok_pos, block_table, nq, nkv, eps):
    """lat [T, >= nq + nkv]: rows (query latent | key/value latent).  Returns the RMS-normed query latents [T, nq]; the RMS-normed
    key/value latent of every token is written into cache [blocks, block_size, >= nkv] at the token's position (columns past nkv
    are padding and are left alone)."""
    T = lat.shape[0]
    assert lat.stride(1) == 1 and cache.dtype == lat.dtype and cache.is_contiguous() and cache.shape[2] >= nkv
    cq = torch.empty(T, nq, dtype=lat.dtype, device=lat.device)
    native.check(native.lib().dsb200_latent_norm_append(native.ptr(lat), lat.stride(0), native.ptr(wq), native.ptr(wkv), native.ptr(cq),
                                                        native.ptr(cache), native.ptr(tok_seq), native.ptr(tok_pos), native.ptr(block_table),
                                                        block_table.stride(0), cache.shape[1], cache.shape[2], T, nq, nkv, float(eps), _dt(lat),
                                                        native.stream_ptr()))
    return cq


def paged_latent_flash(q_abs, cache, tok_seq, tok_pos, block_table, scale, decode=False, max_context=None, n_splits=None, heads=None,
                       sink_logit=None):
    """`latent_attention` on the tensor cores (csrc/attn/paged_flash.cu with one cache plane serving as keys and values).
    q_abs: bf16 view [T, H, rank] with unit stride in rank and any 16-byte-multiple token / head strides (token-major, or the
    head-major output of a batched GEMM seen through `.transpose(0, 1)`); rank 64 / 128.  The kernel works on `heads` heads, a divisor
    of 128 that is >= H (default: the next power of two); heads past H read as zero.  cache [blocks, block_size, rank] bf16 with a
    block size dividing 128.  Returns bf16 [T, heads, rank] (rows of heads >= H are meaningless).  `decode`: (almost) one token per
    sequence -- the small-atom kernel (rank 128, heads dividing 16).  `sink_logit` (fp32, one per head the kernel works on): learned sinks,
    exp(sink_logit[h]) joins head h's softmax denominator."""
    T, H, R = q_abs.shape
    Hp = heads or (1 << (H - 1).bit_length())
    assert sink_logit is None or (sink_logit.dtype == torch.float32 and sink_logit.numel() >= Hp and sink_logit.is_cuda)
    bs = cache.shape[1]
    assert q_abs.stride(2) == 1 and cache.is_contiguous() and q_abs.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and Hp >= H
    decode = bool(decode) and R == 128 and 16 % Hp == 0
    nt = (16 if decode else 128) // Hp
    max_atoms = max(1, min(T, (T + nt - 1) // nt + block_table.shape[0]))
    if n_splits is None:
        pages = -(-(max_context if max_context is not None else block_table.shape[1] * bs) // 128)
        n_splits = _pick_splits(T, Hp, R, max_atoms, pages, page_us=0.45 if decode else 0.7)
    out = torch.empty(T, Hp, R, dtype=torch.bfloat16, device=q_abs.device)
    nbytes = native.lib().dsb200_paged_flash_scratch_bytes(T, Hp, R, max_atoms, n_splits)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=q_abs.device)
    native.check(native.lib().dsb200_paged_flash_latent_sink(native.ptr(q_abs), H, q_abs.stride(1) if H > 1 else R, q_abs.stride(0) if T > 1 else H * R,
                                                             native.ptr(cache), native.ptr(out), native.ptr(tok_seq), native.ptr(tok_pos),
                                                             native.ptr(block_table), T, Hp, R, bs, block_table.shape[1], cache.shape[0], float(scale),
                                                             native.ptr(sink_logit), max_atoms, n_splits, native.ptr(scratch), int(decode),
                                                             native.stream_ptr()), 2 + (n_splits > 1))
    return out


def gate_heads(a, gate):
    """a [H, T, dv] (contiguous result of a per-head batched GEMM), gate [T, H * dv] (unit column stride) -> [T, H * dv]: the heads
    side by side per token, times sigmoid(gate), in one pass."""
    H, T, dv = a.shape
    assert a.is_contiguous() and gate.shape == (T, H * dv) and gate.stride(1) == 1 and gate.dtype == a.dtype
    out = torch.empty(T, H * dv, dtype=a.dtype, device=a.device)
    native.check(native.lib().dsb200_gate_heads(native.ptr(a), native.ptr(gate), gate.stride(0), native.ptr(out), T, H, dv, _dt(a),
                                                native.stream_ptr()))
    return out


def _latent_splits(T, head_groups, max_keys):
    """Key splits per token for the CUDA-core kernel: its CTAs are small (4 warps, ~20 KB of shared memory), so a decode batch wants
    about 8 of them per SM to hide the shared-memory latency of the score loop; at least 128 keys per split, at most 32 splits."""
    ctas = max(1, T * head_groups)
    return max(1, min(-(-max_keys // 128), (8 * 148) // ctas, 32))


def latent_attention(q_abs, cache, tok_seq, tok_pos, block_table, scale, out=None, max_keys=None, n_splits=None):
    """q_abs [T, H, R] (any strides with unit stride in R; bf16 / fp32): queries already mapped into the latent space.
    cache [blocks, block_size, R].  Returns fp32 [T, H, R] (or fills `out`, any token / head strides):
    sum_j softmax_j(scale q . c_j) c_j over the latents 0 .. pos(t) of the token's sequence."""
    T, H, R = q_abs.shape
    assert q_abs.stride(2) == 1 and cache.is_contiguous() and cache.shape[2] == R
    if out is None:
        out = torch.empty(T, H, R, dtype=torch.float32, device=q_abs.device)
    assert out.dtype == torch.float32 and out.stride(2) == 1
    if n_splits is None:
        n_splits = _latent_splits(T, -(-H // 8), max_keys if max_keys is not None else block_table.shape[1] * cache.shape[1])
    nf = native.lib().dsb200_latent_attention_scratch_floats(T, H, R, n_splits)
    scratch = torch.empty(nf, dtype=torch.float32, device=q_abs.device) if nf else None
    native.check(native.lib().dsb200_latent_attention(native.ptr(q_abs), _dt(q_abs), q_abs.stride(0), q_abs.stride(1), native.ptr(cache),
                                                      _dt(cache), native.ptr(out), out.stride(0), out.stride(1), native.ptr(scratch),
                                                      native.ptr(tok_seq), native.ptr(tok_pos), native.ptr(block_table), block_table.stride(0),
                                                      cache.shape[1], T, H, R, float(scale), int(n_splits), native.stream_ptr()),
                 2 if n_splits > 1 else 1)
    return out


def sigmoid_gate_mul(a, g):
    """a *= sigmoid(g), in place; a and g are [rows, cols] views with unit column stride."""
    assert a.shape == g.shape and a.dim() == 2 and a.stride(1) == 1 and g.stride(1) == 1 and a.dtype == g.dtype
    native.check(native.lib().dsb200_sigmoid_gate_mul(native.ptr(a), a.stride(0), native.ptr(g), g.stride(0), a.shape[0], a.shape[1], _dt(a),
                                                      native.stream_ptr()))
    return a


def clamped_swish_gate(gu, alpha, limit, shift):
    """gu [rows, 2F] = (gate | up) -> [rows, F]: g' sigmoid(alpha g') (clamp(u, -limit, limit) + shift) with g' = min(g, limit)."""
    assert gu.is_contiguous() and gu.shape[1] % 2 == 0
    F = gu.shape[1] // 2
    out = torch.empty(gu.shape[0], F, dtype=gu.dtype, device=gu.device)
    native.check(native.lib().dsb200_clamped_swish_gate(native.ptr(gu), native.ptr(out), gu.shape[0], F, float(alpha), float(limit),
                                                        float(shift), _dt(gu), native.stream_ptr()))
    return out


def clamped_swish_gate_cols(gu, gate_col0, up_col0, F, out, alpha, limit, shift):
    """`clamped_swish_gate` on column ranges: gate = gu[:, gate_col0 : gate_col0 + F], up = gu[:, up_col0 : up_col0 + F] of a fused projection,
    result into `out` [rows, F] (a view with unit column stride, e.g. a column range of the next GEMM's input)."""
    assert gu.stride(1) == 1 and out.stride(1) == 1 and out.shape == (gu.shape[0], F) and gu.dtype == out.dtype
    native.check(native.lib().dsb200_clamped_swish_gate_cols(native.ptr(gu), gu.stride(0), int(gate_col0), int(up_col0), native.ptr(out), out.stride(0),
                                                             gu.shape[0], int(F), float(alpha), float(limit), float(shift), _dt(gu), native.stream_ptr()))
    return out


def softcap_(logits, cap):
    """logits <- cap * tanh(logits / cap), in place on an fp32 [rows, cols] view."""
    assert logits.dtype == torch.float32 and logits.is_cuda and logits.stride(1) == 1
    native.check(native.lib().dsb200_softcap(native.ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], float(cap),
                                             native.stream_ptr()))
    return logits


def grouped_topk_gating(logits, k, correction=None, groups=1, keep=1, normalize=False, sigmoid_scores=False):
    """Router with a selection bias and contiguous expert groups (see csrc/ragged/latent_ops.cu).  logits [T, E] fp32 ->
    (expert_counts [E] int32, scores [T, k] fp32, assignments [T, k] int32, offsets [T, k] int32), as `top_k_gating`.
    `sigmoid_scores`: an expert's score is the sigmoid of its own logit instead of its softmax probability."""
    assert logits.dtype == torch.float32 and logits.is_cuda and logits.is_contiguous()
    T, E = logits.shape
    counts = torch.zeros(E, dtype=torch.int32, device=logits.device)
    scores = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    asg = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    off = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    native.check(native.lib().dsb200_grouped_topk_gating(native.ptr(logits), native.ptr(correction), native.ptr(counts), native.ptr(scores),
                                                         native.ptr(asg), native.ptr(off), T, E, k, groups, keep, int(normalize),
                                                         int(sigmoid_scores), native.stream_ptr()))
    return counts, scores, asg, off


def moe_scatter_rows(x, counts, assignments, offsets, row_scale=None):
    """`moe_scatter` for any width and bf16 / fp32 rows.  `row_scale` (fp32 [T, k]): copy k of token t is multiplied by it."""
    T, dim = x.shape
    k, E = assignments.shape[1], counts.numel()
    assert x.is_contiguous()
    moe_in = torch.empty(T * k, dim, dtype=x.dtype, device=x.device)
    cumsum = torch.empty(E, dtype=torch.int64, device=x.device)
    slots = torch.empty(T, k, dtype=torch.int32, device=x.device)
    native.check(native.lib().dsb200_moe_scatter_rows(native.ptr(x), native.ptr(counts), native.ptr(assignments), native.ptr(offsets),
                                                      native.ptr(cumsum), native.ptr(moe_in), native.ptr(slots), T, E, dim, k, _dt(x),
                                                      native.ptr(row_scale), native.stream_ptr()), 2)
    return moe_in, cumsum, slots


def moe_gather_rows(moe_out, scores, mapped_slots, assignments=None, n_real=0, identity_src=None):
    """fp32 [T, dim]: sum_k scores[t, k] * moe_out[mapped_slots[t, k]] (`scores` None: the plain sum).  With `assignments` [T, k]: experts
    `n_real` and above are identity experts -- their output is the token's row of `identity_src` (fp32 [T, dim])."""
    T, k = mapped_slots.shape
    assert moe_out.is_contiguous()
    if assignments is not None:
        assert identity_src is not None and identity_src.dtype == torch.float32 and identity_src.is_contiguous() and identity_src.shape == (T, moe_out.shape[1])
    out = torch.empty(T, moe_out.shape[1], dtype=torch.float32, device=moe_out.device)
    native.check(native.lib().dsb200_moe_gather_rows(native.ptr(moe_out), native.ptr(scores), native.ptr(mapped_slots), native.ptr(out), T,
                                                     moe_out.shape[1], k, _dt(moe_out), native.ptr(assignments), int(n_real),
                                                     native.ptr(identity_src), native.stream_ptr()))
    return out


def moe_gemm_rows(x, w, cumsum):
    """Grouped expert GEMM on CUDA cores (bf16 or fp32, fp32 accumulation, any shape): out[r] = w[expert(r)] @ x[r]."""
    assert x.is_contiguous() and w.is_contiguous() and x.dtype == w.dtype and x.shape[1] == w.shape[2]
    R, K = x.shape
    E, N, _ = w.shape
    out = torch.empty(R, N, dtype=x.dtype, device=x.device)
    native.check(native.lib().dsb200_moe_gemm_rows(native.ptr(x), native.ptr(w), native.ptr(out), native.ptr(cumsum), R, N, K, E, _dt(x),
                                                   native.stream_ptr()))
    return out


# ---- kernels of csrc/ragged/recurrent_ops.cu: short convolutions with per-sequence state, windowed attention that keeps the first
# tokens visible, recurrent matrix memories.  Device only (their oracles live with the tests).  `seq_desc` is the batch's
# [n_seqs, 4] int32 (first row, new tokens, tokens seen before, state slot).
native.register_sigs({
    "dsb200_scan_state_floats": "ii",
    "dsb200_paged_flash_window": "p l pp l ppp iiiiiii ff ii ii p i p",
    "dsb200_window_qk_prepare": "p l ii pppp p ppp p ii pp l p iiiiii f i p",
    "dsb200_conv_state_update": "p l i p ii p iii i p",
    "dsb200_window_attention": "p l p ppp ii p l iiiiii ff i p",
    "dsb200_matrix_memory_scan": "p l iii ppp f p ppp p iiii i p",
    "dsb200_delta_prepare": "p l iii ppp p pp ppp pppp iiiiii i p",
    "dsb200_delta_rule_scan": "ppppp p pp iiiii p",
    "dsb200_head_norm_gate": "pp i p l p l iii ff i p",
    "dsb200_tied_gate_scan": "p l iii pp p pp iiii i p",
    "dsb200_head_norm_rotary_append": "p l iii pp p f ppp ii p l p l p l iiiii i f i iii i p",
    "dsb200_sink_attention": "p l p l p l ppp ii p l iiiii fff i p",
    "dsb200_paged_flash_sink": "p l pp l ppp iiiiiii fff ii p i p",
    "dsb200_paged_flash_sink_ex": "p l pp l ppp iiiiiii fff ppp i ii p i p",
}, restype_long=("dsb200_scan_state_floats", ))


def scan_state_floats(d, dv):
    """fp32 values per (slot, head) of a d x dv recurrent state in the scan kernels' own layout."""
    n = native.lib().dsb200_scan_state_floats(int(d), int(dv))
    if n < 0:
        raise native.NativeError(f"a {d} x {dv} recurrent state per head is not supported")
    return int(n)


def window_qk_prepare(proj, q_col0, k_col0, conv_q, conv_k, norm_q, norm_k, state, seq_desc, tok_seq, tok_pos, block_table, cache, q_out, freq,
                      H, G, d, taps, rot_dims, eps):
    """Short convolution of the query / key projections held in columns q_col0 / k_col0 of proj [T, ld], whole-projection RMS norms,
    interleaved rotary on the first `rot_dims` entries of every head; the convolved keys go to cache plane 1 (they are the values), the
    finished keys to plane 0 and the queries to q_out [T, >= H d].  cache [blocks, 2, block_size, G, d].  Follow with `conv_state_update`."""
    T = proj.shape[0]
    assert proj.stride(1) == 1 and cache.is_contiguous() and cache.dtype == proj.dtype and q_out.dtype == proj.dtype and q_out.stride(1) == 1
    native.check(native.lib().dsb200_window_qk_prepare(native.ptr(proj), proj.stride(0), q_col0, k_col0, native.ptr(conv_q), native.ptr(conv_k),
                                                       native.ptr(norm_q), native.ptr(norm_k), native.ptr(state), native.ptr(seq_desc),
                                                       native.ptr(tok_seq), native.ptr(tok_pos), native.ptr(block_table), block_table.stride(0),
                                                       cache.shape[2], native.ptr(cache), native.ptr(q_out), q_out.stride(0), native.ptr(freq), T,
                                                       H, G, d, taps, rot_dims, float(eps), _dt(proj), native.stream_ptr()))
    return q_out


def conv_state_update(proj, col0, n_cols, state, st_col0, seq_desc, n_seqs, taps):
    """state [slots, taps - 1, C] columns st_col0 .. + n_cols <- the last taps - 1 rows of columns col0 .. + n_cols of proj, per sequence."""
    if taps <= 1:
        return
    assert state.is_contiguous() and state.dtype == proj.dtype and state.shape[1] == taps - 1
    native.check(native.lib().dsb200_conv_state_update(native.ptr(proj), proj.stride(0), col0, native.ptr(state), state.shape[2], st_col0,
                                                       native.ptr(seq_desc), n_seqs, n_cols, taps, _dt(proj), native.stream_ptr()))


def window_attention(q, cache, tok_seq, tok_pos, block_table, out, H, G, d, window, keep_first, scale, out_scale=1.0):
    """CUDA-core attention over the paged cache [blocks, 2, block_size, G, d]: a query at position p sees the keys j <= p with
    p - j < window or j < keep_first.  q [T, >= H d], out [T, >= H d] (views with unit column stride); fp32 softmax and accumulation."""
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and cache.is_contiguous() and q.dtype == cache.dtype == out.dtype
    native.check(native.lib().dsb200_window_attention(native.ptr(q), q.stride(0), native.ptr(cache), native.ptr(tok_seq), native.ptr(tok_pos),
                                                      native.ptr(block_table), block_table.stride(0), cache.shape[2], native.ptr(out),
                                                      out.stride(0), T, H, G, d, int(window), int(keep_first), float(scale), float(out_scale),
                                                      _dt(q), native.stream_ptr()))
    return out


def paged_flash_window_ok(q, cache, out, H, G, d):
    """Whether the tensor-core kernels take this windowed attention: bf16, head size 64 / 128, a q:kv head ratio dividing 128, cache blocks
    dividing 128, 16-byte aligned rows."""
    return (q.is_cuda and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and d in (64, 128) and H % G == 0 and
            128 % (H // G) == 0 and cache.shape[2] >= 8 and 128 % cache.shape[2] == 0 and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and
            q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and os.environ.get("DSB200_PAGED_FLASH", "1") != "0")


def paged_flash_window(q, cache, tok_seq, tok_pos, block_table, out, H, G, d, window, keep_first, scale, out_scale=1.0, decode=False, max_context=None,
                       n_splits=None):
    """`window_attention` on the tensor cores (csrc/attn/paged_flash.cu: TMA pages through the block table, S / P / O in TMEM); only the
    pages of the kept first keys and of the window are visited.  `decode`: (almost) one token per sequence -- the small-atom kernel."""
    T = q.shape[0]
    bs, group = cache.shape[2], H // G
    decode = bool(decode) and d == 128 and 16 % group == 0 and os.environ.get("DSB200_PAGED_DECODE", "1") != "0"
    nt = (16 if decode else 128) // group
    max_atoms = max(1, min(T, (T + nt - 1) // nt + block_table.shape[0]))
    if n_splits is None:
        ctx = max_context if max_context is not None else block_table.shape[1] * bs
        pages = -(-min(ctx, window + keep_first + 256) // 128)
        n_splits = _pick_splits(T, H, d, max_atoms * G, pages, page_us=0.45 if decode else 0.7)
    nbytes = native.lib().dsb200_paged_flash_scratch_bytes(T, H, d, max_atoms, n_splits)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    native.check(native.lib().dsb200_paged_flash_window(native.ptr(q), q.stride(0), native.ptr(cache), native.ptr(out), out.stride(0), native.ptr(tok_seq),
                                                        native.ptr(tok_pos), native.ptr(block_table), T, H, G, d, bs, block_table.shape[1], cache.shape[0],
                                                        float(scale), float(out_scale), int(window), int(keep_first), max_atoms, n_splits,
                                                        native.ptr(scratch), int(decode), native.stream_ptr()), 2 + (n_splits > 1))
    return out


def matrix_memory_scan(proj, q_col0, k_col0, v_col0, gates, bias_i, bias_f, cap, seq_desc, n_seqs, state_S, state_n, state_m, H, d, dv):
    """Matrix memory with exponential gating over every sequence's new tokens -> fp32 [T, H dv] read-outs (before the head norm)."""
    T = proj.shape[0]
    assert proj.stride(1) == 1 and gates.dtype == torch.float32 and gates.is_contiguous() and gates.shape == (T, 2 * H)
    out = torch.empty(T, H * dv, dtype=torch.float32, device=proj.device)
    native.check(native.lib().dsb200_matrix_memory_scan(native.ptr(proj), proj.stride(0), q_col0, k_col0, v_col0, native.ptr(gates),
                                                        native.ptr(bias_i), native.ptr(bias_f), float(cap), native.ptr(seq_desc),
                                                        native.ptr(state_S), native.ptr(state_n), native.ptr(state_m), native.ptr(out), n_seqs, H,
                                                        d, dv, _dt(proj), native.stream_ptr()))
    return out


def delta_prepare(proj, q_col0, k_col0, v_col0, conv_q, conv_k, conv_v, state, seq_desc, tok_seq, a_pre, beta_pre, A_log, dt_bias, G, H, d, dv, taps):
    """Short convolution + silu of the q / k / v projections, q and k to unit length per head (q also times d^-1/2) ->
    fp32 (q [T, G d], k [T, G d], v [T, H dv]).  In place: a_pre fp32 [T, H d] becomes the decays exp(-exp(A_log) softplus(a_pre + dt_bias))
    and beta_pre fp32 [T, H] becomes sigmoid(beta_pre).  Follow with `conv_state_update`."""
    T = proj.shape[0]
    assert proj.stride(1) == 1
    for t, shape in ((a_pre, (T, H * d)), (beta_pre, (T, H))):
        assert t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape) == shape
    qn = torch.empty(T, G * d, dtype=torch.float32, device=proj.device)
    kn = torch.empty(T, G * d, dtype=torch.float32, device=proj.device)
    vo = torch.empty(T, H * dv, dtype=torch.float32, device=proj.device)
    native.check(native.lib().dsb200_delta_prepare(native.ptr(proj), proj.stride(0), q_col0, k_col0, v_col0, native.ptr(conv_q), native.ptr(conv_k),
                                                   native.ptr(conv_v), native.ptr(state), native.ptr(seq_desc), native.ptr(tok_seq), native.ptr(qn),
                                                   native.ptr(kn), native.ptr(vo), native.ptr(a_pre), native.ptr(beta_pre), native.ptr(A_log),
                                                   native.ptr(dt_bias), T, G, H, d, dv, taps, _dt(proj), native.stream_ptr()))
    return qn, kn, vo


def delta_rule_scan(qn, kn, v, beta, decay, seq_desc, n_seqs, state_S, H, G, d, dv):
    """Gated delta rule with per-channel decays over every sequence's new tokens -> fp32 [T, H dv] read-outs.  beta [T, H] and decay
    [T, H d] as `delta_prepare` leaves them."""
    T = qn.shape[0]
    for t in (qn, kn, v, beta, decay):
        assert t.dtype == torch.float32 and t.is_contiguous()
    out = torch.empty(T, H * dv, dtype=torch.float32, device=qn.device)
    native.check(native.lib().dsb200_delta_rule_scan(native.ptr(qn), native.ptr(kn), native.ptr(v), native.ptr(beta), native.ptr(decay),
                                                     native.ptr(seq_desc), native.ptr(state_S), native.ptr(out), n_seqs, H, G, d, dv,
                                                     native.stream_ptr()))
    return out


def head_norm_gate(o, w, gate, out, H, dv, eps, mult=1.0, shared_weight=False):
    """out[:, h dv + c] = rms_norm_over_c(o[:, h, :]) * w * sigmoid(gate) * mult; o fp32 [T, H dv]; w fp32 [H dv] or (shared) [dv];
    gate / out: views [T, >= H dv] of the activation dtype with unit column stride; gate None: no gate factor."""
    T = o.shape[0]
    assert o.dtype == torch.float32 and o.is_contiguous() and out.stride(1) == 1
    assert gate is None or (gate.stride(1) == 1 and gate.dtype == out.dtype)
    native.check(native.lib().dsb200_head_norm_gate(native.ptr(o), native.ptr(w), 0 if shared_weight else dv, native.ptr(gate),
                                                    gate.stride(0) if gate is not None else 0,
                                                    native.ptr(out), out.stride(0), T, H, dv, float(eps), float(mult), _dt(out),
                                                    native.stream_ptr()))
    return out


def tied_gate_scan(proj, q_col0, f_col0, v_col0, f_bias, lower, seq_desc, n_seqs, state_S, H, d, dv):
    """Linear attention whose forget gate also sets the write strength, over every sequence's new tokens -> fp32 [T, H dv] read-outs:
    q = silu(proj[:, q_col0:]), f = lower + (1 - lower) sigmoid(proj[:, f_col0:] + f_bias), S <- diag(f) S + (1 - f) v^T, o = S^T q."""
    T = proj.shape[0]
    assert proj.stride(1) == 1 and f_bias.dtype == torch.float32 and lower.dtype == torch.float32 and f_bias.numel() == H * d == lower.numel()
    out = torch.empty(T, H * dv, dtype=torch.float32, device=proj.device)
    native.check(native.lib().dsb200_tied_gate_scan(native.ptr(proj), proj.stride(0), q_col0, f_col0, v_col0, native.ptr(f_bias), native.ptr(lower),
                                                    native.ptr(seq_desc), native.ptr(state_S), native.ptr(out), n_seqs, H, d, dv, _dt(proj),
                                                    native.stream_ptr()))
    return out


# ---- kernels of csrc/ragged/sink_attention_ops.cu: per-head query / key norms with a partial rotate-half rotation, weightless value norm,
# and causal attention with a soft cap on the scores and a sink in the softmax.  Keys and values are addressed as planes
# (tensor, elements between consecutive blocks): `cache_planes` turns the engine's cache tensors into that form.
def cache_planes(k_cache, v_cache=None):
    """((keys, block stride), (values, block stride)).  One tensor [blocks, 2, block_size, G, d] holds both planes (d = dv); two tensors
    [blocks, block_size, G, d] and [blocks, block_size, G, dv] hold one each."""
    if v_cache is None:
        assert k_cache.dim() == 5 and k_cache.shape[1] == 2 and k_cache.is_contiguous()
        return (k_cache, k_cache.stride(0)), (k_cache[:, 1], k_cache.stride(0))
    assert k_cache.dim() == 4 and v_cache.dim() == 4 and k_cache.is_contiguous() and v_cache.is_contiguous()
    return (k_cache, k_cache.stride(0)), (v_cache, v_cache.stride(0))


def head_norm_rotary_append(proj, q_col0, k_col0, v_col0, wq, wk, freq, mag, tok_seq, tok_pos, block_table, block_size, k_plane, v_plane, q_out,
                            H, G, d, dv, rot_dims, eps, norm_v=True, row=None):
    """Per-head RMS norm (weights wq / wk [d], shared by the heads) and rotation of the first rot_dims entries (entry i with entry
    i + rot_dims / 2, angle pos * freq[i], cosine and sine times `mag`) of the query / key heads in columns q_col0 / k_col0 of proj; value
    heads (columns v_col0) divided by their own root mean square when `norm_v`.  Queries -> q_out [T, >= H d]; keys / values -> their planes.
    `row`: every query head, cached key head and cached value head occupies this many entries (>= d and dv), zeros behind its own."""
    T = proj.shape[0]
    (kc, ks), (vc, vs) = k_plane, v_plane
    assert proj.stride(1) == 1 and q_out.stride(1) == 1 and q_out.dtype == proj.dtype == kc.dtype == vc.dtype
    native.check(native.lib().dsb200_head_norm_rotary_append(native.ptr(proj), proj.stride(0), q_col0, k_col0, v_col0, native.ptr(wq), native.ptr(wk),
                                                             native.ptr(freq), float(mag), native.ptr(tok_seq), native.ptr(tok_pos),
                                                             native.ptr(block_table), block_table.stride(0), int(block_size), native.ptr(kc), ks,
                                                             native.ptr(vc), vs, native.ptr(q_out), q_out.stride(0), T, H, G, d, dv, int(rot_dims),
                                                             float(eps), int(norm_v), int(row or d), int(row or d), int(row or dv), _dt(proj),
                                                             native.stream_ptr()))
    return q_out


def sink_attention(q, k_plane, v_plane, tok_seq, tok_pos, block_table, block_size, out, H, G, d, dv, scale, softcap=0.0, sink=1.0):
    """CUDA-core causal attention over the paged planes: weights exp(s_j) / (sink + sum exp(s_j)) with s_j = scale q . k_j, soft-capped
    as softcap tanh(s_j / softcap) when softcap > 0.  q [T, >= H d], out [T, >= H dv] (views with unit column stride)."""
    T = q.shape[0]
    (kc, ks), (vc, vs) = k_plane, v_plane
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == kc.dtype == vc.dtype == out.dtype
    native.check(native.lib().dsb200_sink_attention(native.ptr(q), q.stride(0), native.ptr(kc), ks, native.ptr(vc), vs, native.ptr(tok_seq),
                                                    native.ptr(tok_pos), native.ptr(block_table), block_table.stride(0), int(block_size),
                                                    native.ptr(out), out.stride(0), T, H, G, d, dv, float(scale), float(softcap), float(sink),
                                                    _dt(q), native.stream_ptr()))
    return out


def paged_flash_sink_ok(q, cache, out, H, G, d, dv):
    """Whether the tensor-core kernels take this attention: bf16, equal key / value head sizes of 64 / 128 in one two-plane cache tensor, a
    q:kv head ratio dividing 128, cache blocks dividing 128, 16-byte aligned rows."""
    return (q.is_cuda and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and d == dv and d in (64, 128) and
            cache.dim() == 5 and H % G == 0 and 128 % (H // G) == 0 and cache.shape[2] >= 8 and 128 % cache.shape[2] == 0 and q.stride(0) % 8 == 0 and
            out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and os.environ.get("DSB200_PAGED_FLASH", "1") != "0")


def paged_flash_sink(q, cache, tok_seq, tok_pos, block_table, out, H, G, d, scale, softcap=0.0, sink=1.0, decode=False, max_context=None, n_splits=None,
                     sink_logit=None, r1=None, r2=None, part=0):
    """`sink_attention` / `sink_attention_ex` on the tensor cores (csrc/attn/paged_flash.cu: TMA pages through the block table, S / P / O in
    TMEM) for a two-plane cache [blocks, 2, block_size, G, d].  `decode`: (almost) one token per sequence -- the small-atom kernel.
    sink_logit / r1, r2 (fp32 [H]) / part: learned sinks, the logarithmic distance term and the mask by parts, as in `sink_attention_ex`."""
    for p in (sink_logit, r1, r2):
        assert p is None or (p.dtype == torch.float32 and p.numel() == H and p.is_cuda)
    T = q.shape[0]
    bs, group = cache.shape[2], H // G
    decode = bool(decode) and d == 128 and 16 % group == 0 and os.environ.get("DSB200_PAGED_DECODE", "1") != "0"
    nt = (16 if decode else 128) // group
    max_atoms = max(1, min(T, (T + nt - 1) // nt + block_table.shape[0]))
    if n_splits is None:
        pages = -(-(max_context if max_context is not None else block_table.shape[1] * bs) // 128)
        n_splits = _pick_splits(T, H, d, max_atoms * G, pages, page_us=0.45 if decode else 0.7)
    nbytes = native.lib().dsb200_paged_flash_scratch_bytes(T, H, d, max_atoms, n_splits)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    native.check(native.lib().dsb200_paged_flash_sink_ex(native.ptr(q), q.stride(0), native.ptr(cache), native.ptr(out), out.stride(0), native.ptr(tok_seq),
                                                         native.ptr(tok_pos), native.ptr(block_table), T, H, G, d, bs, block_table.shape[1],
                                                         cache.shape[0], float(scale), float(softcap), float(sink), native.ptr(sink_logit),
                                                         native.ptr(r1), native.ptr(r2), int(part), max_atoms, n_splits, native.ptr(scratch),
                                                         int(decode), native.stream_ptr()), 2 + (n_splits > 1))
    return out


# ---- blocks whose norm sits behind the residual sum, xIELU, scalar head gates (csrc/ragged/latent_ops.cu); attention inputs behind a short
# convolution, low-rank attention with a shared rotated key part, attention with learned sinks / a distance term / a mask by parts
# (csrc/ragged/sink_attention_ops.cu); the minimal gated recurrence (csrc/ragged/recurrent_ops.cu)
native.register_sigs({
    "dsb200_post_sum_norm": "pp i ppp p i l i ff p",
    "dsb200_xielu": "p l p l i p i p",
    "dsb200_gate_heads_scalar": "pp l p l iii i p",
    "dsb200_mingru_scratch_floats": "iii",
    "dsb200_mingru_scan": "p l iii pp pp p p l iii i p i p",
    "dsb200_sink_attention_ex": "p l l p l i p l i ppp ii p l l iiiii fff ppp i i p",
    "dsb200_latent_rotary_append": "p l ii pp ppp ii p i iiiii i f i p",
    "dsb200_conv_head_norm_append": "p l i pppp p pppp ii p l p l p l p p p iiiiii f iii i p",
}, restype_long=("dsb200_mingru_scratch_floats", ))


def post_sum_norm(x, y=None, w=None, alpha=1.0, eps=1e-6, y32=None, bias=None, out_dtype=torch.bfloat16):
    """On the fp32 residual x [T, dim], in place: x <- rms_norm(alpha x + y + y32 + bias) * w, eps inside the root (y in an activation dtype,
    y32 fp32, bias fp32 [dim]; each optional).  Returns the new stream in `out_dtype` (x itself for fp32)."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.is_cuda and w is not None and w.dtype == torch.float32
    if y is not None:
        assert y.shape == x.shape
        y = y if y.is_contiguous() else y.contiguous()  # a GEMM output whose rows were padded to the TMA stride (odd widths only)
    assert y32 is None or (y32.shape == x.shape and y32.dtype == torch.float32 and y32.is_contiguous())
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == x.shape[1])
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device) if out_dtype != torch.float32 else None
    native.check(native.lib().dsb200_post_sum_norm(native.ptr(x), native.ptr(y), _dt(y) if y is not None else 0, native.ptr(y32), native.ptr(bias),
                                                   native.ptr(w), native.ptr(out), _DT[out_dtype], x.shape[0], x.shape[1], float(alpha), float(eps),
                                                   native.stream_ptr()))
    return out if out is not None else x


def xielu_coefficients(p, q):
    """(softplus(p), 1/2 + softplus(q)) as the fp32 pair the kernel reads, formed in double precision."""
    return torch.tensor([math.log1p(math.exp(float(p))), 0.5 + math.log1p(math.exp(float(q)))], dtype=torch.float32)


def xielu(u, coef):
    """u [rows, F] (unit column stride) -> [rows, F]: z > 0: coef[0] z^2 + z / 2; z <= 0: coef[1] (exp(z) - 1 - z) + z / 2; coef fp32 [2] on the device."""
    assert u.stride(1) == 1 and coef.dtype == torch.float32 and coef.numel() == 2 and coef.is_cuda
    out = torch.empty(u.shape, dtype=u.dtype, device=u.device)
    native.check(native.lib().dsb200_xielu(native.ptr(u), u.stride(0), native.ptr(out), u.shape[0], u.shape[1], native.ptr(coef), _dt(u),
                                           native.stream_ptr()))
    return out


def gate_heads_scalar(a, gate, out=None):
    """a [H, T, dv] (contiguous result of a per-head batched GEMM), gate [T, >= H] (unit column stride): one number per token and head ->
    [T, H * dv]: the heads side by side, each times the sigmoid of its number."""
    H, T, dv = a.shape
    assert a.is_contiguous() and gate.shape[0] == T and gate.stride(1) == 1 and gate.dtype == a.dtype
    if out is None:
        out = torch.empty(T, H * dv, dtype=a.dtype, device=a.device)
    assert out.stride(1) == 1 and out.dtype == a.dtype
    native.check(native.lib().dsb200_gate_heads_scalar(native.ptr(a), native.ptr(gate), gate.stride(0), native.ptr(out), out.stride(0), T, H, dv, _dt(a),
                                                       native.stream_ptr()))
    return out


def mingru_scan(proj, z_col0, x_col0, g_col0, z_bias, x_bias, tok_seq, seq_desc, n_seqs, state, out, W, pieces=None):
    """Minimal gated recurrence over every sequence's new tokens: z = sigmoid(proj[:, z_col0:] + z_bias), u = proj[:, x_col0:] + x_bias,
    S <- (1 - z) S + z (u + 1/2 if u >= 0 else sigmoid(u)), out = S silu(proj[:, g_col0:]); state fp32 [slots, W] (a sequence at position 0
    starts from zero).  `pieces`: cut the batch's rows into pieces that are walked side by side (default: when there are more rows than
    sequences x 64); else one thread per (sequence, channel) walks its tokens in order."""
    T = proj.shape[0]
    assert proj.stride(1) == 1 and out.stride(1) == 1 and out.dtype == proj.dtype and state.dtype == torch.float32 and state.shape[1] == W
    assert z_bias.dtype == torch.float32 and x_bias.dtype == torch.float32 and z_bias.numel() == W == x_bias.numel()
    if pieces is None:
        pieces = T > 64 * n_seqs
    scratch = None
    if pieces:
        scratch = torch.empty(native.lib().dsb200_mingru_scratch_floats(T, n_seqs, W), dtype=torch.float32, device=proj.device)
    native.check(native.lib().dsb200_mingru_scan(native.ptr(proj), proj.stride(0), z_col0, x_col0, g_col0, native.ptr(z_bias), native.ptr(x_bias),
                                                 native.ptr(tok_seq), native.ptr(seq_desc), native.ptr(state), native.ptr(out), out.stride(0), T, n_seqs,
                                                 W, int(bool(pieces)), native.ptr(scratch), _dt(proj), native.stream_ptr()), 3 if pieces else 1)
    return out


def sink_attention_ex(q, q_head_stride, k_plane, k_row, v_plane, v_row, tok_seq, tok_pos, block_table, block_size, out, out_head_stride, H, G, d, dv,
                      scale, softcap=0.0, sink=0.0, sink_logit=None, r1=None, r2=None, part=0):
    """`sink_attention` with learned sinks (sink_logit fp32 [H]: exp of it joins the head's denominator), a distance term (r1, r2 fp32 [H]: the
    score of key j loses r1 ln(1 + r2 (pos - j))), a mask by parts (`part` > 0: a query sees only the keys of its own part of that many
    positions, counted from the sequence's start) and free strides: q / out are addressed [t * stride(0) + h * head_stride + c], a cached
    key / value head starts every k_row / v_row elements of its token's row."""
    T = q.shape[0]
    (kc, ks), (vc, vs) = k_plane, v_plane
    assert q.dtype == kc.dtype == vc.dtype == out.dtype
    for p in (sink_logit, r1, r2):
        assert p is None or (p.dtype == torch.float32 and p.numel() == H and p.is_cuda)
    native.check(native.lib().dsb200_sink_attention_ex(native.ptr(q), q.stride(0), int(q_head_stride), native.ptr(kc), ks, int(k_row), native.ptr(vc), vs,
                                                       int(v_row), native.ptr(tok_seq), native.ptr(tok_pos), native.ptr(block_table),
                                                       block_table.stride(0), int(block_size), native.ptr(out), out.stride(0), int(out_head_stride), T,
                                                       H, G, d, dv, float(scale), float(softcap), float(sink), native.ptr(sink_logit), native.ptr(r1),
                                                       native.ptr(r2), int(part), _dt(q), native.stream_ptr()))
    return out


def latent_rotary_append(proj, q_col0, kv_col0, wkv, freq, tok_seq, tok_pos, block_table, cache, H, d, dr, R, rot_dims, eps):
    """proj [T, N] holds the H query heads (d plain + dr rotated entries each) from q_col0 and the low-rank row (R + dr entries) from kv_col0.
    The rotated parts of the query heads are rotated in place (rotate-half pairs over the first rot_dims of the dr entries, angle pos * freq[i]);
    the RMS-normed (weight wkv) first R entries of the low-rank row and its rotated last dr entries go to the token's row of
    cache [blocks, block_size, row >= R + dr] (zeros behind)."""
    assert proj.stride(1) == 1 and cache.is_contiguous() and cache.dim() == 3 and cache.dtype == proj.dtype
    native.check(native.lib().dsb200_latent_rotary_append(native.ptr(proj), proj.stride(0), q_col0, kv_col0, native.ptr(wkv), native.ptr(freq),
                                                          native.ptr(tok_seq), native.ptr(tok_pos), native.ptr(block_table), block_table.stride(0),
                                                          cache.shape[1], native.ptr(cache), cache.shape[2], proj.shape[0], H, d, dr, R, int(rot_dims),
                                                          float(eps), _dt(proj), native.stream_ptr()))


def conv_head_norm_append(proj, col0, bias, conv_w, wq, wk, state, seq_desc, tok_seq, tok_pos, block_table, block_size, k_plane, v_plane, q_out,
                          H, G, d, dv, taps, eps, v_other=None, mix=None, v_own=None, row=None):
    """Query heads [H d], key heads [G d] and value heads [G dv] lie side by side in proj from column col0.  Every channel gets its bias
    (fp32, or None) and a short causal convolution (conv_w fp32 [taps, channels]; rows before this step's come from state
    [slots, taps - 1, channels], rows before the sequence are zeros); query / key heads are RMS-normed with wq / wk [d] (shared by the heads);
    queries -> q_out, keys / values -> their planes.  v_own ([T, G dv]): receives the convolved values; v_other + mix (fp32 [1]): the cached
    value is (1 - mix) v + mix v_other.  `row`: heads are padded with zeros to this width."""
    (kc, ks), (vc, vs) = k_plane, v_plane
    assert proj.stride(1) == 1 and q_out.stride(1) == 1 and q_out.dtype == proj.dtype == kc.dtype == vc.dtype
    for v in (v_other, v_own):
        assert v is None or (v.is_contiguous() and v.dtype == proj.dtype and v.shape == (proj.shape[0], G * dv))
    assert state is None or (state.dtype == proj.dtype and state.is_contiguous())
    assert conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape == (taps, (H + G) * d + G * dv)
    native.check(native.lib().dsb200_conv_head_norm_append(native.ptr(proj), proj.stride(0), col0, native.ptr(bias), native.ptr(conv_w), native.ptr(wq),
                                                           native.ptr(wk), native.ptr(state), native.ptr(seq_desc), native.ptr(tok_seq),
                                                           native.ptr(tok_pos), native.ptr(block_table), block_table.stride(0), int(block_size),
                                                           native.ptr(kc), ks, native.ptr(vc), vs, native.ptr(q_out), q_out.stride(0),
                                                           native.ptr(v_other), native.ptr(mix), native.ptr(v_own), proj.shape[0], H, G, d, dv, int(taps),
                                                           float(eps), int(row or d), int(row or d), int(row or dv), _dt(proj), native.stream_ptr()))
    return q_out
