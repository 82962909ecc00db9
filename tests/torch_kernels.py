"""Plain PyTorch restatement of every kernel, with the signatures of
``deterministic_inference_b200.kernels.ops``.

Two uses, both in tests only: (1) the float32 reference each CUDA kernel is
compared with; (2) patched over ``ops`` (fixture ``torch_ops`` in conftest.py) so
that the engine's host logic (cache, batch building, step function, scheduler)
can be exercised on a machine without a GPU.  The package never imports this
file.

Formulas: the reference project's kernels, cited per function (paths relative to
Aayaan-Sahu/deterministic-inference).
"""

from __future__ import annotations

import torch


def embedding(ids, table):
    """sid/model/qwen3.py:93"""
    return table[ids.long()]


def patch_token_ids(input_ids, patch_dst, patch_src, prev_tokens):
    ok = patch_dst >= 0
    input_ids[patch_dst[ok].long()] = prev_tokens[patch_src[ok].long()]


def _rms(x32, w, eps):
    """sid/kernels/rmsnorm.py:14-24"""
    var = (x32 * x32).mean(dim=-1, keepdim=True)
    return x32 * (1.0 / torch.sqrt(var + eps)) * w.float()


def rms_norm(x, weight, eps):
    return _rms(x.float(), weight, eps).to(x.dtype)


def add_rms_norm(x, residual, weight, eps):
    """In place like the kernel (sid/kernels/rmsnorm.py:27-42): the residual is
    stored rounded, the norm reads the unrounded sum."""
    s = x.float() + residual.float()
    residual.copy_(s.to(residual.dtype))
    x.copy_(_rms(s, weight, eps).to(x.dtype))
    return x, residual


def qk_norm_rope_cache(qkv, num_heads, num_kv_heads, head_dim, q_norm_weight, k_norm_weight, eps,
                       cos_sin, positions, kv_cache, slot_mapping, page_size):
    """sid/model/qwen3.py:49-61, sid/kernels/rmsnorm.py:72-75, sid/kernels/rope.py:15-37,
    sid/csrc/flash_decode.cu:275-296 (cache layout [pages, 2, Hkv, page, D] is this
    package's own)."""
    t = qkv.shape[0]
    d = head_dim
    x = qkv.float()
    q = x[:, :num_heads * d].reshape(t, num_heads, d)
    k = x[:, num_heads * d:(num_heads + num_kv_heads) * d].reshape(t, num_kv_heads, d)
    v = x[:, (num_heads + num_kv_heads) * d:].reshape(t, num_kv_heads, d)
    if q_norm_weight is not None:
        q = _rms(q, q_norm_weight, eps)
    if k_norm_weight is not None:
        k = _rms(k, k_norm_weight, eps)
    if cos_sin is not None:
        r = cos_sin.shape[1]
        half = r // 2
        tab = cos_sin[positions.long()]
        cos, sin = tab[:, None, :half], tab[:, None, half:]

        def rot(y):
            y1, y2, rest = y[..., :half], y[..., half:r], y[..., r:]
            return torch.cat([y1 * cos - y2 * sin, y2 * cos + y1 * sin, rest], dim=-1)
        q, k = rot(q), rot(k)
    if kv_cache is not None:
        sm = slot_mapping.long()
        ok = sm >= 0
        page, off = sm[ok] // page_size, sm[ok] % page_size
        kv_cache[page, 0, :, off, :] = k[ok].to(kv_cache.dtype)
        kv_cache[page, 1, :, off, :] = v[ok].to(kv_cache.dtype)
    return q.to(qkv.dtype).contiguous()


def reshape_and_cache(k, v, kv_cache, slot_mapping):
    """sid/csrc/flash_decode.cu:275-296"""
    page_size = kv_cache.shape[3]
    sm = slot_mapping.long()
    ok = sm >= 0
    page, off = sm[ok] // page_size, sm[ok] % page_size
    kv_cache[page, 0, :, off, :] = k[ok]
    kv_cache[page, 1, :, off, :] = v[ok]


def paged_attention(q, kv_cache, meta, scale, window=None, defer=False):
    """Every token against the cached keys of its sequence, causal by absolute
    position, float32 softmax (sid/kernels/extend_attention.py:80-109,
    tests/conftest.py:11-32)."""
    t, hq, d = q.shape
    _, _, hkv, page_size, _ = kv_cache.shape
    group = hq // hkv
    out = torch.empty(t, hq, d, dtype=torch.float32, device=q.device)
    token_seq = meta.token_seq.tolist()
    positions = meta.positions.tolist()
    bt = meta.block_table
    for i in range(t):
        s, p = token_seq[i], positions[i]
        first = max(0, p - window + 1) if window else 0
        keys = torch.arange(first, p + 1, device=q.device)
        pages = bt[s, (keys // page_size)].long()
        offs = keys % page_size
        k = kv_cache[pages, 0, :, offs, :].float()      # [n, Hkv, D]
        v = kv_cache[pages, 1, :, offs, :].float()
        for h in range(hq):
            kh = h // group
            sc = (k[:, kh] @ q[i, h].float()) * scale
            out[i, h] = torch.softmax(sc, dim=-1) @ v[:, kh]
    return out.to(q.dtype)


def silu_mul(gate_up):
    """sid/model/qwen3.py:85-86"""
    i = gate_up.shape[1] // 2
    g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
    return (g * torch.sigmoid(g) * u).to(gate_up.dtype)


def gated_linear(x, w_gate_up):
    """sid/model/qwen3.py:84-86"""
    return silu_mul(linear(x, w_gate_up))


def gather_rows(x, index):
    """sid/model/qwen3.py:113"""
    if hasattr(x, "eps") and hasattr(x, "weight"):       # a norm works row by row: gather first
        return type(x)(gather_rows(x.x, index), x.weight, x.eps)
    if hasattr(x, "terms"):
        x = _plain(x)
    return x[index.long()].contiguous()


def linear(x, weight, out_dtype=None):
    """sid/model/qwen3.py:38 (float32 accumulation)."""
    y = x.float() @ weight.float().T
    return y.to(out_dtype or x.dtype)     # (x is a norm's output or a kernel's: a tensor)


def argmax(logits):
    """sid/engine/sampler.py:36-38"""
    return torch.argmax(logits, dim=-1).to(torch.int32)


def seeded_gumbel(seeds, sample_pos, num_cols):
    """sid/engine/sampler.py:22-29"""
    step = seeds * 19349663 ^ sample_pos * 73856093
    cols = torch.arange(num_cols, dtype=torch.int64, device=seeds.device)
    hashed = step.unsqueeze(-1) * 8589934591 ^ cols * 479001599
    u = (hashed % (2 ** 24)).float() / (2 ** 24)
    return -torch.log(-torch.log(u + 1e-10) + 1e-10)


def gumbel_scores(logits, temperatures, seeds, sample_positions, keep=None):
    """log(p + 1e-10) + gumbel for kept ids, -inf elsewhere (sid/engine/sampler.py:44-66)."""
    temps = torch.where(temperatures > 0, temperatures, torch.ones_like(temperatures))
    probs = torch.softmax(logits / temps.unsqueeze(-1), dim=-1)
    logp = torch.log(probs + 1e-10)
    if keep is not None:
        logp = torch.where(keep.bool(), logp, torch.full_like(logp, float("-inf")))
    return logp + seeded_gumbel(seeds, sample_positions, logits.shape[1])


def keep_mask(logits, temperatures, top_ks, top_ps):
    """uint8 [R, V]: 1 for ids that survive top-k / top-p by the reference's rule
    (sid/engine/sampler.py:44-62): probabilities sorted descending; a token is dropped when
    the mass before it exceeds top_p or its rank reaches top_k; the first stays."""
    temps = torch.where(temperatures > 0, temperatures, torch.ones_like(temperatures))
    p = torch.softmax(logits / temps.unsqueeze(-1), dim=-1)
    order = torch.argsort(p, dim=-1, descending=True, stable=True)
    sorted_p = torch.gather(p, -1, order)
    before = torch.cumsum(sorted_p, dim=-1) - sorted_p
    rank = torch.arange(p.shape[-1], device=p.device).unsqueeze(0)
    limit = torch.where(top_ks > 0, top_ks, torch.full_like(top_ks, p.shape[-1])).unsqueeze(-1)
    stays = (before <= top_ps.unsqueeze(-1)) & (rank < limit)
    stays[:, 0] = True
    mask = torch.zeros_like(stays)
    mask.scatter_(-1, order, stays)
    return mask.to(torch.uint8).contiguous()


def gumbel_sample(logits, temperatures, seeds, sample_positions, keep=None, top_ks=None, top_ps=None):
    """sid/engine/sampler.py:32-69"""
    if top_ks is not None:
        keep = keep_mask(logits, temperatures, top_ks, top_ps)
    greedy = torch.argmax(logits, dim=-1)
    sampled = torch.argmax(gumbel_scores(logits, temperatures, seeds, sample_positions, keep), dim=-1)
    return torch.where(temperatures > 0, sampled, greedy).to(torch.int32)


# ---- kernels of models with a float32 residual stream, attention without a softmax and a
# ---- delta-rule recurrence (each from its equations; signatures of ``ops``)

def _plain(x):
    """A float32 tensor of a weighted sum that is not added up yet, or of a tensor."""
    if hasattr(x, "eps") and hasattr(x, "weight"):       # a part's output under its post norm
        return _rms(_plain(x.x), x.weight, x.eps)
    if hasattr(x, "parts"):                               # split-k partial products
        total = x.parts[0].float().clone()
        for i in range(1, x.parts.shape[0]):
            total += x.parts[i].float()
        return total
    if hasattr(x, "terms"):
        total = None
        for a, t in x.terms:
            total = a * _plain(t) if total is None else total + a * _plain(t)
        return total
    return x.float()


def embedding_positions(ids, positions, table, pos_table):
    return table[ids.long()].float() + pos_table[positions[:ids.shape[0]].long()].float()


def stream_rms_norm(stream, weight, eps, out_dtype, add=None):
    if add is not None:
        stream += _plain(add)
    return _rms(stream, weight, eps).to(out_dtype)


def xielu(z, alpha_p, alpha_n, out_dtype):
    z = _plain(z)
    pos = alpha_p * z * z + 0.5 * z
    neg = alpha_n * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg).to(out_dtype)


def scale_(x, a):
    x.mul_(a)
    return x


def softcap_(logits, cap):
    logits.copy_(cap * torch.tanh(logits / cap))
    return logits


def qkv_bias_cache(qkv, bias, num_heads, num_kv_heads, head_dim, v_head_dim, kv_cache, slot_mapping,
                   page_size, out_dtype):
    x = _plain(qkv)
    if bias is not None:
        x = x + bias
    t = x.shape[0]
    nq, nk = num_heads * head_dim, num_kv_heads * head_dim
    if kv_cache is not None:
        flat = kv_cache.view(kv_cache.shape[0], -1)
        k = x[:, nq:nq + nk].view(t, num_kv_heads, head_dim).to(out_dtype)
        v = x[:, nq + nk:].view(t, num_kv_heads, v_head_dim).to(out_dtype)
        v_base = num_kv_heads * page_size * head_dim
        for i, slot in enumerate(slot_mapping.tolist()[:t]):
            if slot < 0:
                continue
            page, off = divmod(slot, page_size)
            for g in range(num_kv_heads):
                a = (g * page_size + off) * head_dim
                flat[page, a:a + head_dim] = k[i, g]
                a = v_base + (g * page_size + off) * v_head_dim
                flat[page, a:a + v_head_dim] = v[i, g]
    return x[:, :nq].reshape(t, num_heads, head_dim).to(out_dtype)


def sigmoid_attention(q, kv_cache, meta, scale, head_bias, v_head_dim, page_size, window=None, keep_first=0):
    t, hq, d = q.shape
    flat = kv_cache.view(kv_cache.shape[0], -1)
    hkv = flat.shape[1] // (page_size * (d + v_head_dim))
    keys_of = flat[:, :hkv * page_size * d].view(-1, hkv, page_size, d)
    values_of = flat[:, hkv * page_size * d:].view(-1, hkv, page_size, v_head_dim)
    out = torch.zeros(t, hq, v_head_dim, dtype=torch.float32)
    seqs, positions = meta.token_seq.tolist(), meta.positions.tolist()
    for i in range(t):
        p = positions[i]
        js = [j for j in range(p + 1) if not window or p - j < window or j < keep_first]
        idx = torch.tensor(js)
        pages = meta.block_table[seqs[i], idx // page_size].long()
        k = keys_of[pages, :, idx % page_size].float()        # [n, Hkv, D]
        v = values_of[pages, :, idx % page_size].float()
        for h in range(hq):
            g = h // (hq // hkv)
            sc = (k[:, g] @ q[i, h].float()) * scale
            if head_bias is not None:
                sc = sc + head_bias[h]
            out[i, h] = torch.sigmoid(sc) @ v[:, g]
    return out.to(q.dtype)


def delta_rule(proj, w2_t, w0, a_bias, norm_weight, state, step, num_heads, head_dim, lora_rank,
               decay_scale, key_eps, norm_eps, out_dtype):
    x = _plain(proj)
    t, hd = x.shape[0], num_heads * head_dim
    shape = (t, num_heads, head_dim)
    r, k, v, g = (x[:, i * hd:(i + 1) * hd].reshape(shape) for i in range(4))
    a = x[:, 4 * hd:5 * hd]
    if a_bias is not None:
        a = a + a_bias
    a = torch.sigmoid(a).reshape(shape)
    w = torch.exp(-decay_scale * torch.sigmoid(torch.tanh(x[:, 5 * hd:]) @ w2_t.float() + w0)).reshape(shape)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + key_eps)
    o = torch.zeros(shape)
    cu, slots = step.cu_q_lens.tolist(), step.state_slots.tolist()
    for b in range(len(slots)):
        # state slot 0 is no request's: a sequence on it starts from zero and leaves nothing
        s = state[slots[b]] if slots[b] else torch.zeros_like(state[0])
        for i in range(cu[b], cu[b + 1]):
            us = torch.einsum("hk,hkv->hv", u[i], s)
            s = w[i][:, :, None] * s - (a[i] * u[i])[:, :, None] * us[:, None, :] + k[i][:, :, None] * v[i][:, None, :]
            o[i] = torch.einsum("hkv,hk->hv", s, r[i])
        if slots[b]:
            state[slots[b]] = s
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + norm_eps)
    return (o.reshape(t, hd) * norm_weight * torch.sigmoid(g.reshape(t, hd))).to(out_dtype)


# ---- softmax attention with a mask kind, latent rows, the float32 stream's other kernels

def embedding_scaled(ids, table, scale):
    return table[ids.long()].float() * scale


def stream_add_(stream, term=None, bias=None, norm_weight=None, norm_eps=0.0, out=None):
    if term is not None:
        stream += _plain(term)
    if bias is not None:
        stream += bias
    if out is not None:
        out.copy_((stream if norm_weight is None else _rms(stream, norm_weight, norm_eps)).to(out.dtype))
    return stream


def stream_read(stream, term, out_dtype):
    if term is not None:
        stream += _plain(term)
    return stream if out_dtype == torch.float32 else stream.to(out_dtype)


def limited_gate(gate_up, limit, alpha, out_dtype):
    x = _plain(gate_up)
    i = x.shape[1] // 2
    g, u = torch.clamp(x[:, :i], max=limit), torch.clamp(x[:, i:], -limit, limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(out_dtype)


def _rotate_first(x, positions, freq, rot):
    """x [T, heads, D] float32: elements i and i + rot / 2 (i < rot / 2) turned by position * freq[i]."""
    if freq is None or rot == 0:
        return x
    half = rot // 2
    a = positions[:x.shape[0]].float()[:, None] * freq[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:rot]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., rot:]], dim=-1)


def _rotate_pairs(x, positions, freq, rot):
    """x [T, heads, D] float32: elements 2i and 2i + 1 (i < rot / 2) turned by position * freq[i]."""
    if freq is None or rot == 0:
        return x
    a = positions[:x.shape[0]].float()[:, None] * freq[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:rot:2], x[..., 1:rot:2]
    out = x.clone()
    out[..., 0:rot:2] = u * c - v * s
    out[..., 1:rot:2] = v * c + u * s
    return out


def attn_prepare(proj, num_heads, num_kv_heads, head_dim, v_head_dim, q_norm_weight, k_norm_weight, eps, freq,
                 rotary_dim, positions, kv_cache, slot_mapping, page_size, out_dtype, bias=None, norm_scope="head",
                 rotary_layout="halves", conv_weight=None, conv_state=None, step=None):
    t = proj.shape[0]
    nq, nk, nv = num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * v_head_dim
    x = _plain(proj)[:, :nq + nk + nv]
    if bias is not None:
        x = x + bias
    if conv_weight is not None:
        taps = conv_weight.shape[1]
        tail = conv_state.view(conv_state.shape[0], taps - 1, nq + nk + nv) if taps > 1 \
            else torch.zeros(int(step.state_slots.max()) + 1, 0, nq + nk + nv)
        x = _conv_with_tail(x.contiguous(), conv_weight, tail, step.cu_q_lens.tolist(), step.state_slots.tolist())
    else:
        x = x.to(out_dtype).float()
    q, k = x[:, :nq], x[:, nq:nq + nk]
    if norm_scope == "head":
        q, k = q.reshape(t, num_heads, head_dim), k.reshape(t, num_kv_heads, head_dim)
    if q_norm_weight is not None:
        q, k = _rms(q, q_norm_weight, eps), _rms(k, k_norm_weight, eps)
    q, k = q.reshape(t, num_heads, head_dim), k.reshape(t, num_kv_heads, head_dim)
    v = x[:, nq + nk:nq + nk + nv].reshape(t, num_kv_heads, v_head_dim)
    rotate = _rotate_pairs if rotary_layout == "pairs" else _rotate_first
    q, k = rotate(q, positions, freq, rotary_dim), rotate(k, positions, freq, rotary_dim)
    if kv_cache is not None:
        flat = kv_cache.view(kv_cache.shape[0], -1)
        v_base = num_kv_heads * page_size * head_dim
        for i, slot in enumerate(slot_mapping.tolist()[:t]):
            if slot < 0:
                continue
            page, off = divmod(slot, page_size)
            for g in range(num_kv_heads):
                a = (g * page_size + off) * head_dim
                flat[page, a:a + head_dim] = k[i, g].to(out_dtype)
                a = v_base + (g * page_size + off) * v_head_dim
                flat[page, a:a + v_head_dim] = v[i, g].to(out_dtype)
    return q.to(out_dtype)


def latent_prepare(proj, num_heads, plain_dim, rot_dim, rank, latent_norm_weight, eps, freq, positions, kv_cache,
                   slot_mapping, page_size, out_dtype):
    x = _plain(proj).to(out_dtype).float()
    t = x.shape[0]
    nq = num_heads * (plain_dim + rot_dim)
    q_rot = x[:, :nq].reshape(t, num_heads, plain_dim + rot_dim)[:, :, plain_dim:]
    q = torch.zeros(t, num_heads, rank + rot_dim, dtype=out_dtype)
    q[:, :, rank:] = _rotate_first(q_rot, positions, freq, rot_dim).to(out_dtype)
    if kv_cache is not None:
        latent = _rms(x[:, nq:nq + rank], latent_norm_weight, eps)
        k_rot = _rotate_first(x[:, None, nq + rank:], positions, freq, rot_dim)[:, 0]
        rows = kv_cache.view(-1, rank + rot_dim)
        for i, slot in enumerate(slot_mapping.tolist()[:t]):
            if slot >= 0:
                rows[slot] = torch.cat([latent[i], k_rot[i]]).to(out_dtype)
    return q


def heads_linear(x, weight, out):
    out.copy_(torch.einsum("mhk,hkn->mhn", x.float(), weight.float()).to(out.dtype))
    return out


def masked_attention(q, kv_cache, meta, scale, num_kv_heads, v_head_dim, page_size, mask="causal", mask_size=None,
                     sink=None, gate=None, gate_col=0, values_in_keys=False, keep_first=0, softcap=None):
    t, hq, dk = q.shape
    flat = kv_cache.view(kv_cache.shape[0], -1)
    keys_of = flat[:, :num_kv_heads * page_size * dk].view(-1, num_kv_heads, page_size, dk)
    values_of = None if values_in_keys else \
        flat[:, num_kv_heads * page_size * dk:].view(-1, num_kv_heads, page_size, v_head_dim)
    out = torch.zeros(t, hq, v_head_dim, dtype=torch.float32)
    seqs, positions = meta.token_seq.tolist(), meta.positions.tolist()
    group = hq // num_kv_heads
    g_all = None if gate is None else _plain(gate).to(q.dtype).float()
    for i in range(t):
        p = positions[i]
        lo = 0 if mask == "causal" else (max(0, p - mask_size + 1) if mask == "window" else p // mask_size * mask_size)
        js = torch.arange(lo, p + 1)
        if keep_first and lo > 0:
            js = torch.cat([torch.arange(0, min(keep_first, lo)), js])
        pages = meta.block_table[seqs[i]][js // page_size].long()
        for h in range(hq):
            k = keys_of[pages, h // group, js % page_size].float()
            v = k[:, :v_head_dim] if values_in_keys else values_of[pages, h // group, js % page_size].float()
            s = (k @ q[i, h].float()) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if sink is not None:
                s = torch.cat([s, sink[h].float().reshape(1)])
            w = torch.softmax(s, dim=0)[:js.shape[0]]
            out[i, h] = w @ v
    out = out.to(q.dtype)
    if g_all is not None:
        cols = g_all[:, gate_col:gate_col + hq * v_head_dim].reshape(t, hq, v_head_dim)
        out = (out.float() * torch.sigmoid(cols)).to(q.dtype)
    return out


# ---- gated delta rule with short convolutions, a gated linear recurrent unit, routed experts

def _conv_with_tail(x, taps_w, tail, cu, slots, conv_bias=None):
    """x [T, C] float32, taps_w [C, K], tail [slots, K - 1, C] (updated in place for slots != 0): per
    sequence of the step the causal convolution over its tokens, the K - 1 inputs before them from the
    tail."""
    k = taps_w.shape[1]
    out = torch.empty_like(x)
    for b in range(len(slots)):
        a, e = cu[b], cu[b + 1]
        if e <= a:
            continue
        old = tail[slots[b]] if slots[b] else torch.zeros_like(tail[0])
        seq = torch.cat([old, x[a:e]], dim=0)
        y = torch.zeros(e - a, x.shape[1])
        for j in range(k):
            y = y + seq[j:j + e - a] * taps_w[:, j]
        out[a:e] = y if conv_bias is None else y + conv_bias
        if slots[b] and k > 1:
            tail[slots[b]] = seq[-(k - 1):]
    return out


def gated_delta_rule(proj, conv_weight, a_log, dt_bias, norm_weight, state, step, num_heads, num_kv_heads,
                     head_dim, v_head_dim, taps, key_eps, norm_eps, out_dtype):
    x = _plain(proj)
    t, h, g, d, e = x.shape[0], num_heads, num_kv_heads, head_dim, v_head_dim
    chan = 2 * g * d + h * e
    cu, slots = step.cu_q_lens.tolist(), step.state_slots.tolist()
    n_state = h * d * e
    tail = state[:, n_state:].view(state.shape[0], taps - 1, chan)
    c = _conv_with_tail(x[:, :chan], conv_weight, tail, cu, slots)
    c = c * torch.sigmoid(c)
    q, k = c[:, :g * d].reshape(t, g, d), c[:, g * d:2 * g * d].reshape(t, g, d)
    v = c[:, 2 * g * d:].reshape(t, h, e)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + key_eps) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + key_eps)
    q, k = q.repeat_interleave(h // g, dim=1), k.repeat_interleave(h // g, dim=1)
    gate = x[:, chan:chan + h * e].reshape(t, h, e)
    beta = torch.sigmoid(x[:, chan + h * e:chan + h * e + h])
    decay = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(x[:, chan + h * e + h:chan + h * e + 2 * h] + dt_bias))
    o = torch.zeros(t, h, e)
    for b in range(len(slots)):
        s = state[slots[b], :n_state].view(h, d, e).clone() if slots[b] else torch.zeros(h, d, e)
        for i in range(cu[b], cu[b + 1]):
            s = s * decay[i][:, None, None]
            u = beta[i][:, None] * (v[i] - torch.einsum("hde,hd->he", s, k[i]))
            s = s + k[i][:, :, None] * u[:, None, :]
            o[i] = torch.einsum("hde,hd->he", s, q[i])
        if slots[b]:
            state[slots[b], :n_state] = s.reshape(-1)
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + norm_eps) * norm_weight
    return (o * gate * torch.sigmoid(gate)).reshape(t, h * e).to(out_dtype)


def gated_linear_recurrence(proj, bias, conv_weight, conv_bias, gates, gate_bias, neg_rate, state, step, width,
                            blocks, taps, out_dtype):
    x = _plain(proj) + bias
    t, c = x.shape[0], width
    cu, slots = step.cu_q_lens.tolist(), step.state_slots.tolist()
    tail = state[:, c:].view(state.shape[0], taps - 1, c)
    z = x[:, :c]
    y = 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    u = _conv_with_tail(x[:, c:], conv_weight, tail, cu, slots, conv_bias)
    ub = u.view(t, blocks, c // blocks)
    r = torch.sigmoid(torch.einsum("nbi,bio->nbo", ub, gates[0]).reshape(t, c) + gate_bias[0])
    i = torch.sigmoid(torch.einsum("nbi,bio->nbo", ub, gates[1]).reshape(t, c) + gate_bias[1])
    a = torch.exp(r * neg_rate)
    xin = torch.sqrt(1.0 - a * a) * i * u
    out = torch.empty(t, c)
    for b in range(len(slots)):
        s = state[slots[b], :c].clone() if slots[b] else torch.zeros(c)
        for j in range(cu[b], cu[b + 1]):
            s = a[j] * s + xin[j]
            out[j] = s * y[j]
        if slots[b]:
            state[slots[b], :c] = s
    return out.to(out_dtype)


def state_space(proj, conv_weight, conv_bias, a_log, dt_bias, d_skip, norm_weight, state, step, num_heads,
                head_dim, state_dim, groups, norm_groups, taps, norm_eps, out_dtype):
    x_all = _plain(proj)
    t, h, p, n, g = x_all.shape[0], num_heads, head_dim, state_dim, groups
    inner, chan = h * p, h * p + 2 * g * n
    cu, slots = step.cu_q_lens.tolist(), step.state_slots.tolist()
    n_state = h * n * p
    tail = state[:, n_state:].view(state.shape[0], taps - 1, chan)
    z = x_all[:, :inner]
    c = _conv_with_tail(x_all[:, inner:inner + chan], conv_weight, tail, cu, slots, conv_bias)
    c = c * torch.sigmoid(c)
    x = c[:, :inner].reshape(t, h, p)
    pick = torch.arange(h) // (h // g)
    bm = c[:, inner:inner + g * n].reshape(t, g, n)[:, pick]
    cm = c[:, inner + g * n:].reshape(t, g, n)[:, pick]
    dt = torch.nn.functional.softplus(x_all[:, inner + chan:inner + chan + h] + dt_bias)
    decay = torch.exp(-torch.exp(a_log) * dt)
    y = torch.zeros(t, h, p)
    for b in range(len(slots)):
        s = state[slots[b], :n_state].view(h, n, p).clone() if slots[b] else torch.zeros(h, n, p)
        for i in range(cu[b], cu[b + 1]):
            s = decay[i][:, None, None] * s + dt[i][:, None, None] * bm[i][:, :, None] * x[i][:, None, :]
            y[i] = torch.einsum("hnp,hn->hp", s, cm[i]) + d_skip[:, None] * x[i]
        if slots[b]:
            state[slots[b], :n_state] = s.reshape(-1)
    u = (y.reshape(t, inner) * (z * torch.sigmoid(z))).reshape(t, norm_groups, inner // norm_groups)
    u = u / torch.sqrt((u * u).mean(-1, keepdim=True) + norm_eps)
    return (u.reshape(t, inner) * norm_weight).to(out_dtype)


def route_experts(logits, correction, num_experts, top, group_count, group_keep, scale, eps, score="sigmoid",
                  group_top=2, normalize=True):
    z = _plain(logits)[:, :num_experts]
    s = torch.softmax(z, dim=-1) if score == "softmax" else torch.sigmoid(z)
    choice = s + correction
    per = num_experts // group_count
    by_group = choice.view(-1, group_count, per)
    group_score = by_group.topk(min(group_top, per), dim=-1).values.sum(-1)
    best = group_score.topk(group_keep, dim=-1).indices
    allowed = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, best, True)
    masked = by_group.masked_fill(~allowed[:, :, None], float("-inf")).reshape(-1, num_experts)
    ids = masked.topk(top, dim=-1).indices
    w = s.gather(1, ids)
    w = w / (w.sum(-1, keepdim=True) + eps) * scale if normalize else w * scale
    return ids.to(torch.int32), w


def routed_experts(x, ids, weights, w_gate_up, w_down, shared, logits, shared_gate_col, out_dtype):
    t, w = x.shape
    f = w_gate_up.shape[1] // 2
    out = torch.zeros(t, w)
    for i in range(t):
        for j in range(ids.shape[1]):
            e = int(ids[i, j])
            gu = w_gate_up[e].float() @ x[i].float()
            hdn = (gu[:f] * torch.sigmoid(gu[:f]) * gu[f:]).to(x.dtype).float()
            out[i] += weights[i, j] * (w_down[e].float() @ hdn)
    if shared is not None and shared_gate_col < 0:
        out = out + _plain(shared)
    elif shared is not None:
        out = out + torch.sigmoid(_plain(logits)[:, shared_gate_col:shared_gate_col + 1]) * _plain(shared)
    return out


ALL = ("state_space", "scale_", "stream_read", "gated_delta_rule", "gated_linear_recurrence", "route_experts", "routed_experts",
       "embedding_scaled", "stream_add_", "limited_gate", "attn_prepare", "latent_prepare", "heads_linear",
       "masked_attention", "embedding_positions", "stream_rms_norm", "xielu", "softcap_", "qkv_bias_cache", "sigmoid_attention",
       "delta_rule", "patch_token_ids", "embedding", "rms_norm", "add_rms_norm", "qk_norm_rope_cache", "reshape_and_cache",
       "paged_attention", "silu_mul", "gated_linear", "gather_rows", "linear", "argmax", "gumbel_sample")
