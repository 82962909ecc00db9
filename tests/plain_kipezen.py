"""A plain, slow implementation of the Kipezen design: whole sequences, no cache, no batches,
float64 by default, one function per mechanism, written from the design's equations.  It shares
no code with the package; the tests compare the package with it.

Notation: n tokens, width W.  Delta mixer: H value heads of size E, G query/key heads of size D.
Attention: H query heads, G key/value heads, key size D, value size E.  Recurrent unit: C
channels in B blocks.  ``rnd`` rounds what a bfloat16 engine stores (a yardstick for its tests);
by default nothing is rounded.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

DT = torch.float64


def read_model_dir(model_dir, dtype=DT):
    """(config dict, {name: tensor}) of a folder with config.json and model.safetensors."""
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    raw = (model_dir / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[meta["dtype"]]).reshape(meta["shape"])
        out[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, out


def _keep(x):
    return x


def as_stored_bf16(x):
    return x.to(torch.bfloat16).to(x.dtype)


# ---- small functions -------------------------------------------------------------------------

def rms(x, eps):
    """x over its root mean square over the last dimension, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def one_plus_norm(x, w, eps):
    """The layer norm of the design: the weight is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(x, taps, bias=None):
    """x [n, C], taps [C, K]: y_t = sum_j taps[:, j] * x_(t - (K - 1) + j), zeros before the start
    (the last column multiplies the current token)."""
    n, c = x.shape
    k = taps.shape[1]
    padded = torch.cat([torch.zeros(k - 1, c, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for j in range(k):
        y = y + padded[j:j + n] * taps[:, j]
    return y if bias is None else y + bias


# ---- the 'delta' mixer ----------------------------------------------------------------------------

def gated_delta_rule(q, k, v, beta, decay):
    """Per head a state S [D, E] from zero: S <- decay_t S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T;
    o_t = S^T q_t (the read-out sees the token's own write).  q, k [n, H, D]; v [n, H, E];
    beta, decay [n, H].  Returns (o [n, H, E], the last state [H, D, E])."""
    n, h, d = q.shape
    e = v.shape[-1]
    s = torch.zeros(h, d, e, dtype=q.dtype)
    out = torch.empty(n, h, e, dtype=q.dtype)
    for t in range(n):
        s = s * decay[t, :, None, None]
        u = beta[t, :, None] * (v[t] - torch.einsum("hde,hd->he", s, k[t]))
        s = s + k[t, :, :, None] * u[:, None, :]
        out[t] = torch.einsum("hde,hd->he", s, q[t])
    return out, s


def delta_mixer(h, w, p, c, eps, rnd=_keep):
    n = h.shape[0]
    heads, groups, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    rep = heads // groups
    q = silu(causal_conv(rnd(h @ w[p + "q"].T), w[p + "q.conv"])).view(n, groups, d)
    k = silu(causal_conv(rnd(h @ w[p + "k"].T), w[p + "k.conv"])).view(n, groups, d)
    v = silu(causal_conv(rnd(h @ w[p + "v"].T), w[p + "v.conv"])).view(n, heads, e)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)    # head j reads q/k head j // rep
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o, _ = gated_delta_rule(q, k, v, beta, decay)
    gate = silu(rnd(h @ w[p + "g"].T)).view(n, heads, e)
    y = rms(o, eps) * w[p + "norm"] * gate
    return rnd(rnd(y).reshape(n, heads * e) @ w[p + "o"].T)


# ---- the 'parallel' mixer: attention beside a gated linear recurrent unit ------------------------

def rotate_pairs(x, positions, dims, base):
    """x [n, heads, D]: the pair (x[2i], x[2i + 1]), i < dims / 2, is turned by the angle
    position * base^(-2i / dims); elements from ``dims`` on pass."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=DT)
    ang = positions.to(DT)[:, None] * f[None, :]
    cos, sin = torch.cos(ang)[:, None, :].to(x.dtype), torch.sin(ang)[:, None, :].to(x.dtype)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def window_keep_first_mask(n, size, keep_first):
    """[n, n] bool: query i sees key j if j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def softmax_attention(q, k, v, scale, mask):
    """q [n, H, D], k [n, G, D], v [n, G, E]; query head j reads key/value head j // (H / G)."""
    n, heads, _ = q.shape
    rep = heads // k.shape[1]
    out = torch.empty(n, heads, v.shape[-1], dtype=q.dtype)
    for j in range(heads):
        s = (q[:, j] @ k[:, j // rep].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out[:, j] = torch.softmax(s, dim=-1) @ v[:, j // rep]
    return out


def windowed_attention(h, positions, w, p, c, eps, rnd=_keep):
    n = h.shape[0]
    heads, groups, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = rnd(h @ w[p + "v"].T + w[p + "v.b"]).view(n, groups, e)
    # the norm runs over the whole projection, all heads at once, with a plain weight
    q = (rms(q, eps) * w[p + "q.norm"]).view(n, heads, d)
    k = (rms(k, eps) * w[p + "k.norm"]).view(n, groups, d)
    q = rnd(rotate_pairs(q, positions, c["rot"]["dims"], c["rot"]["base"]))
    k = rnd(rotate_pairs(k, positions, c["rot"]["dims"], c["rot"]["base"]))
    mask = window_keep_first_mask(n, c["mask"]["size"], c["mask"].get("keep_first", 0))
    o = softmax_attention(q, k, v, c["scale"], mask)
    return rnd(rnd(o).reshape(n, heads * e) @ w[p + "o"].T)


def gated_linear_recurrence(u, r, i, lam):
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t from S = 0 (the first token too), with
    log a_t = -8 r_t softplus(lam).  All [n, C]; returns (S for every token, the last S)."""
    a = torch.exp(-8.0 * r * softplus(lam))
    x = torch.sqrt(1.0 - a * a) * i * u
    s = torch.zeros(u.shape[1], dtype=u.dtype)
    out = torch.empty_like(u)
    for t in range(u.shape[0]):
        s = a[t] * s + x[t]
        out[t] = s
    return out, s


def recurrent_unit(h, w, p, c, rnd=_keep):
    n = h.shape[0]
    width, blocks = c["width"], c["blocks"]
    y = gelu_tanh(rnd(h @ w[p + "y"].T + w[p + "y.b"]))
    u = causal_conv(rnd(h @ w[p + "x"].T + w[p + "x.b"]), w[p + "conv"], w[p + "conv.b"])
    ub = u.view(n, blocks, width // blocks)
    r = torch.sigmoid(torch.einsum("nbi,boi->nbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(n, width)
    i = torch.sigmoid(torch.einsum("nbi,boi->nbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(n, width)
    s, _ = gated_linear_recurrence(u, r, i, w[p + "lam"])
    return rnd(rnd(s * y) @ w[p + "o"].T)


def parallel_mixer(h, positions, w, p, c, eps, rnd=_keep):
    left = windowed_attention(h, positions, w, p + "left.", c["left"], eps, rnd)
    right = recurrent_unit(h, w, p + "right.", c["right"], rnd)
    return c["left_scale"] * left + c["right_scale"] * right


# ---- the feed-forward: routed experts and a gated shared expert ----------------------------------

def route(h, w, p, c, forced=None):
    """(chosen experts [n, top], their weights [n, top], gap [n]).  Scores sigmoid(W_router h); the
    choice adds the stored correction, the weights do not; only experts of the ``keep`` best groups
    (a group's score: the sum of its two largest choice scores) can be chosen.  ``forced`` [n, top]:
    experts to take instead of the rule's own choice (what an engine chose under its rounding); ``gap``
    then says by how much a choice score, or a group's score, would have to move for the rule to make
    that choice (0 where it is the rule's own)."""
    r = c["router"]
    n_exp, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    per = n_exp // count
    by_group = choice.view(-1, count, per)
    group_score = by_group.topk(min(2, per), dim=-1).values.sum(-1)
    best = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, best, True)
    masked = by_group.masked_fill(~allowed[:, :, None], float("-inf")).reshape(-1, n_exp)
    chosen = masked.topk(top, dim=-1).indices
    gap = torch.zeros(h.shape[0], dtype=choice.dtype)
    if forced is not None:
        forced = torch.as_tensor(forced, dtype=torch.long)
        for t in range(h.shape[0]):
            ids = forced[t].tolist()
            if sorted(ids) == sorted(chosen[t].tolist()):
                continue
            if len(set(ids)) != top:
                gap[t] = float("inf")
                continue
            # its groups must be among the best up to the gap ...
            mine = sorted({e // per for e in ids})
            kth = group_score[t].topk(keep).values[-1]
            g_gap = max(float(kth - group_score[t, g]) for g in mine)
            # ... and, within its groups filled up with the best others, its experts the best up to the gap
            rest = [g for g in group_score[t].argsort(descending=True).tolist() if g not in mine]
            mine = mine + rest[:max(keep - len(mine), 0)]
            inside = torch.cat([by_group[t, g] for g in mine])
            e_gap = float(inside.topk(top).values[-1] - choice[t, ids].min())
            gap[t] = float("inf") if len(mine) > keep else max(g_gap, e_gap, 0.0)
        chosen = forced
    weights = s.gather(1, chosen)
    weights = weights / (weights.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    return chosen, weights, gap


def expert(h, w, p, rnd=_keep):
    return rnd(rnd(silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T)


def moe_feed_forward(h, w, p, c, rnd=_keep, route_input=None, forced=None, gaps=None):
    """``route_input``: what the router reads (the unrounded h when h itself is a rounding).  ``forced``,
    ``gaps``: see ``route``; the tokens' gaps are appended to the list ``gaps``."""
    chosen, weights, gap = route(h if route_input is None else route_input, w, p, c, forced)
    if gaps is not None:
        gaps.append(gap)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            out[t] = out[t] + a * expert(h[t:t + 1], w, f"{p}e{e}.", rnd)[0]
    if c.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * expert(h, w, p + "shared.", rnd)
    return out


# ---- the model ----------------------------------------------------------------------------------------

def forward(cfg, w, tokens, bf16_storage=False, return_layers=False, forced=None, gaps=None):
    """Logits [n, vocab] of one whole sequence.  ``forced`` {layer: [n, top]}: the experts to take in
    that layer's feed-forward; ``gaps``: a list that receives, per such layer, how far each token's
    forced choice is from the rule's own (see ``route``)."""
    rnd = as_stored_bf16 if bf16_storage else _keep
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.shape[0])
    x = w["embed"][tokens]
    layers_out = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rnd(x)                  # the sublayers read the stream itself: no norm in front of them
        if layer["type"] == "delta":
            m = delta_mixer(h, w, p + "mix.", layer["mixer"], eps, rnd)
        elif layer["type"] == "parallel":
            m = parallel_mixer(h, positions, w, p + "mix.", layer["mixer"], eps, rnd)
        else:
            raise ValueError(layer["type"])
        x = x + one_plus_norm(m, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + one_plus_norm(moe_feed_forward(rnd(x), w, p + "mlp.", layer["mlp"], rnd, route_input=x,
                                                   forced=None if forced is None else forced.get(i), gaps=gaps),
                                  w[p + "norm2"], eps)
        layers_out.append(x)
    logits = rnd(one_plus_norm(x, w["final.norm"], eps)) @ w["embed"].T
    if return_layers:
        return logits, torch.stack(layers_out)
    return logits
