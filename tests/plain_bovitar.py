"""A plain, slow implementation of the Bovitar design: whole sequences, no cache, no batches,
float64 by default, one function per mechanism, written from the design's equations.  It shares
no code with the package; the tests compare the package with it.

Notation: n tokens, width W.  ``w`` maps tensor names to tensors, ``p`` is a part's prefix
("l3.mix.left." and the like), ``c`` the part's entry of config.json.  ``rnd`` rounds what a
bfloat16 engine stores (a yardstick for its tests); by default nothing is rounded.

A layer is x <- x + mixer(norm1(x)), then x <- x + ff(norm2(x)).  Mixers: "delta" (a gated delta
rule behind short convolutions) and "parallel" (softmax attention behind short convolutions,
with soft-capped scores, beside a state-space recurrence with a scalar decay per head; each
branch's output is normed and the two are averaged).  The feed-forward is a mixture of experts
with a softmax router.  A layer may run with another layer's weights.
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

def unit_rms(x, eps):
    """x over its root mean square over the last dimension, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def short_conv(x, taps, bias=None):
    """x [n, C], taps [C, K]: y_t = sum_j taps[:, j] * x_(t - K + 1 + j), with zeros before the
    first token; the last column belongs to the current token."""
    n, ch = x.shape
    k = taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(n):
        for j in range(k):
            src = t - k + 1 + j
            if src >= 0:
                y[t] = y[t] + taps[:, j] * x[src]
    return y if bias is None else y + bias


# ---- mixer "delta" ------------------------------------------------------------------------------

def delta_recurrence(q, k, v, beta, g):
    """q, k [n, H, D]; v [n, H, E]; beta, g [n, H].  Per head, from S = 0 [D, E]:
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    n, heads, d = q.shape
    e = v.shape[-1]
    out = torch.zeros(n, heads, e, dtype=q.dtype)
    for h in range(heads):
        s = torch.zeros(d, e, dtype=q.dtype)
        for t in range(n):
            s = g[t, h] * s
            u = beta[t, h] * (v[t, h] - s.T @ k[t, h])
            s = s + torch.outer(k[t, h], u)
            out[t, h] = s.T @ q[t, h]
    return out


def delta_mixer(h, w, p, c, eps, rnd=_keep):
    n = h.shape[0]
    heads, groups, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    per = heads // groups

    def branch(name, count, size):
        u = silu(short_conv(rnd(h @ w[p + name].T), w[p + name + ".conv"]))
        return u.reshape(n, count, size)

    q, k, v = branch("q", groups, d), branch("k", groups, d), branch("v", heads, e)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    pick = torch.arange(heads) // per
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = delta_recurrence(q[:, pick], k[:, pick], v, beta, g)
    gate = silu(rnd(h @ w[p + "g"].T)).reshape(n, heads, e)
    y = unit_rms(o, eps) * w[p + "norm"] * gate
    return rnd(rnd(y).reshape(n, heads * e) @ w[p + "o"].T)


# ---- mixer "parallel", left: attention ------------------------------------------------------------

def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims) for i < dims/2; long wavelengths stretched: with l = 2 pi / f, f stays
    where l < original/high, becomes f/factor where l > original/low, and is blended between."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, original = (float(scaling[x]) for x in ("factor", "low", "high", "original"))
            l = 2.0 * math.pi / f
            if l > original / low:
                f = f / factor
            elif not l < original / high:
                s = (original / l - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate_halves(x, positions, freqs):
    """x [n, heads, D]; element i < dims/2 turns with element i + dims/2 by the angle position * f_i;
    elements from dims on pass."""
    half = len(freqs)
    if half == 0:
        return x
    a = positions.to(x.dtype)[:, None] * torch.tensor(freqs, dtype=x.dtype)[None, :]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., 2 * half:]], dim=-1)


def capped_causal_attention(q, k, v, scale, softcap):
    """q [n, H, D], k [n, G, D], v [n, G, E]: softmax over j <= i of cap * tanh(q_i . k_j * scale / cap)."""
    n, heads, _ = q.shape
    per = heads // k.shape[1]
    out = torch.zeros(n, heads, v.shape[-1], dtype=q.dtype)
    for h in range(heads):
        g = h // per
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(torch.ones(n, n, dtype=torch.bool).triu(1), -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def attention_branch(h, w, p, c, eps, rnd=_keep):
    n = h.shape[0]
    heads, groups, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = short_conv(rnd(h @ w[p + "q"].T), w[p + "q.conv"])
    k = short_conv(rnd(h @ w[p + "k"].T), w[p + "k.conv"])
    v = short_conv(rnd(h @ w[p + "v"].T), w[p + "v.conv"])
    q = rms_norm(q, w[p + "q.norm"], eps).reshape(n, heads, d)       # over the whole projection
    k = rms_norm(k, w[p + "k.norm"], eps).reshape(n, groups, d)
    rot = c["rot"]
    freqs = rotary_frequencies(rot["dims"], float(rot["base"]), rot.get("scaling"))
    pos = torch.arange(n)
    q, k = rnd(rotate_halves(q, pos, freqs)), rnd(rotate_halves(k, pos, freqs))
    o = capped_causal_attention(q, k, rnd(v).reshape(n, groups, e), float(c["scale"]), c.get("softcap"))
    return rnd(rnd(o).reshape(n, heads * e) @ w[p + "o"].T)


# ---- mixer "parallel", right: state-space recurrence ----------------------------------------------

def state_space_recurrence(x, b, c, dt, a, d_skip):
    """x [n, H, P], b and c [n, H, N] (already picked per head), dt [n, H], a [H] = exp(A_log), d_skip [H].
    Per head from S = 0 [N, P]: S <- exp(-a dt) S + dt b x^T;  y = S^T c + d_skip x."""
    n, heads, pdim = x.shape
    out = torch.zeros_like(x)
    for h in range(heads):
        s = torch.zeros(b.shape[-1], pdim, dtype=x.dtype)
        for t in range(n):
            s = torch.exp(-a[h] * dt[t, h]) * s + dt[t, h] * torch.outer(b[t, h], x[t, h])
            out[t, h] = s.T @ c[t, h] + d_skip[h] * x[t, h]
    return out


def state_space_branch(h, w, p, c, eps, rnd=_keep):
    n = h.shape[0]
    heads, pdim, ns, groups, parts = c["heads"], c["vdim"], c["state"], c["groups"], c["norm_groups"]
    inner = heads * pdim
    proj = rnd(h @ w[p + "in"].T)
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * groups * ns], proj[:, 2 * inner + 2 * groups * ns:]
    xbc = silu(short_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(n, heads, pdim)
    b = xbc[:, inner:inner + groups * ns].reshape(n, groups, ns)
    cc = xbc[:, inner + groups * ns:].reshape(n, groups, ns)
    pick = torch.arange(heads) // (heads // groups)
    dt = softplus(dt + w[p + "dt_bias"])
    y = state_space_recurrence(x, b[:, pick], cc[:, pick], dt, torch.exp(w[p + "A_log"]), w[p + "D"])
    y = y.reshape(n, inner) * silu(z)                         # gated first, normed second
    y = unit_rms(y.reshape(n, parts, inner // parts), eps).reshape(n, inner) * w[p + "norm"]
    return rnd(rnd(y) @ w[p + "o"].T)


def parallel_mixer(h, w, p, c, eps, rnd=_keep):
    left = attention_branch(h, w, p + "left.", c["left"], eps, rnd)
    right = state_space_branch(h, w, p + "right.", c["right"], eps, rnd)
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


# ---- feed-forward ---------------------------------------------------------------------------------

def route(h, w, p, r, follow=None):
    """(chosen experts [n, top], weights [n, top], scores): softmax scores; the choice is made on
    scores + correction among the experts of the best groups (a group's score is its largest choice
    score; other groups count as minus infinity); the weights are the plain scores times scale.
    ``follow``: take these experts instead of the rule's own (an engine's choice)."""
    experts, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"]
    n = h.shape[0]
    per = experts // groups["count"]
    gscore = choice.reshape(n, groups["count"], per).max(-1).values
    kept = torch.zeros(n, groups["count"], dtype=torch.bool)
    kept.scatter_(1, gscore.topk(groups["keep"], dim=-1).indices, True)
    masked = choice.masked_fill(~kept.repeat_interleave(per, dim=1), -math.inf)
    ids = masked.topk(top, dim=-1).indices if follow is None else follow
    return ids, s.gather(1, ids) * float(r["scale"]), masked


def expert(h, w, p, rnd=_keep):
    a = rnd(silu(rnd(h @ w[p + "gate"].T)) * rnd(h @ w[p + "up"].T))
    return rnd(a @ w[p + "down"].T)


def route_gap(h, w, p, r, ids):
    """How far a given choice ``ids`` [n, top] is from the rule's own, per token, in units of the choice
    scores: the larger of (a) how far the worst group it uses lies below the rule's worst kept group and
    (b) how far its worst expert lies below the worst expert the rule would choose among the groups the
    choice must have kept (the groups it uses, filled up with the best of the others).  0 where the
    choice is the rule's."""
    experts, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    n, per = h.shape[0], experts // groups["count"]
    choice = torch.softmax(h @ w[p + "router"].T, dim=-1) + w[p + "correction"]
    gscore = choice.reshape(n, groups["count"], per).max(-1).values
    kept_worst = gscore.topk(groups["keep"], dim=-1).values.min(-1).values
    used = torch.zeros(n, groups["count"], dtype=torch.bool).scatter_(1, ids // per, True)
    used_worst = gscore.masked_fill(~used, math.inf).min(-1).values
    kept = torch.zeros(n, groups["count"], dtype=torch.bool)
    kept.scatter_(1, gscore.masked_fill(used, math.inf).topk(groups["keep"], dim=-1).indices, True)
    masked = choice.masked_fill(~kept.repeat_interleave(per, dim=1), -math.inf)
    own = masked.topk(top, dim=-1).values.min(-1).values
    return torch.maximum(kept_worst - used_worst, own - choice.gather(1, ids).min(-1).values).clamp(min=0.0)


def moe_feed_forward(h, w, p, c, rnd=_keep, follow=None, gaps=None):
    """``gaps`` (a list, with ``follow``): receives ``route_gap`` of the followed choice."""
    ids, weights, _ = route(h, w, p, c["router"], follow)
    if gaps is not None and follow is not None:
        gaps.append(route_gap(h, w, p, c["router"], ids))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            out[t] = out[t] + weights[t, j] * expert(h[t:t + 1], w, f"{p}e{int(ids[t, j])}.", rnd)[0]
    if c.get("shared") is not None:
        out = out + expert(h, w, p + "shared.", rnd)
    return out


# ---- the model ------------------------------------------------------------------------------------

def forward(cfg, w, tokens, rnd=_keep, layers_out=None, follow=None, gaps=None):
    """Logits [n, vocab] of one sequence.  ``layers_out``: a list that receives the residual stream
    after every layer run.  ``follow``: {layer run: chosen experts [n, top]}; ``gaps``: see
    ``moe_feed_forward``."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        h = rnd(rms_norm(x, w[p + "norm1"], eps))
        if layer["type"] == "delta":
            x = x + delta_mixer(h, w, p + "mix.", layer["mixer"], eps, rnd)
        elif layer["type"] == "parallel":
            x = x + parallel_mixer(h, w, p + "mix.", layer["mixer"], eps, rnd)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        if layer.get("mlp") is not None:
            h = rnd(rms_norm(x, w[p + "norm2"], eps))
            x = x + moe_feed_forward(h, w, p + "mlp.", layer["mlp"], rnd,
                                     None if follow is None else follow.get(i), gaps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rnd(rms_norm(x, w["final.norm"], eps))
    return (x @ w["head"].T) * float(cfg["logit_scale"])
