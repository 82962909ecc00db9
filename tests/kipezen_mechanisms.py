"""One mechanism of the Kipezen design at a time: a model of ONE layer in which everything else is
switched off (the other branch's scale is zero, no feed-forward), with weights and a prompt made so
that a fault shows (a token whose key takes nearly all of a later query's weight just inside or just
outside the window and the kept first keys, at and beside a page's border; a write to the recurrent
state that is read a hundred tokens later), run through the engine's step function under every
cutting, against the plain implementation.  Each case also checks that it WOULD show the fault: the
plain implementation with the constant one off, or with the far token taken away, moves the probed
rows by far more than the tolerance.  Used on the CPU (kernel wrappers replaced by their PyTorch
restatements) and on the GPU."""

from __future__ import annotations

import copy

import torch

from tests import kipezen_util as ku
from tests import plain_kipezen as pk

FILLERS = slice(8, None)          # token ids 0..7 are the marked ones
QUERY, MARKS = 0, (1, 2, 3, 4, 5, 6)


def row_errors(got, want):
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt()


CLOSE_CALL = 0.06      # a bfloat16 engine may choose another expert where choice scores are this close


def compare(model_dir, reqs, dtype, device, page, tail, what, **engine):
    """Every schedule's logits against the plain implementation's.  A bfloat16 engine's router sees
    rounded inputs and may decide a close call the other way, which changes everything behind it; so
    its choices are recorded, checked to be the rule's own up to CLOSE_CALL, and the plain
    implementation follows them.  Returns (config, weights, the plain logits, the tolerance per
    request) for the caller's own checks."""
    cfg, w = pk.read_model_dir(model_dir)
    exact = [pk.forward(cfg, w, r) for r in reqs]
    moe_layers = [i for i, layer in enumerate(cfg["layers"]) if layer.get("mlp") is not None]
    lens = [len(r) for r in reqs]
    for name, steps in ku.schedules(lens, tail).items():
        routes = {} if dtype == "bfloat16" and moe_layers else None
        if routes is not None:
            engine = dict(engine, cuda_graphs=False)      # a replayed graph does not show its router's choices
        runner = ku.runner_for(model_dir, dtype, device, page, lens, **engine)
        got = ku.replay(runner, reqs, steps, routes)
        for i, (g, r) in enumerate(zip(got, reqs)):
            if dtype == "float32":
                e = exact[i]
                bound = 1e-4 * float(e.std())
            else:
                forced = None if routes is None else {layer: routes[i][k] for k, layer in enumerate(moe_layers)}
                gaps = []
                e = pk.forward(cfg, w, r, forced=forced, gaps=gaps)
                for layer, gap in zip(moe_layers, gaps):
                    assert float(gap.max()) <= CLOSE_CALL, \
                        f"{what} ({dtype}, {name}): request {i}, layer {layer}, position {int(gap.argmax())}: the " \
                        f"engine chose experts whose scores are {float(gap.max()):.3g} from the rule's choice"
                stored = pk.forward(cfg, w, r, bf16_storage=True, forced=forced)
                bound = max(3.0 * float(row_errors(stored, e).max()), 2e-2 * float(e.std()))
            err = row_errors(g, e)
            worst = int(err.argmax())
            assert float(err[worst]) <= bound, \
                f"{what} ({dtype}, {name}): request {i} position {worst} of {len(e)}: {float(err[worst]):.4g} " \
                f"exceeds {bound:.4g}"
    return cfg, w, exact, [1e-4 * float(e.std()) for e in exact]


def shows(cfg, w, req, exact, bound, rows, what, change_cfg=None, change_req=None, factor=30.0):
    """The plain implementation with the change applied moves the probed rows by ``factor`` times the
    float32 engine's tolerance (the bfloat16 engine runs the same case at its own tolerance)."""
    cfg2, req2 = copy.deepcopy(cfg), list(req)
    if change_cfg is not None:
        change_cfg(cfg2)
    if change_req is not None:
        change_req(req2)
    moved = row_errors(pk.forward(cfg2, w, req2)[rows], exact[rows])
    assert float(moved.max()) > factor * bound, \
        f"{what}: the case would not show it (rows move by {float(moved.max()):.3g}, tolerance {bound:.3g})"


def marked_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(8, vocab, (n,), generator=g)).tolist()


# ---- attention with a window and kept first keys ---------------------------------------------------

def attention_case(tmp, dtype, device, heads, kv_heads, dim, vdim, window, keep, rot, page, n=150, seed=1):
    layer = ku.parallel(heads, kv_heads, dim, vdim, window, keep, rot, 5000.0, 16, 1, 2, scales=(1.0, 0.0),
                        scale=8.0 / dim, mlp=None)
    config = ku.one_layer(layer, vocab=97, width=48)

    def edit(t):
        # hidden channel 0 marks a key, channel 1 a query; both map onto the same direction of every
        # head, so a marked key takes nearly all of a marked query's weight; channels 2.. tell the
        # marked keys' values apart
        e = t["embed"]
        e[:, :8] = 0.0
        e[list(MARKS), 0] = 6.0
        e[QUERY, 1] = 6.0
        for j, m in enumerate(MARKS):
            e[m, 2 + j] = 8.0
        direction = torch.ones(dim)
        direction[:rot] = 0.0 if rot < dim else 1.0       # where it can, outside the rotated part
        t["l0.mix.left.k"][:, 0] = direction.repeat(kv_heads)
        t["l0.mix.left.q"][:, 1] = direction.repeat(heads)
        t["l0.mix.left.q.norm"].fill_(1.0)
        t["l0.mix.left.k.norm"].fill_(1.0)

    d = ku.write_model(config, seed, tmp, edit)
    toks = marked_tokens(97, n, seed)
    last = n - 1
    # for the last query: the edge of the kept first keys, the window's edge, and a far key in between
    places = {keep - 1: 1, keep: 2, last - window: 3, last - window + 1: 4, (keep + last - window) // 2: 5}
    if keep == 0:
        places = {0: 2, last - window: 3, last - window + 1: 4, (last - window) // 2: 5}
    for p, m in places.items():
        toks[p] = m
    toks[last - 3:] = [QUERY] * 4                   # four queries: the window's edge passes over the marked keys
    other = marked_tokens(97, 37, seed + 1)
    other[3], other[-1] = 6, QUERY
    reqs = [toks, other, marked_tokens(97, 2 * page + 1, seed + 2)]
    cfg, w, exact, bounds = compare(d, reqs, dtype, device, page, tail=n - (last - window) + 3, what="attention")
    rows = list(range(last - 3, n))
    mask = lambda c: c["layers"][0]["mixer"]["left"]["mask"]
    for name, change in (("a window one longer", lambda c: mask(c).update(size=window + 1)),
                         ("a window one shorter", lambda c: mask(c).update(size=window - 1)),
                         ("one more kept key", lambda c: mask(c).update(keep_first=keep + 1)),
                         ("one kept key fewer", lambda c: mask(c).update(keep_first=max(keep - 1, 0)))):
        if keep == 0 and "fewer" in name:
            continue
        shows(cfg, w, toks, exact[0], bounds[0], rows, name, change_cfg=change)
    return exact


# ---- the gated delta rule ---------------------------------------------------------------------------

def delta_case(tmp, dtype, device, heads, kv_heads, dim, vdim, taps, page=16, n=140, seed=2):
    config = ku.one_layer(ku.delta(heads, kv_heads, dim, vdim, taps, mlp=None), vocab=97, width=48)

    def edit(t):
        # a marked token writes a large value under a key that only the marked query, far behind, asks for
        e = t["embed"]
        e[:, :8] = 0.0
        e[MARKS[0], 0] = 6.0
        e[QUERY, 1] = 6.0
        e[MARKS[0], 2] = 8.0
        t["l0.mix.q"][:, 1] = t["l0.mix.k"][:, 0]
        t["l0.mix.A_log"].fill_(-5.0)               # slow decays: the state keeps a hundred tokens
        t["l0.mix.b"][:, 0] = 1.0                   # the marked token writes with a rate near one

    d = ku.write_model(config, seed, tmp, edit)
    toks = marked_tokens(97, n, seed)
    toks[2] = MARKS[0]
    toks[n - 2:] = [QUERY] * 2
    other = marked_tokens(97, 29, seed + 1)
    reqs = [toks, other, marked_tokens(97, 3, seed + 2), marked_tokens(97, 50, seed + 3)]
    cfg, w, exact, bounds = compare(d, reqs, dtype, device, page, tail=100, what="gated delta rule")

    def unmark(r):
        r[2] = 50
    shows(cfg, w, toks, exact[0], bounds[0], [n - 2, n - 1], "a write lost from the state", change_req=unmark,
          factor=20.0)


# ---- the gated linear recurrent unit ------------------------------------------------------------------

def recurrence_case(tmp, dtype, device, width, blocks, taps, page=16, n=130, seed=3):
    layer = ku.parallel(2, 1, 16, 16, 8, 0, 16, 100.0, width, blocks, taps, scales=(0.0, 1.0), mlp=None)
    config = ku.one_layer(layer, vocab=97, width=48)

    def edit(t):
        t["l0.mix.right.lam"].fill_(-5.0)           # slow decays: the state keeps the first tokens
        e = t["embed"]
        e[:, :8] = 0.0
        e[MARKS[0], 0] = 8.0
        t["l0.mix.right.x"][:, 0] = 1.0             # the marked token drives every channel

    d = ku.write_model(config, seed, tmp, edit)
    toks = marked_tokens(97, n, seed)
    toks[0] = MARKS[0]
    reqs = [toks, marked_tokens(97, 31, seed + 1), marked_tokens(97, 2, seed + 2), marked_tokens(97, 64, seed + 3)]
    cfg, w, exact, bounds = compare(d, reqs, dtype, device, page, tail=100, what="gated linear recurrence")

    def unmark(r):
        r[0] = 50
    shows(cfg, w, toks, exact[0], bounds[0], [n - 1], "a first token lost from the state", change_req=unmark,
          factor=20.0)


# ---- routed experts -------------------------------------------------------------------------------------

def experts_case(tmp, dtype, device, experts, top, ff, groups, shared, correction, page=16, seed=4):
    """``correction``: the size of the stored correction; -2.0 makes every choice score negative, so an
    expert of a group that is left out must count as minus infinity, not as zero."""
    mlp = ku.moe(experts, top, ff, 2.5, groups=groups, shared=shared)
    config = ku.one_layer(ku.delta(1, 1, 8, 8, 2, mlp=mlp), vocab=97, width=48)

    def edit(t):
        g = torch.Generator().manual_seed(seed)
        c = torch.randn(experts, generator=g) * 0.5
        t["l0.mlp.correction"] = c if correction >= 0 else c * 0.2 - 2.0
        t["l0.norm1"].fill_(-0.9)                   # the mixer nearly silent: the feed-forward reads the embedding

    d = ku.write_model(config, seed, tmp, edit)
    reqs = [marked_tokens(97, n, seed + i) for i, n in enumerate((90, 17, 1, 300))]
    cfg, w, exact, bounds = compare(d, reqs, dtype, device, page, tail=20, what="routed experts")
    rows = list(range(90))
    router = lambda c: c["layers"][0]["mlp"]["router"]
    if groups is not None and groups[1] < groups[0]:
        shows(cfg, w, reqs[0], exact[0], bounds[0], rows, "groups ignored",
              change_cfg=lambda c: router(c).update(groups={"count": 1, "keep": 1}), factor=20.0)
    w0 = dict(w)
    w0["l0.mlp.correction"] = torch.zeros_like(w["l0.mlp.correction"])
    moved = row_errors(pk.forward(cfg, w0, reqs[0]), exact[0])
    assert top == experts or float(moved.max()) > 20.0 * bounds[0], "the correction would not show"
    if shared is not None:
        w1 = dict(w)
        w1["l0.mlp.shared.sg"] = torch.zeros_like(w["l0.mlp.shared.sg"])
        moved = row_errors(pk.forward(cfg, w1, reqs[0]), exact[0])
        assert float(moved.max()) > 20.0 * bounds[0], "the shared expert's gate would not show"
