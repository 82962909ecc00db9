"""One mechanism of the Bovitar design at a time: a model of ONE layer in which everything else is
quiet (the other branch's output norm weight is zero, no feed-forward), with weights and a prompt
made so that a fault shows (a token whose key takes nearly all of a later query's weight from far
back, at and beside a page's border; scores far beyond the soft cap; convolution taps that reach
back over the start of a portion and of the sequence; a write to a recurrent state that is read a
hundred tokens later), run through the engine's step function under every cutting, against the
plain implementation.  Each case also checks that it WOULD show the fault: the plain implementation
with the constant changed, or with the far token taken away, moves the probed rows by far more than
the tolerance.  Used on the CPU (kernel wrappers replaced by their PyTorch restatements) and on the
GPU."""

from __future__ import annotations

import copy

import torch

from tests import bovitar_util as bu
from tests import plain_bovitar as pb

QUERY, MARKS = 0, (1, 2, 3, 4, 5, 6)       # token ids 0..7 are the marked ones
CLOSE_CALL = 0.05      # a bfloat16 engine may choose another expert where choice scores are this close


def row_errors(got, want):
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt()


def compare(model_dir, reqs, dtype, device, page, tail, what, **engine):
    """Every schedule's logits against the plain implementation's.  A bfloat16 engine's router sees
    rounded inputs and may decide a close call the other way, which changes everything behind it; so
    its choices are recorded, checked to be the rule's own up to CLOSE_CALL, and the plain
    implementation follows them.  Returns (config, weights, the plain logits, the float32 tolerance
    per request)."""
    cfg, w = pb.read_model_dir(model_dir)
    exact = [pb.forward(cfg, w, r) for r in reqs]
    moe_runs = [i for i, layer in enumerate(cfg["layers"]) if layer.get("mlp") is not None]
    lens = [len(r) for r in reqs]
    for name, steps in bu.schedules(lens, tail).items():
        routes = {} if dtype == "bfloat16" and moe_runs else None
        if routes is not None:
            engine = dict(engine, cuda_graphs=False)      # a replayed graph does not show its router's choices
        runner = bu.runner_for(model_dir, dtype, device, page, lens, **engine)
        got = bu.replay(runner, reqs, steps, routes)
        for i, (g, r) in enumerate(zip(got, reqs)):
            if dtype == "float32":
                e = exact[i]
                bound = 1e-4 * float(e.std())
            else:
                follow = None if routes is None else {run: routes[i][k] for k, run in enumerate(moe_runs)}
                gaps = []
                e = pb.forward(cfg, w, r, follow=follow, gaps=gaps)
                for run, gap in zip(moe_runs, gaps):
                    assert float(gap.max()) <= CLOSE_CALL, \
                        f"{what} ({dtype}, {name}): request {i}, layer run {run}, position {int(gap.argmax())}: the " \
                        f"engine chose experts whose scores are {float(gap.max()):.3g} from the rule's choice"
                stored = pb.forward(cfg, w, r, rnd=pb.as_stored_bf16, follow=follow)
                bound = max(3.0 * float(row_errors(stored, e).max()), 2e-2 * float(e.std()))
            err = row_errors(g, e)
            worst = int(err.argmax())
            assert float(err[worst]) <= bound, \
                f"{what} ({dtype}, {name}): request {i} position {worst} of {len(e)}: {float(err[worst]):.4g} " \
                f"exceeds {bound:.4g}"
    return cfg, w, exact, [1e-4 * float(e.std()) for e in exact]


def shows(cfg, w, req, exact, bound, rows, what, change_cfg=None, change_req=None, change_w=None, factor=30.0):
    """The plain implementation with the change applied moves the probed rows by ``factor`` times the
    float32 engine's tolerance (the bfloat16 engine runs the same case at its own tolerance)."""
    cfg2, req2, w2 = copy.deepcopy(cfg), list(req), dict(w)
    if change_cfg is not None:
        change_cfg(cfg2)
    if change_req is not None:
        change_req(req2)
    if change_w is not None:
        change_w(w2)
    moved = row_errors(pb.forward(cfg2, w2, req2)[rows], exact[rows])
    assert float(moved.max()) > factor * bound, \
        f"{what}: the case would not show it (rows move by {float(moved.max()):.3g}, tolerance {bound:.3g})"


def filler_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(8, vocab, (n,), generator=g)).tolist()


QUIET_STATE_SPACE = bu.state_space(2, 8, 8, 1, 1, 2)
QUIET_ATTENTION = bu.attention(2, 1, 16, 16, 2, 16, 100.0)


# ---- attention: far keys, page borders, the soft cap, the rotation, the convolutions ----------------

def attention_case(tmp, dtype, device, heads, kv_heads, dim, vdim, taps, rot, page, softcap, scaling=None, n=330,
                   seed=1, repeat=False):
    left = bu.attention(heads, kv_heads, dim, vdim, taps, rot, 5000.0, scaling=scaling, softcap=softcap,
                        scale=3.0 / dim)
    config = bu.one_layer(bu.parallel(left, QUIET_STATE_SPACE, mlp=None), vocab=97, width=48, repeat=repeat)
    chan_q, chan_k = heads * dim, kv_heads * dim

    def edit(t):
        # hidden channel 0 marks a key, channel 1 a query; both map onto the same direction of every
        # head, so a marked key takes most of a marked query's weight (as far as the soft cap lets it);
        # channels 2.. tell the marked keys' values apart.  The convolutions pass the current token and
        # mix a little of the tokens before it in, so that a lost tail still shows.
        e = t["embed"]
        e[:, :8] = 0.0
        e[list(MARKS), 0] = 6.0
        e[QUERY, 1] = 6.0
        for j, m in enumerate(MARKS):
            e[m, 2 + j] = 8.0
        direction = torch.ones(dim)
        if 0 < rot < dim:
            direction[:rot] = 0.0                 # where it can, outside the rotated part
        t["l0.mix.left.k"][:, 0] = direction.repeat(kv_heads)
        t["l0.mix.left.q"][:, 1] = direction.repeat(heads)
        t["l0.mix.left.q.norm"].fill_(2.0)
        t["l0.mix.left.k.norm"].fill_(2.0)
        for x in ("q", "k", "v"):
            c = t[f"l0.mix.left.{x}.conv"]
            c.mul_(0.3)
            c[:, -1] = 1.0
        t["l0.mix.right.out"].zero_()             # the other branch is silent

    d = bu.write_model(config, seed, tmp, edit)
    toks = filler_tokens(97, n, seed)
    last = n - 1
    # marked keys: the first token, both sides of a page's border far back, the middle, right before the queries
    places = {0: 1, 2 * page - 1: 2, 2 * page: 3, n // 2: 4, last - 4: 5}
    for p, m in places.items():
        toks[p] = m
    toks[last - 2:] = [QUERY] * 3
    other = filler_tokens(97, 37, seed + 1)
    other[3], other[-1] = 6, QUERY
    reqs = [toks, other, filler_tokens(97, 2 * page + 1, seed + 2)]
    cfg, w, exact, bounds = compare(d, reqs, dtype, device, page, tail=40, what="attention")
    rows = list(range(last - 2, n))
    att = lambda c: c["layers"][0]["mixer"]["left"]
    for p in (0, 2 * page - 1, 2 * page):
        def unmark(r, p=p):
            r[p] = 50
        # (a rotation over the whole head weakens a far key's match; it still weighs many tolerances)
        shows(cfg, w, toks, exact[0], bounds[0], rows, f"the far key at {p} lost", change_req=unmark,
              factor=30.0 if rot < dim else 8.0)
    if softcap is not None:
        shows(cfg, w, toks, exact[0], bounds[0], rows, "no soft cap", change_cfg=lambda c: att(c).update(softcap=None))
        shows(cfg, w, toks, exact[0], bounds[0], rows, "another soft cap",
              change_cfg=lambda c: att(c).update(softcap=softcap * 1.25))
    if taps > 1:
        def cut_tap(w2):
            for x in ("q", "k", "v"):
                c = w2[f"l0.mix.left.{x}.conv"].clone()
                c[:, 0] = 0.0
                w2[f"l0.mix.left.{x}.conv"] = c
        shows(cfg, w, toks, exact[0], bounds[0], list(range(n)), "the oldest tap lost", change_w=cut_tap)
    if scaling is not None:
        shows(cfg, w, toks, exact[0], bounds[0], list(range(n)), "plain frequencies",
              change_cfg=lambda c: att(c)["rot"].pop("scaling"))
    return exact


# ---- the gated delta rule ---------------------------------------------------------------------------

def delta_case(tmp, dtype, device, heads, kv_heads, dim, vdim, taps, page=16, n=140, seed=2, repeat=False):
    config = bu.one_layer(bu.delta(heads, kv_heads, dim, vdim, taps, mlp=None), vocab=97, width=48, repeat=repeat)

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

    d = bu.write_model(config, seed, tmp, edit)
    toks = filler_tokens(97, n, seed)
    toks[2] = MARKS[0]
    toks[n - 2:] = [QUERY] * 2
    reqs = [toks, filler_tokens(97, 29, seed + 1), filler_tokens(97, 3, seed + 2), filler_tokens(97, 50, seed + 3)]
    cfg, w, exact, bounds = compare(d, reqs, dtype, device, page, tail=100, what="gated delta rule")

    def unmark(r):
        r[2] = 50
    shows(cfg, w, toks, exact[0], bounds[0], [n - 2, n - 1], "a write lost from the state", change_req=unmark,
          factor=20.0)


# ---- the state-space recurrence -------------------------------------------------------------------------

def state_space_case(tmp, dtype, device, heads, vdim, state, groups, norm_groups, taps, page=16, n=130, seed=3,
                     repeat=False):
    right = bu.state_space(heads, vdim, state, groups, norm_groups, taps)
    config = bu.one_layer(bu.parallel(QUIET_ATTENTION, right, mlp=None), vocab=97, width=48, repeat=repeat)
    inner = heads * vdim

    def edit(t):
        t["l0.mix.right.A_log"].fill_(-5.0)         # slow decays: the state keeps the first tokens
        t["l0.mix.right.dt_bias"].fill_(0.5)
        e = t["embed"]
        e[:, :8] = 0.0
        e[MARKS[0], 0] = 8.0
        t["l0.mix.right.in"][inner:2 * inner + groups * state, 0] = 1.0     # the marked token drives x and B
        t["l0.mix.right.D"].mul_(0.1)               # what the state gives back outweighs the skip
        t["l0.mix.left.out"].zero_()                # the other branch is silent

    d = bu.write_model(config, seed, tmp, edit)
    toks = filler_tokens(97, n, seed)
    toks[0] = MARKS[0]
    reqs = [toks, filler_tokens(97, 31, seed + 1), filler_tokens(97, 2, seed + 2), filler_tokens(97, 64, seed + 3)]
    cfg, w, exact, bounds = compare(d, reqs, dtype, device, page, tail=100, what="state-space recurrence")

    def unmark(r):
        r[0] = 50
    shows(cfg, w, toks, exact[0], bounds[0], [n - 1], "a first token lost from the state", change_req=unmark,
          factor=20.0)
    ssm = lambda c: c["layers"][0]["mixer"]["right"]
    if norm_groups > 1:
        shows(cfg, w, toks, exact[0], bounds[0], list(range(n)), "one part in the gated norm",
              change_cfg=lambda c: ssm(c).update(norm_groups=1), factor=20.0)
    if groups > 1 and heads > groups:
        def other_groups(w2):       # the heads read their own group's B and C: swapping two groups' rows shows
            m = w2["l0.mix.right.in"].clone()
            a, b = 2 * inner, 2 * inner + state
            m[a:a + state], m[b:b + state] = w2["l0.mix.right.in"][b:b + state], w2["l0.mix.right.in"][a:a + state]
            w2["l0.mix.right.in"] = m
        shows(cfg, w, toks, exact[0], bounds[0], list(range(n)), "heads on another group", change_w=other_groups,
              factor=20.0)


# ---- routed experts -------------------------------------------------------------------------------------

def experts_case(tmp, dtype, device, experts, top, ff, groups, shared, correction, page=16, seed=4):
    """``correction``: positive: corrections of both signs and of the scores' size; negative: every choice
    score is negative, so an expert of a group that is left out must count as minus infinity, not as
    zero."""
    mlp = bu.moe(experts, top, ff, 2.5, groups=groups, shared=shared)
    config = bu.one_layer(bu.delta(1, 1, 8, 8, 2, mlp=mlp), vocab=97, width=48)

    def edit(t):
        g = torch.Generator().manual_seed(seed)
        c = torch.randn(experts, generator=g) * (0.6 / experts)
        t["l0.mlp.correction"] = c if correction >= 0 else c - 2.0
        t["l0.mix.o"].mul_(0.05)                    # the mixer nearly silent: the feed-forward reads the embedding

    d = bu.write_model(config, seed, tmp, edit)
    reqs = [filler_tokens(97, n, seed + i) for i, n in enumerate((90, 17, 1, 300))]
    cfg, w, exact, bounds = compare(d, reqs, dtype, device, page, tail=20, what="routed experts")
    rows = list(range(90))
    router = lambda c: c["layers"][0]["mlp"]["router"]
    if groups is not None and groups[1] < groups[0]:
        shows(cfg, w, reqs[0], exact[0], bounds[0], rows, "groups ignored",
              change_cfg=lambda c: router(c).update(groups={"count": 1, "keep": 1}), factor=20.0)
    if top < experts:
        def no_correction(w2):
            w2["l0.mlp.correction"] = torch.zeros_like(w2["l0.mlp.correction"])
        shows(cfg, w, reqs[0], exact[0], bounds[0], rows, "no correction", change_w=no_correction, factor=20.0)
    shows(cfg, w, reqs[0], exact[0], bounds[0], rows, "another scale of the weights",
          change_cfg=lambda c: router(c).update(scale=2.0), factor=20.0)
    if shared is not None:
        def no_shared(w2):
            w2["l0.mlp.shared.down"] = torch.zeros_like(w2["l0.mlp.shared.down"])
        shows(cfg, w, reqs[0], exact[0], bounds[0], rows, "no shared expert", change_w=no_shared, factor=20.0)
