"""The Bovitar design on the GPU against the plain implementation of ``tests/plain_bovitar.py``:
each mechanism alone (``tests/bovitar_mechanisms.py``: one-layer models whose weights and prompts
make a lost far key, a missing soft cap, a lost convolution tap, a lost state or a left-out group
show, under every cutting of the engine's step function), the new kernels alone against their
equations, then whole models under the same cuttings (whole prompts, the last tokens one by one,
portions down to two tokens, mixed batches in a pool so small that pages and slots are used again):
float32 through ``bin/trace_run``, bfloat16 through the step function in this process, where the
router's choices can be read and followed; and greedy generation through ``Engine.generate``."""

import copy
import math

import pytest
import torch

from tests import bovitar_mechanisms as bm
from tests import bovitar_util as bu
from tests import plain_bovitar as pb
from tests import replay_util as ru

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: bu.write_tiny(name, tmp_path_factory.mktemp(f"bovitar_{name}")) for name in bu.CONFIGS}


# ---- one mechanism at a time --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, taps, rot, page, softcap, scaling", [
    (4, 2, 32, 16, 4, 8, 16, 5.0, (4.0, 1.0, 4.0, 64)),       # a partial rotation with stretched frequencies
    (2, 2, 16, 24, 2, 16, 16, None, None),                    # no soft cap; a full rotation
    (3, 1, 24, 24, 1, 0, 8, 3.0, None),                       # one tap, no rotation; sizes that are multiples of nothing
    (4, 2, 64, 64, 3, 32, 16, 8.0, (8.0, 1.0, 4.0, 128)),     # heads of 64: the tensor-core form
    (8, 2, 128, 64, 4, 128, 32, 20.0, None),                  # heads of 128, values half as wide, pages of 32
])
def test_attention_alone(tmp_path, dtype, heads, kv_heads, dim, vdim, taps, rot, page, softcap, scaling):
    bm.attention_case(tmp_path, dtype, "cuda", heads, kv_heads, dim, vdim, taps, rot, page, softcap, scaling,
                      repeat=heads == 4 and dim == 32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, taps", [
    (4, 2, 16, 24, 4), (2, 2, 32, 16, 1), (2, 1, 64, 128, 3)])
def test_gated_delta_rule_alone(tmp_path, dtype, heads, kv_heads, dim, vdim, taps):
    bm.delta_case(tmp_path, dtype, "cuda", heads, kv_heads, dim, vdim, taps, repeat=taps == 4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, vdim, state, groups, norm_groups, taps", [
    (4, 8, 16, 2, 2, 4), (1, 24, 8, 1, 1, 1), (6, 4, 20, 6, 3, 2), (4, 64, 128, 1, 2, 4), (2, 20, 200, 2, 1, 3)])
def test_state_space_recurrence_alone(tmp_path, dtype, heads, vdim, state, groups, norm_groups, taps):
    bm.state_space_case(tmp_path, dtype, "cuda", heads, vdim, state, groups, norm_groups, taps, repeat=heads == 4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts, top, ff, groups, shared, correction", [
    (12, 3, 20, (4, 2), 24, 0.5),
    (8, 2, 16, (2, 1), None, -2.0),       # every choice score negative: a group left out is minus infinity, not zero
    (5, 1, 24, None, 16, 0.5),            # one chosen expert, no groups
    (6, 6, 8, (3, 3), 8, -2.0),           # every expert chosen
    (64, 6, 32, (8, 3), 64, 0.5),         # many experts: most tiles hold one expert's few rows
])
def test_routed_experts_alone(tmp_path, dtype, experts, top, ff, groups, shared, correction):
    bm.experts_case(tmp_path, dtype, "cuda", experts, top, ff, groups, shared, correction)


# ---- the new kernels against their equations, at sizes the one-layer models do not reach --------------

@pytest.mark.parametrize("experts, top, count, keep", [(16, 3, 2, 1), (12, 3, 4, 2), (8, 8, 1, 1), (6, 1, 6, 3),
                                                        (64, 6, 8, 3), (256, 8, 8, 4), (10, 4, 5, 5)])
def test_the_softmax_router_alone(experts, top, count, keep):
    """The choice and the weights for many rows at once, corrections of both signs, against the plain
    router fed with the same logits (W = the identity)."""
    from deterministic_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(experts)
    for t, shift in ((1, 0.0), (77, 0.0), (700, -1.5)):
        logits = torch.randn(t, experts + 4, generator=g) * 1.5
        correction = torch.randn(experts, generator=g) * (0.5 / experts) + shift
        ids, weights = ops.route_experts(logits.cuda(), correction.cuda(), experts, top, count, keep, 2.5, 0.0,
                                         score="softmax", group_top=1, normalize=False)
        w = {"r.router": torch.eye(experts, dtype=torch.float64), "r.correction": correction.double()}
        c = {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": count, "keep": keep}}
        want_ids, want_w, masked = pb.route(logits[:, :experts].double(), w, "r.", c)
        got_ids = ids.long().cpu()
        # the same experts, up to calls closer than float32 resolves
        worst = masked.topk(top, dim=-1).values.min(-1).values - masked.gather(1, got_ids).min(-1).values
        assert float(worst.max()) < 1e-6
        same = (got_ids.sort(-1).values == want_ids.sort(-1).values).all(-1)
        got = {(r, int(e)): float(x) for r in range(t) for e, x in zip(got_ids[r], weights[r].cpu()) if same[r]}
        want = {(r, int(e)): float(x) for r in range(t) for e, x in zip(want_ids[r], want_w[r]) if same[r]}
        assert got.keys() == want.keys() and int(same.sum()) >= t - 2
        assert max(abs(got[k] - want[k]) for k in want) < 1e-5


class _Step:
    def __init__(self, lens, slots):
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        self.cu_q_lens = torch.tensor(cu, dtype=torch.int32, device="cuda")
        self.state_slots = torch.tensor(slots, dtype=torch.int32, device="cuda")
        self.token_seq = torch.tensor([b for b, n in enumerate(lens) for _ in range(n)], dtype=torch.int32,
                                      device="cuda")
        self.num_seqs = len(lens)


@pytest.mark.parametrize("heads, pdim, state, groups, parts, taps", [
    (8, 64, 128, 2, 2, 4), (3, 20, 24, 3, 1, 2), (16, 32, 64, 1, 4, 4), (2, 12, 256, 2, 2, 1), (2, 8, 300, 1, 1, 2)])
def test_the_state_space_kernels_alone(heads, pdim, state, groups, parts, taps):
    """Sequences of unequal lengths in one launch, then their next tokens from the state the launch
    left, against the plain recurrence over the whole sequences."""
    from deterministic_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(heads * 7 + state)
    inner, chan = heads * pdim, heads * pdim + 2 * groups * state
    width = (2 * inner + 2 * groups * state + heads + 7) // 8 * 8
    lens, more = [70, 1, 33, 2], [1, 5, 1, 40]
    w = {"m.in": torch.eye(width, dtype=torch.float64)[:2 * inner + 2 * groups * state + heads],
         "m.conv": torch.randn(chan, taps, generator=g).double() * 0.5,
         "m.conv.b": torch.randn(chan, generator=g).double() * 0.3,
         "m.dt_bias": torch.randn(heads, generator=g).double(), "m.A_log": torch.randn(heads, generator=g).double() - 1.0,
         "m.D": torch.randn(heads, generator=g).double(), "m.norm": 1.0 + 0.1 * torch.randn(inner, generator=g).double(),
         "m.o": torch.eye(inner, dtype=torch.float64)}
    c = {"heads": heads, "vdim": pdim, "state": state, "groups": groups, "norm_groups": parts}
    seqs = [torch.randn(a + b, width, generator=g) for a, b in zip(lens, more)]
    want = [pb.state_space_branch(s.double(), w, "m.", c, 1e-5) for s in seqs]
    f32 = lambda name: w[name].float().cuda().contiguous()
    slots = [3, 1, 4, 2]
    st = torch.zeros(5, heads * state * pdim + (taps - 1) * chan, device="cuda")
    st[0] = float("nan")               # slot 0 is no request's: nothing reads it
    got = [[] for _ in seqs]
    for part, counts in ((0, lens), (1, more)):
        rows = torch.cat([s[:lens[i]] if part == 0 else s[lens[i]:] for i, s in enumerate(seqs)]).cuda().contiguous()
        out = ops.state_space(rows, f32("m.conv"), f32("m.conv.b"), f32("m.A_log"), f32("m.dt_bias"), f32("m.D"),
                              f32("m.norm"), st, _Step(counts, slots), heads, pdim, state, groups, parts, taps, 1e-5,
                              torch.float32)
        at = 0
        for i, n in enumerate(counts):
            got[i].append(out[at:at + n].double().cpu())
            at += n
    for i, ref in enumerate(want):
        err = float((torch.cat(got[i]) - ref).abs().max())
        assert err <= 2e-5 * float(ref.abs().max()), (i, err)


@pytest.mark.parametrize("dtype", DTYPES)
def test_normed_branches_join_the_stream(dtype):
    """stream += a0 n0(x0) + a1 n1(x1), then the stream's norm: against the formula, for inputs of both
    storage types; and as a plain tensor."""
    from deterministic_inference_b200.kernels import ops
    dt = getattr(torch, dtype)
    g = torch.Generator().manual_seed(5)
    for rows, width in ((7, 72), (33, 1024), (3, 4100)):
        stream = torch.randn(rows, width, generator=g).cuda()
        x0, x1 = (torch.randn(rows, width, generator=g).to(dt).cuda() for _ in range(2))
        w0, w1, wn = (1.0 + 0.2 * torch.randn(width, generator=g).cuda() for _ in range(3))
        terms = ops.WeightedSum([(0.5, ops.NormedTerm(x0, w0, 1e-5)), (0.25, ops.NormedTerm(x1, w1, 1e-6))])
        want = stream.double() + 0.5 * pb.rms_norm(x0.double(), w0.double(), 1e-5) \
            + 0.25 * pb.rms_norm(x1.double(), w1.double(), 1e-6)
        assert float((terms.tensor().double() - (want - stream.double())).abs().max()) < 2e-5
        out = ops.stream_rms_norm(stream, wn, 1e-5, dt, add=terms)
        assert float((stream.double() - want).abs().max()) < 2e-5
        normed = pb.rms_norm(want, wn.double(), 1e-5)
        assert float((out.double() - normed).abs().max()) < (2e-5 if dtype == "float32" else 4e-2)


# ---- whole models ------------------------------------------------------------------------------------------

CASES = {       # configuration -> request lengths, seed
    "b1": ([1, 2, 17, 48, 131, 260], 31),
    "b2": ([5, 33, 64, 200], 32),
    "b3": ([3, 22, 57, 130, 333], 33),
    "b4": ([2, 30, 75, 180], 36),
}


@pytest.fixture(scope="module")
def plain_logits(model_dirs):
    out = {}
    for name, (lens, seed) in CASES.items():
        cfg, w = pb.read_model_dir(model_dirs[name])
        reqs = bu.requests(cfg["vocab"], lens, seed)
        out[name] = (cfg, reqs, [pb.forward(cfg, w, r) for r in reqs])
    return out


@pytest.mark.parametrize("name", list(CASES))
def test_whole_models_in_bfloat16_under_all_cuttings(name, model_dirs):
    """Through the engine's step function in this process, where the router's choices can be read: a
    bfloat16 engine may decide a close call the other way, and the plain implementation follows it."""
    cfg, _ = pb.read_model_dir(model_dirs[name])
    lens, seed = CASES[name]
    reqs = bu.requests(cfg["vocab"], [min(n, 200) for n in lens], seed)
    bm.compare(model_dirs[name], reqs, "bfloat16", "cuda", bu.CONFIGS[name]["page_size"], tail=110, what=name)


@pytest.mark.parametrize("name", list(CASES))
def test_replay_all_cuttings_in_float32(name, model_dirs, plain_logits, tmp_path):
    cfg, reqs, exact = plain_logits[name]
    trace = ru.Trace()
    ru.mixed(trace, reqs)                             # sizes the pool; four live requests at most
    ru.whole(trace, reqs)
    ru.last_one_by_one(trace, reqs, tail=150)         # long decoding
    ru.portions(trace, reqs)
    out = ru.run_trace(model_dirs[name], "float32", trace, tmp_path / "out", page_size=bu.CONFIGS[name]["page_size"])
    got = ru.read_rows(out, trace, cfg["vocab"])
    for kind in "mwtp":
        for i, r in enumerate(reqs):
            assert all((f"{kind}{i}", p) in got for p in range(len(r))), (kind, i)
    for (key, pos), row in got.items():
        i = int(key[1:])
        scale = float(exact[i].std())
        err = float(bm.row_errors(row, exact[i][pos]))
        assert err <= 1e-4 * scale, f"{name}: request {key} position {pos}: {err:.4g} exceeds {1e-4 * scale:.4g}"


def test_replay_with_captured_graphs(model_dirs, tmp_path):
    """The step function as generation runs it: pure-decode steps replayed as captured CUDA graphs."""
    name = "b1"
    cfg, w = pb.read_model_dir(model_dirs[name])
    same = bu.requests(cfg["vocab"], [120] * 4, 41)
    other = bu.requests(cfg["vocab"], [33, 150, 77], 42)
    reqs = same + other
    exact = [pb.forward(cfg, w, r) for r in reqs]
    trace = ru.Trace()
    for prefix in ("", "x"):
        ru.lockstep(trace, same, portion=48, tail=30, prefix=prefix)
    ru.mixed(trace, reqs)
    out = ru.run_trace(model_dirs[name], "float32", trace, tmp_path / "out", page_size=bu.CONFIGS[name]["page_size"],
                       cuda_graphs=True)
    for (key, pos), row in ru.read_rows(out, trace, cfg["vocab"]).items():
        i = int(key.lstrip("xyz")[1:])
        scale = float(exact[i].std())
        err = float(bm.row_errors(row, exact[i][pos]))
        assert err <= 1e-4 * scale, f"{name}: request {key} position {pos}: {err:.4g} exceeds {1e-4 * scale:.4g}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_stream_after_every_layer_run(dtype, model_dirs):
    """The residual stream stays float32 whatever the engine's type; a layer that runs twice counts twice."""
    d = model_dirs["b3"]
    cfg, w = pb.read_model_dir(d)
    (toks,) = bu.requests(cfg["vocab"], [40], 5)
    runner = bu.runner_for(d, dtype, "cuda", 8, [40], cuda_graphs=False)
    seen = []

    def hook(entry, hidden, residual):
        term = hidden.tensor() if hasattr(hidden, "tensor") else hidden
        assert residual.dtype == torch.float32
        seen.append((residual + term.float()).double().cpu())
    runner.model.after_layer = hook
    routes = {}
    bu.replay(runner, [toks], [[(0, 40)]], routes)
    runs = [i for i, layer in enumerate(cfg["layers"]) if layer.get("mlp") is not None]
    follow = {run: routes[0][k] for k, run in enumerate(runs)} if dtype == "bfloat16" else None
    want = []
    pb.forward(cfg, w, toks, rnd=pb.as_stored_bf16 if dtype == "bfloat16" else (lambda x: x), layers_out=want,
               follow=follow)
    assert len(seen) == len(want) == 5
    for i, (got, ref) in enumerate(zip(seen, want)):
        err, scale = float((got - ref).abs().max()), float(ref.abs().max())
        assert err <= (1e-4 if dtype == "float32" else 6e-2) * scale, f"layer run {i}: {err:.4g} of {scale:.4g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["b1", "b3"])
def test_greedy_generation_through_the_entry_point(name, dtype, model_dirs, tmp_path):
    from deterministic_inference_b200 import Engine, EngineConfig, SamplingParams
    d = model_dirs[name]
    if dtype == "bfloat16":
        # a bfloat16 router may decide a close call the other way, and every later token then differs; so
        # this engine's models choose all their experts (the float32 engines route as configured)
        config = copy.deepcopy(bu.CONFIGS[name]["config"])
        for layer in config["layers"]:
            if layer.get("mlp") is not None:
                layer["mlp"]["router"].update(top=layer["mlp"]["router"]["experts"], groups=None)
        d = bu.write_model(config, bu.CONFIGS[name]["seed"], tmp_path / "all_experts")
    cfg, w = pb.read_model_dir(d)
    prompts = bu.requests(cfg["vocab"], [3, 40, 9, 77, 15], 9)
    new = 40
    eng = Engine(EngineConfig(model_path=str(d), dtype=dtype, kv_pool_tokens=384, page_size=bu.CONFIGS[name]["page_size"],
                              max_reqs=3, max_seq_len=160, max_prefill_tokens=48))
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    eng.cache.check_invariants()
    spread = math.sqrt(2.0)
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == new
        ids = list(p)
        for t in o.token_ids:
            logits = pb.forward(cfg, w, ids)[-1]
            best = int(torch.argmax(logits))
            if t != best:
                # another token only where rounding can flip the choice; from there on the
                # engine's own continuation is followed
                gap = float(logits[best] - logits[t])
                assert dtype == "bfloat16" and gap < 0.25 * spread, f"token {t} instead of {best}, logits {gap:.3g} apart"
            ids.append(t)
