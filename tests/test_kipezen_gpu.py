"""The Kipezen design on the GPU against the plain implementation of ``tests/plain_kipezen.py``:
each mechanism alone (``tests/kipezen_mechanisms.py``: one-layer models whose weights and prompts
make a wrong edge, a lost state or a left-out group show, under every cutting of the engine's step
function), then whole models under the same cuttings (whole prompts, the last tokens one by one over
more tokens than the windows are long, portions down to two tokens, mixed batches in a pool so small
that pages and slots are used again): float32 through ``bin/trace_run``, bfloat16 through the step
function in this process, where the router's choices can be read and followed; the router and the
experts' products against their equations at sizes the one-layer models do not reach; and greedy
generation through ``Engine.generate``."""

import pytest
import torch

from tests import kipezen_mechanisms as km
from tests import kipezen_util as ku
from tests import plain_kipezen as pk
from tests import replay_util as ru

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: ku.write_tiny(name, tmp_path_factory.mktemp(f"kipezen_{name}")) for name in ku.CONFIGS}


# ---- one mechanism at a time --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, keep, rot, page", [
    (4, 2, 32, 16, 40, 6, 8, 16),         # edges inside pages
    (2, 2, 16, 24, 32, 16, 16, 16),       # a window of two pages, kept keys of one; a full rotation
    (3, 1, 24, 24, 21, 0, 12, 8),         # no kept keys; sizes that are multiples of nothing
    (2, 1, 16, 16, 9, 30, 4, 8),          # kept keys reach beyond the window
    (4, 2, 64, 64, 50, 19, 32, 16),       # heads of 64: the tensor-core kernels
    (8, 2, 128, 64, 33, 17, 64, 32),      # heads of 128, values half as wide, pages of 32
])
def test_windowed_attention_alone(tmp_path, dtype, heads, kv_heads, dim, vdim, window, keep, rot, page):
    km.attention_case(tmp_path, dtype, "cuda", heads, kv_heads, dim, vdim, window, keep, rot, page)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, vdim, taps", [
    (4, 2, 16, 24, 4), (2, 2, 32, 16, 1), (3, 1, 8, 8, 2), (2, 1, 64, 128, 3), (4, 4, 128, 64, 2)])
def test_gated_delta_rule_alone(tmp_path, dtype, heads, kv_heads, dim, vdim, taps):
    km.delta_case(tmp_path, dtype, "cuda", heads, kv_heads, dim, vdim, taps)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width, blocks, taps", [(40, 2, 3), (24, 1, 1), (36, 6, 4), (256, 4, 2)])
def test_gated_linear_recurrence_alone(tmp_path, dtype, width, blocks, taps):
    km.recurrence_case(tmp_path, dtype, "cuda", width, blocks, taps)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts, top, ff, groups, shared, correction", [
    (12, 3, 20, (4, 2), 24, 0.5),
    (8, 2, 16, (2, 1), None, -2.0),       # every choice score negative: a group left out is minus infinity, not zero
    (5, 1, 24, None, 16, 0.5),            # one chosen expert, no groups
    (6, 6, 8, (3, 3), 8, -2.0),           # every expert chosen
    (64, 6, 32, (8, 3), 64, 0.5),         # many experts: most tiles hold one expert's few rows
])
def test_routed_experts_alone(tmp_path, dtype, experts, top, ff, groups, shared, correction):
    km.experts_case(tmp_path, dtype, "cuda", experts, top, ff, groups, shared, correction)


@pytest.mark.parametrize("experts, top, count, keep", [(16, 3, 2, 1), (12, 3, 4, 2), (8, 8, 1, 1), (6, 1, 6, 3),
                                                        (64, 6, 8, 3), (256, 8, 8, 4), (10, 4, 5, 5)])
def test_the_router_alone(experts, top, count, keep):
    """The choice and the weights for many rows at once, corrections of both signs, against the plain
    router fed with the same logits (W = the identity)."""
    from deterministic_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(experts)
    for t, shift in ((1, 0.0), (77, 0.0), (700, -1.5)):
        logits = torch.randn(t, experts + 4, generator=g) * 1.5
        correction = torch.randn(experts, generator=g) * 0.4 + shift
        ids, weights = ops.route_experts(logits.cuda(), correction.cuda(), experts, top, count, keep, 2.5, 1e-20)
        w = {"r.router": torch.eye(experts, dtype=torch.float64), "r.correction": correction.double()}
        c = {"router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": count, "keep": keep}}}
        want_ids, want_w, _ = pk.route(logits[:, :experts].double(), w, "r.", c)
        got = {(r, int(e)): float(x) for r in range(t) for e, x in zip(ids[r].cpu(), weights[r].cpu())}
        want = {(r, int(e)): float(x) for r in range(t) for e, x in zip(want_ids[r], want_w[r])}
        assert got.keys() == want.keys()
        assert max(abs(got[k] - want[k]) for k in want) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts, top, width, ff, rows", [(8, 2, 256, 128, 700), (32, 4, 128, 64, 3000), (4, 4, 64, 40, 5),
                                                           (8, 2, 512, 384, 2100), (3, 1, 256, 128, 1000)])
def test_the_experts_products_alone(dtype, experts, top, width, ff, rows):
    """The grouped products at row counts that fill large tiles, and a row's independence of the step:
    the same token gives the same bits alone and among thousands."""
    from deterministic_inference_b200.kernels import ops
    dt = getattr(torch, dtype)
    rnd = pk.as_stored_bf16 if dtype == "bfloat16" else (lambda x: x)
    g = torch.Generator().manual_seed(rows)
    x = pk.as_stored_bf16(torch.randn(rows, width, generator=g))
    w = {}
    for e in range(experts):
        w[f"m.e{e}.gate"] = pk.as_stored_bf16(torch.randn(ff, width, generator=g) * width ** -0.5).double()
        w[f"m.e{e}.up"] = pk.as_stored_bf16(torch.randn(ff, width, generator=g) * width ** -0.5).double()
        w[f"m.e{e}.down"] = pk.as_stored_bf16(torch.randn(width, ff, generator=g) * ff ** -0.5).double()
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).int()
    weights = torch.rand(rows, top, generator=g) + 0.2
    gate_up = torch.stack([torch.cat([w[f"m.e{e}.gate"], w[f"m.e{e}.up"]]) for e in range(experts)]).to(dt).cuda()
    down = torch.stack([w[f"m.e{e}.down"] for e in range(experts)]).to(dt).cuda()
    got = ops.routed_experts(x.to(dt).cuda(), ids.cuda(), weights.cuda(), gate_up, down, None, None, experts, dt)
    assert got.dtype == torch.float32
    check = list(range(0, rows, max(rows // 40, 1)))
    want = torch.stack([sum(weights[r, j].double() * pk.expert(x[r:r + 1].double(), w, f"m.e{int(ids[r, j])}.", rnd)[0]
                            for j in range(top)) for r in check])
    err = float((got[check].double().cpu() - want).abs().max())
    assert err <= (2e-5 if dtype == "float32" else 2e-2) * float(want.abs().max()), err
    few = ops.routed_experts(x[:3].to(dt).cuda(), ids[:3].cuda(), weights[:3].cuda(), gate_up, down, None, None,
                             experts, dt)
    on_tensor_cores = dtype == "bfloat16" and rows * top >= ops.EXPERT_TILE_ROWS_TC * experts and ff % 128 == 0 \
        and width % 256 == 0
    if on_tensor_cores:       # another kernel form for many rows: the same up to rounding
        assert float((few - got[:3]).abs().max()) <= 1e-2 * float(got[:3].abs().max())
    else:
        assert torch.equal(few, got[:3])


# ---- whole models ------------------------------------------------------------------------------------------

CASES = {       # configuration -> request lengths, seed
    "k1": ([1, 2, 17, 48, 131, 260], 31),
    "k2": ([5, 33, 64, 200], 32),
    "k3": ([3, 22, 57, 130, 333], 33),
    "k4": ([1, 9, 40, 150, 300], 34),
    "k5": ([2, 30, 75, 180], 36),
    "k6": ([40, 300, 520], 37),
}


def row_error(got, want):
    return float(km.row_errors(got, want))


@pytest.fixture(scope="module")
def plain_logits(model_dirs):
    out = {}
    for name, (lens, seed) in CASES.items():
        cfg, w = pk.read_model_dir(model_dirs[name])
        reqs = ku.requests(cfg["vocab"], lens, seed)
        exact = [pk.forward(cfg, w, r) for r in reqs]
        stored = [pk.forward(cfg, w, r, bf16_storage=True) for r in reqs]
        out[name] = (cfg, reqs, exact, stored)
    return out


@pytest.mark.parametrize("name", list(CASES))
def test_whole_models_in_bfloat16_under_all_cuttings(name, model_dirs):
    """Through the engine's step function in this process, where the router's choices can be read: a
    bfloat16 engine may decide a close call the other way, and the plain implementation follows it."""
    cfg, _ = pk.read_model_dir(model_dirs[name])
    lens, seed = CASES[name]
    reqs = ku.requests(cfg["vocab"], [min(n, 200) if name != "k6" else n for n in lens], seed)
    km.compare(model_dirs[name], reqs, "bfloat16", "cuda", ku.CONFIGS[name]["page_size"], tail=110, what=name)


@pytest.mark.parametrize("dtype", ["float32"])
@pytest.mark.parametrize("name", list(CASES))
def test_replay_all_cuttings(name, dtype, model_dirs, plain_logits, tmp_path):
    cfg, reqs, exact, stored = plain_logits[name]
    trace = ru.Trace()
    ru.mixed(trace, reqs)                             # sizes the pool; four live requests at most
    ru.whole(trace, reqs)
    ru.last_one_by_one(trace, reqs, tail=150)         # decoding over more tokens than any window is long
    ru.portions(trace, reqs)
    out = ru.run_trace(model_dirs[name], dtype, trace, tmp_path / "out", page_size=ku.CONFIGS[name]["page_size"])
    got = ru.read_rows(out, trace, cfg["vocab"])
    for kind in "mwtp":
        for i, r in enumerate(reqs):
            assert all((f"{kind}{i}", p) in got for p in range(len(r))), (kind, i)
    worst = 0.0
    for (key, pos), row in got.items():
        i = int(key[1:])
        scale = float(exact[i].std())
        err = row_error(row, exact[i][pos])
        if dtype == "float32":
            bound = 1e-4 * scale
        else:
            # what bfloat16 storage alone does to this request's logits, three times over
            yard = max(row_error(a, b) for a, b in zip(stored[i], exact[i]))
            bound = max(3.0 * yard, 2e-2 * scale)
        assert err <= bound, f"{name}/{dtype}: request {key} position {pos}: {err:.4g} exceeds {bound:.4g}"
        worst = max(worst, err / scale)
    print(f"{name}/{dtype}: worst difference {worst:.3e} of the logits' spread")


@pytest.mark.parametrize("name, dtype", [("k4", "float32"), ("k1", "float32")])
def test_replay_with_captured_graphs(name, dtype, model_dirs, tmp_path):
    """The step function as generation runs it: pure-decode steps (and, where the design's state allows,
    steps whose shape has come twice before) replayed as captured CUDA graphs, against the plain
    implementation (float32: a replayed graph does not show its router's choices; the bfloat16 engine
    replays graphs in the generation test below)."""
    cfg, w = pk.read_model_dir(model_dirs[name])
    same = ku.requests(cfg["vocab"], [120] * 4, 41)
    other = ku.requests(cfg["vocab"], [33, 150, 77], 42)
    reqs = same + other
    exact = [pk.forward(cfg, w, r) for r in reqs]
    stored = [pk.forward(cfg, w, r, bf16_storage=True) for r in reqs]
    trace = ru.Trace()
    for prefix, portion in {"": 48, "x": 48, "y": 48}.items():
        ru.lockstep(trace, same, portion=portion, prefix=prefix)
    ru.mixed(trace, reqs)
    out = ru.run_trace(model_dirs[name], dtype, trace, tmp_path / "out", page_size=ku.CONFIGS[name]["page_size"],
                       cuda_graphs=True)
    for (key, pos), row in ru.read_rows(out, trace, cfg["vocab"]).items():
        i = int(key.lstrip("xyz")[1:])
        scale = float(exact[i].std())
        err = row_error(row, exact[i][pos])
        yard = max(row_error(a, b) for a, b in zip(stored[i], exact[i]))
        bound = 1e-4 * scale if dtype == "float32" else max(3.0 * yard, 2e-2 * scale)
        assert err <= bound, f"{name}/{dtype}: request {key} position {pos}: {err:.4g} exceeds {bound:.4g}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_stream_after_every_layer(dtype, model_dirs):
    """The residual stream stays float32 whatever the engine's type."""
    d = model_dirs["k4"]
    cfg, w = pk.read_model_dir(d)
    (toks,) = ku.requests(cfg["vocab"], [40], 5)
    runner = ku.runner_for(d, dtype, "cuda", 16, [40], cuda_graphs=False)
    seen = []

    def hook(entry, hidden, residual):
        term = hidden.tensor() if hasattr(hidden, "tensor") else hidden
        assert residual.dtype == torch.float32
        seen.append((residual + term.float()).double().cpu())
    runner.model.after_layer = hook
    routes = {}
    ku.replay(runner, [toks], [[(0, 40)]], routes)
    moe_layers = [i for i, layer in enumerate(cfg["layers"]) if layer.get("mlp") is not None]
    forced = {layer: routes[0][k] for k, layer in enumerate(moe_layers)} if dtype == "bfloat16" else None
    _, want = pk.forward(cfg, w, toks, bf16_storage=dtype == "bfloat16", return_layers=True, forced=forced)
    assert len(seen) == want.shape[0]
    for i, (got, ref) in enumerate(zip(seen, want)):
        err, scale = float((got - ref).abs().max()), float(ref.abs().max())
        assert err <= (1e-4 if dtype == "float32" else 6e-2) * scale, f"layer {i}: {err:.4g} of {scale:.4g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["k1", "k4"])
def test_greedy_generation_through_the_entry_point(name, dtype, model_dirs):
    from deterministic_inference_b200 import Engine, EngineConfig, SamplingParams
    d = model_dirs[name]
    cfg, w = pk.read_model_dir(d)
    prompts = ku.requests(cfg["vocab"], [3, 40, 9, 77, 15], 9)
    new = 40
    eng = Engine(EngineConfig(model_path=str(d), dtype=dtype, kv_pool_tokens=384, page_size=ku.CONFIGS[name]["page_size"],
                              max_reqs=3, max_seq_len=160, max_prefill_tokens=48))
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    eng.cache.check_invariants()
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == new
        ids = list(p)
        for t in o.token_ids:
            logits = pk.forward(cfg, w, ids)[-1]
            best = int(torch.argmax(logits))
            if t != best:
                # another token only where rounding can flip the choice; from there on the
                # engine's own continuation is followed
                gap = float(logits[best] - logits[t])
                assert dtype == "bfloat16" and gap < 0.25, f"token {t} instead of {best}, logits {gap:.3g} apart"
            ids.append(t)
