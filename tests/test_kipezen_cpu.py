"""The Kipezen design without a GPU: configuration and registry, weights, the cache manager's share
(a window's pages with kept first keys, state slots of two kinds beside paged keys), and the engine's
host logic with the kernel wrappers replaced by plain PyTorch restatements (fixture ``torch_ops``),
against the plain implementation of ``tests/plain_kipezen.py``."""

import copy

import pytest
import torch

from deterministic_inference_b200.cache.manager import CacheManager
from deterministic_inference_b200.config import EngineConfig, SamplingParams
from deterministic_inference_b200.config.kipezen_config import KipezenConfig
from deterministic_inference_b200.config.model_config import ConfigError
from deterministic_inference_b200.engine import Engine, ModelRunner, SequenceInput
from deterministic_inference_b200.models.registry import build_model, config_from_dir
from deterministic_inference_b200.parts.spec import CompositeSpec, PagedKVSpec, StateSpec
from deterministic_inference_b200.weights.loader import WeightsError, load_weights
from tests import kipezen_mechanisms as km
from tests import kipezen_util as ku
from tests import plain_kipezen as pk


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: ku.write_tiny(name, tmp_path_factory.mktemp(f"kipezen_{name}")) for name in ku.CONFIGS}


# ---- configuration, registry, weights ---------------------------------------------------------

def test_the_registry_picks_the_design_by_its_name_and_reads_every_size(model_dirs):
    cfg = config_from_dir(model_dirs["k1"])
    assert isinstance(cfg, KipezenConfig)
    raw = ku.CONFIGS["k1"]["config"]
    assert (cfg.vocab, cfg.width, cfg.norm_eps) == (150, 72, 2e-5)
    plan = cfg.plan()
    assert [l.mixer.kind for l in plan.layers] == ["parallel", "gated_delta_rule", "gated_delta_rule"]
    assert [l.feed_forward.kind for l in plan.layers] == ["routed_experts", "routed_experts", "none"]
    left, right = plan.layers[0].mixer.params["branches"]
    a = left.params
    assert (a["num_heads"], a["num_kv_heads"], a["head_dim"], a["v_head_dim"]) == (6, 3, 20, 12)
    assert (a["mask"], a["mask_size"], a["keep_first"], a["bias"]) == ("window", 13, 5, True)
    assert (a["qk_norm_scope"], a["rotary_layout"], a["qk_norm_eps"]) == ("projection", "pairs", 2e-5)
    assert a["position_encoding"].params["rotary_dim"] == 10 and a["position_encoding"].params["theta"] == 777.0
    b = right.params
    assert (b["width"], b["blocks"], b["conv_taps"], b["decay_scale"]) == (60, 3, 4, 8.0)
    assert plan.layers[0].mixer.params["scales"] == [0.7, 1.3]
    d = plan.layers[1].mixer.params
    assert (d["num_heads"], d["num_kv_heads"], d["head_dim"], d["v_head_dim"], d["conv_taps"]) == (3, 1, 24, 40, 4)
    f = plan.layers[0].feed_forward.params
    assert (f["num_experts"], f["top"], f["intermediate_size"], f["route_scale"]) == (6, 3, 28, 1.5)
    assert (f["group_count"], f["group_keep"], f["shared_intermediate_size"]) == (3, 2, 36)
    g = plan.layers[1].feed_forward.params          # no groups given: one group of all experts, no shared expert
    assert (g["group_count"], g["group_keep"], g["shared_intermediate_size"]) == (1, 1, None)
    assert KipezenConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.to_dict()["layers"] == raw["layers"]
    model = build_model(cfg, torch.float32, "cpu")
    assert sum(int(torch.tensor(s.shape).prod()) for s in model.tensor_specs()) == cfg.num_parameters()


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=2), "multiple"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(blocks=7), "blocks"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_a_configuration_that_cannot_run_is_refused_with_the_reason(change, text):
    raw = copy.deepcopy(ku.CONFIGS["k1"]["config"])
    change(raw)
    with pytest.raises(ConfigError) as e:
        KipezenConfig.from_dict(raw)
    assert text in str(e.value)


def test_missing_and_misshapen_tensors_are_listed(model_dirs, tmp_path):
    from safetensors.torch import load_file, save_file
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text((model_dirs["k1"] / "config.json").read_text())
    tensors = load_file(str(model_dirs["k1"] / "model.safetensors"))
    del tensors["l0.mix.right.lam"], tensors["l1.mix.q.conv"], tensors["l0.mlp.correction"]
    tensors["l0.mix.left.q.norm"] = tensors["l0.mix.left.q.norm"][:20].contiguous()     # one head's, not all rows'
    save_file(tensors, str(d / "model.safetensors"))
    model = build_model(config_from_dir(d), torch.float32, "cpu")
    with pytest.raises(WeightsError) as e:
        load_weights(d, model.tensor_specs(), model.plan, torch.float32, "cpu")
    assert all(n in str(e.value) for n in ("l0.mix.right.lam", "l1.mix.q.conv", "l0.mlp.correction",
                                           "l0.mix.left.q.norm"))


# ---- cache manager ----------------------------------------------------------------------------------

def test_pages_of_kept_first_keys_stay_while_the_window_moves_on():
    spec = PagedKVSpec(2, 8, window=20, v_head_dim=12, keep_first=11)
    assert spec.group_key() != PagedKVSpec(2, 8, window=20, v_head_dim=12).group_key()
    cm = CacheManager({0: spec}, num_pages=12, page_size=8, max_reqs=3, max_seq_len=88, allocate_device=False)
    (g,) = cm.page_groups.values()
    s = cm.allocate_slot()
    cm.allocate(s, 60)
    # a query at 60 reads keys 41..60 and 0..10: pages 2, 3 and 4 (positions 16..39) go back, 0 and 1 stay
    assert cm.release_passed(s, 60) == 3
    assert [p != 0 for p in g.pages[s]] == [True, True, False, False, False, True, True, True]
    cm.allocate(s, 75)
    assert cm.release_passed(s, 75) == 2          # keys from 56 on: pages 5 and 6 (40..55)
    cm.check_invariants()
    # the freed pages serve another request while the first goes on
    t = cm.allocate_slot()
    cm.allocate(t, 40)
    assert set(g.pages[t]) & set(g.pages[s]) <= {0}
    cm.release_slot(s)
    cm.release_slot(t)
    cm.check_invariants()
    assert g.num_free == 11
    # kept keys that end on a page's border keep exactly those pages
    cm2 = CacheManager({0: PagedKVSpec(1, 8, window=9, keep_first=16)}, num_pages=12, page_size=8, max_reqs=2,
                       max_seq_len=88, allocate_device=False)
    u = cm2.allocate_slot()
    cm2.allocate(u, 50)
    assert cm2.release_passed(u, 50) == 3         # keys from 42 on: pages 2, 3, 4; page 5 holds 40..47
    (g2,) = cm2.page_groups.values()
    assert [p != 0 for p in g2.pages[u]] == [True, True, False, False, False, True, True]


def test_the_cache_of_every_layer_kind(model_dirs):
    cfg = config_from_dir(model_dirs["k1"])
    model = build_model(cfg, torch.float32, "cpu")
    specs = model.cache_specs()
    assert len(specs) == 3
    both = specs[0]
    assert isinstance(both, CompositeSpec)
    assert both.members[0] == PagedKVSpec(3, 20, window=13, v_head_dim=12, keep_first=5)
    assert both.members[1] == StateSpec((4 * 60,), "float32")                 # the state and three earlier inputs
    # delta: three heads of a 24 x 40 state, then three earlier inputs of the q, k and v channels
    assert specs[1] == StateSpec((3 * 24 * 40 + 3 * (24 + 24 + 120),), "float32")
    assert specs[2] == StateSpec((4 * 12 * 20 + 1 * (24 + 24 + 80),), "float32")
    # one tap: nothing of the convolution is kept
    one_tap = build_model(config_from_dir(model_dirs["k2"]), torch.float32, "cpu").cache_specs()
    assert one_tap[0] == StateSpec((2 * 32 * 32,), "float32")
    assert one_tap[1].members[1] == StateSpec((40,), "float32")


# ---- one mechanism at a time, through the engine's step function on the CPU ---------------------------

@pytest.mark.parametrize("heads, kv_heads, dim, vdim, window, keep, rot, page", [
    (4, 2, 32, 16, 40, 6, 8, 16),         # edges inside pages
    (2, 2, 16, 24, 32, 16, 16, 16),       # a window of two pages, kept keys of one; a full rotation
    (3, 1, 24, 24, 21, 0, 12, 8),         # no kept keys
    (2, 1, 16, 16, 9, 30, 4, 8),          # kept keys reach beyond the window
])
def test_windowed_attention_alone(tmp_path, torch_ops, heads, kv_heads, dim, vdim, window, keep, rot, page):
    km.attention_case(tmp_path, "float32", "cpu", heads, kv_heads, dim, vdim, window, keep, rot, page)


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, taps", [(4, 2, 16, 24, 4), (2, 2, 32, 16, 1), (3, 1, 8, 8, 2)])
def test_gated_delta_rule_alone(tmp_path, torch_ops, heads, kv_heads, dim, vdim, taps):
    km.delta_case(tmp_path, "float32", "cpu", heads, kv_heads, dim, vdim, taps)


@pytest.mark.parametrize("width, blocks, taps", [(40, 2, 3), (24, 1, 1), (36, 6, 4)])
def test_gated_linear_recurrence_alone(tmp_path, torch_ops, width, blocks, taps):
    km.recurrence_case(tmp_path, "float32", "cpu", width, blocks, taps)


@pytest.mark.parametrize("experts, top, ff, groups, shared, correction", [
    (12, 3, 20, (4, 2), 24, 0.5),
    (8, 2, 16, (2, 1), None, -2.0),       # every choice score negative: a group left out is minus infinity, not zero
    (5, 1, 24, None, 16, 0.5),            # one chosen expert, no groups
    (6, 6, 8, (3, 3), 8, -2.0),           # every expert chosen
])
def test_routed_experts_alone(tmp_path, torch_ops, experts, top, ff, groups, shared, correction):
    km.experts_case(tmp_path, "float32", "cpu", experts, top, ff, groups, shared, correction)


# ---- whole models: the engine's host logic on the CPU -------------------------------------------------

@pytest.mark.parametrize("name", list(ku.CONFIGS))
def test_cuttings_batches_and_reused_slots_on_cpu(name, model_dirs, torch_ops):
    d = model_dirs[name]
    cfg, w = pk.read_model_dir(d)
    lens = [70, 41, 2, 26, 55]
    reqs = ku.requests(cfg["vocab"], lens, 3)
    exact = [pk.forward(cfg, w, r) for r in reqs]
    for what, steps in ku.schedules(lens, tail=45).items():
        runner = ku.runner_for(d, "float32", "cpu", ku.CONFIGS[name]["page_size"], lens)
        got = ku.replay(runner, reqs, steps)
        for i, (g, e) in enumerate(zip(got, exact)):
            err = km.row_errors(g, e)
            assert float(err.max()) <= 1e-4 * float(e.std()), (name, what, i, int(err.argmax()), float(err.max()))


def test_the_stream_after_every_layer(model_dirs, torch_ops):
    """The float32 residual stream (pending term added) after each layer."""
    from tests.torch_kernels import _plain
    d = model_dirs["k4"]
    cfg, w = pk.read_model_dir(d, torch.float32)
    (toks,) = ku.requests(cfg["vocab"], [19], 5)
    _, want = pk.forward(cfg, w, toks, return_layers=True)
    runner = ku.runner_for(d, "float32", "cpu", 16, [19])
    seen = []
    runner.model.after_layer = lambda e, hidden, residual: seen.append(residual + _plain(hidden))
    s = runner.cache.allocate_slot()
    runner.step([SequenceInput(s, toks, 0, [18])])
    assert len(seen) == want.shape[0] == 5
    for i, (got, ref) in enumerate(zip(seen, want)):
        assert got.dtype == torch.float32
        torch.testing.assert_close(got, ref, atol=3e-4, rtol=1e-4, msg=lambda m, i=i: f"layer {i}: {m}")


def generate_plain(cfg, w, prompt, new):
    ids = list(prompt)
    for _ in range(new):
        ids.append(int(torch.argmax(pk.forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]


def test_greedy_generation_through_the_entry_point_on_cpu(model_dirs, torch_ops):
    d = model_dirs["k3"]
    cfg, w = pk.read_model_dir(d, torch.float32)
    prompts = ku.requests(cfg["vocab"], [3, 20, 9], 7)
    want = [generate_plain(cfg, w, p, 10) for p in prompts]
    eng = Engine(EngineConfig(model_path=str(d), dtype="float32", device="cpu", kv_pool_tokens=96, page_size=8,
                              max_reqs=2, max_seq_len=64, max_prefill_tokens=12, cuda_graphs=False,
                              async_scheduling=False))
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=10, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    eng.cache.check_invariants()


def test_the_command_line_writes_a_model_folder_the_registry_reads_back(tmp_path):
    from deterministic_inference_b200.__main__ import main
    from deterministic_inference_b200.config import preset
    cfg = preset("kipezen_tiny")
    assert isinstance(cfg, KipezenConfig)
    out = tmp_path / "model"
    assert main(["random", "--preset", "kipezen_tiny", "--seed", "3", "--out", str(out)]) == 0
    back = config_from_dir(out)
    assert back.to_dict() == cfg.to_dict()
    model = build_model(back, torch.float32, "cpu")
    load_weights(out, model.tensor_specs(), model.plan, torch.float32, "cpu")
