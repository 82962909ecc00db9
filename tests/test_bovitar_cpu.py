"""The Bovitar design without a GPU: configuration and registry, weights, the cache manager's share
(pages and a convolution tail for the attention inside a pair of mixers, state slots, a cache of its
own for a layer that runs with another's weights), and the engine's host logic with the kernel
wrappers replaced by plain PyTorch restatements (fixture ``torch_ops``), against the plain
implementation of ``tests/plain_bovitar.py``."""

import copy

import pytest
import torch

from deterministic_inference_b200.cache.manager import CacheManager
from deterministic_inference_b200.config import EngineConfig, SamplingParams
from deterministic_inference_b200.config.bovitar_config import BovitarConfig
from deterministic_inference_b200.config.model_config import ConfigError
from deterministic_inference_b200.engine import Engine, SequenceInput
from deterministic_inference_b200.models.registry import build_model, config_from_dir
from deterministic_inference_b200.parts.spec import CompositeSpec, PagedKVSpec, StateSpec, flatten_cache_specs
from deterministic_inference_b200.weights.loader import WeightsError, load_weights
from tests import bovitar_mechanisms as bm
from tests import bovitar_util as bu
from tests import plain_bovitar as pb


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {name: bu.write_tiny(name, tmp_path_factory.mktemp(f"bovitar_{name}")) for name in bu.CONFIGS}


# ---- configuration, registry, weights ---------------------------------------------------------

def test_the_registry_picks_the_design_by_its_name_and_reads_every_size(model_dirs):
    cfg = config_from_dir(model_dirs["b1"])
    assert isinstance(cfg, BovitarConfig)
    raw = bu.CONFIGS["b1"]["config"]
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.logit_scale) == (150, 72, 2e-5, 0.7)
    plan = cfg.plan()
    # four layer runs on three layers with tensors: the last run uses the first layer's
    assert [l.mixer.kind for l in plan.layers] == ["parallel", "gated_delta_rule", "gated_delta_rule"]
    assert [(e.layer, e.cache) for e in plan.schedule] == [(0, 0), (1, 1), (2, 2), (0, 3)]
    assert [l.feed_forward.kind for l in plan.layers] == ["routed_experts", "routed_experts", "none"]
    assert [l.block.kind for l in plan.layers] == ["pre_norm_f32_stream"] * 3
    mix = plan.layers[0].mixer.params
    assert mix["scales"] == [0.5, 0.5]
    assert [n["name"] for n in mix["branch_norms"]] == ["l0.mix.left.out", "l0.mix.right.out"]
    left, right = mix["branches"]
    a = left.params
    assert (a["num_heads"], a["num_kv_heads"], a["head_dim"], a["v_head_dim"], a["conv_taps"]) == (6, 3, 20, 12, 4)
    assert (a["mask"], a["softcap"], a["qk_norm_scope"], a["rotary_layout"], a["qk_norm_eps"]) == \
        ("causal", 4.0, "projection", "halves", 2e-5)
    rope = a["position_encoding"].params
    assert (rope["rotary_dim"], rope["theta"]) == (10, 777.0)
    assert rope["scaling"] == {"factor": 3.0, "low": 1.0, "high": 5.0, "original": 24}
    b = right.params
    assert (b["num_heads"], b["head_dim"], b["state_dim"], b["groups"], b["norm_groups"], b["conv_taps"]) == \
        (6, 10, 12, 3, 2, 3)
    d = plan.layers[1].mixer.params
    assert (d["num_heads"], d["num_kv_heads"], d["head_dim"], d["v_head_dim"], d["conv_taps"]) == (3, 1, 24, 40, 4)
    f = plan.layers[0].feed_forward.params
    assert (f["num_experts"], f["top"], f["intermediate_size"], f["route_scale"]) == (6, 3, 28, 1.5)
    assert (f["group_count"], f["group_keep"], f["shared_intermediate_size"]) == (3, 2, 36)
    assert (f["score"], f["group_top"], f["normalize"], f["shared_gate"]) == ("softmax", 1, False, False)
    g = plan.layers[1].feed_forward.params          # no groups given: one group of all experts, no shared expert
    assert (g["group_count"], g["group_keep"], g["shared_intermediate_size"]) == (1, 1, None)
    assert plan.head.params["scale"] == 0.7 and plan.head.params["name"] == "head"
    assert BovitarConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.to_dict()["layers"] == raw["layers"]
    model = build_model(cfg, torch.float32, "cpu")
    assert sum(int(torch.tensor(s.shape).prod()) for s in model.tensor_specs()) == cfg.num_parameters()
    assert not any(s.name.startswith("l3.") for s in model.tensor_specs())


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("low"), "scaling"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(softcap=0.0), "softcap"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=2), "multiple"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(groups=4), "groups"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(norm_groups=7), "equal parts"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][3].update(weights_of=9), "weights_of"),
    (lambda c: c["layers"][3].update(weights_of=1), "differs"),
    (lambda c: c["layers"][0].update(weights_of=3), "circle"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_a_configuration_that_cannot_run_is_refused_with_the_reason(change, text):
    raw = copy.deepcopy(bu.CONFIGS["b1"]["config"])
    change(raw)
    with pytest.raises(ConfigError) as e:
        BovitarConfig.from_dict(raw)
    assert text in str(e.value)


def test_missing_and_misshapen_tensors_are_listed(model_dirs, tmp_path):
    from safetensors.torch import load_file, save_file
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text((model_dirs["b1"] / "config.json").read_text())
    tensors = load_file(str(model_dirs["b1"] / "model.safetensors"))
    del tensors["l0.mix.right.D"], tensors["l0.mix.left.k.conv"], tensors["l0.mlp.correction"], tensors["head"]
    tensors["l0.mix.left.q.norm"] = tensors["l0.mix.left.q.norm"][:20].contiguous()     # one head's, not all rows'
    tensors["l3.norm1"] = tensors["l0.norm1"].clone()       # a layer that runs with another's weights has none
    save_file(tensors, str(d / "model.safetensors"))
    model = build_model(config_from_dir(d), torch.float32, "cpu")
    with pytest.raises(WeightsError) as e:
        load_weights(d, model.tensor_specs(), model.plan, torch.float32, "cpu")
    assert all(n in str(e.value) for n in ("l0.mix.right.D", "l0.mix.left.k.conv", "l0.mlp.correction", "head",
                                           "l0.mix.left.q.norm", "l3.norm1"))


# ---- cache manager ----------------------------------------------------------------------------------

def test_the_cache_of_every_layer_run(model_dirs):
    cfg = config_from_dir(model_dirs["b1"])
    model = build_model(cfg, torch.float32, "cpu")
    specs = model.cache_specs()
    assert sorted(specs) == [0, 1, 2, 3]           # the run with another layer's weights has a cache of its own
    both = specs[0]
    assert isinstance(both, CompositeSpec) and isinstance(both.members[0], CompositeSpec)
    assert both.members[0].members[0] == PagedKVSpec(3, 20, window=None, v_head_dim=12)
    # three earlier inputs of the q, k and v channels
    assert both.members[0].members[1] == StateSpec((3 * (120 + 60 + 36),), "float32")
    # six heads of a 12 x 10 state, then two earlier inputs of the x, B and C channels
    assert both.members[1] == StateSpec((6 * 12 * 10 + 2 * (60 + 2 * 3 * 12),), "float32")
    assert specs[3].group_key() == both.group_key()
    assert specs[1] == StateSpec((3 * 24 * 40 + 3 * (24 + 24 + 120),), "float32")
    flat = flatten_cache_specs(specs)
    assert set(flat) == {((0, 0), 0), ((0, 0), 1), (0, 1), 1, 2, ((3, 0), 0), ((3, 0), 1), (3, 1)}
    # one tap: nothing of a convolution is kept, and the attention's cache is its pages alone
    one_tap = build_model(config_from_dir(model_dirs["b2"]), torch.float32, "cpu").cache_specs()
    assert one_tap[0] == StateSpec((2 * 32 * 32,), "float32")
    assert one_tap[1].members[0] == PagedKVSpec(1, 48, window=None, v_head_dim=48)
    assert one_tap[1].members[1] == StateSpec((16 * 40,), "float32")


def test_a_pair_inside_a_pair_gets_its_views_and_slots_are_used_again(model_dirs):
    model = build_model(config_from_dir(model_dirs["b1"]), torch.float32, "cpu")
    cm = CacheManager(model.cache_specs(), num_pages=9, page_size=16, max_reqs=3, max_seq_len=128,
                      dtype=torch.float32, device="cpu")
    assert len(cm.page_groups) == 1 and len(cm.state_groups) == 4
    (g,) = cm.page_groups.values()
    assert sorted(g.cache_ids, key=str) == sorted([((0, 0), 0), ((3, 0), 0)], key=str)
    a = cm.allocate_slot()
    cm.allocate(a, 100)
    for grp in cm.state_groups.values():
        grp.array[:, a] = 7.0
    cm.reset_fresh_state()
    assert all(float(grp.array[:, a].abs().max()) == 0.0 for grp in cm.state_groups.values())
    for grp in cm.state_groups.values():
        grp.array[:, a] = 7.0
    cm.release_slot(a)
    b = cm.allocate_slot()
    assert b == a                                   # the slot freed last is handed out first
    cm.allocate(b, 128)
    cm.reset_fresh_state()                          # and starts from zeros again
    assert all(float(grp.array[:, b].abs().max()) == 0.0 for grp in cm.state_groups.values())
    cm.check_invariants()


# ---- one mechanism at a time, through the engine's step function on the CPU ---------------------------

@pytest.mark.parametrize("heads, kv_heads, dim, vdim, taps, rot, page, softcap, scaling", [
    (4, 2, 32, 16, 4, 8, 16, 5.0, (4.0, 1.0, 4.0, 64)),       # a partial rotation with stretched frequencies
    (2, 2, 16, 24, 2, 16, 16, None, None),                    # no soft cap; a full rotation
    (3, 1, 24, 24, 1, 0, 8, 3.0, None),                       # one tap, no rotation
])
def test_attention_alone(tmp_path, torch_ops, heads, kv_heads, dim, vdim, taps, rot, page, softcap, scaling):
    bm.attention_case(tmp_path, "float32", "cpu", heads, kv_heads, dim, vdim, taps, rot, page, softcap, scaling,
                      n=150)


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, taps", [(4, 2, 16, 24, 4), (2, 2, 32, 16, 1)])
def test_gated_delta_rule_alone(tmp_path, torch_ops, heads, kv_heads, dim, vdim, taps):
    bm.delta_case(tmp_path, "float32", "cpu", heads, kv_heads, dim, vdim, taps, repeat=taps == 4)


@pytest.mark.parametrize("heads, vdim, state, groups, norm_groups, taps", [
    (4, 8, 16, 2, 2, 4), (1, 24, 8, 1, 1, 1), (6, 4, 20, 6, 3, 2)])
def test_state_space_recurrence_alone(tmp_path, torch_ops, heads, vdim, state, groups, norm_groups, taps):
    bm.state_space_case(tmp_path, "float32", "cpu", heads, vdim, state, groups, norm_groups, taps,
                        repeat=heads == 4)


@pytest.mark.parametrize("experts, top, ff, groups, shared, correction", [
    (12, 3, 20, (4, 2), 24, 0.5),
    (8, 2, 16, (2, 1), None, -2.0),       # every choice score negative: a group left out is minus infinity, not zero
    (5, 1, 24, None, 16, 0.5),            # one chosen expert, no groups
    (6, 6, 8, (3, 3), 8, -2.0),           # every expert chosen
])
def test_routed_experts_alone(tmp_path, torch_ops, experts, top, ff, groups, shared, correction):
    bm.experts_case(tmp_path, "float32", "cpu", experts, top, ff, groups, shared, correction)


# ---- whole models: the engine's host logic on the CPU -------------------------------------------------

@pytest.mark.parametrize("name", list(bu.CONFIGS))
def test_cuttings_batches_and_reused_slots_on_cpu(name, model_dirs, torch_ops):
    d = model_dirs[name]
    cfg, w = pb.read_model_dir(d)
    lens = [70, 41, 2, 26, 55]
    reqs = bu.requests(cfg["vocab"], lens, 3)
    exact = [pb.forward(cfg, w, r) for r in reqs]
    for what, steps in bu.schedules(lens, tail=45).items():
        runner = bu.runner_for(d, "float32", "cpu", bu.CONFIGS[name]["page_size"], lens)
        got = bu.replay(runner, reqs, steps)
        for i, (g, e) in enumerate(zip(got, exact)):
            err = bm.row_errors(g, e)
            assert float(err.max()) <= 1e-4 * float(e.std()), (name, what, i, int(err.argmax()), float(err.max()))


def test_the_stream_after_every_layer_run(model_dirs, torch_ops):
    """The float32 residual stream (pending term added) after each layer run; a layer that runs twice
    counts twice."""
    from tests.torch_kernels import _plain
    d = model_dirs["b3"]
    cfg, w = pb.read_model_dir(d, torch.float32)
    (toks,) = bu.requests(cfg["vocab"], [19], 5)
    want = []
    pb.forward(cfg, w, toks, layers_out=want)
    runner = bu.runner_for(d, "float32", "cpu", 8, [19])
    seen = []
    runner.model.after_layer = lambda e, hidden, residual: seen.append(residual + _plain(hidden))
    s = runner.cache.allocate_slot()
    runner.step([SequenceInput(s, toks, 0, [18])])
    assert len(seen) == len(want) == 5
    for i, (got, ref) in enumerate(zip(seen, want)):
        assert got.dtype == torch.float32
        torch.testing.assert_close(got, ref, atol=3e-4, rtol=1e-4, msg=lambda m, i=i: f"layer run {i}: {m}")


def generate_plain(cfg, w, prompt, new):
    ids = list(prompt)
    for _ in range(new):
        ids.append(int(torch.argmax(pb.forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]


def test_greedy_generation_through_the_entry_point_on_cpu(model_dirs, torch_ops):
    d = model_dirs["b1"]
    cfg, w = pb.read_model_dir(d, torch.float32)
    prompts = bu.requests(cfg["vocab"], [3, 20, 9], 7)
    want = [generate_plain(cfg, w, p, 10) for p in prompts]
    eng = Engine(EngineConfig(model_path=str(d), dtype="float32", device="cpu", kv_pool_tokens=96, page_size=16,
                              max_reqs=2, max_seq_len=64, max_prefill_tokens=12, cuda_graphs=False,
                              async_scheduling=False))
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=10, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    eng.cache.check_invariants()


def test_the_command_line_writes_a_model_folder_the_registry_reads_back(tmp_path):
    from deterministic_inference_b200.__main__ import main
    from deterministic_inference_b200.config import preset
    cfg = preset("bovitar_tiny")
    assert isinstance(cfg, BovitarConfig)
    out = tmp_path / "model"
    assert main(["random", "--preset", "bovitar_tiny", "--seed", "3", "--out", str(out)]) == 0
    back = config_from_dir(out)
    assert back.to_dict() == cfg.to_dict()
    model = build_model(back, torch.float32, "cpu")
    load_weights(out, model.tensor_specs(), model.plan, torch.float32, "cpu")
