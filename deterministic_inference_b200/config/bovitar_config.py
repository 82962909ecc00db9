"""Typed configuration of the Bovitar design, read from the keys of its config.json.

A pre-norm decoder with a residual stream in float32 (x <- x + mixer(norm1(x)), then
x <- x + ff(norm2(x)), RMS norms with plain weights) and two kinds of mixer in any order: "delta", a
gated delta rule with short causal convolutions in front of it, and "parallel", causal softmax
attention (short convolutions on q, k and v, an RMS norm over the whole q and k projections, a
rotation in halves with stretched long wavelengths, soft-capped scores) beside a state-space
recurrence with a scalar decay per head, each branch's output RMS-normed over the model width and the
two averaged.  The feed-forward is a mixture of experts with a softmax router, groups of experts that
are scored by their best member, weights that are not renormalised and an ungated shared expert.  A
layer may run with the weights of another layer and a cache of its own.  The head has a matrix of
its own; the logits are scaled by a constant.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``logit_scale`` and ``layers``:
per layer ``type``, ``mixer`` (delta: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``; parallel:
``left`` with ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``, ``scale``, ``softcap``, ``rot.base``,
``rot.dims``, ``rot.scaling`` (``factor``, ``low``, ``high``, ``original``) and ``right`` with ``heads``,
``vdim``, ``state``, ``groups``, ``norm_groups``, ``conv``), ``mlp`` (``kind`` "moe" with ``expert.ff``,
``router.experts``, ``router.top``, ``router.scale``, ``router.groups.count``, ``router.groups.keep``,
``shared.ff``; or null) and optionally ``weights_of``: the index of the layer whose tensors this layer
uses.  ``max_positions`` is optional (no part of the design needs a longest position; it bounds the
engine's block tables).  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass
from pathlib import Path

from ..parts.spec import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from .model_config import ConfigError

# fixed by the design
DELTA_KEY_EPS = 1e-6             # inside the root of the unit query and key
BRANCH_SCALE = 0.5               # the two normed branches of a parallel mixer are averaged
DEFAULT_MAX_POSITIONS = 1 << 20


def _positive(what: str, v) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v < 1:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return v


def _check_delta(i: int, m: dict) -> None:
    for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
        _positive(f"layer {i}: mixer.{k}", m.get(k))
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"layer {i}: mixer.heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")


def _check_parallel(i: int, m: dict) -> None:
    for k in ("left", "right"):
        if not isinstance(m.get(k), dict):
            raise ConfigError(f"layer {i}: mixer.{k} is missing")
    left, right = m["left"], m["right"]
    for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
        _positive(f"layer {i}: left.{k}", left.get(k))
    if left["heads"] % left["kv_heads"]:
        raise ConfigError(f"layer {i}: left.heads {left['heads']} is not a multiple of kv_heads "
                          f"{left['kv_heads']}")
    if "scale" not in left:
        raise ConfigError(f"layer {i}: left.scale is missing")
    cap = left.get("softcap")
    if cap is not None and not float(cap) > 0:
        raise ConfigError(f"layer {i}: left.softcap must be positive or null, got {cap!r}")
    rot = left.get("rot")
    if rot is not None:
        if not isinstance(rot, dict) or "base" not in rot or "dims" not in rot:
            raise ConfigError(f"layer {i}: left.rot.base and left.rot.dims are needed")
        dims = rot["dims"]
        if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > left["dim"]:
            raise ConfigError(f"layer {i}: left.rot.dims {dims!r} must be even and at most {left['dim']}")
        if float(rot["base"]) <= 0:
            raise ConfigError(f"layer {i}: left.rot.base must be positive")
        sc = rot.get("scaling")
        if sc is not None:
            missing = [k for k in ("factor", "low", "high", "original") if k not in sc]
            if missing:
                raise ConfigError(f"layer {i}: left.rot.scaling lacks {missing}")
            if float(sc["high"]) <= float(sc["low"]) or float(sc["factor"]) <= 0 or float(sc["original"]) <= 0:
                raise ConfigError(f"layer {i}: left.rot.scaling needs high > low and positive factor, original")
    for k in ("heads", "vdim", "state", "groups", "norm_groups", "conv"):
        _positive(f"layer {i}: right.{k}", right.get(k))
    if right["heads"] % right["groups"]:
        raise ConfigError(f"layer {i}: right.heads {right['heads']} is not a multiple of groups {right['groups']}")
    if (right["heads"] * right["vdim"]) % right["norm_groups"]:
        raise ConfigError(f"layer {i}: right.heads x vdim {right['heads'] * right['vdim']} does not split into "
                          f"{right['norm_groups']} equal parts")


def _check_moe(i: int, mlp: dict) -> None:
    if mlp.get("kind") != "moe":
        raise ConfigError(f"layer {i}: mlp.kind {mlp.get('kind')!r} is not known (only 'moe')")
    _positive(f"layer {i}: mlp.expert.ff", (mlp.get("expert") or {}).get("ff"))
    r = mlp.get("router") or {}
    for k in ("experts", "top"):
        _positive(f"layer {i}: mlp.router.{k}", r.get(k))
    if "scale" not in r:
        raise ConfigError(f"layer {i}: mlp.router.scale is missing")
    g = r.get("groups")
    count, keep = 1, 1
    if g is not None:
        count, keep = _positive(f"layer {i}: router.groups.count", g.get("count")), \
            _positive(f"layer {i}: router.groups.keep", g.get("keep"))
    if r["experts"] % count or keep > count:
        raise ConfigError(f"layer {i}: router.groups {count} / {keep} do not fit {r['experts']} experts")
    if r["top"] > keep * (r["experts"] // count):
        raise ConfigError(f"layer {i}: router.top {r['top']} is more than the kept groups hold")
    if mlp.get("shared") is not None:
        _positive(f"layer {i}: mlp.shared.ff", mlp["shared"].get("ff"))


@dataclass(frozen=True)
class BovitarConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple                  # the ``layers`` list of config.json
    logit_scale: float = 1.0
    max_positions: int = DEFAULT_MAX_POSITIONS
    architecture: str = "Bovitar"

    # ---- construction -----------------------------------------------------

    @classmethod
    def from_dict(cls, cfg: dict) -> "BovitarConfig":
        missing = [k for k in ("vocab", "width", "norm", "layers") if k not in cfg]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        if not isinstance(cfg["norm"], dict) or "eps" not in cfg["norm"]:
            raise ConfigError("config.json: norm.eps is missing")
        layers = copy.deepcopy(list(cfg["layers"]))
        if not layers:
            raise ConfigError("config.json lists no layers")
        for i, layer in enumerate(layers):
            kind, mixer = layer.get("type"), layer.get("mixer") or {}
            if kind == "delta":
                _check_delta(i, mixer)
            elif kind == "parallel":
                _check_parallel(i, mixer)
            else:
                raise ConfigError(f"layer {i}: type {kind!r} is not known ('delta', 'parallel')")
            if layer.get("mlp") is not None:
                _check_moe(i, layer["mlp"])
        out = cls(vocab=_positive("vocab", cfg["vocab"]), width=_positive("width", cfg["width"]),
                  norm_eps=float(cfg["norm"]["eps"]), layers=tuple(layers),
                  logit_scale=float(cfg.get("logit_scale", 1.0)),
                  max_positions=_positive("max_positions", cfg.get("max_positions", DEFAULT_MAX_POSITIONS)),
                  architecture=str(cfg.get("architecture", "Bovitar")))
        if out.norm_eps <= 0:
            raise ConfigError("norm.eps must be positive")
        for i in range(len(layers)):
            out.weights_owner(i)
        return out

    @classmethod
    def from_json(cls, model_dir) -> "BovitarConfig":
        return cls.from_dict(json.loads((Path(model_dir) / "config.json").read_text()))

    def to_dict(self) -> dict:
        """The config.json content that ``from_dict`` reads back unchanged."""
        out = {"architecture": self.architecture, "layers": copy.deepcopy(list(self.layers)),
               "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
               "width": self.width}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    def validate(self) -> None:
        BovitarConfig.from_dict(self.to_dict())

    # ---- derived -----------------------------------------------------------

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def weights_owner(self, i: int) -> int:
        """The layer whose tensors layer ``i`` runs with (itself, unless it names another)."""
        seen = []
        while self.layers[i].get("weights_of") is not None:
            j = self.layers[i]["weights_of"]
            if not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < len(self.layers):
                raise ConfigError(f"layer {i}: weights_of {j!r} names no layer")
            if j == i or j in seen:
                raise ConfigError(f"layer {i}: weights_of runs in a circle")
            if self.layers[j]["type"] != self.layers[i]["type"] \
                    or self.layers[j]["mixer"] != self.layers[i]["mixer"] \
                    or self.layers[j].get("mlp") != self.layers[i].get("mlp"):
                raise ConfigError(f"layer {i} uses the weights of layer {j}, whose entry differs")
            seen.append(i)
            i = j
        return i

    def num_parameters(self) -> int:
        w = self.width
        n = 2 * self.vocab * w + w
        for i, layer in enumerate(self.layers):
            if self.weights_owner(i) != i:
                continue
            m = layer["mixer"]
            n += w
            if layer["type"] == "delta":
                qk, v = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
                n += (2 * qk + 3 * v + 2 * m["heads"]) * w + (2 * qk + v) * m["conv"] + 2 * m["heads"] + m["vdim"]
            else:
                left, right = m["left"], m["right"]
                q, k, v = left["heads"] * left["dim"], left["kv_heads"] * left["dim"], left["kv_heads"] * left["vdim"]
                n += (q + k + v) * (w + left["conv"]) + q + k + left["heads"] * left["vdim"] * w
                inner = right["heads"] * right["vdim"]
                chan = inner + 2 * right["groups"] * right["state"]
                n += (inner + chan + right["heads"]) * w + chan * (right["conv"] + 1) + 3 * right["heads"] \
                    + inner + inner * w + 2 * w
            mlp = layer.get("mlp")
            if mlp is not None:
                r = mlp["router"]
                n += w + r["experts"] * (3 * mlp["expert"]["ff"] * w + w + 1)
                if mlp.get("shared") is not None:
                    n += 3 * mlp["shared"]["ff"] * w
        return n

    # ---- the plan ------------------------------------------------------------

    def _layer_spec(self, i: int) -> tuple:
        """(LayerSpec, ignored tensor names) of layer ``i``, which owns its tensors."""
        layer, w, eps = self.layers[i], self.width, self.norm_eps
        p = f"l{i}."
        m = layer["mixer"]
        ignored = []
        if layer["type"] == "delta":
            mixer = PartSpec("gated_delta_rule", dict(
                prefix=p + "mix.", hidden_size=w, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
                head_dim=m["dim"], v_head_dim=m["vdim"], conv_taps=m["conv"], norm_eps=eps,
                key_eps=DELTA_KEY_EPS))
        else:
            left, right = m["left"], m["right"]
            rot = left.get("rot")
            left_spec = PartSpec("masked_attention", dict(
                prefix=p + "mix.left.", hidden_size=w, num_heads=left["heads"], num_kv_heads=left["kv_heads"],
                head_dim=left["dim"], v_head_dim=left["vdim"], scale=float(left["scale"]),
                position_encoding=None if rot is None or not rot["dims"] else PartSpec("rope", dict(
                    head_dim=left["dim"], rotary_dim=rot["dims"], theta=float(rot["base"]),
                    scaling=rot.get("scaling"))),
                rotary_layout="halves", qk_norm_eps=eps, qk_norm_scope="projection", mask="causal",
                softcap=None if left.get("softcap") is None else float(left["softcap"]),
                conv_taps=left["conv"]))
            right_spec = PartSpec("state_space", dict(
                prefix=p + "mix.right.", hidden_size=w, num_heads=right["heads"], head_dim=right["vdim"],
                state_dim=right["state"], groups=right["groups"], norm_groups=right["norm_groups"],
                conv_taps=right["conv"], norm_eps=eps))
            mixer = PartSpec("parallel", dict(
                branches=[left_spec, right_spec], scales=[BRANCH_SCALE, BRANCH_SCALE], hidden_size=w,
                branch_norms=[dict(name=p + "mix.left.out", eps=eps), dict(name=p + "mix.right.out", eps=eps)]))
        mlp = layer.get("mlp")
        if mlp is None:
            ff, ff_norm = PartSpec("none", {}), PartSpec("none", {})
            ignored.append(p + "norm2")
        else:
            r = mlp["router"]
            groups = r.get("groups") or {"count": 1, "keep": 1}
            shared = mlp.get("shared")
            ff = PartSpec("routed_experts", dict(
                prefix=p + "mlp.", hidden_size=w, intermediate_size=mlp["expert"]["ff"],
                num_experts=r["experts"], top=r["top"], route_scale=float(r["scale"]),
                group_count=groups["count"], group_keep=groups["keep"],
                shared_intermediate_size=None if shared is None else shared["ff"],
                score="softmax", group_top=1, normalize=False, shared_gate=False))
            ff_norm = PartSpec("stream_rms_norm", dict(name=p + "norm2", size=w, eps=eps))
        spec = LayerSpec(block=PartSpec("pre_norm_f32_stream", {}), mixer=mixer, feed_forward=ff,
                         mixer_norm=PartSpec("stream_rms_norm", dict(name=p + "norm1", size=w, eps=eps)),
                         feed_forward_norm=ff_norm)
        return spec, ignored

    def plan(self) -> ModelPlan:
        w = self.width
        # the plan holds the layers that own tensors; a layer that runs with another's weights is a
        # second schedule entry of that layer with a cache (pages, state) of its own
        owners = [i for i in range(len(self.layers)) if self.weights_owner(i) == i]
        index_of = {i: n for n, i in enumerate(owners)}
        layers, ignored = [], []
        for i in owners:
            spec, ign = self._layer_spec(i)
            layers.append(spec)
            ignored += ign
        schedule = tuple(ScheduleEntry(layer=index_of[self.weights_owner(i)], cache=i, writes_cache=True)
                         for i in range(len(self.layers)))
        return ModelPlan(
            hidden_size=w, vocab_size=self.vocab,
            embedding=PartSpec("scaled_token_embedding", dict(name="embed", vocab_size=self.vocab,
                                                              hidden_size=w, scale=1.0)),
            head=PartSpec("linear_head", dict(name="head", vocab_size=self.vocab, hidden_size=w,
                                              scale=self.logit_scale)),
            final_norm=PartSpec("stream_rms_norm", dict(name="final.norm", size=w, eps=self.norm_eps)),
            layers=tuple(layers),
            schedule=schedule,
            max_positions=self.max_positions,
            eos_token_ids=(),
            ignored_names=tuple(ignored),
        )
