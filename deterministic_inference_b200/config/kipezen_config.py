"""Typed configuration of the Kipezen design, read from the keys of its config.json.

A decoder with a residual stream in float32 whose sublayers read the stream itself and whose
OUTPUTS are normed before they join it (x <- x + norm1(mixer(x)), then x <- x + norm2(ff(x)),
RMS norms with weights stored around zero), two kinds of mixer in any order -- a gated delta rule
with short causal convolutions in front of it ("delta"), and softmax attention with a sliding
window that keeps the first tokens beside a gated linear recurrent unit ("parallel") -- a
feed-forward of routed experts with a gated shared expert, and a head that shares the embedding.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps`` and ``layers``: per layer
``type``, ``mixer`` (delta: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``; parallel:
``left`` with ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``,
``mask.keep_first``, ``rot.base``, ``rot.dims``; ``right`` with ``width``, ``blocks``, ``conv``;
``left_scale``, ``right_scale``) and ``mlp`` (``kind`` "moe" with ``expert.ff``,
``router.experts``, ``router.top``, ``router.scale``, ``router.groups.count``,
``router.groups.keep``, ``shared.ff``; or null).  ``max_positions`` is optional (no part of the
design needs a longest position; it bounds the engine's block tables).  Tensor names: ``embed``,
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
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
RECURRENT_DECAY_SCALE = 8.0      # log a = -8 r softplus(lam)
ROUTER_WEIGHT_EPS = 1e-20        # added to the sum the chosen experts' scores are divided by
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
    for k in ("left", "right", "left_scale", "right_scale"):
        if k not in m:
            raise ConfigError(f"layer {i}: mixer.{k} is missing")
    left, right = m["left"], m["right"]
    for k in ("heads", "kv_heads", "dim", "vdim"):
        _positive(f"layer {i}: left.{k}", left.get(k))
    if left["heads"] % left["kv_heads"]:
        raise ConfigError(f"layer {i}: left.heads {left['heads']} is not a multiple of kv_heads "
                          f"{left['kv_heads']}")
    if "scale" not in left:
        raise ConfigError(f"layer {i}: left.scale is missing")
    mask = left.get("mask") or {}
    _positive(f"layer {i}: left.mask.size", mask.get("size"))
    keep = mask.get("keep_first", 0)
    if not isinstance(keep, int) or isinstance(keep, bool) or keep < 0:
        raise ConfigError(f"layer {i}: left.mask.keep_first must be a non-negative integer")
    rot = left.get("rot")
    if not isinstance(rot, dict) or "base" not in rot or "dims" not in rot:
        raise ConfigError(f"layer {i}: left.rot.base and left.rot.dims are needed")
    dims = rot["dims"]
    if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > left["dim"]:
        raise ConfigError(f"layer {i}: left.rot.dims {dims!r} must be even and at most {left['dim']}")
    if float(rot["base"]) <= 0:
        raise ConfigError(f"layer {i}: left.rot.base must be positive")
    for k in ("width", "blocks", "conv"):
        _positive(f"layer {i}: right.{k}", right.get(k))
    if right["width"] % right["blocks"]:
        raise ConfigError(f"layer {i}: right.width {right['width']} is not a multiple of blocks {right['blocks']}")


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
class KipezenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple                  # the ``layers`` list of config.json
    max_positions: int = DEFAULT_MAX_POSITIONS
    architecture: str = "Kipezen"

    # ---- construction -----------------------------------------------------

    @classmethod
    def from_dict(cls, cfg: dict) -> "KipezenConfig":
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
                  max_positions=_positive("max_positions", cfg.get("max_positions", DEFAULT_MAX_POSITIONS)),
                  architecture=str(cfg.get("architecture", "Kipezen")))
        if out.norm_eps <= 0:
            raise ConfigError("norm.eps must be positive")
        return out

    @classmethod
    def from_json(cls, model_dir) -> "KipezenConfig":
        return cls.from_dict(json.loads((Path(model_dir) / "config.json").read_text()))

    def to_dict(self) -> dict:
        """The config.json content that ``from_dict`` reads back unchanged."""
        out = {"architecture": self.architecture, "layers": copy.deepcopy(list(self.layers)),
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    def validate(self) -> None:
        KipezenConfig.from_dict(self.to_dict())

    # ---- derived -----------------------------------------------------------

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def num_parameters(self) -> int:
        w = self.width
        n = self.vocab * w + w
        for layer in self.layers:
            m = layer["mixer"]
            n += w
            if layer["type"] == "delta":
                qk, v = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
                n += (2 * qk + 3 * v + 2 * m["heads"]) * w + (2 * qk + v) * m["conv"] + 2 * m["heads"] + m["vdim"]
            else:
                left, right = m["left"], m["right"]
                q, k, v = left["heads"] * left["dim"], left["kv_heads"] * left["dim"], left["kv_heads"] * left["vdim"]
                n += (q + k + v) * (w + 1) + q + k + left["heads"] * left["vdim"] * w
                c = right["width"]
                n += 2 * c * (w + 1) + c * (right["conv"] + 1) + 2 * c * (c // right["blocks"] + 1) + c + c * w
            mlp = layer.get("mlp")
            if mlp is not None:
                r = mlp["router"]
                n += w + r["experts"] * (3 * mlp["expert"]["ff"] * w + w + 1)
                if mlp.get("shared") is not None:
                    n += 3 * mlp["shared"]["ff"] * w + w
        return n

    # ---- the plan ------------------------------------------------------------

    def plan(self) -> ModelPlan:
        w = self.width
        post = dict(size=w, eps=self.norm_eps, weight_offset=1.0)
        layers, ignored = [], []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            m = layer["mixer"]
            if layer["type"] == "delta":
                mixer = PartSpec("gated_delta_rule", dict(
                    prefix=p + "mix.", hidden_size=w, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
                    head_dim=m["dim"], v_head_dim=m["vdim"], conv_taps=m["conv"], norm_eps=self.norm_eps,
                    key_eps=DELTA_KEY_EPS))
            else:
                left, right = m["left"], m["right"]
                rot = left["rot"]
                left_spec = PartSpec("masked_attention", dict(
                    prefix=p + "mix.left.", hidden_size=w, num_heads=left["heads"], num_kv_heads=left["kv_heads"],
                    head_dim=left["dim"], v_head_dim=left["vdim"], scale=float(left["scale"]),
                    position_encoding=None if not rot["dims"] else PartSpec("rope", dict(
                        head_dim=left["dim"], rotary_dim=rot["dims"], theta=float(rot["base"]))),
                    rotary_layout="pairs", qk_norm_eps=self.norm_eps, qk_norm_scope="projection", bias=True,
                    mask="window", mask_size=left["mask"]["size"], keep_first=left["mask"].get("keep_first", 0)))
                right_spec = PartSpec("gated_linear_recurrence", dict(
                    prefix=p + "mix.right.", hidden_size=w, width=right["width"], blocks=right["blocks"],
                    conv_taps=right["conv"], decay_scale=RECURRENT_DECAY_SCALE))
                mixer = PartSpec("parallel", dict(branches=[left_spec, right_spec],
                                                  scales=[float(m["left_scale"]), float(m["right_scale"])]))
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
                    weight_eps=ROUTER_WEIGHT_EPS))
                ff_norm = PartSpec("stream_post_norm", dict(name=p + "norm2", **post))
            layers.append(LayerSpec(
                block=PartSpec("post_norm_f32_stream", {}),
                mixer=mixer, feed_forward=ff,
                mixer_norm=PartSpec("stream_post_norm", dict(name=p + "norm1", **post)),
                feed_forward_norm=ff_norm))
        return ModelPlan(
            hidden_size=w, vocab_size=self.vocab,
            embedding=PartSpec("scaled_token_embedding", dict(name="embed", vocab_size=self.vocab,
                                                              hidden_size=w, scale=1.0)),
            head=PartSpec("linear_head", dict(name=None, vocab_size=self.vocab, hidden_size=w)),
            final_norm=PartSpec("stream_rms_norm", dict(name="final.norm", size=w, eps=self.norm_eps,
                                                        weight_offset=1.0)),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(layer=i, cache=i, writes_cache=True) for i in range(len(layers))),
            max_positions=self.max_positions,
            eos_token_ids=(),
            ignored_names=tuple(ignored),
        )
