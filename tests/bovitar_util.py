"""Tiny Bovitar models for the tests: configurations that differ in every size and option (also in
values that may happen to be equal or 1 elsewhere: as many key heads as query heads or one, key and
value sizes equal or not, one tap or several, one group of state-space heads or one per head, one
part or several in the gated norm, one group of experts, one chosen expert or all of them, a full, a
partial or no rotation, stretched frequencies or plain ones, a soft cap or none, a layer without a
feed-forward, no shared expert, layers that run with another layer's weights), written with random
weights by the package's writer and then rescaled so that every mechanism weighs in the logits:
streams of unit size, scores that reach the soft cap, decays that neither forget everything nor
nothing, routers whose choice changes from token to token.  The schedules and the replay through the
step function are those of ``tests/kipezen_util.py`` (they know no design)."""

from __future__ import annotations

import copy
import math
from pathlib import Path

import torch

from tests.kipezen_util import (last_one_by_one, mixed, portions, replay, requests, runner_for,  # noqa: F401
                                schedules, whole)


def moe(experts, top, ff, scale, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router,
            "shared": None if shared is None else {"ff": shared}}


def delta(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, conv, rot_dims, base, scaling=None, softcap=None, scale=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
            "scale": scale if scale is not None else 3.0 / math.sqrt(dim), "softcap": softcap,
            "rot": {"base": base, "dims": rot_dims}}
    if scaling is not None:
        left["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return left


def state_space(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def parallel(left, right, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def again(layers, j):
    """Layer ``j`` once more: the same entry, run with layer j's weights and a cache of its own."""
    out = copy.deepcopy(layers[j])
    out["weights_of"] = j
    return out


def _with_repeats(layers, repeats):
    layers = list(layers)
    for j in repeats:
        layers.append(again(layers, j))
    return layers


CONFIGS = {
    # sizes that are multiples of nothing (the kernels that take any size); a partial rotation with
    # stretched frequencies; a layer without a feed-forward; the first layer runs a second time
    "b1": dict(page_size=16, seed=61, config={
        "architecture": "Bovitar", "vocab": 150, "width": 72, "norm": {"eps": 2e-5}, "logit_scale": 0.7,
        "layers": _with_repeats([
            parallel(attention(6, 3, 20, 12, 4, 10, 777.0, scaling=(3.0, 1.0, 5.0, 24), softcap=4.0),
                     state_space(6, 10, 12, 3, 2, 3), mlp=moe(6, 3, 28, 1.5, groups=(3, 2), shared=36)),
            delta(3, 1, 24, 40, 4, mlp=moe(5, 2, 20, 2.0, shared=None)),
            delta(4, 2, 12, 20, 2, mlp=None)], repeats=(0,))}),
    # everything that can be 1 is 1: one tap (no convolution tails), one head, one group, one part in the
    # gated norm, one group of experts, one chosen expert, no soft cap, plain frequencies, a logit
    # scale of 1; pages of 32
    "b2": dict(page_size=32, seed=62, config={
        "architecture": "Bovitar", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
        "layers": [delta(2, 2, 32, 32, 1, mlp=moe(4, 1, 48, 1.0, groups=(1, 1), shared=64)),
                   parallel(attention(1, 1, 48, 48, 1, 48, 30000.0),
                            state_space(1, 40, 16, 1, 1, 1), mlp=moe(3, 3, 40, 3.0, shared=24))]}),
    # sizes the tensor-core kernels take; many experts in groups; a group per state-space head; two
    # layers that run twice, in another order than their owners; pages of 8
    "b3": dict(page_size=8, seed=63, config={
        "architecture": "Bovitar", "vocab": 211, "width": 128, "norm": {"eps": 3e-6}, "logit_scale": 0.3,
        "layers": _with_repeats([
            delta(4, 4, 128, 64, 2, mlp=moe(32, 4, 64, 2.5, groups=(8, 3), shared=128)),
            parallel(attention(8, 2, 64, 32, 2, 32, 10000.0, scaling=(8.0, 1.0, 4.0, 64), softcap=30.0),
                     state_space(4, 32, 64, 4, 4, 4), mlp=moe(8, 2, 96, 1.0, groups=(4, 2), shared=None)),
            parallel(attention(4, 4, 32, 64, 3, 16, 500.0, softcap=6.0),
                     state_space(8, 16, 32, 2, 1, 2), mlp=moe(16, 6, 32, 2.0, groups=(2, 2), shared=48))],
            repeats=(2, 0))}),
    # a width that is a multiple of 4 only, five heads, groups of ONE expert (a group's score is that
    # expert's), no rotation at all, a wide state
    "b4": dict(page_size=16, seed=64, config={
        "architecture": "Bovitar", "vocab": 131, "width": 100, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
        "layers": [delta(5, 5, 12, 20, 3, mlp=moe(6, 2, 36, 1.0, groups=(6, 3), shared=20)),
                   parallel(attention(5, 5, 12, 20, 2, 0, 3000.0, softcap=2.5),
                            state_space(5, 8, 136, 5, 5, 2), mlp=moe(9, 4, 28, 1.5, groups=(3, 2), shared=None))]}),
}


def sharpen(model_dir) -> None:
    from safetensors.torch import load_file, save_file

    path = Path(model_dir) / "model.safetensors"
    tensors = load_file(str(path))

    def unit(t, gain):      # a matrix drawn with std 0.02 -> std gain / sqrt(inputs)
        return t.float() * (gain / (0.02 * math.sqrt(t.shape[-1])))

    for name, t in list(tensors.items()):
        end = name.split(".", 1)[-1] if name.startswith("l") and name[1].isdigit() else name
        leaf = end.rsplit(".", 1)[-1]
        x = None
        if name == "embed":
            x = t.float() * 50.0
        elif name == "head":
            x = unit(t, 1.5)
        elif end in ("mix.left.q", "mix.left.k", "mix.b", "mix.a", "mlp.router"):
            x = unit(t, 2.0)
        elif leaf in ("gate", "up", "down") or end in ("mix.q", "mix.k", "mix.v", "mix.g", "mix.o", "mix.left.v",
                                                        "mix.left.o", "mix.right.in", "mix.right.o"):
            x = unit(t, 1.2)
        elif leaf == "conv":
            x = t.float() * 25.0                          # taps of size one half
        elif end in ("mix.A_log", "mix.dt_bias", "mix.right.A_log", "mix.right.dt_bias"):
            x = t.float() * 25.0
        elif end == "mix.right.conv.b":
            x = t.float() * 15.0                          # biases of size 0.3
        elif end == "mlp.correction":
            x = t.float() * 4.0                           # of the size of a score's spread
        elif end in ("mix.left.q.norm", "mix.left.k.norm"):
            x = t.float() * 1.4                           # scores that reach a soft cap
        if x is not None:
            tensors[name] = x.to(t.dtype)
    save_file(tensors, str(path), metadata={"format": "pt"})


def write_model(config: dict, seed: int, out_dir, edit=None) -> Path:
    """Random weights, rescaled as for the tiny models, then changed by ``edit(tensors)`` (float32 in,
    stored as bfloat16)."""
    from safetensors.torch import load_file, save_file

    from deterministic_inference_b200.config.bovitar_config import BovitarConfig
    from deterministic_inference_b200.weights import write_random_model

    write_random_model(BovitarConfig.from_dict(config), seed, out_dir)
    sharpen(out_dir)
    if edit is not None:
        path = Path(out_dir) / "model.safetensors"
        stored = load_file(str(path))
        tensors = {k: v.float() for k, v in stored.items()}
        edit(tensors)
        save_file({k: v.to(stored[k].dtype).contiguous() for k, v in tensors.items()}, str(path),
                  metadata={"format": "pt"})
    return Path(out_dir)


def write_tiny(name: str, out_dir) -> Path:
    spec = CONFIGS[name]
    return write_model(spec["config"], spec["seed"], out_dir)


def one_layer(layer, vocab=97, width=48, eps=1e-5, logit_scale=1.0, repeat=False) -> dict:
    layers = [layer] + ([again([layer], 0)] if repeat else [])
    return {"architecture": "Bovitar", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "logit_scale": logit_scale, "layers": layers}
