"""Tiny Kipezen models for the tests: configurations that differ in every size and option (also in
values that may happen to be equal or 1 elsewhere: as many key heads as value heads or one, key and
value sizes equal or not, one tap or several, one block of channels, one group of experts, one chosen
expert, a window that no prompt reaches or that is shorter than a page, kept first keys that reach
beyond the window or none, a full or a partial rotation, a layer without a feed-forward, no shared
expert), written with random weights by the package's writer and then rescaled so that every
mechanism weighs in the logits: streams of unit size, scores of unit size, decays that neither
forget everything nor nothing, routers whose choice changes from token to token."""

from __future__ import annotations

import math
from pathlib import Path

import torch


def moe(experts, top, ff, scale, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router,
            "shared": None if shared is None else {"ff": shared}}


def delta(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": mlp}


def parallel(heads, kv_heads, dim, vdim, window, keep_first, rot_dims, base, width, blocks, conv, scales=(1.0, 1.0),
             scale=None, mlp=None):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                               "scale": scale if scale is not None else 1.0 / math.sqrt(dim),
                               "mask": {"size": window, "keep_first": keep_first},
                               "rot": {"base": base, "dims": rot_dims}},
                      "right": {"width": width, "blocks": blocks, "conv": conv},
                      "left_scale": scales[0], "right_scale": scales[1]},
            "mlp": mlp}


CONFIGS = {
    # sizes that are multiples of nothing (the kernels that take any size); a window shorter than a page;
    # a layer without a feed-forward
    "k1": dict(page_size=16, seed=51, config={
        "architecture": "Kipezen", "vocab": 150, "width": 72, "norm": {"eps": 2e-5},
        "layers": [parallel(6, 3, 20, 12, 13, 5, 10, 777.0, 60, 3, 4, scales=(0.7, 1.3),
                            mlp=moe(6, 3, 28, 1.5, groups=(3, 2), shared=36)),
                   delta(3, 1, 24, 40, 4, mlp=moe(5, 2, 20, 2.0, shared=None)),
                   delta(4, 2, 12, 20, 2, mlp=None)]}),
    # everything that can be 1 is 1: one tap (no convolution tail), one block of channels, one group of
    # experts, one chosen expert, as many key heads as value heads, no kept keys, a full rotation; pages of 32
    "k2": dict(page_size=32, seed=52, config={
        "architecture": "Kipezen", "vocab": 300, "width": 96, "norm": {"eps": 1e-6},
        "layers": [delta(2, 2, 32, 32, 1, mlp=moe(4, 1, 48, 1.0, groups=(1, 1), shared=64)),
                   parallel(1, 1, 48, 48, 4096, 0, 48, 20000.0, 40, 1, 1, scales=(1.0, 0.5),
                            mlp=moe(3, 3, 40, 3.0, shared=24))]}),
    # sizes the tensor-core kernels take; kept first keys that reach beyond the window; a window that ends
    # inside a page; many experts in groups; pages of 8
    "k3": dict(page_size=8, seed=53, config={
        "architecture": "Kipezen", "vocab": 211, "width": 128, "norm": {"eps": 1e-5},
        "layers": [delta(4, 4, 128, 64, 2, mlp=moe(32, 4, 64, 2.5, groups=(8, 3), shared=128)),
                   parallel(8, 2, 64, 32, 40, 70, 32, 10000.0, 256, 4, 2, scales=(0.9, 0.8),
                            mlp=moe(8, 2, 96, 1.0, groups=(4, 2), shared=None)),
                   parallel(4, 4, 32, 64, 100, 3, 16, 500.0, 64, 2, 3, scales=(1.2, 0.6),
                            mlp=moe(16, 6, 32, 2.0, groups=(2, 2), shared=48))]}),
    # five layers in another order; value heads wider than key heads; a window and kept keys of whole pages
    "k4": dict(page_size=16, seed=54, config={
        "architecture": "Kipezen", "vocab": 512, "width": 192, "norm": {"eps": 1e-6},
        "layers": [parallel(4, 2, 64, 64, 64, 16, 64, 30000.0, 192, 6, 4, mlp=None),
                   delta(6, 2, 32, 64, 3, mlp=moe(12, 2, 64, 2.0, groups=(4, 1), shared=96)),
                   delta(2, 1, 64, 128, 4, mlp=moe(8, 8, 32, 1.0, shared=32)),
                   parallel(6, 1, 32, 16, 30, 40, 8, 100.0, 96, 1, 2, scales=(0.5, 1.5),
                            mlp=moe(10, 3, 48, 1.5, groups=(5, 3), shared=64)),
                   delta(4, 4, 16, 16, 2, mlp=None)]}),
    # a width that is a multiple of 4 only, five heads, groups of ONE expert (a group's score is that
    # expert's), a window shorter than a page, state sizes that are multiples of nothing
    "k5": dict(page_size=16, seed=55, config={
        "architecture": "Kipezen", "vocab": 131, "width": 100, "norm": {"eps": 1e-5},
        "layers": [delta(5, 5, 12, 20, 3, mlp=moe(6, 2, 36, 1.0, groups=(6, 3), shared=20)),
                   parallel(5, 5, 12, 20, 7, 2, 6, 3000.0, 50, 5, 2, scales=(1.1, 0.9),
                            mlp=moe(9, 4, 28, 1.5, groups=(3, 2), shared=None))]}),
    # few wide experts: a prompt of some hundred tokens brings each of them 128 rows or more, so a
    # bfloat16 engine runs their products on the tensor-core kernel of the dense layers
    "k6": dict(page_size=16, seed=56, config={
        "architecture": "Kipezen", "vocab": 160, "width": 256, "norm": {"eps": 1e-5},
        "layers": [parallel(2, 1, 32, 32, 50, 3, 16, 10000.0, 64, 2, 2,
                            mlp=moe(4, 2, 128, 2.0, groups=(2, 2), shared=128)),
                   delta(2, 1, 32, 32, 3, mlp=moe(3, 1, 256, 1.5, shared=None))]}),
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
            x = t.float() * 50.0                          # the sublayers read the stream itself
        elif end in ("mix.left.q", "mix.left.k"):
            x = unit(t, 2.0)
        elif leaf in ("gate", "up", "down") or end in ("mix.q", "mix.k", "mix.v", "mix.g", "mix.o", "mix.left.v",
                                                        "mix.left.o", "mix.right.y", "mix.right.x", "mix.right.o"):
            x = unit(t, 1.2)
        elif end in ("mix.b", "mix.a", "mlp.router", "mlp.shared.sg"):
            x = unit(t, 2.0)
        elif end in ("mix.right.ra", "mix.right.ri"):
            x = unit(t, 2.0)
        elif leaf == "conv":
            x = t.float() * 25.0                          # taps of size one half
        elif end in ("mix.A_log", "mix.dt_bias", "mix.right.lam", "mlp.correction"):
            x = t.float() * 25.0
        elif leaf == "b" or end == "mix.right.conv.b":
            x = t.float() * 15.0                          # biases of size 0.3
        elif end in ("norm1", "norm2") or name == "final.norm":
            x = t.float() * 10.0                          # weights around zero, of size 0.2
        if x is not None:
            tensors[name] = x.to(t.dtype)
    save_file(tensors, str(path), metadata={"format": "pt"})


def write_tiny(name: str, out_dir) -> Path:
    from deterministic_inference_b200.config.kipezen_config import KipezenConfig
    from deterministic_inference_b200.weights import write_random_model

    spec = CONFIGS[name]
    write_random_model(KipezenConfig.from_dict(spec["config"]), spec["seed"], out_dir)
    sharpen(out_dir)
    return Path(out_dir)


def requests(vocab: int, lens, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


# ---- one-layer models that show one mechanism, and schedules for the engine's step function -------

def one_layer(layer, vocab=97, width=48, eps=1e-5) -> dict:
    return {"architecture": "Kipezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": [layer]}


def write_model(config: dict, seed: int, out_dir, edit=None) -> Path:
    """Random weights, rescaled as for the tiny models, then changed by ``edit(tensors)`` (float32 in,
    stored as bfloat16)."""
    from safetensors.torch import load_file, save_file

    from deterministic_inference_b200.config.kipezen_config import KipezenConfig
    from deterministic_inference_b200.weights import write_random_model

    write_random_model(KipezenConfig.from_dict(config), seed, out_dir)
    sharpen(out_dir)
    if edit is not None:
        path = Path(out_dir) / "model.safetensors"
        stored = load_file(str(path))
        tensors = {k: v.float() for k, v in stored.items()}
        edit(tensors)
        save_file({k: v.to(stored[k].dtype).contiguous() for k, v in tensors.items()}, str(path),
                  metadata={"format": "pt"})
    return Path(out_dir)


def whole(lens):
    return [[(i, n)] for i, n in enumerate(lens)]


def last_one_by_one(lens, tail):
    steps = []
    for i, n in enumerate(lens):
        head = max(n - tail, 0)
        steps += ([[(i, head)]] if head else []) + [[(i, 1)]] * (n - head)
    return steps


def portions(lens, sizes=(13, 2, 7, 2, 25, 5, 16, 3, 40, 2, 2, 9)):
    steps, at = [], 0
    for i, n in enumerate(lens):
        left = n
        while left:
            m = min(sizes[at % len(sizes)], left)
            at += 1
            steps.append([(i, m)])
            left -= m
    return steps


def mixed(lens, live=3, tail=12, seed=0):
    """Up to ``live`` requests at a time: a request brings portions of 2 to 30 tokens until its last
    ``tail`` tokens, which come one by one; now and then a request sits a step out.  When one ends,
    the next takes its slot and pages."""
    g = torch.Generator().manual_seed(seed)
    left = {}
    waiting = list(range(len(lens)))
    steps = []
    while waiting or left:
        while waiting and len(left) < live:
            i = waiting.pop(0)
            left[i] = lens[i]
        entries = []
        for i in list(left):
            if len(left) > 1 and int(torch.randint(0, 5, (1,), generator=g)) == 0:
                continue
            n = 1 if left[i] <= tail else min(int(torch.randint(2, 31, (1,), generator=g)), left[i] - tail)
            entries.append((i, n))
            left[i] -= n
            if not left[i]:
                del left[i]
        if entries:
            steps.append(entries)
    return steps


def replay(runner, reqs, steps, routes=None):
    """Runs the schedule (steps of (request, how many of its next tokens)) through the runner's step
    function; a request gets its slot at its first entry and gives slot and pages back with its last
    token.  Returns the logits of every position, one tensor per request.  ``routes`` (a dict): it
    receives routes[request][k] = the experts [tokens, top] that the k-th feed-forward with a router
    chose for the request's tokens (what its bfloat16 rounding made of close calls)."""
    from deterministic_inference_b200.engine import SequenceInput
    from deterministic_inference_b200.kernels import ops

    got = [None] * len(reqs)
    done, slots = {}, {}
    calls = []
    real = ops.route_experts

    def spy(*args, **kw):
        ids, weights = real(*args, **kw)
        calls.append(ids)
        return ids, weights
    if routes is not None:
        ops.route_experts = spy
    try:
        for entries in steps:
            ins = []
            for i, n in entries:
                if i not in slots:
                    slots[i], done[i] = runner.cache.allocate_slot(), 0
                ins.append(SequenceInput(slots[i], reqs[i][done[i]:done[i] + n], done[i], list(range(n))))
            calls.clear()
            logits, batch = runner.step(ins)
            logits = logits.detach().double().cpu()
            if routes is not None:
                at = 0
                for j in batch.order:               # the step's tokens lie in batch order
                    i, n = entries[j]
                    for k, ids in enumerate(calls):
                        mine = routes.setdefault(i, {}).setdefault(k, torch.zeros(len(reqs[i]), ids.shape[1], dtype=torch.long))
                        mine[done[i]:done[i] + n] = ids[at:at + n].long().cpu()
                    at += n
            for j, (i, n) in enumerate(entries):
                if got[i] is None:
                    got[i] = torch.full((len(reqs[i]), logits.shape[1]), float("nan"), dtype=torch.float64)
                got[i][done[i]:done[i] + n] = logits[torch.as_tensor(batch.logit_rows[j], dtype=torch.long)]
                done[i] += n
                if done[i] == len(reqs[i]):
                    runner.cache.release_slot(slots.pop(i))
    finally:
        ops.route_experts = real
    runner.cache.check_invariants()
    assert not slots, f"requests {sorted(slots)} were not finished by the schedule"
    return got


def schedules(lens, tail):
    return {"whole": whole(lens), "last tokens one by one": last_one_by_one(lens, tail),
            "portions": portions(lens), "mixed": mixed(lens, tail=min(tail, 12), seed=sum(lens))}


def runner_for(model_dir, dtype, device, page, lens, live=3, **kw):
    """A runner whose pool holds the ``live`` longest requests and no more, so that pages come back
    into use."""
    from deterministic_inference_b200.config import EngineConfig
    from deterministic_inference_b200.engine import ModelRunner

    longest = sorted(lens)[-live:]
    pool = sum(-(-n // page) * page for n in longest) + page
    return ModelRunner(EngineConfig(model_path=str(model_dir), dtype=dtype, device=device, kv_pool_tokens=pool,
                                    page_size=page, max_reqs=live, max_seq_len=-(-max(lens) // page) * page,
                                    debug_checks=True, **kw))
