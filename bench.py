"""Benchmark of the engine on one B200: decode tokens/s (batch 8 by default, also
batch 1 and 64), prefill tokens/s at 2,048 tokens, both with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  Default model: the layer sizes of
Qwen3-0.6B (28 layers, hidden 1024, 16/8 heads of 128, intermediate 3072,
vocabulary 151936, tied head), random weights N(0, 0.02) from seed 0, bfloat16,
page size 16; each request holds 2,048 cached tokens when decoding starts.

``value``   decode tokens/s timed on the device (CUDA events): K decode steps through
            ``ModelRunner.step`` and the sampler (argmax), the sampled tokens handed to
            the next step on the device; nothing is read on the host in between.
``e2e``     the same through ``Engine.step()``: scheduler, packing, one
            host-to-device copy of the step's metadata from pinned memory, the
            graph, sampling, and the device-to-host read of the sampled tokens,
            every step.
``prefill`` a prompt of 2,048 tokens, whole, of a length not run before, through the
            captured graph of its bucket of prompt lengths (``value``, ``ms``); the same
            launched kernel by kernel (``launched_ms``, ``cold_ms``: a bucket's first two
            prompts) and replayed again (``replayed_ms``).
``points``  decode at batch 1 and 64; ``points_<preset>``: decode and prefill at a larger
            model's layer sizes with fewer layers (``config.second_model`` names both
            layer counts).
``--impl reference`` runs the unmodified reference engine on the same workload.
Every decode step reads all weights and the live cache (about 3 GB at batch 8),
far more than the 126 MB L2, so no L2 flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


REF_TREE = ROOT / "baseline" / "_ref"


def _stub_tokenizer(folder: Path) -> None:
    """The reference's ``Engine`` builds a tokenizer from the model folder whatever the
    prompts are; a three-word one satisfies it (requests come as token ids)."""
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    tok = Tokenizer(WordLevel({"<unk>": 0, "a": 1, "b": 2}, unk_token="<unk>"))
    tok.pre_tokenizer = Whitespace()
    tok.save(str(folder / "tokenizer.json"))
    (folder / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>"}))


def reference_arm(a) -> int:
    """The unmodified reference (a copy of its tree under ``baseline/_ref``; it has no
    packaging metadata, so it is put on the module path instead of installed) through its
    own public API: ``sid.engine.engine.Engine(EngineConfig(mode=NONDET))``,
    ``add_request(prompt_ids=...)`` and ``step()``.  Same model shape, random weights,
    batch, context, steps and warm-up as this repository's arm.  Its ``step()`` ends with
    the device-to-host read of the sampled tokens, so one timing gives both ``value`` and
    ``e2e``.  Nothing of this package's kernels is loaded in this process: only the
    random-weights writer (plain torch on the CPU) makes the model folder."""
    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
        return 0

    if a.gpus != 1:
        return unavailable("the reference is a single-GPU engine (no collective code); N>1 is not run")
    if not (REF_TREE / "sid" / "engine" / "engine.py").exists():
        return unavailable("no copy of the reference's tree under baseline/_ref")
    import tempfile
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        from deterministic_inference_b200.config import preset
        from deterministic_inference_b200.weights import write_random_model
        full = preset(a.preset)
        layers = a.layers or full.num_hidden_layers
        cfg = preset(a.preset, num_hidden_layers=layers, max_window_layers=layers)
        pk = peaks()
        sizes = sorted({a.batch, *[int(x) for x in a.points.split(",") if x.strip()]})
        max_b = max(sizes)
        new_tokens = max(a.steps, a.point_steps) + a.warmup + 32
        with tempfile.TemporaryDirectory(prefix="dib200_ref_model_") as folder:
            folder = Path(folder)
            write_random_model(cfg, 0, folder)
            _stub_tokenizer(folder)
            sys.path.insert(0, str(REF_TREE))
            from sid.config import EngineConfig as RefEngineConfig, Mode, SamplingParams as RefParams
            from sid.engine.engine import Engine as RefEngine
            pool = max_b * (a.context + new_tokens + 64) + a.prefill_tokens + 4096
            eng = RefEngine(RefEngineConfig(
                model_path=str(folder), mode=Mode.NONDET, kv_pool_tokens=pool,
                max_reqs=max(256, max_b + 8), max_seq_len=max(8192, a.context + new_tokens + 64),
                max_prompt_len=max(a.context, a.prefill_tokens), max_prefill_tokens=8192,
                max_decode_batch=max(256, max_b), device="cuda"))
            gen = torch.Generator().manual_seed(1)

            def random_prompt(n):
                return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

            def timed(fn):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                s.record()
                fn()
                e.record()
                torch.cuda.synchronize()
                return s.elapsed_time(e)

            def drain():
                while eng.scheduler.has_work():
                    eng.step()
                eng._done.clear()

            # prefill of one whole prompt: the step that admits it runs it and samples one token
            prompt = random_prompt(a.prefill_tokens)
            flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
            ms_list = []
            for it in range(0 if a.no_prefill else 6):
                eng.add_request(prompt_ids=prompt, params=RefParams(max_new_tokens=1, ignore_eos=True))
                flush.zero_()
                ms = timed(eng.step)
                drain()
                if it >= 3:
                    ms_list.append(ms)
            prefill = None
            if ms_list:
                pms = sorted(ms_list)[len(ms_list) // 2]
                _, flops = model_bytes_and_flops(cfg, layers, 1, 0, a.prefill_tokens)
                prefill = {"value": a.prefill_tokens / (pms / 1e3), "tokens": a.prefill_tokens, "ms": pms,
                           "frac": flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12)}

            def decode(batch, steps, sample_clocks=False):
                sp = RefParams(max_new_tokens=steps + a.warmup + 32, ignore_eos=True)
                for _ in range(batch):
                    eng.add_request(prompt_ids=random_prompt(a.context), params=sp)
                eng.step()                          # admits all and prefills them, untimed
                assert len(eng.scheduler.active) == batch and not eng.scheduler.waiting
                for _ in range(a.warmup):
                    eng.step()
                sampler = ClockSampler()
                if sample_clocks:
                    sampler.start()
                ms = timed(lambda: [eng.step() for _ in range(steps)])
                clocks = sampler.stop() if sample_clocks else None
                assert all(len(r.output_ids) >= steps + a.warmup for r in eng.scheduler.active)
                for r in eng.scheduler.active:      # stop them: the next step retires them
                    r.params.max_new_tokens = len(r.output_ids)
                    r.check_finished()
                drain()
                return ms, clocks

            ms, clocks = decode(a.batch, a.steps, sample_clocks=True)
            points = {}
            for b in sizes:
                if b != a.batch:
                    pms, _ = decode(b, a.point_steps)
                    points[f"decode_b{b}"] = b * a.point_steps / (pms / 1e3)
    except Exception as exc:  # the reference's kernels or its build failed here: say so, run nothing again
        return unavailable(f"{type(exc).__name__}: {exc}")
    value = a.batch * a.steps / (ms / 1e3)
    mean_ctx = a.context + a.warmup + a.steps / 2
    decode_bytes, _ = model_bytes_and_flops(cfg, layers, a.batch, mean_ctx, 0)
    achieved = decode_bytes / (ms / a.steps / 1e3) / 1e9
    print(json.dumps({
        "metric": "decode tok/s (bf16, 1 B200)", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference",
        "config": dict(bench_config(a, cfg, full, layers), page_size=1),
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": None,
                "d2h_bytes_per_step": a.batch * 8,
                "note": "the reference's step() reads the sampled tokens on the host every step; "
                        "value and e2e are the same timing"},
        "clocks": clocks, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"]},
        "points": points}))
    return 0


def bench_config(a, cfg, full, layers: int) -> dict:
    return {"model": a.preset, "layers": layers, "layers_full": full.num_hidden_layers,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "tied_head": cfg.tie_word_embeddings, "global_batch": a.batch,
            "seq_len": a.context, "context": 4096, "page_size": 16,
            "weights": "random N(0,0.02) seed 0", "parallelism": "1 GPU",
            "l2": "inputs larger than L2 (weights+cache per step)"}


def model_bytes_and_flops(cfg, layers: int, batch: int, ctx: float, prefill_tokens: int):
    h, i, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    hq, hkv, v = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.vocab_size
    layer_params = (hq + 2 * hkv) * d * h + h * hq * d + 3 * h * i
    weight_bytes = 2 * (layers * layer_params + v * h)            # every matrix once, head once
    kv_bytes_per_token = 2 * hkv * d * 2 * layers
    decode_bytes = weight_bytes + batch * ctx * kv_bytes_per_token
    t = prefill_tokens
    prefill_flops = 2 * t * layers * layer_params + layers * 2 * t * t * d * hq + 2 * v * h
    return decode_bytes, prefill_flops


# ---- another design beside the closest existing model, at equal layer sizes -------------------

DESIGN_SIZES = {
    # name -> (the Qwen3 preset of these layer sizes, the Gamilorn mixer sizes that go with them)
    "0_6b": ("qwen3_0_6b", dict(window=1024, keep=4, r_heads=16, r_dim=64)),
    "8b": ("qwen3_8b", dict(window=4096, keep=4, r_heads=64, r_dim=64)),
}


def gamilorn_like(q, layers: int, window: int, keep: int, r_heads: int, r_dim: int):
    """A Gamilorn configuration with the layer sizes of the Qwen3 configuration ``q``."""
    from deterministic_inference_b200.config.gamilorn_config import GamilornConfig
    layer = {"type": "parallel",
             "mixer": {"left": {"heads": q.num_attention_heads, "kv_heads": q.num_key_value_heads,
                                "dim": q.head_dim, "vdim": q.head_dim, "scale": q.head_dim ** -0.5,
                                "mask": {"size": window, "keep_first": keep}},
                       "left_scale": 1.0,
                       "right": {"heads": r_heads, "dim": r_dim, "decay_rank": 64},
                       "right_scale": 1.0},
             "mlp": {"kind": "dense", "ff": q.intermediate_size}}
    return GamilornConfig.from_dict({
        "architecture": "Gamilorn", "vocab": q.vocab_size, "width": q.hidden_size,
        "max_positions": 8192, "norm": {"eps": 1e-6}, "logit_softcap": 30.0, "layers": [layer] * layers})


ZATIRAX_SIZES = {
    # name -> the Zatirax mixer sizes that go with the Qwen3 preset of DESIGN_SIZES[name]: the attention
    # layers take Qwen3's heads; the latent layers as many heads of 64 plain + 64 rotated dimensions
    "0_6b": dict(chunk=1024, window=1024, rank=192, rot=64),
    "8b": dict(chunk=4096, window=4096, rank=192, rot=64),
}


def zatirax_like(q, layers: int, chunk: int, window: int, rank: int, rot: int):
    """A Zatirax configuration with the layer sizes of the Qwen3 configuration ``q``: an attention layer
    and a latent-attention layer, run ``layers`` / 2 times in a row (one loop over both)."""
    from deterministic_inference_b200.config.zatirax_config import ZatiraxConfig
    d = q.head_dim
    mlp = {"kind": "dense", "ff": q.intermediate_size, "limit": 7.0}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": q.num_attention_heads, "kv_heads": q.num_key_value_heads, "dim": d, "vdim": d,
                     "scale": d ** -0.5, "mask": {"size": chunk},
                     "rot": {"base": 500000.0, "dims": d // 2,
                             "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": q.num_attention_heads, "dim": d - rot, "rot_dim": rot, "vdim": d, "kv_rank": rank,
                     "scale": d ** -0.5, "mask": {"size": window}, "rot": {"base": 10000.0, "dims": rot}}}
    return ZatiraxConfig.from_dict({
        "architecture": "Zatirax", "vocab": q.vocab_size, "width": q.hidden_size, "norm": {"eps": 1e-6},
        "embedding": {"scale": 1.0}, "loop": {"start": 0, "stop": 2, "times": max(1, layers // 2)},
        "layers": [att, lat]})


KIPEZEN_SIZES = {
    # name -> the Kipezen sizes that go with the Qwen3 preset of DESIGN_SIZES[name]: the delta and the attention
    # heads are Qwen3's, the recurrent unit is as wide as the model in blocks of 128 channels, and a token's
    # experts (the chosen ones and the shared one) hold as many weights as Qwen3's dense feed-forward
    "0_6b": dict(window=1024, keep=4, taps=4, experts=16, top=2, expert_ff=768, shared_ff=1536, groups=(4, 2)),
    "8b": dict(window=4096, keep=4, taps=4, experts=32, top=4, expert_ff=1536, shared_ff=6144, groups=(8, 4)),
}


def kipezen_like(q, layers: int, window: int, keep: int, taps: int, experts: int, top: int, expert_ff: int,
                 shared_ff: int, groups: tuple):
    """A Kipezen configuration with the layer sizes of the Qwen3 configuration ``q``: delta layers and
    parallel layers (attention beside the recurrent unit) in turn, every one with routed experts."""
    from deterministic_inference_b200.config.kipezen_config import KipezenConfig
    d = q.head_dim
    mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "shared": {"ff": shared_ff},
           "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups[0], "keep": groups[1]}}}
    delta = {"type": "delta", "mlp": mlp,
             "mixer": {"heads": q.num_attention_heads, "kv_heads": q.num_key_value_heads, "dim": d, "vdim": d,
                       "conv": taps}}
    par = {"type": "parallel", "mlp": mlp,
           "mixer": {"left": {"heads": q.num_attention_heads, "kv_heads": q.num_key_value_heads, "dim": d, "vdim": d,
                              "scale": d ** -0.5, "mask": {"size": window, "keep_first": keep},
                              "rot": {"base": 10000.0, "dims": d // 2}},
                     "left_scale": 1.0,
                     "right": {"width": q.hidden_size, "blocks": q.hidden_size // 128, "conv": taps},
                     "right_scale": 1.0}}
    return KipezenConfig.from_dict({
        "architecture": "Kipezen", "vocab": q.vocab_size, "width": q.hidden_size, "max_positions": 8192,
        "norm": {"eps": 1e-6}, "layers": [delta if i % 2 == 0 else par for i in range(layers)]})


BOVITAR_SIZES = {
    # name -> the Bovitar sizes that go with the Qwen3 preset of DESIGN_SIZES[name]: the delta and the attention
    # heads are Qwen3's, the state-space branch is as wide as the model in heads of 64 with a state of 128, and
    # the experts are Kipezen's
    "0_6b": dict(taps=4, softcap=30.0, state=128, ssm_groups=1, norm_groups=1, experts=16, top=2, expert_ff=768,
                 shared_ff=1536, groups=(4, 2)),
    "8b": dict(taps=4, softcap=30.0, state=128, ssm_groups=8, norm_groups=8, experts=32, top=4, expert_ff=1536,
               shared_ff=6144, groups=(8, 4)),
}


def bovitar_like(q, layers: int, taps: int, softcap: float, state: int, ssm_groups: int, norm_groups: int,
                 experts: int, top: int, expert_ff: int, shared_ff: int, groups: tuple):
    """A Bovitar configuration with the layer sizes of the Qwen3 configuration ``q``: delta layers and
    parallel layers (attention beside the state-space branch) in turn, every one with routed experts; the
    second half of the layers runs with the weights of the first half."""
    from deterministic_inference_b200.config.bovitar_config import BovitarConfig
    d = q.head_dim
    mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "shared": {"ff": shared_ff},
           "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups[0], "keep": groups[1]}}}
    delta = {"type": "delta", "mlp": mlp,
             "mixer": {"heads": q.num_attention_heads, "kv_heads": q.num_key_value_heads, "dim": d, "vdim": d,
                       "conv": taps}}
    par = {"type": "parallel", "mlp": mlp,
           "mixer": {"left": {"heads": q.num_attention_heads, "kv_heads": q.num_key_value_heads, "dim": d, "vdim": d,
                              "conv": taps, "scale": d ** -0.5, "softcap": softcap,
                              "rot": {"base": 500000.0, "dims": d // 2,
                                      "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}},
                     "right": {"heads": q.hidden_size // 64, "vdim": 64, "state": state, "groups": ssm_groups,
                               "norm_groups": norm_groups, "conv": taps}}}
    own = max(2, layers // 2)
    entries = [dict(delta if i % 2 == 0 else par) for i in range(layers)]
    for i in range(own, layers):
        entries[i] = dict(entries[i], weights_of=i - own) if (i - own) % 2 == i % 2 else entries[i]
    return BovitarConfig.from_dict({
        "architecture": "Bovitar", "vocab": q.vocab_size, "width": q.hidden_size, "max_positions": 8192,
        "norm": {"eps": 1e-6}, "logit_scale": 0.5, "layers": entries})


def design_arm(a) -> int:
    """``--design zatirax``: the same for the Zatirax design; ``--design kipezen``: for the Kipezen design,
    beside Gamilorn (the closest design) instead of Qwen3.  ``--design gamilorn``: prompt and decode throughput of the Gamilorn design at layer sizes of
    real models (random weights, ``--design-layers`` layers), beside Qwen3 at the same sizes, and
    the new design's kernels one by one beside the like kernels of Qwen3, each with its share of
    the measured roofline.  Prints one JSON line of its own; the default benchmark is untouched."""
    import torch

    from deterministic_inference_b200 import EngineConfig, SamplingParams, preset
    from deterministic_inference_b200.engine.batch import SequenceInput, build_step_batch
    from deterministic_inference_b200.engine.engine import Engine
    from deterministic_inference_b200.kernels import ops
    from deterministic_inference_b200.sampling.sampler import sample

    pk = peaks()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    gen = torch.Generator().manual_seed(1)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)     # > L2
    greedy = SamplingParams(max_new_tokens=1 << 20, ignore_eos=True)
    n_layers, n_prompt, ctx = a.design_layers, a.prefill_tokens, a.context
    batches = sorted({int(x) for x in a.design_batches.split(",") if x.strip()})

    def timed(fn, repeats=5):
        """Median device time of ``fn`` in ms, L2 flushed before every run."""
        out = []
        for _ in range(repeats):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            out.append(s.elapsed_time(e))
        return sorted(out)[len(out) // 2]

    def prompt_of(vocab, n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    def engine_for(mcfg):
        per_req = ctx + a.point_steps + a.warmup + 96
        pool = max(batches) * (-(-per_req // 16) * 16) + n_prompt + 1024
        return Engine(EngineConfig(model_config=mcfg, random_seed=0, dtype="bfloat16", kv_pool_tokens=pool,
                                   page_size=16, max_reqs=max(batches) + 8, max_seq_len=8192,
                                   max_prefill_tokens=8192, max_decode_batch=max(256, max(batches)),
                                   device="cuda:0"))

    def prefill_ms(engine, vocab):
        runner, cache = engine.runner, engine.cache

        def once(n):
            slot = cache.allocate_slot()
            toks = prompt_of(vocab, n)
            ms = timed(lambda: runner.step([SequenceInput(slot, toks, 0, [n - 1])]), repeats=1)
            cache.release_slot(slot)
            return ms
        once(n_prompt - 40)
        return min(once(n_prompt) for _ in range(3))

    def decode_ms(engine, vocab, batch):
        runner, cache = engine.runner, engine.cache
        slots = [cache.allocate_slot() for _ in range(batch)]
        group = max(1, 8192 // ctx)
        for i in range(0, batch, group):
            runner.step([SequenceInput(s, prompt_of(vocab, ctx), 0, []) for s in slots[i:i + group]])
        state = {"tokens": None}

        def one(k):
            pend = state["tokens"] is not None
            entries = [SequenceInput(s, [0], ctx + k, [0], i if pend else -1) for i, s in enumerate(slots)]
            logits, _ = runner.step(entries, state["tokens"])
            state["tokens"] = sample(logits, [greedy] * batch, [ctx + k + 1] * batch)
        for k in range(a.warmup):
            one(k)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for k in range(a.warmup, a.warmup + a.point_steps):
            one(k)
        e.record()
        torch.cuda.synchronize()
        for sl in slots:
            cache.release_slot(sl)
        return s.elapsed_time(e) / a.point_steps

    def kernel_rows(eng_g, eng_q, gcfg, qcfg):
        """The new kernels and the like kernels of Qwen3 on one layer's shapes: a prompt of
        ``n_prompt`` tokens, and a decode step of 8 requests with ``ctx`` cached tokens."""
        rows = {}
        hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
        left = gcfg.layers[0]["mixer"]["left"]
        right = gcfg.layers[0]["mixer"]["right"]
        hq, hkv, d, w = left["heads"], left["kv_heads"], left["dim"], gcfg.width
        win, keep = left["mask"]["size"], left["mask"]["keep_first"]
        rh, rd, rank = right["heads"], right["dim"], right["decay_rank"]
        bf = torch.bfloat16

        def row(name, ms, nbytes, flops):
            floor = max(nbytes / hbm, flops / tf) * 1e3
            rows[name] = {"ms": round(ms, 4), "roofline_ms": round(floor, 4), "of_roofline": round(floor / ms, 4)}

        for what, batch, q_len, before in (("prompt", 1, n_prompt, 0), ("decode_b8", 8, 1, ctx)):
            t = batch * q_len
            for eng, mine in ((eng_g, True), (eng_q, False)):
                runner, cache = eng.runner, eng.cache
                slots = [cache.allocate_slot() for _ in range(batch)]
                if before:
                    for sl in slots:
                        runner.step([SequenceInput(sl, prompt_of(1000, before), 0, [])])
                entries = [SequenceInput(sl, [1] * q_len, before, []) for sl in slots]
                for e_ in entries:
                    cache.allocate(e_.slot, before + q_len)
                cache.reset_fresh_state()
                step = build_step_batch(entries, cache, dev)
                view = cache.view(0, step)
                q = torch.randn(t, hq, d, device=dev).to(bf)
                keys = batch * sum(min(p + 1, win + keep) if mine else p + 1 for p in range(before, before + q_len))
                att_flops = 4 * keys * hq * d
                att_bytes = 2 * (2 * t * hq * d + batch * hkv * 2 * d * min(before + q_len, (win + keep) if mine else 1 << 30))
                if mine:
                    kv = view.members[0]
                    pb = torch.zeros(hq, device=dev)
                    row(f"{what}: sigmoid attention", timed(lambda: ops.sigmoid_attention(
                        q, kv.kv, kv.attention_meta, d ** -0.5, pb, d, kv.page_size, win, keep)), att_bytes, att_flops)
                    width = 5 * rh * rd + rank
                    proj = torch.randn(t, width, device=dev)
                    w2 = (torch.randn(rank, rh * rd, device=dev) * 0.1).to(bf)
                    vec = torch.zeros(rh * rd, device=dev)
                    one = torch.ones(rh * rd, device=dev)
                    state = view.members[1].state
                    st_bytes = batch * rh * rd * rd * 4 * 2 + t * (width * 4 + rh * rd * 2)
                    row(f"{what}: delta rule (prepare, recurrence, output)", timed(lambda: ops.delta_rule(
                        proj, w2, vec, vec, one, state, step, rh, rd, rank, 0.6, 1e-6, 1e-6, bf)),
                        st_bytes, 8 * t * rh * rd * rd)
                    stream = torch.randn(t, w, device=dev)
                    x0 = torch.randn(t, w, device=dev).to(bf)
                    row(f"{what}: add + norm of the float32 stream (two terms)", timed(lambda: ops.stream_rms_norm(
                        stream, one[:1].expand(w).contiguous(), 1e-6, bf, add=ops.WeightedSum([(1.0, x0), (1.0, x0)]))),
                        t * w * (4 + 4 + 2 + 2 + 2), 0)
                    z = torch.randn(t, gcfg.layers[0]["mlp"]["ff"], device=dev)
                    row(f"{what}: xielu", timed(lambda: ops.xielu(z, 0.7, 1.2, bf)), z.numel() * 6, 0)
                    qkv = torch.randn(t, (hq + 2 * hkv) * d, device=dev)
                    bias = torch.zeros((hq + 2 * hkv) * d, device=dev)
                    row(f"{what}: q/k/v bias + cache write", timed(lambda: ops.qkv_bias_cache(
                        qkv, bias, hq, hkv, d, d, kv.kv, kv.slot_mapping, kv.page_size, bf)), qkv.numel() * 6, 0)
                else:
                    row(f"{what}: qwen3 softmax attention", timed(lambda: ops.paged_attention(
                        q, view.kv, view.attention_meta, d ** -0.5, None)), att_bytes, att_flops)
                    x0 = torch.randn(t, w, device=dev).to(bf)
                    res = torch.randn(t, w, device=dev).to(bf)
                    row(f"{what}: qwen3 add + norm", timed(lambda: ops.add_rms_norm(
                        x0, res, torch.ones(w, device=dev), 1e-6)), t * w * 2 * 4, 0)
                    gu = torch.randn(t, 2 * qcfg.intermediate_size, device=dev).to(bf)
                    row(f"{what}: qwen3 silu gate", timed(lambda: ops.silu_mul(gu)), gu.numel() * 3, 0)
                    qkv = torch.randn(t, (hq + 2 * hkv) * d, device=dev).to(bf)
                    nw = torch.ones(d, device=dev)
                    rope = runner.model.mixers[0].position_encoding.rotary_table()
                    row(f"{what}: qwen3 q/k norm + rotation + cache write", timed(lambda: ops.qk_norm_rope_cache(
                        qkv, hq, hkv, d, nw, nw, 1e-6, rope, step.positions, view.kv, view.slot_mapping,
                        view.page_size)), qkv.numel() * 4, 0)
                for sl in slots:
                    cache.release_slot(sl)
        return rows

    def zatirax_kernel_rows(eng_z, eng_q, zcfg, qcfg):
        """Zatirax's kernels and the like kernels of Qwen3 on one layer's shapes: a prompt of ``n_prompt``
        tokens, and a decode step of 8 requests with ``ctx`` cached tokens."""
        rows = {}
        hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
        att, lat = zcfg.layers[0]["mixer"], zcfg.layers[1]["mixer"]
        hq, hkv, d, w = att["heads"], att["kv_heads"], att["dim"], zcfg.width
        chunk, win = att["mask"]["size"], lat["mask"]["size"]
        lh, ld, lr, le, lc = lat["heads"], lat["dim"], lat["rot_dim"], lat["vdim"], lat["kv_rank"]
        ff = zcfg.layers[0]["mlp"]["ff"]
        bf = torch.bfloat16

        def row(name, ms, nbytes, flops):
            floor = max(nbytes / hbm, flops / tf) * 1e3
            rows[name] = {"ms": round(ms, 4), "roofline_ms": round(floor, 4), "of_roofline": round(floor / ms, 4)}

        for what, batch, q_len, before in (("prompt", 1, n_prompt, 0), ("decode_b8", 8, 1, ctx)):
            t = batch * q_len
            span = range(before, before + q_len)
            for eng, mine in ((eng_z, True), (eng_q, False)):
                runner, cache = eng.runner, eng.cache
                slots = [cache.allocate_slot() for _ in range(batch)]
                if before:
                    for sl in slots:
                        runner.step([SequenceInput(sl, prompt_of(1000, before), 0, [])])
                entries = [SequenceInput(sl, [1] * q_len, before, []) for sl in slots]
                for e_ in entries:
                    cache.allocate(e_.slot, before + q_len)
                cache.reset_fresh_state()
                step = build_step_batch(entries, cache, dev)
                q = torch.randn(t, hq, d, device=dev).to(bf)
                one_w = torch.ones(w, device=dev)
                if mine:
                    kv, lkv = cache.view(0, step), cache.view(1, step)
                    # chunked softmax attention with a sink (the tensor-core kernels Qwen3 runs on), then the gate
                    keys = batch * sum(p % chunk + 1 for p in span)
                    held = min(before + q_len, chunk)
                    sink = torch.zeros(hq, device=dev)
                    row(f"{what}: attention, chunk mask + sink", timed(lambda: ops.masked_attention(
                        q, kv.kv, kv.attention_meta, d ** -0.5, hkv, d, kv.page_size, "chunk", chunk, sink)),
                        2 * (2 * t * hq * d + batch * hkv * 2 * d * held), 4 * keys * hq * d)
                    proj = torch.randn(t, (2 * hq + 2 * hkv) * d, device=dev)
                    o = torch.randn(t, hq * d, device=dev).to(bf)
                    from ctypes import c_int, c_longlong
                    row(f"{what}: sigmoid gate on the heads", timed(lambda: ops._check(ops._lib("masked_attention").dib_sigmoid_gate_(
                        ops._ptr(o), *ops._source_args(proj), c_longlong(proj.shape[1]), c_longlong((hq + 2 * hkv) * d),
                        c_int(t), c_int(hq * d), c_int(1), ops._stream()), "gate")), t * hq * d * (2 + 2 + 4), 0)
                    freq = runner.model.mixers[0].freq
                    row(f"{what}: q/k norm + partial rotation + cache write", timed(lambda: ops.attn_prepare(
                        proj, hq, hkv, d, d, one_w[:d].contiguous(), one_w[:d].contiguous(), 1e-6, freq, d // 2,
                        step.positions, kv.kv, kv.slot_mapping, kv.page_size, bf)), t * (hq + 2 * hkv) * d * 6, 0)
                    # latent attention: one key head of rank + rot, values read out of the keys
                    ql = torch.randn(t, lh, lc + lr, device=dev).to(bf)
                    keys = batch * sum(min(p + 1, win) for p in span)
                    held = min(before + q_len, win)
                    row(f"{what}: latent attention (window)", timed(lambda: ops.masked_attention(
                        ql, lkv.kv, lkv.attention_meta, d ** -0.5, 1, lc, lkv.page_size, "window", win,
                        values_in_keys=True)), 2 * (t * lh * (2 * lc + lr) + batch * (lc + lr) * held),
                        2 * keys * lh * (2 * lc + lr))
                    lproj = torch.randn(t, lh * (ld + lr) + lc + lr, device=dev).to(bf)
                    mixer = runner.model.mixers[1]
                    def latent_rows():
                        qq = ops.latent_prepare(lproj, lh, ld, lr, lc, mixer.latent_norm, 1e-6, mixer.freq, step.positions,
                                                lkv.kv, lkv.slot_mapping, lkv.page_size, bf)
                        ops.heads_linear(lproj.as_strided((t, lh, ld), (lproj.shape[1], ld + lr, 1)), mixer.w_key, qq[:, :, :lc])
                        oo = torch.empty(t, lh, le, dtype=bf, device=dev)
                        ops.heads_linear(ql[:, :, :lc], mixer.w_value, oo)
                    row(f"{what}: latent rows + the two products per head", timed(latent_rows),
                        2 * (lproj.numel() + t * lh * (2 * lc + lr + le) + lh * lc * (ld + le)),
                        2 * t * lh * lc * (ld + le))
                    stream = torch.randn(t, w, device=dev)
                    x0 = torch.randn(t, w, device=dev).to(bf)
                    row(f"{what}: post norm + add + norm of the float32 stream", timed(lambda: ops.stream_rms_norm(
                        stream, one_w, 1e-6, bf, add=ops.NormedTerm(x0, one_w, 1e-6))), t * w * (4 + 4 + 2 + 2), 0)
                    gu = torch.randn(t, 2 * ff, device=dev)
                    row(f"{what}: limited gate", timed(lambda: ops.limited_gate(gu, 7.0, 1.702, bf)), gu.numel() * 4 + t * ff * 2, 0)
                else:
                    view = cache.view(0, step)
                    keys = batch * sum(p + 1 for p in span)
                    row(f"{what}: qwen3 softmax attention", timed(lambda: ops.paged_attention(
                        q, view.kv, view.attention_meta, d ** -0.5, None)),
                        2 * (2 * t * hq * d + batch * hkv * 2 * d * (before + q_len)), 4 * keys * hq * d)
                    x0 = torch.randn(t, w, device=dev).to(bf)
                    res = torch.randn(t, w, device=dev).to(bf)
                    row(f"{what}: qwen3 add + norm", timed(lambda: ops.add_rms_norm(x0, res, one_w, 1e-6)), t * w * 2 * 4, 0)
                    gu = torch.randn(t, 2 * qcfg.intermediate_size, device=dev).to(bf)
                    row(f"{what}: qwen3 silu gate", timed(lambda: ops.silu_mul(gu)), gu.numel() * 3, 0)
                    qkv = torch.randn(t, (hq + 2 * hkv) * d, device=dev).to(bf)
                    rope = runner.model.mixers[0].position_encoding.rotary_table()
                    row(f"{what}: qwen3 q/k norm + rotation + cache write", timed(lambda: ops.qk_norm_rope_cache(
                        qkv, hq, hkv, d, one_w[:d].contiguous(), one_w[:d].contiguous(), 1e-6, rope, step.positions,
                        view.kv, view.slot_mapping, view.page_size)), qkv.numel() * 4, 0)
                for sl in slots:
                    cache.release_slot(sl)
        return rows

    def kipezen_kernel_rows(eng_k, eng_g, kcfg, gcfg):
        """Kipezen's kernels and the like kernels of Gamilorn (the closest design: attention with a window
        and kept first keys beside a delta rule, a float32 stream) on one layer's shapes: a prompt of
        ``n_prompt`` tokens, and a decode step of 8 requests with ``ctx`` cached tokens."""
        rows = {}
        hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
        dl, par = kcfg.layers[0]["mixer"], kcfg.layers[1]["mixer"]
        left, right, mlp = par["left"], par["right"], kcfg.layers[0]["mlp"]
        hq, hkv, d, w = left["heads"], left["kv_heads"], left["dim"], kcfg.width
        win, keep = left["mask"]["size"], left["mask"]["keep_first"]
        n_exp, top, eff, sff = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"], mlp["shared"]["ff"]
        g_right = gcfg.layers[0]["mixer"]["right"]
        rh, rd, rank = g_right["heads"], g_right["dim"], g_right["decay_rank"]
        g_ff = gcfg.layers[0]["mlp"]["ff"]
        bf = torch.bfloat16

        def row(name, ms, nbytes, flops):
            floor = max(nbytes / hbm, flops / tf) * 1e3
            rows[name] = {"ms": round(ms, 4), "roofline_ms": round(floor, 4), "of_roofline": round(floor / ms, 4)}

        for what, batch, q_len, before in (("prompt", 1, n_prompt, 0), ("decode_b8", 8, 1, ctx)):
            t = batch * q_len
            span = range(before, before + q_len)
            keys = batch * sum(min(p + 1, win + keep) for p in span)
            held = min(before + q_len, win + keep)
            att_bytes, att_flops = 2 * (2 * t * hq * d + batch * hkv * 2 * d * held), 4 * keys * hq * d
            for eng, mine in ((eng_k, True), (eng_g, False)):
                runner, cache = eng.runner, eng.cache
                slots = [cache.allocate_slot() for _ in range(batch)]
                if before:
                    for sl in slots:
                        runner.step([SequenceInput(sl, prompt_of(1000, before), 0, [])])
                entries = [SequenceInput(sl, [1] * q_len, before, []) for sl in slots]
                for e_ in entries:
                    cache.allocate(e_.slot, before + q_len)
                cache.reset_fresh_state()
                step = build_step_batch(entries, cache, dev)
                q = torch.randn(t, hq, d, device=dev).to(bf)
                x = torch.randn(t, w, device=dev).to(bf)
                stream = torch.randn(t, w, device=dev)
                one_w = torch.ones(w, device=dev)
                blocks = runner.model.blocks
                if mine:
                    dview, pview = cache.view(0, step), cache.view(1, step)
                    kv, rstate = pview.members[0], pview.members[1].state
                    delta, att, glr = blocks[0].mixer, blocks[1].mixer.branches[0], blocks[1].mixer.branches[1]
                    ff = blocks[0].feed_forward
                    row(f"{what}: attention, window + kept first keys", timed(lambda: ops.masked_attention(
                        q, kv.kv, kv.attention_meta, d ** -0.5, hkv, d, kv.page_size, "window", win, keep_first=keep)),
                        att_bytes, att_flops)
                    proj = torch.randn(t, (hq + 2 * hkv) * d, device=dev)
                    row(f"{what}: q/k/v bias + norm over the projection + pair rotation + cache write", timed(
                        lambda: ops.attn_prepare(proj, hq, hkv, d, d, att.q_norm, att.k_norm, 1e-6, att.freq,
                                                 att.rotary_dim, step.positions, kv.kv, kv.slot_mapping, kv.page_size, bf,
                                                 bias=att.b_in, norm_scope="projection", rotary_layout="pairs")),
                        proj.numel() * 6, 0)
                    h, g, e = dl["heads"], dl["kv_heads"], dl["vdim"]
                    dproj = torch.randn(t, delta.w_in.shape[0], device=dev)
                    row(f"{what}: gated delta rule (convolutions, recurrence, output)", timed(lambda: ops.gated_delta_rule(
                        dproj, delta.conv, delta.a_log, delta.dt_bias, delta.norm_weight, dview.state, step, h, g, d, e,
                        dl["conv"], 1e-6, 1e-6, bf)),
                        batch * h * d * e * 4 * 2 + t * (dproj.shape[1] * 4 + h * e * 2), 8 * t * h * d * e)
                    c, per = right["width"], right["width"] // right["blocks"]
                    rproj = torch.randn(t, 2 * c, device=dev)
                    row(f"{what}: gated linear recurrence (convolution, gates, scan)", timed(
                        lambda: ops.gated_linear_recurrence(rproj, glr.b_in, glr.conv, glr.conv_bias, glr.gates,
                                                            glr.gate_bias, glr.neg_rate, rstate, step, c, right["blocks"],
                                                            right["conv"], bf)),
                        t * c * (8 + 2) + batch * right["conv"] * c * 8 + 2 * c * per * 4, 4 * t * c * per)
                    row(f"{what}: post norm + add into the float32 stream + read", timed(lambda: ops.stream_read(
                        stream, ops.NormedTerm(x, one_w, 1e-6), bf)), t * w * (4 + 4 + 2 + 2), 0)
                    logits = torch.randn(t, ff.w_router.shape[0], device=dev)
                    row(f"{what}: router", timed(lambda: ops.route_experts(
                        logits, ff.correction, n_exp, top, ff.group_count, ff.group_keep, 2.5, 1e-20)),
                        t * (logits.shape[1] * 4 + top * 8), 0)
                    ids, wts = ops.route_experts(logits, ff.correction, n_exp, top, ff.group_count, ff.group_keep, 2.5, 1e-20)
                    row(f"{what}: routed experts (sort, gate and up, down, sum)", timed(lambda: ops.routed_experts(
                        x, ids, wts, ff.w_gate_up, ff.w_down, None, None, n_exp, bf)),
                        min(n_exp, t * top) * 3 * eff * w * 2 + t * w * 6, 2 * t * top * 3 * eff * w)
                    row(f"{what}: feed-forward (router, shared expert, routed experts)", timed(lambda: ff.forward(x)),
                        (min(n_exp, t * top) * eff + sff) * 3 * w * 2 + t * w * 6, 2 * t * 3 * (top * eff + sff) * w)
                else:
                    view = cache.view(0, step)
                    kv = view.members[0]
                    pb = torch.zeros(hq, device=dev)
                    row(f"{what}: gamilorn sigmoid attention (window + kept first keys)", timed(lambda: ops.sigmoid_attention(
                        q, kv.kv, kv.attention_meta, d ** -0.5, pb, d, kv.page_size, win, keep)), att_bytes, att_flops)
                    qkv = torch.randn(t, (hq + 2 * hkv) * d, device=dev)
                    bias = torch.zeros((hq + 2 * hkv) * d, device=dev)
                    row(f"{what}: gamilorn q/k/v bias + cache write", timed(lambda: ops.qkv_bias_cache(
                        qkv, bias, hq, hkv, d, d, kv.kv, kv.slot_mapping, kv.page_size, bf)), qkv.numel() * 6, 0)
                    width = 5 * rh * rd + rank
                    proj = torch.randn(t, width, device=dev)
                    w2 = (torch.randn(rank, rh * rd, device=dev) * 0.1).to(bf)
                    vec, one = torch.zeros(rh * rd, device=dev), torch.ones(rh * rd, device=dev)
                    state = view.members[1].state
                    row(f"{what}: gamilorn delta rule (prepare, recurrence, output)", timed(lambda: ops.delta_rule(
                        proj, w2, vec, vec, one, state, step, rh, rd, rank, 0.6, 1e-6, 1e-6, bf)),
                        batch * rh * rd * rd * 4 * 2 + t * (width * 4 + rh * rd * 2), 8 * t * rh * rd * rd)
                    row(f"{what}: gamilorn add + norm of the float32 stream (two terms)", timed(lambda: ops.stream_rms_norm(
                        stream, one_w, 1e-6, bf, add=ops.WeightedSum([(1.0, x), (1.0, x)]))), t * w * (4 + 4 + 2 + 2 + 2), 0)
                    ff = blocks[0].feed_forward
                    row(f"{what}: gamilorn dense feed-forward", timed(lambda: ff.forward(x)),
                        3 * g_ff * w * 2 + t * w * 4, 2 * t * 3 * g_ff * w)
                for sl in slots:
                    cache.release_slot(sl)
        return rows

    def bovitar_kernel_rows(eng_b, eng_k, bcfg, kcfg):
        """Bovitar's kernels and the like kernels of Kipezen (the closest design: a gated delta rule, softmax
        attention beside a recurrent unit, routed experts, a float32 stream) on one layer's shapes: a prompt of
        ``n_prompt`` tokens, and a decode step of 8 requests with ``ctx`` cached tokens."""
        rows = {}
        hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
        par = bcfg.layers[1]["mixer"]
        left, right, mlp = par["left"], par["right"], bcfg.layers[0]["mlp"]
        hq, hkv, d, w = left["heads"], left["kv_heads"], left["dim"], bcfg.width
        n_exp, top = mlp["router"]["experts"], mlp["router"]["top"]
        k_left, k_right = kcfg.layers[1]["mixer"]["left"], kcfg.layers[1]["mixer"]["right"]
        win, keep = k_left["mask"]["size"], k_left["mask"]["keep_first"]
        sh, sp, sn, sg = right["heads"], right["vdim"], right["state"], right["groups"]
        inner, chan = sh * sp, sh * sp + 2 * sg * sn
        bf = torch.bfloat16

        def row(name, ms, nbytes, flops):
            floor = max(nbytes / hbm, flops / tf) * 1e3
            rows[name] = {"ms": round(ms, 4), "roofline_ms": round(floor, 4), "of_roofline": round(floor / ms, 4)}

        for what, batch, q_len, before in (("prompt", 1, n_prompt, 0), ("decode_b8", 8, 1, ctx)):
            t = batch * q_len
            span = range(before, before + q_len)
            for eng, mine in ((eng_b, True), (eng_k, False)):
                runner, cache = eng.runner, eng.cache
                slots = [cache.allocate_slot() for _ in range(batch)]
                if before:
                    for sl in slots:
                        runner.step([SequenceInput(sl, prompt_of(1000, before), 0, [])])
                entries = [SequenceInput(sl, [1] * q_len, before, []) for sl in slots]
                for e_ in entries:
                    cache.allocate(e_.slot, before + q_len)
                cache.reset_fresh_state()
                step = build_step_batch(entries, cache, dev)
                q = torch.randn(t, hq, d, device=dev).to(bf)
                x = torch.randn(t, w, device=dev).to(bf)
                stream = torch.randn(t, w, device=dev)
                one_w = torch.ones(w, device=dev)
                blocks = runner.model.blocks
                pview = cache.view(1, step)
                ff = blocks[0].feed_forward
                logits = torch.randn(t, ff.w_router.shape[0], device=dev)
                proj = torch.randn(t, (hq + 2 * hkv) * d, device=dev)
                if mine:
                    att, ssm = blocks[1].mixer.branches[0], blocks[1].mixer.branches[1]
                    kv, tail, sstate = pview.members[0].members[0], pview.members[0].members[1].state, pview.members[1].state
                    keys = batch * sum(p + 1 for p in span)
                    held = before + q_len
                    row(f"{what}: attention, causal, soft-capped scores", timed(lambda: ops.masked_attention(
                        q, kv.kv, kv.attention_meta, d ** -0.5, hkv, d, kv.page_size, "causal", None,
                        softcap=left["softcap"])),
                        2 * (2 * t * hq * d + batch * hkv * 2 * d * held), 4 * keys * hq * d)
                    row(f"{what}: q/k/v convolutions + norm over the projection + rotation + cache write", timed(
                        lambda: ops.attn_prepare(proj, hq, hkv, d, d, att.q_norm, att.k_norm, 1e-6, att.freq,
                                                 att.rotary_dim, step.positions, kv.kv, kv.slot_mapping, kv.page_size, bf,
                                                 norm_scope="projection", rotary_layout="halves", conv_weight=att.conv,
                                                 conv_state=tail, step=step)),
                        proj.numel() * 6 + batch * tail.shape[1] * 8, 0)
                    sproj = torch.randn(t, ssm.w_in.shape[0], device=dev)
                    row(f"{what}: state-space branch (convolution, recurrence, gated norm)", timed(lambda: ops.state_space(
                        sproj, ssm.conv, ssm.conv_bias, ssm.a_log, ssm.dt_bias, ssm.d_skip, ssm.norm_weight, sstate, step,
                        sh, sp, sn, sg, right["norm_groups"], right["conv"], 1e-6, bf)),
                        batch * sh * sn * sp * 4 * 2 + t * (sproj.shape[1] * 4 + chan * 8 + inner * 10),
                        5 * t * sh * sn * sp)
                    row(f"{what}: two normed branches + add + norm of the float32 stream", timed(
                        lambda: ops.stream_rms_norm(stream, one_w, 1e-6, bf, add=ops.WeightedSum(
                            [(0.5, ops.NormedTerm(x, one_w, 1e-6)), (0.5, ops.NormedTerm(x, one_w, 1e-6))]))),
                        t * w * (4 + 4 + 2 + 2 + 2), 0)
                    row(f"{what}: softmax router", timed(lambda: ops.route_experts(
                        logits, ff.correction, n_exp, top, ff.group_count, ff.group_keep, 2.5, 0.0, score="softmax",
                        group_top=1, normalize=False)), t * (logits.shape[1] * 4 + top * 8), 0)
                else:
                    att, glr = blocks[1].mixer.branches[0], blocks[1].mixer.branches[1]
                    kv, rstate = pview.members[0], pview.members[1].state
                    keys = batch * sum(min(p + 1, win + keep) for p in span)
                    held = min(before + q_len, win + keep)
                    row(f"{what}: kipezen attention, window + kept first keys", timed(lambda: ops.masked_attention(
                        q, kv.kv, kv.attention_meta, d ** -0.5, hkv, d, kv.page_size, "window", win, keep_first=keep)),
                        2 * (2 * t * hq * d + batch * hkv * 2 * d * held), 4 * keys * hq * d)
                    row(f"{what}: kipezen q/k/v bias + norm over the projection + pair rotation + cache write", timed(
                        lambda: ops.attn_prepare(proj, hq, hkv, d, d, att.q_norm, att.k_norm, 1e-6, att.freq,
                                                 att.rotary_dim, step.positions, kv.kv, kv.slot_mapping, kv.page_size, bf,
                                                 bias=att.b_in, norm_scope="projection", rotary_layout="pairs")),
                        proj.numel() * 6, 0)
                    c, per = k_right["width"], k_right["width"] // k_right["blocks"]
                    rproj = torch.randn(t, 2 * c, device=dev)
                    row(f"{what}: kipezen gated linear recurrence (convolution, gates, scan)", timed(
                        lambda: ops.gated_linear_recurrence(rproj, glr.b_in, glr.conv, glr.conv_bias, glr.gates,
                                                            glr.gate_bias, glr.neg_rate, rstate, step, c, k_right["blocks"],
                                                            k_right["conv"], bf)),
                        t * c * (8 + 2) + batch * k_right["conv"] * c * 8 + 2 * c * per * 4, 4 * t * c * per)
                    dl = kcfg.layers[0]["mixer"]
                    delta, dview = blocks[0].mixer, cache.view(0, step)
                    h, g, e = dl["heads"], dl["kv_heads"], dl["vdim"]
                    dproj = torch.randn(t, delta.w_in.shape[0], device=dev)
                    row(f"{what}: kipezen gated delta rule (convolutions, recurrence, output; the same kernels serve both designs)",
                        timed(lambda: ops.gated_delta_rule(
                            dproj, delta.conv, delta.a_log, delta.dt_bias, delta.norm_weight, dview.state, step, h, g, d, e,
                            dl["conv"], 1e-6, 1e-6, bf)),
                        batch * h * d * e * 4 * 2 + t * (dproj.shape[1] * 4 + h * e * 2), 8 * t * h * d * e)
                    row(f"{what}: kipezen post norm + add into the float32 stream + read", timed(lambda: ops.stream_read(
                        stream, ops.NormedTerm(x, one_w, 1e-6), bf)), t * w * (4 + 4 + 2 + 2), 0)
                    row(f"{what}: kipezen sigmoid router", timed(lambda: ops.route_experts(
                        logits, ff.correction, n_exp, top, ff.group_count, ff.group_keep, 2.5, 1e-20)),
                        t * (logits.shape[1] * 4 + top * 8), 0)
                eff, sff = mlp["expert"]["ff"], mlp["shared"]["ff"]
                row(f"{what}: {'' if mine else 'kipezen '}feed-forward (router, shared expert, routed experts)",
                    timed(lambda: ff.forward(x)),
                    (min(n_exp, t * top) * eff + sff) * 3 * w * 2 + t * w * 6, 2 * t * 3 * (top * eff + sff) * w)
                for sl in slots:
                    cache.release_slot(sl)
        return rows

    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    for name in [x for x in a.design_sizes.split(",") if x.strip()]:
        preset_name, extra = DESIGN_SIZES[name]
        qcfg = preset(preset_name, num_hidden_layers=n_layers, max_window_layers=n_layers)
        beside, bcfg = "qwen3", qcfg
        if a.design == "zatirax":
            extra = ZATIRAX_SIZES[name]
            gcfg = zatirax_like(qcfg, n_layers, **extra)
        elif a.design == "kipezen":
            # beside Gamilorn, the closest design, at the same layer sizes
            beside, bcfg = "gamilorn", gamilorn_like(qcfg, n_layers, **extra)
            extra = KIPEZEN_SIZES[name]
            gcfg = kipezen_like(qcfg, n_layers, **extra)
        elif a.design == "bovitar":
            # beside Kipezen, the closest design, at the same layer sizes
            beside, bcfg = "kipezen", kipezen_like(qcfg, n_layers, **KIPEZEN_SIZES[name])
            extra = BOVITAR_SIZES[name]
            gcfg = bovitar_like(qcfg, n_layers, **extra)
        else:
            gcfg = gamilorn_like(qcfg, n_layers, **extra)
        out = {"layers": n_layers, "width": qcfg.hidden_size, "heads": f"{qcfg.num_attention_heads}/{qcfg.num_key_value_heads} x {qcfg.head_dim}",
               "ff": qcfg.intermediate_size, a.design: dict(extra, parameters=gcfg.num_parameters()),
               f"{beside}_parameters": bcfg.num_parameters()}
        engines = {}
        for label, mcfg in ((a.design, gcfg), (beside, bcfg)):
            eng = engines[label] = engine_for(mcfg)
            ms = prefill_ms(eng, mcfg.vocab_size)
            r = {"prefill_ms": round(ms, 3), "prefill_tok_s": round(n_prompt / (ms / 1e3))}
            for b in batches:
                dms = decode_ms(eng, mcfg.vocab_size, b)
                r[f"decode_b{b}_ms"] = round(dms, 4)
                r[f"decode_b{b}_tok_s"] = round(b / (dms / 1e3))
            out[label + "_result"] = r
        rows_of = {"zatirax": zatirax_kernel_rows, "kipezen": kipezen_kernel_rows,
                   "bovitar": bovitar_kernel_rows}.get(a.design, kernel_rows)
        out["kernels"] = rows_of(engines[a.design], engines[beside], gcfg, bcfg)
        sizes[name] = out
        del engines
        import gc
        gc.collect()
        torch.cuda.empty_cache()
    beside = {"kipezen": "gamilorn", "bovitar": "kipezen"}.get(a.design, "qwen3")
    print(json.dumps({"metric": f"{a.design} beside {beside} at equal layer sizes (bf16, 1 B200)", "impl": "ours",
                      "dtype": "bf16", "data": "synthetic, random weights", "n_gpus": 1,
                      "prompt_tokens": n_prompt, "decode_context": ctx, "decode_steps": a.point_steps,
                      "warmup": a.warmup, "l2": "flushed before every timed kernel; steps hold more than L2",
                      "peaks": pk, "clocks": sampler.stop(), "sizes": sizes}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--preset", default="qwen3_0_6b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048, help="cached tokens per request")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the preset has")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--points", default="1,64", help="extra decode batch sizes")
    ap.add_argument("--point-steps", type=int, default=64)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"],
                    help="mixed: the continuous-batching run of the benchmark configurations "
                         "(64 requests, prompts uniform in [128, 2048], 256 outputs each, "
                         "temperature 0.7) through Engine.generate; prints its own line")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--second-preset", default="qwen3_8b",
                    help="layer sizes measured after the main model (decode batch 8 and 64, prefill), "
                         "with --second-layers layers; 'none' to skip")
    ap.add_argument("--second-layers", type=int, default=12)
    ap.add_argument("--profile", default=None, choices=["decode", "prefill"],
                    help="bracket this region with cudaProfilerStart/Stop (for ncu "
                         "--profile-from-start off); the numbers of such a run are not a result")
    ap.add_argument("--design", default=None, choices=["gamilorn", "zatirax", "kipezen", "bovitar"],
                    help="measure this design beside Qwen3 (kipezen: beside Gamilorn; bovitar: beside Kipezen) at equal layer sizes instead of the default "
                         "workload (prints a line of its own)")
    ap.add_argument("--design-sizes", default="0_6b,8b", help=f"of {sorted(DESIGN_SIZES)}")
    ap.add_argument("--design-layers", type=int, default=4)
    ap.add_argument("--design-batches", default="1,8,64")
    a = ap.parse_args()

    if a.warmup < 3:
        a.warmup = 3
    if a.impl == "reference":
        return reference_arm(a)
    if a.design is not None:
        return design_arm(a)
    if a.gpus != 1:
        print(f"bench.py measures one GPU only (this engine is single-GPU); --gpus {a.gpus} is not run")
        return 2

    import torch

    from deterministic_inference_b200 import EngineConfig, SamplingParams, preset
    from deterministic_inference_b200.engine.batch import SequenceInput
    from deterministic_inference_b200.engine.engine import Engine
    from deterministic_inference_b200.kernels import ops
    from deterministic_inference_b200.sampling.sampler import sample

    full = preset(a.preset)
    layers = a.layers or full.num_hidden_layers
    cfg = preset(a.preset, num_hidden_layers=layers, max_window_layers=layers)
    pk = peaks()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    gen = torch.Generator().manual_seed(1)
    greedy = SamplingParams(max_new_tokens=1 << 20, ignore_eos=True)

    def random_prompt(vocab, n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    def timed(fn):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e)

    def make_engine(mcfg, sizes, steps_most):
        max_b = max(sizes)
        per_req = a.context + steps_most + a.warmup + 96
        pool = max_b * (-(-per_req // 16) * 16) + a.prefill_tokens + 1024
        longest_prompt = a.prefill_tokens + 64        # the prefill run also feeds a few tokens more
        return Engine(EngineConfig(
            model_config=mcfg, random_seed=0, dtype="bfloat16", kv_pool_tokens=pool, page_size=16,
            max_reqs=max(256, max_b + 8),
            max_seq_len=max(8192, -(-per_req // 1024) * 1024, longest_prompt),
            max_prefill_tokens=max(8192, longest_prompt), max_decode_batch=max(256, max_b),
            device="cuda:0"))

    def launches_now(runner):
        """Kernels launched so far: the wrappers' own count plus what replayed graphs hold."""
        n = ops.launch_count
        for g in (runner.decode_graphs, runner.step_graphs):
            if g is not None:
                n += g.kernels_replayed
        return n

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > L2

    def measure_prefill(engine, mcfg, n_layers, profile=False):
        """One prompt of ``--prefill-tokens`` tokens, whole, to its first logits.  The engine
        launches a step kernel by kernel the first two times its bucket of shapes is seen
        (prompt lengths rounded up by a sixteenth of an octave) and replays the bucket's
        captured graph from the third time on, whatever the length inside the bucket.  Timed:
        ``launched_ms``: the prompt launched, bucket and libraries new (first) and known
        (second); ``value``/``ms``: a prompt of a length NOT run before, its bucket's graph
        captured (what a prompt costs in a running engine); ``replayed_ms``: the same length
        again.  Every timed prompt goes through ``ModelRunner.step`` from host tokens."""
        runner, cache = engine.runner, engine.cache
        n = a.prefill_tokens
        prompt = random_prompt(mcfg.vocab_size, n + 1)

        def once(tokens, profiled=False):
            slot = cache.allocate_slot()
            flush.zero_()
            if profiled:
                torch.cuda.synchronize()
                torch.cuda.profiler.start()
            ms = timed(lambda: runner.step([SequenceInput(slot, tokens, 0, [len(tokens) - 1])]))
            if profiled:
                torch.cuda.profiler.stop()
            cache.release_slot(slot)
            return ms

        once(prompt[:n + 40])                    # another bucket: load the libraries, warm the clocks
        launched = [once(prompt[:n - 2]), once(prompt[:n - 1])]      # the bucket's first and second time
        once(prompt[:n - 3])                     # the third: captured, then replayed
        sg = runner.step_graphs
        replays0 = sg.replays if sg is not None else 0
        fresh = once(prompt[:n], profiled=profile)                   # a length not run before
        replayed = [once(prompt[:n]) for _ in range(3)]
        in_graph = sg is not None and sg.replays - replays0 == 4
        ms = fresh if in_graph else min(launched + [fresh] + replayed)   # never captured: all were launched
        replayed_ms = sorted(replayed)[1] if in_graph else None
        _, flops = model_bytes_and_flops(mcfg, n_layers, 1, 0, n)
        frac = lambda t: flops / (t / 1e3) / (pk["bf16_tflops"] * 1e12)
        return {"value": n / (ms / 1e3), "tokens": n, "ms": ms, "cold_ms": min(launched),
                "launched_ms": [round(x, 3) for x in launched], "replayed_ms": replayed_ms,
                "frac": frac(ms), "frac_launched": frac(min(launched)),
                "note": ("value, ms and frac: a prompt length not run before, replayed through the "
                         "captured graph of its bucket of lengths; launched_ms: kernel by kernel, "
                         "the bucket's first and second time" if in_graph else
                         "value, ms and frac: launched kernel by kernel (the device bounds this step, so "
                         "its bucket is not captured before it has come many times)")}

    def fill_requests(engine, mcfg, batch):
        slots = [engine.cache.allocate_slot() for _ in range(batch)]
        group = max(1, 8192 // a.context)
        for i in range(0, batch, group):
            engine.runner.step([SequenceInput(s, random_prompt(mcfg.vocab_size, a.context), 0, [])
                                for s in slots[i:i + group]])
        return slots

    def device_decode(engine, mcfg, batch, steps, warmup, sample_clocks=False, profile=False):
        """``steps`` decode steps of ``batch`` requests through ``ModelRunner.step`` and the
        sampler, the sampled tokens handed to the next step on the device; nothing is read
        on the host inside the timed region."""
        runner = engine.runner
        slots = fill_requests(engine, mcfg, batch)
        params = [greedy] * batch
        state = {"tokens": None}

        def one(k):
            pend = state["tokens"] is not None
            entries = [SequenceInput(s, [0], a.context + k, [0], i if pend else -1)
                       for i, s in enumerate(slots)]
            logits, _ = runner.step(entries, state["tokens"])
            state["tokens"] = sample(logits, params, [a.context + k + 1] * batch)

        for k in range(warmup):
            one(k)
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
        n0 = launches_now(runner)
        if profile:
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
        ms = timed(lambda: [one(k) for k in range(warmup, warmup + steps)])
        if profile:
            torch.cuda.profiler.stop()
        launches = launches_now(runner) - n0
        clocks = sampler.stop() if sample_clocks else None
        for s in slots:
            engine.cache.release_slot(s)
        return ms, launches, clocks

    def decode_roofline(mcfg, n_layers, batch, steps, warmup, ms):
        mean_ctx = a.context + warmup + steps / 2
        nbytes, _ = model_bytes_and_flops(mcfg, n_layers, batch, mean_ctx, 0)
        achieved = nbytes / (ms / steps / 1e3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"]}

    sizes = sorted({a.batch, *[int(x) for x in a.points.split(",") if x.strip()]})
    engine = make_engine(cfg, sizes, max(a.steps, a.point_steps))
    graphs = engine.runner.decode_graphs

    if a.workload == "mixed":
        n_req, n_out = 64, 256
        lens = torch.randint(128, 2049, (n_req,), generator=gen).tolist()
        prompts = [random_prompt(cfg.vocab_size, n) for n in lens]
        sp = SamplingParams(max_new_tokens=n_out, temperature=0.7, seed=7, ignore_eos=True)
        # the first pass captures the CUDA graphs this workload needs (one per bucket of batch
        # size and context length, tens of milliseconds each); the second is the steady state
        runs = []
        for _ in range(2):
            steps0, replays0 = engine.runner.steps_run, (graphs.replays if graphs else 0)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            outs = engine.generate(prompts, sp)
            torch.cuda.synchronize()
            runs.append(time.perf_counter() - t0)
            assert all(len(o.token_ids) == n_out for o in outs)
        dt = runs[1]
        print(json.dumps({
            "metric": "continuous batching output tok/s (bf16, 1 B200)", "value": n_req * n_out / dt,
            "first_pass_value": n_req * n_out / runs[0],
            "graph_captures": {"decode": graphs.captures if graphs else 0,
                               "decode_seconds": graphs.capture_seconds if graphs else 0.0,
                               "steps": engine.runner.step_graphs.captures if engine.runner.step_graphs else 0,
                               "steps_seconds": engine.runner.step_graphs.capture_seconds
                               if engine.runner.step_graphs else 0.0},
            "unit": "tokens/s", "n_gpus": 1, "seconds": dt, "requests": n_req,
            "prompt_tokens": sum(lens), "output_tokens": n_req * n_out, "temperature": 0.7,
            "steps": engine.runner.steps_run - steps0, "preemptions": engine.scheduler.num_preemptions,
            "graph_replays": (graphs.replays if graphs else 0) - replays0, "dtype": "bf16", "data": "synthetic",
            "config": {"model": a.preset, "layers": layers, "layers_full": full.num_hidden_layers,
                       "max_prefill_tokens": engine.cfg.max_prefill_tokens}}))
        return 0

    prefill = None if a.no_prefill else measure_prefill(engine, cfg, layers, a.profile == "prefill")

    # ---------------- decode, timed on the device ----------------
    ms, launches, clocks = device_decode(engine, cfg, a.batch, a.steps, a.warmup, sample_clocks=True,
                                         profile=a.profile == "decode")
    value = a.batch * a.steps / (ms / 1e3)
    roofline = decode_roofline(cfg, layers, a.batch, a.steps, a.warmup, ms)
    points = {}
    for b in sizes:
        if b != a.batch:
            pms, _, _ = device_decode(engine, cfg, b, a.point_steps, a.warmup)
            points[f"decode_b{b}"] = b * a.point_steps / (pms / 1e3)
            points[f"decode_b{b}_frac"] = decode_roofline(cfg, layers, b, a.point_steps, a.warmup, pms)["frac"]

    # ---------------- decode end to end through Engine.step() ----------------
    e2e = None
    if not a.no_e2e:
        sp = SamplingParams(max_new_tokens=a.steps + a.warmup + 32, ignore_eos=True)   # nobody finishes inside the timed steps
        for _ in range(a.batch):
            engine.add_request(prompt_ids=random_prompt(cfg.vocab_size, a.context), params=sp)
        while any(r.num_output == 0 for r in list(engine.scheduler.running) + list(engine.scheduler.waiting)):
            engine.step()                       # prefill, untimed
        for _ in range(a.warmup):
            engine.step()
        e2e_ms = timed(lambda: [engine.step() for _ in range(a.steps)])
        assert all(r.num_output + r.num_pending >= a.steps for r in engine.scheduler.running)
        meta_bytes = max(c.layout.size for c in graphs.graphs.values()) * 4 if graphs and graphs.graphs else 0
        e2e = {"value": a.batch * a.steps / (e2e_ms / 1e3), "unit": "tokens/s",
               "ms_per_step": e2e_ms / a.steps,
               "h2d_bytes_per_step": meta_bytes, "d2h_bytes_per_step": a.batch * 4}
        while engine.has_work():
            engine.step()

    # ---------------- the same at a larger model's layer sizes, fewer layers ----------------
    second = None
    if a.second_preset and a.second_preset != "none" and a.profile is None:
        del engine, graphs
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        full2 = preset(a.second_preset)
        l2 = min(a.second_layers, full2.num_hidden_layers)
        cfg2 = preset(a.second_preset, num_hidden_layers=l2, max_window_layers=l2)
        eng2 = make_engine(cfg2, [8, 64], a.point_steps)
        second = {"model": a.second_preset, "layers": l2, "layers_full": full2.num_hidden_layers,
                  "hidden": cfg2.hidden_size, "heads": cfg2.num_attention_heads,
                  "kv_heads": cfg2.num_key_value_heads, "intermediate": cfg2.intermediate_size}
        if not a.no_prefill:
            pf = measure_prefill(eng2, cfg2, l2)
            second.update(prefill_tok_s=pf["value"], prefill_ms=pf["ms"], prefill_frac=pf["frac"],
                          prefill_launched_ms=pf["cold_ms"])
        for b in (8, 64):
            pms, _, _ = device_decode(eng2, cfg2, b, a.point_steps, a.warmup)
            second[f"decode_b{b}"] = b * a.point_steps / (pms / 1e3)
            second[f"decode_b{b}_frac"] = decode_roofline(cfg2, l2, b, a.point_steps, a.warmup, pms)["frac"]
        del eng2

    config = bench_config(a, cfg, full, layers)
    if second is not None:
        config["second_model"] = f"{second['model']} layer sizes, {second['layers']} of {second['layers_full']} layers"
    line = {
        "metric": "decode tok/s (bf16, 1 B200)", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours", "config": config,
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "prefill": prefill,
        "roofline": roofline, "points": points, "points_" + (a.second_preset or "none"): second,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
