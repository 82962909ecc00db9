"""Grouped-query softmax attention over a paged cache, with everything that differs between
designs as a parameter.

One product of the concatenated weights gives [q | k | v | gate]; query head h reads key/value head
h // (heads / kv_heads); key heads have ``head_dim`` elements, value heads ``v_head_dim``.
``bias``: q, k and v take a bias each (``<name>.b``), added to the projection's float32 accumulator.
Optional RMS norm of q and k (``qk_norm_scope`` "head": per head, one weight of size head_dim each,
shared by the heads; "projection": over all heads of q (of k) at once, before they are split into
heads, one weight of that size each), then the position encoding's rotation of the first
``rotary_dim`` elements of every q and k head (the rest pass; ``rotary_layout`` "halves": element i
turns with i + rotary_dim / 2, "pairs": element 2i with 2i + 1).  score = q . k * scale.  ``mask``:
"causal" (every key up to the query), "window" (the last ``mask_size`` keys, the query's own
included; with ``keep_first`` also the sequence's first ``keep_first`` keys, at their true
positions) or "chunk" (the keys of the query's own chunk of ``mask_size`` positions, chunks counted
from position 0).  ``sink``: the softmax's denominator also
holds one more term exp(s_h), s_h a learned number per head, that brings nothing into the output.  ``gate``: the concatenated
heads are multiplied by sigmoid(W_g x) before the output projection.  ``softcap`` c: a score becomes
c * tanh(score / c) before the softmax.  ``conv_taps`` K: each channel of q, k and v passes a causal
convolution over time right after the projection, before norm and rotation (``<name>.conv`` [channels,
K], no bias, the last column the current token's, zeros before the sequence's start); a request's last
K - 1 projected values are float32 state beside its pages, so the part's cache is a composite of the
two.  Norms, angles, scores and the softmax are float32.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer
from .registry import POSITION_ENCODINGS, register_mixer
from .spec import CompositeSpec, PagedKVSpec, PartSpec, StateSpec, TensorSpec


@register_mixer("masked_attention")
class MaskedAttention(Mixer):
    def __init__(self, ctx, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 v_head_dim: int, scale: float, position_encoding: Optional[PartSpec] = None,
                 qk_norm_eps: Optional[float] = None, mask: str = "causal", mask_size: Optional[int] = None,
                 sink: bool = False, gate: bool = False, names: Optional[dict] = None, bias: bool = False,
                 qk_norm_scope: str = "head", rotary_layout: str = "halves", keep_first: int = 0,
                 softcap: Optional[float] = None, conv_taps: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if mask not in ("causal", "window", "chunk"):
            raise ValueError(f"mask {mask!r} is not known ('causal', 'window', 'chunk')")
        if mask != "causal" and (mask_size is None or int(mask_size) < 1):
            raise ValueError(f"a {mask} mask needs a positive mask_size")
        if qk_norm_scope not in ("head", "projection") or rotary_layout not in ("halves", "pairs"):
            raise ValueError(f"qk_norm_scope {qk_norm_scope!r} ('head', 'projection') or rotary_layout "
                             f"{rotary_layout!r} ('halves', 'pairs') is not known")
        if int(keep_first) < 0 or (int(keep_first) and mask != "window"):
            raise ValueError("keep_first belongs to a window mask and is not negative")
        if softcap is not None and not float(softcap) > 0:
            raise ValueError(f"a soft cap is positive, got {softcap!r}")
        if conv_taps is not None and int(conv_taps) < 1:
            raise ValueError(f"conv_taps {conv_taps!r}: a convolution has at least one tap")
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.scale = float(scale)
        self.softcap = None if softcap is None else float(softcap)
        self.conv_taps = None if conv_taps is None else int(conv_taps)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.mask, self.mask_size = mask, None if mask == "causal" else int(mask_size)
        self.sink, self.gate, self.bias = bool(sink), bool(gate), bool(bias)
        self.qk_norm_scope, self.rotary_layout, self.keep_first = qk_norm_scope, rotary_layout, int(keep_first)
        # checkpoint names of the part's tensors, after the prefix
        self.names = dict(q="q", k="k", v="v", o="o", gate="g", q_norm="q.norm", k_norm="k.norm", sink="sink",
                          bias_suffix=".b", conv_suffix=".conv")
        self.names.update(names or {})
        self.position_encoding = None if position_encoding is None \
            else POSITION_ENCODINGS.build(position_encoding, ctx)
        self.rotary_dim = getattr(self.position_encoding, "rotary_dim", 0)
        self.out_dtype = ctx.dtype
        self.w_in = self.w_o = self.q_norm = self.k_norm = self.sinks = self.freq = self.b_in = self.conv = None

    # (the convolution's kernels take state slots from the step's device metadata; a sequence on
    # state slot 0 starts from zeros and stores nothing)
    state_on_device = True

    def _sizes(self) -> dict:
        return dict(q=self.num_heads * self.head_dim, k=self.num_kv_heads * self.head_dim,
                    v=self.num_kv_heads * self.v_head_dim, gate=self.num_heads * self.v_head_dim)

    def _inputs(self) -> tuple:
        return ("q", "k", "v", "gate") if self.gate else ("q", "k", "v")

    def tensor_specs(self):
        p, n, w, sizes = self.prefix, self.names, self.hidden_size, self._sizes()
        specs = [TensorSpec(p + n[x], (sizes[x], w)) for x in self._inputs()]
        if self.bias:
            specs += [TensorSpec(p + n[x] + n["bias_suffix"], (sizes[x],), role="vector", init="normal")
                      for x in ("q", "k", "v")]
        if self.conv_taps is not None:
            specs += [TensorSpec(p + n[x] + n["conv_suffix"], (sizes[x], self.conv_taps), role="vector", init="normal")
                      for x in ("q", "k", "v")]
        if self.qk_norm_eps is not None:
            whole = self.qk_norm_scope == "projection"
            specs += [TensorSpec(p + n["q_norm"], (sizes["q"] if whole else self.head_dim,), role="vector",
                                 init="one_plus_normal"),
                      TensorSpec(p + n["k_norm"], (sizes["k"] if whole else self.head_dim,), role="vector",
                                 init="one_plus_normal")]
        if self.sink:
            specs.append(TensorSpec(p + n["sink"], (self.num_heads,), role="vector", init="normal"))
        specs.append(TensorSpec(p + n["o"], (w, self.num_heads * self.v_head_dim)))
        return specs

    def load(self, tensors):
        p, n = self.prefix, self.names
        self.w_in = torch.cat([tensors[p + n[x]] for x in self._inputs()], dim=0).contiguous()
        self.w_o = tensors[p + n["o"]]
        if self.bias:
            self.b_in = torch.cat([tensors[p + n[x] + n["bias_suffix"]] for x in ("q", "k", "v")]).contiguous()
        if self.conv_taps is not None:
            self.conv = torch.cat([tensors[p + n[x] + n["conv_suffix"]] for x in ("q", "k", "v")], dim=0).contiguous()
        if self.qk_norm_eps is not None:
            self.q_norm, self.k_norm = tensors[p + n["q_norm"]], tensors[p + n["k_norm"]]
        if self.sink:
            self.sinks = tensors[p + n["sink"]]
        if self.position_encoding is not None and self.rotary_dim:
            self.freq = self.position_encoding.frequencies()

    @property
    def _conv_state(self) -> bool:
        return self.conv_taps is not None and self.conv_taps > 1

    def cache_spec(self):
        pages = PagedKVSpec(self.num_kv_heads, self.head_dim, self.mask_size, v_head_dim=self.v_head_dim,
                            mask="chunk" if self.mask == "chunk" else "window", keep_first=self.keep_first)
        if not self._conv_state:
            return pages
        # beside the pages, one row of a slot: the convolutions' last taps - 1 inputs [taps - 1, q + k + v]
        sizes = self._sizes()
        return CompositeSpec((pages, StateSpec(((self.conv_taps - 1) * (sizes["q"] + sizes["k"] + sizes["v"]),),
                                               "float32")))

    def forward(self, x, step, cache):
        conv_state = None
        if self._conv_state:
            cache, conv_state = cache.members[0], cache.members[1].state
        # (few rows: the product's split-k partial sums, which the readers add in float32 while they load)
        if (self.bias or self.conv is not None) and x.dtype != torch.float32:
            # the biases join the projection's float32 accumulator, before anything is rounded
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        else:
            proj = ops.linear(x, self.w_in)
        q = ops.attn_prepare(proj, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim,
                             self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, self.freq, self.rotary_dim,
                             step.positions, cache.kv if cache.writes else None, cache.slot_mapping,
                             cache.page_size, self.out_dtype, bias=self.b_in, norm_scope=self.qk_norm_scope,
                             rotary_layout=self.rotary_layout, conv_weight=self.conv, conv_state=conv_state,
                             step=step)
        sizes = self._sizes()
        o = ops.masked_attention(q, cache.kv, cache.attention_meta, self.scale, self.num_kv_heads,
                                 self.v_head_dim, cache.page_size, self.mask, self.mask_size, self.sinks,
                                 gate=proj if self.gate else None,
                                 gate_col=sizes["q"] + sizes["k"] + sizes["v"], keep_first=self.keep_first,
                                 softcap=self.softcap)
        return ops.linear(o.view(o.shape[0], self.num_heads * self.v_head_dim), self.w_o)
