"""Gated delta rule: a linear recurrence with a matrix state per head, one decay per head and short
causal convolutions in front of it.

q = W_q x and k = W_k x (``num_kv_heads`` heads of ``head_dim``), v = W_v x (``num_heads`` heads of
``v_head_dim``); value head h reads q/k head h // (num_heads / num_kv_heads).  Each of q, k, v
passes a causal convolution over time per channel (``conv_taps`` taps, the last one the current
token's, zeros before the sequence's start) and silu; q and k become unit vectors per head
(x / sqrt(sum(x^2) + key_eps)), q also times head_dim^(-1/2).  Per head beta = sigmoid(W_b x) and
the decay g = exp(-exp(A_log) * softplus(W_a x + dt_bias)).  The state S [head_dim, v_head_dim]
moves as
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
(the read-out sees the token's own write).  Each head's o is divided by its root mean square
(``norm_eps``), multiplied by a weight of size v_head_dim that the heads share and by silu(W_g x),
then projected by W_o.  The state starts at zero, is float32 and lives in the request's state slot
together with the convolutions' last ``conv_taps`` - 1 inputs; decays, rates, unit vectors and the
recurrence are float32 whatever the engine's storage type.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer
from .registry import register_mixer
from .spec import StateSpec, TensorSpec


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    # the kernels take the sequences' state slots from the step's device metadata, and a
    # sequence on state slot 0 (padding) starts from zero and stores nothing
    state_on_device = True

    def __init__(self, ctx, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 v_head_dim: int, conv_taps: int, norm_eps: float, key_eps: float = 1e-6,
                 names: Optional[dict] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim, self.conv_taps = int(head_dim), int(v_head_dim), int(conv_taps)
        self.norm_eps, self.key_eps = float(norm_eps), float(key_eps)
        self.names = dict(q="q", k="k", v="v", g="g", b="b", a="a", a_log="A_log", dt_bias="dt_bias",
                          norm="norm", o="o", conv_suffix=".conv")
        self.names.update(names or {})
        self.out_dtype = ctx.dtype
        self.w_in = self.conv = self.a_log = self.dt_bias = self.norm_weight = self.w_o = None

    def _sizes(self) -> dict:
        qk, v = self.num_kv_heads * self.head_dim, self.num_heads * self.v_head_dim
        return dict(q=qk, k=qk, v=v, g=v, b=self.num_heads, a=self.num_heads)

    @property
    def conv_channels(self) -> int:
        s = self._sizes()
        return s["q"] + s["k"] + s["v"]

    def tensor_specs(self):
        p, n, w, s = self.prefix, self.names, self.hidden_size, self._sizes()
        specs = []
        for x in ("q", "k", "v"):
            specs.append(TensorSpec(p + n[x], (s[x], w)))
            specs.append(TensorSpec(p + n[x] + n["conv_suffix"], (s[x], self.conv_taps), role="vector", init="normal"))
        specs += [TensorSpec(p + n[x], (s[x], w)) for x in ("b", "a", "g")]
        specs += [TensorSpec(p + n["a_log"], (self.num_heads,), role="vector", init="normal"),
                  TensorSpec(p + n["dt_bias"], (self.num_heads,), role="vector", init="normal"),
                  TensorSpec(p + n["norm"], (self.v_head_dim,), role="vector", init="one_plus_normal"),
                  TensorSpec(p + n["o"], (w, s["v"]))]
        return specs

    def load(self, tensors):
        p, n = self.prefix, self.names
        # one product for everything that is read from x: [q | k | v | g | b | a], its rows filled up
        # to a multiple of 8 with zeros
        mats = [tensors[p + n[x]] for x in ("q", "k", "v", "g", "b", "a")]
        rows = sum(m.shape[0] for m in mats)
        if rows % 8:
            mats.append(torch.zeros(8 - rows % 8, self.hidden_size, dtype=mats[0].dtype, device=mats[0].device))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.conv = torch.cat([tensors[p + n[x] + n["conv_suffix"]] for x in ("q", "k", "v")], dim=0).contiguous()
        self.a_log, self.dt_bias = tensors[p + n["a_log"]], tensors[p + n["dt_bias"]]
        self.norm_weight, self.w_o = tensors[p + n["norm"]], tensors[p + n["o"]]

    def cache_spec(self):
        # one row of a slot: the heads' states [H, D, E], then the convolutions' tail [taps - 1, channels]
        return StateSpec((self.num_heads * self.head_dim * self.v_head_dim
                          + (self.conv_taps - 1) * self.conv_channels,), "float32")

    def forward(self, x, step, cache):
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32 if x.dtype != torch.float32 else None)
        y = ops.gated_delta_rule(proj, self.conv, self.a_log, self.dt_bias, self.norm_weight, cache.state, step,
                                 self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim,
                                 self.conv_taps, self.key_eps, self.norm_eps, self.out_dtype)
        return ops.linear(y, self.w_o)
