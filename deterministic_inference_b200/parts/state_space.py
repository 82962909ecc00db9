"""A state-space mixer with one scalar decay per head (the recurrent form of state-space duality).

One product W_in x gives [z: inner | x: inner | B: G N | C: G N | dt: H] with inner = ``num_heads`` *
``head_dim``, N = ``state_dim`` and G = ``groups``.  x, B and C together pass a causal convolution
over time per channel (``conv_taps`` taps, the last one the current token's, zeros before the
sequence's start) with a bias, and silu.  dt = softplus(dt + dt_bias), not clamped.  Head h reads the B
and C of group h // (H / G); its state S [N, head_dim] moves as
    S <- exp(-exp(A_log_h) dt) S + dt B x^T;     y = S^T C + D_h x.
y (the heads side by side) is multiplied by silu(z) and then RMS-normed in ``norm_groups`` equal parts,
each by its own root mean square (``norm_eps``), times a weight of size inner; then W_o.  The state
starts at zero, is float32 and lives in the request's state slot together with the convolution's last
``conv_taps`` - 1 inputs; dt, the decay, the convolution and the recurrence are float32 whatever the
engine's storage type.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer
from .registry import register_mixer
from .spec import StateSpec, TensorSpec


@register_mixer("state_space")
class StateSpace(Mixer):
    # the kernels take the sequences' state slots from the step's device metadata, and a
    # sequence on state slot 0 (padding) starts from zero and stores nothing
    state_on_device = True

    def __init__(self, ctx, prefix: str, hidden_size: int, num_heads: int, head_dim: int, state_dim: int,
                 groups: int, norm_groups: int, conv_taps: int, norm_eps: float, names: Optional[dict] = None):
        if num_heads % groups:
            raise ValueError(f"num_heads {num_heads} is not a multiple of groups {groups}")
        if (num_heads * head_dim) % norm_groups:
            raise ValueError(f"{num_heads} heads of {head_dim} do not split into {norm_groups} equal parts")
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.head_dim = int(hidden_size), int(num_heads), int(head_dim)
        self.state_dim, self.groups, self.norm_groups = int(state_dim), int(groups), int(norm_groups)
        self.conv_taps, self.norm_eps = int(conv_taps), float(norm_eps)
        self.names = dict(w_in="in", conv="conv", conv_bias="conv.b", dt_bias="dt_bias", a_log="A_log", d="D",
                          norm="norm", o="o")
        self.names.update(names or {})
        self.out_dtype = ctx.dtype
        self.w_in = self.conv = self.conv_bias = self.dt_bias = self.a_log = self.d_skip = None
        self.norm_weight = self.w_o = None

    @property
    def inner(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state_dim

    def tensor_specs(self):
        p, n, w, h = self.prefix, self.names, self.hidden_size, self.num_heads
        return [TensorSpec(p + n["w_in"], (self.inner + self.conv_channels + h, w)),
                TensorSpec(p + n["conv"], (self.conv_channels, self.conv_taps), role="vector", init="normal"),
                TensorSpec(p + n["conv_bias"], (self.conv_channels,), role="vector", init="normal"),
                TensorSpec(p + n["dt_bias"], (h,), role="vector", init="normal"),
                TensorSpec(p + n["a_log"], (h,), role="vector", init="normal"),
                TensorSpec(p + n["d"], (h,), role="vector", init="one_plus_normal"),
                TensorSpec(p + n["norm"], (self.inner,), role="vector", init="one_plus_normal"),
                TensorSpec(p + n["o"], (w, self.inner))]

    def load(self, tensors):
        p, n = self.prefix, self.names
        w_in = tensors[p + n["w_in"]]
        if w_in.shape[0] % 8:        # the product's rows filled up to a multiple of 8 with zeros
            w_in = torch.cat([w_in, torch.zeros(8 - w_in.shape[0] % 8, self.hidden_size, dtype=w_in.dtype,
                                                device=w_in.device)], dim=0)
        self.w_in = w_in.contiguous()
        self.conv, self.conv_bias = tensors[p + n["conv"]], tensors[p + n["conv_bias"]]
        self.dt_bias, self.a_log, self.d_skip = tensors[p + n["dt_bias"]], tensors[p + n["a_log"]], tensors[p + n["d"]]
        self.norm_weight, self.w_o = tensors[p + n["norm"]], tensors[p + n["o"]]

    def cache_spec(self):
        # one row of a slot: the heads' states [H, N, P], then the convolution's tail [taps - 1, channels]
        return StateSpec((self.num_heads * self.state_dim * self.head_dim
                          + (self.conv_taps - 1) * self.conv_channels,), "float32")

    def forward(self, x, step, cache):
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32 if x.dtype != torch.float32 else None)
        y = ops.state_space(proj, self.conv, self.conv_bias, self.a_log, self.dt_bias, self.d_skip, self.norm_weight,
                            cache.state, step, self.num_heads, self.head_dim, self.state_dim, self.groups,
                            self.norm_groups, self.conv_taps, self.norm_eps, self.out_dtype)
        return ops.linear(y, self.w_o)
