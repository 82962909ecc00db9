"""A recurrent block around a real-gated linear recurrent unit.

Two branches of ``width`` channels read the input: y = gelu_tanh(W_y x + b_y) and
u = conv(W_x x + b_x), a causal convolution over time per channel with a bias (``conv_taps`` taps,
the last one the current token's, zeros before the sequence's start, no activation).  u is cut into
``blocks`` equal parts; in part b the gates are r = sigmoid(R_b u_b + c_b) and i = sigmoid(I_b u_b +
d_b) with square matrices R_b, I_b ([out, in]).  With log a = -decay_scale * r * softplus(lam) the
state moves as
    S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t,   S = 0 before the first token,
and the output is W_o (S_t * y_t).  The state is float32 and lives in the request's state slot
together with the convolution's last ``conv_taps`` - 1 inputs; the convolution, the gates, the
decay and the recurrence are float32 whatever the engine's storage type.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer
from .registry import register_mixer
from .spec import StateSpec, TensorSpec


@register_mixer("gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    # (state slots from the step's device metadata; state slot 0 starts from zero and stores nothing)
    state_on_device = True

    def __init__(self, ctx, prefix: str, hidden_size: int, width: int, blocks: int, conv_taps: int,
                 decay_scale: float = 8.0, names: Optional[dict] = None):
        if width % blocks:
            raise ValueError(f"width {width} is not a multiple of blocks {blocks}")
        self.prefix = prefix
        self.hidden_size, self.width, self.blocks = int(hidden_size), int(width), int(blocks)
        self.conv_taps, self.decay_scale = int(conv_taps), float(decay_scale)
        self.names = dict(y="y", x="x", conv="conv", conv_bias="conv.b", recurrence_gate="ra", input_gate="ri",
                          lam="lam", o="o", bias_suffix=".b")
        self.names.update(names or {})
        self.out_dtype = ctx.dtype
        self.w_in = self.b_in = self.conv = self.conv_bias = self.gates = self.gate_bias = None
        self.neg_rate = self.w_o = None

    def tensor_specs(self):
        p, n, w, c, per = self.prefix, self.names, self.hidden_size, self.width, self.width // self.blocks
        s = n["bias_suffix"]
        return [TensorSpec(p + n["y"], (c, w)), TensorSpec(p + n["y"] + s, (c,), role="vector", init="normal"),
                TensorSpec(p + n["x"], (c, w)), TensorSpec(p + n["x"] + s, (c,), role="vector", init="normal"),
                TensorSpec(p + n["conv"], (c, self.conv_taps), role="vector", init="normal"),
                TensorSpec(p + n["conv_bias"], (c,), role="vector", init="normal"),
                TensorSpec(p + n["recurrence_gate"], (self.blocks, per, per), role="vector", init="normal"),
                TensorSpec(p + n["recurrence_gate"] + s, (self.blocks, per), role="vector", init="normal"),
                TensorSpec(p + n["input_gate"], (self.blocks, per, per), role="vector", init="normal"),
                TensorSpec(p + n["input_gate"] + s, (self.blocks, per), role="vector", init="normal"),
                TensorSpec(p + n["lam"], (c,), role="vector", init="normal"),
                TensorSpec(p + n["o"], (w, c))]

    def load(self, tensors):
        p, n, s = self.prefix, self.names, self.names["bias_suffix"]
        self.w_in = torch.cat([tensors[p + n["y"]], tensors[p + n["x"]]], dim=0).contiguous()
        self.b_in = torch.cat([tensors[p + n["y"] + s], tensors[p + n["x"] + s]]).contiguous()
        self.conv, self.conv_bias = tensors[p + n["conv"]], tensors[p + n["conv_bias"]]
        # the gates' matrices as [2, blocks, in, out] (the kernel's threads walk the outputs), float32
        self.gates = torch.stack([tensors[p + n["recurrence_gate"]].transpose(1, 2),
                                  tensors[p + n["input_gate"]].transpose(1, 2)]).contiguous()
        self.gate_bias = torch.stack([tensors[p + n["recurrence_gate"] + s].reshape(-1),
                                      tensors[p + n["input_gate"] + s].reshape(-1)]).contiguous()
        # log a = r * (-decay_scale * softplus(lam)): the factor is a constant of the channel
        self.neg_rate = (-self.decay_scale * torch.nn.functional.softplus(tensors[p + n["lam"]].float())).contiguous()
        self.w_o = tensors[p + n["o"]]

    def cache_spec(self):
        # one row of a slot: the state [width], then the convolution's tail [taps - 1, width]
        return StateSpec((self.conv_taps * self.width,), "float32")

    def forward(self, x, step, cache):
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32 if x.dtype != torch.float32 else None)
        y = ops.gated_linear_recurrence(proj, self.b_in, self.conv, self.conv_bias, self.gates, self.gate_bias,
                                        self.neg_rate, cache.state, step, self.width, self.blocks,
                                        self.conv_taps, self.out_dtype)
        return ops.linear(y, self.w_o)
