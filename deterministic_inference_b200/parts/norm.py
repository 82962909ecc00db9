"""RMSNorm part: y = x / sqrt(mean(x^2) + eps) * w, float32 arithmetic, eps
inside the root, the weight multiplies directly (sid/kernels/rmsnorm.py:14-24).
``add_forward`` is the fused residual form: residual += x, then the norm of the
unrounded sum, both in place (sid/kernels/rmsnorm.py:27-42)."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm
from .registry import register_norm
from .spec import TensorSpec


@register_norm("rms_norm")
class RMSNorm(Norm):
    def __init__(self, ctx, name: str, size: int, eps: float):
        self.name, self.size, self.eps = name, int(size), float(eps)
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.size,), role="vector", init="one_plus_normal")]

    def load(self, tensors):
        self.weight = tensors[self.name]

    def forward(self, x):
        return ops.rms_norm(x, self.weight, self.eps)

    def add_forward(self, x, residual):
        return ops.add_rms_norm(x, residual, self.weight, self.eps)


@register_norm("stream_rms_norm")
class StreamRMSNorm(Norm):
    """RMSNorm of a residual stream that is kept in float32 whatever the engine's storage type:
    y = x / sqrt(mean(x^2) + eps) * (weight_offset + w), written in the engine's type.
    ``weight_offset`` 1: the weight is stored around zero.  ``add_forward`` adds what the part
    before left (a tensor, split-k partial products or a weighted sum of several mixers'
    outputs) to the stream in float32, in place, and norms the sum."""

    def __init__(self, ctx, name: str, size: int, eps: float, weight_offset: float = 0.0):
        self.name, self.size, self.eps = name, int(size), float(eps)
        self.weight_offset = float(weight_offset)
        self.out_dtype = ctx.dtype
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.size,), role="vector",
                           init="normal" if self.weight_offset else "one_plus_normal")]

    def load(self, tensors):
        w = tensors[self.name]
        self.weight = (w + self.weight_offset).contiguous() if self.weight_offset else w

    def forward(self, x):
        return ops.stream_rms_norm(x, self.weight, self.eps, self.out_dtype)

    def add_forward(self, x, residual):
        return ops.stream_rms_norm(residual, self.weight, self.eps, self.out_dtype, add=x), residual


@register_norm("stream_post_norm")
class StreamPostNorm(Norm):
    """RMSNorm of a part's OUTPUT on its way into a float32 residual stream:
    stream += x / sqrt(mean(x^2) + eps) * (weight_offset + w).  ``forward`` only wraps its input
    (``ops.NormedTerm``); the stream's next reader (its next norm, ``ops.stream_read`` or
    ``ops.stream_add_``) computes it in float32 and adds it unrounded.  ``weight_offset`` 1: the
    weight is stored around zero."""

    def __init__(self, ctx, name: str, size: int, eps: float, weight_offset: float = 0.0):
        self.name, self.size, self.eps = name, int(size), float(eps)
        self.weight_offset = float(weight_offset)
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.size,), role="vector",
                           init="normal" if self.weight_offset else "one_plus_normal")]

    def load(self, tensors):
        w = tensors[self.name]
        self.weight = (w + self.weight_offset).contiguous() if self.weight_offset else w

    def forward(self, x):
        # (a tensor, split sums, or a weighted sum of several mixers' outputs: the reader adds it up)
        return ops.NormedTerm(x, self.weight, self.eps)


@register_norm("none")
class NoNorm(Norm):
    """The norm in front of a part that the layer does not have."""

    def __init__(self, ctx, **_):
        pass
