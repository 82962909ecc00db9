"""The two ends of the decoder as parts: the token embedding (a row gather,
sid/model/qwen3.py:93; or a row gather plus a learned position vector) and the head on the wanted rows (a matrix product whose float32
accumulator is the logits, sid/model/qwen3.py:113-115).  The head has a weight of its own
or shares the embedding's table (sid/model/loader.py:74-82)."""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Head, Part, TokenEmbedding
from .registry import register_embedding, register_head, register_stream_addend
from .spec import TensorSpec


@register_embedding("token_embedding")
class GatherEmbedding(TokenEmbedding):
    def __init__(self, ctx, name: str, vocab_size: int, hidden_size: int):
        self.name, self.vocab_size, self.hidden_size = name, int(vocab_size), int(hidden_size)
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), role="table")]

    def load(self, tensors):
        self.weight = tensors[self.name]

    def table(self):
        return self.weight

    def forward(self, ids):
        return ops.embedding(ids, self.weight)


@register_embedding("token_position_embedding")
class TokenPositionEmbedding(TokenEmbedding):
    """x = table[token] + positions[p]: a learned vector per position (counted from 0 in each
    sequence) is added, unscaled, to the token's row.  The sum is float32: this embedding
    opens a residual stream that is kept in float32."""

    needs_positions = True

    def __init__(self, ctx, name: str, position_name: str, vocab_size: int, hidden_size: int,
                 max_positions: int):
        self.name, self.position_name = name, position_name
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.max_positions = int(max_positions)
        self.weight = self.positions = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), role="table"),
                TensorSpec(self.position_name, (self.max_positions, self.hidden_size), role="table")]

    def load(self, tensors):
        self.weight, self.positions = tensors[self.name], tensors[self.position_name]

    def table(self):
        return self.weight

    def forward(self, ids, positions=None):
        return ops.embedding_positions(ids, positions, self.weight, self.positions)


@register_embedding("scaled_token_embedding")
class ScaledTokenEmbedding(TokenEmbedding):
    """x = table[token] * scale, in float32: this embedding opens a residual stream that is kept
    in float32."""

    def __init__(self, ctx, name: str, vocab_size: int, hidden_size: int, scale: float):
        self.name, self.vocab_size, self.hidden_size = name, int(vocab_size), int(hidden_size)
        self.scale = float(scale)
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), role="table")]

    def load(self, tensors):
        self.weight = tensors[self.name]

    def table(self):
        return self.weight

    def forward(self, ids):
        return ops.embedding_scaled(ids, self.weight, self.scale)


@register_stream_addend("row_vectors")
class RowVectors(Part):
    """``count`` learned vectors of the stream's width; ``forward(stream, i)`` adds vector i to every
    row of the float32 stream, in place."""

    def __init__(self, ctx, name: str, count: int, hidden_size: int):
        self.name, self.count, self.hidden_size = name, int(count), int(hidden_size)
        self.vectors = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.count, self.hidden_size), role="vector", init="normal")]

    def load(self, tensors):
        self.vectors = tensors[self.name]

    def forward(self, stream, index: int):
        if not 0 <= index < self.count:
            raise IndexError(f"{self.name}: vector {index} of {self.count}")
        return ops.stream_add_(stream, bias=self.vectors[index])


@register_head("linear_head")
class LinearHead(Head):
    """logits = rows @ W^T in float32, times ``scale`` (when it is not 1).  ``name`` None: W is the
    embedding's table."""

    def __init__(self, ctx, name: Optional[str], vocab_size: int, hidden_size: int,
                 softcap: Optional[float] = None, scale: float = 1.0):
        self.name, self.vocab_size, self.hidden_size = name, int(vocab_size), int(hidden_size)
        # softcap c: logits <- c * tanh(logits / c)
        self.softcap = None if softcap is None else float(softcap)
        self.scale = float(scale)
        self.tied = name is None
        self.weight = None

    def tensor_specs(self):
        return [] if self.tied else [TensorSpec(self.name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors):
        self.weight = tensors[None] if self.tied else tensors[self.name]
        if self.weight is None or tuple(self.weight.shape) != (self.vocab_size, self.hidden_size):
            raise ValueError(f"head: no [{self.vocab_size}, {self.hidden_size}] table to share or load")

    def forward(self, rows):
        # logits leave as a plain tensor (the product may come as split-k partials)
        logits = ops.as_tensor(ops.linear(rows, self.weight, out_dtype=torch.float32))
        if self.scale != 1.0:
            logits = ops.scale_(logits, self.scale)
        return logits if self.softcap is None else ops.softcap_(logits, self.softcap)
