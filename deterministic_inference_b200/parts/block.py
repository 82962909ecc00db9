"""Arrangement of a layer's parts and of the residual stream.

``pre_norm``: norm -> mixer -> norm -> feed-forward, the residual carried beside
the hidden state: the first norm site takes the embedding as the residual, every
later one adds the previous part's output to the residual and norms the sum
(sid/model/qwen3.py:94-108).  The float32-stream forms below keep the residual
stream in float32 whatever type the parts compute in."""

from __future__ import annotations

from ..kernels import ops
from .base import Block
from .registry import NORMS, register_block
from .spec import PartSpec


@register_block("pre_norm")
class PreNormBlock(Block):
    def __init__(self, ctx, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def forward(self, hidden, residual, step, cache):
        if residual is None:
            residual = hidden
            hidden = self.mixer_norm.forward(hidden)
        else:
            hidden, residual = self.mixer_norm.add_forward(hidden, residual)
        hidden = self.mixer.forward(hidden, step, cache)
        hidden, residual = self.feed_forward_norm.add_forward(hidden, residual)
        hidden = self.feed_forward.forward(hidden)
        return hidden, residual


@register_block("pre_norm_f32_stream")
class PreNormStreamBlock(Block):
    """The same arrangement with the residual stream in float32: x <- x + mixer(norm(x)), then
    x <- x + feed_forward(norm(x)), every addition in float32 whatever type the parts
    compute in.  The stream comes in as float32 (from the embedding, or as the stream and
    the pending output of the layer before); a layer without a feed-forward (kind "none")
    hands its mixer's output on as the pending term."""

    def __init__(self, ctx, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def forward(self, hidden, residual, step, cache):
        if residual is None:
            residual = hidden
            hidden = self.mixer_norm.forward(residual)
        else:
            hidden, residual = self.mixer_norm.add_forward(hidden, residual)
        hidden = self.mixer.forward(hidden, step, cache)
        if self.feed_forward.kind == "none":
            return hidden, residual
        hidden, residual = self.feed_forward_norm.add_forward(hidden, residual)
        hidden = self.feed_forward.forward(hidden)
        return hidden, residual


@register_block("sandwich_f32_stream")
class SandwichStreamBlock(Block):
    """A norm in front of and behind each sublayer, the residual stream in float32:
    x <- x + post1(mixer(pre1(x))), then x <- x + post2(feed_forward(pre2(x))).  The post norms are
    ``stream_post_norm`` parts given as parameters; what they return is added to the stream inside the
    next norm's kernel (this layer's second norm, the next layer's first, or the model's last), so the
    block hands its last sublayer's normed output on as the pending term.  A layer without a
    feed-forward (kind "none") hands on its mixer's."""

    def __init__(self, ctx, mixer, feed_forward, mixer_norm, feed_forward_norm, mixer_post_norm: PartSpec,
                 feed_forward_post_norm: PartSpec):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.mixer_post_norm = NORMS.build(mixer_post_norm, ctx)
        self.feed_forward_post_norm = NORMS.build(feed_forward_post_norm, ctx)
        # parts of this block beyond the four every block has (the model loads their tensors)
        self.extra_parts = (self.mixer_post_norm, self.feed_forward_post_norm)

    def forward(self, hidden, residual, step, cache):
        if residual is None:
            residual = hidden
            hidden = self.mixer_norm.forward(residual)
        else:
            hidden, residual = self.mixer_norm.add_forward(hidden, residual)
        hidden = self.mixer_post_norm.forward(self.mixer.forward(hidden, step, cache))
        if self.feed_forward.kind == "none":
            return hidden, residual
        hidden, residual = self.feed_forward_norm.add_forward(hidden, residual)
        hidden = self.feed_forward_post_norm.forward(self.feed_forward.forward(hidden))
        return hidden, residual


@register_block("post_norm_f32_stream")
class PostNormStreamBlock(Block):
    """The norm sits on a sublayer's OUTPUT only, the residual stream is float32, and the sublayers
    read the stream itself: x <- x + norm1(mixer(x)), then x <- x + norm2(feed_forward(x)).  The two
    norms are ``stream_post_norm`` parts; what they return joins the stream inside the kernel that
    hands the stream to the next sublayer (``ops.stream_read``: the sum stays float32, the copy the
    sublayer reads is of the engine's type), so the block hands its last sublayer's normed output on
    as the pending term.  A layer without a feed-forward (kind "none") hands on its mixer's."""

    def __init__(self, ctx, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.dtype = ctx.dtype

    def forward(self, hidden, residual, step, cache):
        if residual is None:
            residual, hidden = hidden, None
        x = ops.stream_read(residual, hidden, self.dtype)
        hidden = self.mixer_norm.forward(self.mixer.forward(x, step, cache))
        if self.feed_forward.kind == "none":
            return hidden, residual
        x = ops.stream_read(residual, hidden, self.dtype)
        hidden = self.feed_forward_norm.forward(self.feed_forward.forward(x))
        return hidden, residual
