"""Plain data that describes a model as parts.

A model is a ``ModelPlan``: a tuple of ``LayerSpec`` (which mixer, feed-forward,
norms and block arrangement a layer is made of, each with its sizes and
constants as parameters) and a ``schedule``, the order in which layers run.  The
schedule is data too: an entry may name a layer a second time, and it names the
cache its mixer uses, so a layer may read the cache another entry wrote.

Nothing in this module knows an architecture; the architecture's configuration
class produces a plan, and the generic decoder builds and runs it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind and its parameters (sizes, constants,
    checkpoint names)."""

    kind: str
    params: dict = field(default_factory=dict)

    def __hash__(self):  # params is a dict; identity is enough for frozen use
        return id(self)


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec               # arrangement of the parts below and the residual
    mixer: PartSpec               # token mixer (attention here)
    feed_forward: PartSpec        # dense or experts
    mixer_norm: PartSpec          # norm in front of the mixer
    feed_forward_norm: PartSpec   # norm in front of the feed-forward


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  ``cache`` is the id of the cache (or state) its
    mixer works on; exactly one entry writes a given cache, and it runs before
    the entries that only read it."""

    layer: int
    cache: int
    writes_cache: bool = True
    enter_vector: Optional[int] = None   # the plan's ``stream_addend`` adds its vector of this index
                                         # to the residual stream right before the layer runs


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec               # token ids -> hidden states
    head: PartSpec                    # hidden states of the wanted rows -> float32 logits
    final_norm: PartSpec
    layers: tuple
    schedule: tuple
    max_positions: int
    eos_token_ids: tuple = ()
    ignored_names: tuple = ()         # checkpoint tensors that may be present and are not used
    ignored_substrings: tuple = ()
    stream_addend: Optional[PartSpec] = None   # learned vectors that schedule entries add to the stream

    def validate(self) -> None:
        writers: dict[int, int] = {}
        for pos, e in enumerate(self.schedule):
            if e.enter_vector is not None and self.stream_addend is None:
                raise ValueError(f"schedule entry {pos} adds vector {e.enter_vector}, the plan has no stream addend")
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {pos} names layer {e.layer}, "
                                 f"the plan has {len(self.layers)}")
            if e.writes_cache:
                if e.cache in writers:
                    raise ValueError(f"cache {e.cache} is written by schedule entries "
                                     f"{writers[e.cache]} and {pos}")
                writers[e.cache] = pos
        for pos, e in enumerate(self.schedule):
            if not e.writes_cache:
                if e.cache not in writers:
                    raise ValueError(f"schedule entry {pos} reads cache {e.cache} that no entry writes")
                if writers[e.cache] > pos:
                    raise ValueError(f"schedule entry {pos} reads cache {e.cache} before "
                                     f"entry {writers[e.cache]} writes it")


@dataclass(frozen=True)
class TensorSpec:
    """A checkpoint tensor a part needs: name, shape, and what it is.

    role "matrix": a linear weight [out, in], cast to the engine dtype.
    role "table":  the embedding [vocab, hidden], cast to the engine dtype.
    role "vector": a norm weight; kept in float32 whatever it is stored as
                   (norm math is float32).
    ``init`` names the law the random-weights mode draws it from.
    """

    name: str
    shape: tuple
    role: str = "matrix"
    init: str = "normal"          # "normal": N(0, std); "one_plus_normal": 1 + N(0, norm_std)


@dataclass(frozen=True)
class PagedKVSpec:
    """Cache need of an attention-like mixer: keys and values per token.
    ``window`` None: all keys are kept; an int: only the last ``window`` keys are
    ever read, so older pages can be given back.  ``mask`` says what the int means:
    "window": a query at position p reads the keys p - window + 1 .. p; "chunk": the keys of
    its own chunk of ``window`` positions, floor(p / window) * window .. p (chunks counted from
    position 0)."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None   # size of a value head; None: that of a key head; 0: no
                                       # values are stored (the mixer reads them out of the keys)
    keep_first: int = 0                # with a window: the first ``keep_first`` keys stay readable
    mask: str = "window"

    def __post_init__(self):
        if self.mask not in ("window", "chunk"):
            raise ValueError(f"mask {self.mask!r} is not known ('window' or 'chunk')")
        if self.mask == "chunk" and (self.window is None or self.keep_first):
            raise ValueError("a chunk mask needs a size and keeps no first keys")

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim

    def first_needed(self, position: int) -> int:
        """The oldest key a query at ``position`` (or any later one) can read, the kept first
        keys aside."""
        if self.window is None:
            return 0
        if self.mask == "chunk":
            return position // self.window * self.window
        return max(0, position - self.window + 1)

    def group_key(self) -> tuple:
        key = ("paged_kv", self.num_kv_heads, self.head_dim, self.window)
        if self.value_dim != self.head_dim or (self.window is not None and self.keep_first) \
                or self.mask != "window":
            key += (self.value_dim, self.keep_first if self.window is not None else 0)
        if self.mask != "window":
            key += (self.mask,)
        return key


@dataclass(frozen=True)
class StateSpec:
    """Cache need of a mixer with per-request state of fixed size."""

    shape: tuple
    dtype: str = "float32"

    def group_key(self) -> tuple:
        return ("state", tuple(self.shape), self.dtype)


@dataclass(frozen=True)
class CompositeSpec:
    """Cache need of a mixer made of several mixers that run side by side on the same
    input: one member per inner mixer (``None`` for one that keeps nothing).  The cache
    manager keeps every member in the group of its own kind; the mixer sees them as
    ``CacheView.members``, in this order."""

    members: tuple

    def group_key(self) -> tuple:
        return ("composite",) + tuple(None if m is None else m.group_key() for m in self.members)


def flatten_cache_specs(cache_specs: dict) -> dict:
    """cache id -> need, with every ``CompositeSpec`` replaced by its members under the ids
    ``(cache id, member index)``; members that keep nothing are left out.  A member may be a
    composite itself (a mixer that keeps pages and a state row inside a pair of mixers): its
    members get the ids ``((cache id, member index), member index)``."""
    flat = {}

    def walk(cid, spec):
        if isinstance(spec, CompositeSpec):
            for mi, m in enumerate(spec.members):
                if m is not None:
                    walk((cid, mi), m)
        else:
            flat[cid] = spec

    for cid in sorted(cache_specs):
        walk(cid, cache_specs[cid])
    return flat


def composite_cache_ids(cache_specs: dict) -> dict:
    """id of every composite cache (nested ones under their ``(cache id, member index)`` ids) -> its
    number of members."""
    out = {}

    def walk(cid, spec):
        if isinstance(spec, CompositeSpec):
            out[cid] = len(spec.members)
            for mi, m in enumerate(spec.members):
                walk((cid, mi), m)

    for cid, spec in cache_specs.items():
        walk(cid, spec)
    return out
