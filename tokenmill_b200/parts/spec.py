"""Data that describes a model: which parts each layer is made of, and in which order layers run.

Nothing here computes. An architecture's builder turns its typed configuration into a ``ModelSpec``;
``parts.model.DecoderModel`` turns the spec into parts through the registry. Every size and constant
a part needs travels in ``PartSpec.params``, so a part never looks at a model configuration.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class WeightSpec:
    """One tensor of the checkpoint, by its safetensors name.

    dtype: "compute" - held in the run's dtype (bfloat16 or float32);
           "float32" - held in 32-bit whatever the run's dtype (norm weights, biases: small vectors
                       whose arithmetic is 32-bit in the kernels);
           "int32"   - an integer table.
    init:  how the random-weights writer fills it: ("normal", std), ("normal", std, mean),
           ("ones_plus_normal", std) or ("uniform", low, high).
    An empty ``name`` stands for the part's prefix itself (a part whose one tensor has no name of its own).
    """

    name: str
    shape: tuple[int, ...]
    dtype: str = "compute"
    init: tuple = ("normal", 0.02)


@dataclass(frozen=True)
class PagedKVNeed:
    """A mixer that keeps per-token keys and values. window=None: all keys stay; window=w: a query at
    position p reads keys p-w+1..p only, and pages wholly behind every future window are given back.
    planes=2: a key row and a value row per token; planes=1: one row per token (a cache of latents, from
    which keys and values are both derived, or keys and values of different sizes side by side).
    keep_first=n (with a window): the first n positions stay readable for every query, so their pages are never
    given back."""

    kv_heads: int
    head_dim: int
    window: int | None = None
    planes: int = 2
    keep_first: int = 0

    def group_key(self) -> tuple:
        return ("paged_kv", self.kv_heads, self.head_dim, self.window, self.planes, self.keep_first)


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a fixed-size state per request (zeroed when the request is admitted)."""

    shape: tuple[int, ...]
    dtype: str = "float32"


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def __hash__(self) -> int:
        return hash((self.kind, tuple(sorted((k, repr(v)) for k, v in self.params.items()))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a mixer and a feed-forward, each behind a norm, put together by a block kind.
    ``prefix`` is the checkpoint-name prefix of the layer's tensors ("model.layers.3")."""

    prefix: str
    block: str                      # arrangement, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec | None   # None: the layer has no feed-forward (arrangements that allow it)
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec | None
    mixer_name: str = "self_attn"                       # checkpoint sub-prefix of each part's tensors
    feed_forward_name: str = "mlp"
    mixer_norm_name: str = "input_layernorm"
    feed_forward_norm_name: str = "post_attention_layernorm"
    block_params: dict = field(default_factory=dict)    # sizes and constants of the arrangement itself


@dataclass(frozen=True)
class RunEntry:
    """One stop in the order layers run. ``layer`` indexes ``ModelSpec.layers`` and may appear in
    several entries (the same weights run twice; each run keeps a cache of its own). ``cache_of``
    names an EARLIER entry (by its place in the run order) whose cache this entry reads instead of
    keeping one."""

    layer: int
    cache_of: int | None = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding_name: str
    layers: list[LayerSpec]
    run_order: list[RunEntry]
    final_norm: PartSpec
    final_norm_prefix: str
    lm_head_name: str | None          # None: the output matrix is the embedding (tied)
    max_positions: int
    eos_token_ids: list[int] = field(default_factory=list)
    ignored_name_patterns: tuple[str, ...] = ()   # checkpoint names that may be present and are not loaded
    embedding_scale: float = 1.0                  # the stream starts as embedding row * this (multiplied in 32-bit)
    position_table_name: str | None = None        # a learned vector per position [max_positions, hidden], added to the
                                                  # embedding row where the stream starts (norms that take ``pos_table``)
    streams: int = 1                              # copies of the residual stream a token carries (hyper-connections);
                                                  # the blocks say how they are read and written
    logit_softcap: float = 0.0                    # logits <- cap * tanh(logits / cap); 0: none
    logit_scale: float = 1.0                      # the logits are multiplied by this first (before the cap)

    def validate(self) -> None:
        n = len(self.layers)
        for i, e in enumerate(self.run_order):
            if not (0 <= e.layer < n):
                raise ValueError(f"run_order[{i}] names layer {e.layer}, the model has {n}")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ValueError(f"run_order[{i}].cache_of={e.cache_of} must name an earlier entry")
                if self.run_order[e.cache_of].cache_of is not None:
                    raise ValueError(f"run_order[{i}].cache_of={e.cache_of} names an entry that has no cache "
                                     f"of its own")
