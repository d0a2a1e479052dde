"""Plain-data descriptions of a network: which parts each layer is made of, with their sizes
and constants, and in which order the layers run.

A model is data before it is code.  An architecture's factory (``cuinfer_b200/models``) turns
its ``config.json`` into a :class:`ModelSpec`; :func:`cuinfer_b200.parts.model.build_model`
looks every ``kind`` up in the part registries and builds the objects.  The reference makes the
same choices with an ``if`` per layer inside ``CausalLM`` (csrc/model/causal_lm.cpp:41-64) and a
virtual ``FeedForward`` base (csrc/model/layers/mlp.h:10-16); here they are a table.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping


class PartSpec:
    """``kind`` plus free-form parameters, read as attributes (``spec.eps``).

    Immutable and hashable by content so that equal layers compare equal.
    """

    __slots__ = ("kind", "_params")

    def __init__(self, kind: str, **params: Any) -> None:
        object.__setattr__(self, "kind", kind)
        object.__setattr__(self, "_params", MappingProxyType(dict(params)))

    def __getattr__(self, name: str) -> Any:
        params = object.__getattribute__(self, "_params")
        try:
            return params[name]
        except KeyError:
            raise AttributeError(f"{self.kind!r} spec has no parameter {name!r}; it has {sorted(params)}") from None

    def __setattr__(self, name: str, value: Any) -> None:
        raise AttributeError("PartSpec is immutable")

    def get(self, name: str, default: Any = None) -> Any:
        return self._params.get(name, default)

    @property
    def params(self) -> Mapping[str, Any]:
        return self._params

    def replace(self, **changes: Any) -> "PartSpec":
        merged = dict(self._params)
        merged.update(changes)
        return PartSpec(self.kind, **merged)

    def __eq__(self, other: object) -> bool:
        return isinstance(other, PartSpec) and self.kind == other.kind and dict(self._params) == dict(other._params)

    def __hash__(self) -> int:
        return hash((self.kind, tuple(sorted((k, repr(v)) for k, v in self._params.items()))))

    def __repr__(self) -> str:
        inner = ", ".join(f"{k}={v!r}" for k, v in self._params.items())
        return f"PartSpec({self.kind!r}{', ' if inner else ''}{inner})"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (``block``) and the parts it arranges.

    ``prefix`` is the checkpoint name prefix of the layer's tensors (``model.layers.3``).
    ``norm`` describes the layer's norms; the block decides how many it needs and where.
    """

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec


@dataclass(frozen=True)
class ModelSpec:
    """The whole network.

    ``order`` lists layer indices in execution order; an index may appear twice (the layer
    runs twice with the same weights; each run has a cache of its own unless ``cache_source``
    says otherwise).  ``cache_source`` maps a position in ``order`` to an earlier position
    whose cache that run reads instead of writing its own.
    """

    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: tuple[LayerSpec, ...]
    final_norm: PartSpec
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm"
    lm_head_name: str | None = "lm_head.weight"   # None: the output head is the embedding table
    order: tuple[int, ...] | None = None
    cache_source: Mapping[int, int] = field(default_factory=dict)
    eos_token_ids: tuple[int, ...] = ()           # sampling one of these ends a request (unless it ignores them)

    def run_order(self) -> tuple[int, ...]:
        order = self.order if self.order is not None else tuple(range(len(self.layers)))
        for idx in order:
            if not 0 <= idx < len(self.layers):
                raise ValueError(f"order names layer {idx}, but the model has {len(self.layers)} layers")
        for run, src in self.cache_source.items():
            if not (0 <= src < run < len(order)):
                raise ValueError(f"cache_source[{run}]={src}: a run may only read the cache of an earlier run")
            if src in self.cache_source:
                raise ValueError(f"cache_source[{run}]={src}: run {src} has no cache of its own")
        return tuple(order)


@dataclass(frozen=True)
class TensorSpec:
    """A checkpoint tensor a part expects: exact name and shape.

    ``keep_stored_precision``: a tensor stored in 32 bits stays in 32 bits on a bfloat16
    engine (small vectors such as norm gains); matrices are brought to the engine's dtype.
    ``init`` tells the random-weights mode whether the tensor is a matrix or a gain around one.
    """

    name: str
    shape: tuple[int, ...]
    keep_stored_precision: bool = False
    integer: bool = False    # an integer table (kept as int32); a floating tensor in its place is refused, and vice versa
    init: str = "normal"     # how the random-weights mode fills it: "normal" or "ones" (a gain)


@dataclass(frozen=True)
class PagedCacheNeed:
    """What a mixer keeps per token: keys and values of ``num_kv_heads`` × ``head_dim``.

    ``window``: None keeps every token; ``w`` keeps only the last ``w`` (pages that a request's
    next query can no longer see are given back).
    """

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """What a mixer keeps per request, whatever its length: one tensor of ``shape``/``dtype``
    per run, zeroed when a request is admitted."""

    shape: tuple[int, ...]
    dtype: str = "float32"
