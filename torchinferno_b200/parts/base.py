"""Interfaces of the parts a layer is put together from, and their registry.

A model is data: a list of blocks, each naming a mixer, a feed-forward, its
norms and a position encoding by *kind* with their sizes and constants as
parameters (:class:`PartSpec`).  The kinds are looked up here.  A part never
learns which model it is in: it sees its parameters, its weights (by names
relative to its own prefix) and, at run time, a :class:`LayerContext`.

Adding a part: subclass the interface, then ``register_part("mixer", "my_kind",
MyMixer)``; a model description may name it at once.

Interfaces
----------
``Part``           ``weight_specs()``, ``bind(weights)``
``Norm``           ``forward(residual, out, rows)`` / ``add_forward(delta, residual, out, rows)``
``PositionEncoding`` ``encode_and_store(qkv, q_out, ctx, heads, kv_heads, head_dim)``
``Mixer``          ``cache_spec()``, ``side_cache_spec()``, ``state_spec()``, ``forward(x, ctx) -> y``
``FeedForward``    ``forward(x, ctx) -> y``
``Block``          ``forward(stream, ctx)`` on a :class:`ResidualStream`
``StreamStage``    ``forward(stream, ctx)`` between the embedding and the first block
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import torch


# --------------------------------------------------------------------- data
@dataclass(frozen=True)
class PartSpec:
    """A part named by kind, with its sizes and constants."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""  # weight-name prefix relative to the enclosing block


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part reads from the checkpoint, by name relative to its prefix."""
    name: str
    shape: tuple[int, ...]
    init: str = "normal"       # random mode: "normal" (std), "about_one" (1 + normal), "about_identity" (unit matrix + normal),
                               # "ones", "zeros"
    std: float = 0.02
    role: str = "matrix"       # "matrix": kept as stored (bf16 / fp32); "vector": widened to fp32;
                               # "int_table": integer table kept as int32
    optional: bool = False     # may be absent from the file (then the part copes)
    free_dims: tuple[int, ...] = ()   # dimensions whose size the file decides (``shape`` holds what random weights get);
                                      # the part reads the size off the tensor it is bound to


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer keeps per token: for each of ``kv_heads`` heads a key of ``head_dim`` elements and a
    value of ``value_dim`` elements (None: as wide as the key; 0: keys only, e.g. one latent vector).

    ``window``: None keeps every token; w > 0 means a query at position p reads
    keys p-w+1 .. p only, so pages wholly behind the window may be given back.

    ``stride``: s > 1 means the cache holds one entry for every full run of s tokens (entry b stands for the
    positions b*s .. b*s + s - 1 and exists once the last of them has arrived): a summary of the run, such as
    the mean of its keys.  Such a cache grows s times slower than the request.
    """
    kv_heads: int
    head_dim: int
    window: int | None = None
    value_dim: int | None = None
    stride: int = 1

    @property
    def value_width(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim

    @property
    def elements_per_token(self) -> int:
        return self.kv_heads * (self.head_dim + self.value_width)


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size (it does not grow with tokens)."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class KVBinding:
    """The cache one layer call reads and, unless ``writes`` is False, writes."""
    pool: torch.Tensor          # this cache layer's pages: [pages, 2, kv_heads, page_size, head_dim] when keys and
                                # values are equally wide, else the flat pages [pages, elements of a page]
    block_table: torch.Tensor   # [slots, max_pages] int32, on the device
    page_size: int
    window: int | None
    writes: bool = True
    keys: torch.Tensor | None = None     # [pages, kv_heads, page_size, head_dim], a view of the pages
    values: torch.Tensor | None = None   # [pages, kv_heads, page_size, value width], a view of the pages


@dataclass
class LayerContext:
    """What a part sees of the running step."""
    batch: Any                          # engine.batch.StepBatch
    kv: KVBinding | None = None
    state: torch.Tensor | None = None   # [slots, *StateSpec.shape] of this layer, or None
    error_word: torch.Tensor | None = None
    layer_index: int = 0
    call_arg: int = 0                   # the argument of a stage call of the schedule
    side_kv: KVBinding | None = None    # the second cache of a mixer that keeps one (``Mixer.side_cache_spec``)


class ResidualStream:
    """The 32-bit residual sum plus the not-yet-added output of the last part.

    Keeping the last output pending lets a norm fuse the add with itself: one
    pass reads the pending delta and the residual, writes the new residual and
    the normalised rows.
    """

    def __init__(self, residual: torch.Tensor, dtype: torch.dtype) -> None:
        self.residual = residual        # [tokens, hidden] float32
        self.pending: torch.Tensor | None = None
        self.dtype = dtype              # activation dtype of normalised rows
        self.origin: torch.Tensor | None = None    # the embedding output, kept when the model's stages read it
        # [depth, tokens, hidden] fp32 when the model keeps every layer's output (ModelSpec.history_depth): slice 0 is
        # the embedding output, and ``residual`` is one of its slices; a block that averages over the layers so
        # far reads the slices below its own and moves ``residual`` on to the next
        self.history: torch.Tensor | None = None
        # the residual rows in the activation type, left by whoever last changed the residual and had them at
        # hand; whoever changes the residual next drops it
        self.activation_copy: torch.Tensor | None = None
        # [S, tokens, hidden] fp32 when the model carries its residual in S streams (ModelSpec.streams): every stream
        # starts as the embedding output, blocks read them through a weighted sum (:meth:`read_streams`) and write a
        # sublayer's output back through a matrix (:meth:`write_streams`); the model's output is their sum.
        # ``residual`` is then not used.
        self.streams: torch.Tensor | None = None
        self.pending_write: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None     # (y, mix, out weights)
        self._unit_weights: torch.Tensor | None = None

    # ------------------------------------------------------- several streams
    def write_streams(self, y: torch.Tensor, mix: torch.Tensor, out_weights: torch.Tensor) -> None:
        """x_t <- sum_s mix[s, t] x_s + out_weights[t] * y for all streams at once; left pending so that the next read
        does it in its own pass."""
        if self.pending_write is not None:
            self.settle_streams()
        self.pending_write = (y, mix, out_weights)

    def settle_streams(self) -> torch.Tensor:
        if self.pending_write is not None:
            from torchinferno_b200.kernels import ops
            y, mix, out_weights = self.pending_write
            ops.hyper_step(self.streams, y=y, mix=mix, out_weights=out_weights)
            self.pending_write = None
        return self.streams

    def read_streams(self, in_weights: torch.Tensor | None, norm: "Norm", rows: torch.Tensor | None = None) -> torch.Tensor:
        """norm(sum_s in_weights[s] x_s) in the activation type (``in_weights`` None: the plain sum).  A pending write is
        done on the way (with ``rows`` it is only looked through and stays pending).  A norm that needs no statistic of
        the row (``tanh_params``) is computed in the same launch; any other gets the sums in fp32."""
        from torchinferno_b200.kernels import ops
        streams = self.streams
        count, n, width = streams.shape
        if in_weights is None:
            if self._unit_weights is None:
                self._unit_weights = torch.ones(count, dtype=torch.float32, device=streams.device)
            in_weights = self._unit_weights
        y, mix, out_weights = self.pending_write if self.pending_write is not None else (None, None, None)
        n_out = n if rows is None else rows.numel()
        out = torch.empty((n_out, width), dtype=self.dtype, device=streams.device)
        params = getattr(norm, "tanh_params", None)
        if params is not None:
            ops.hyper_step(streams, y=y, mix=mix, out_weights=out_weights, in_weights=in_weights, out=out, rows=rows,
                           tanh_norm=params())
        else:
            sums = torch.empty((n_out, width), dtype=torch.float32, device=streams.device)
            ops.hyper_step(streams, y=y, mix=mix, out_weights=out_weights, in_weights=in_weights, out=sums, rows=rows)
            norm.forward(sums, out)
        if rows is None:
            self.pending_write = None
        return out

    def normed(self, norm: "Norm", rows: torch.Tensor | None = None) -> torch.Tensor:
        if self.streams is not None:
            return self.read_streams(None, norm, rows)
        n = self.residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.residual.shape[1]), dtype=self.dtype, device=self.residual.device)
        if self.pending is None:
            norm.forward(self.residual, out, rows)
        else:
            norm.add_forward(self.pending, self.residual, out, rows)
            if rows is None:
                self.pending = None
        return out

    def add(self, delta: torch.Tensor) -> None:
        if self.pending is not None:
            raise RuntimeError("a delta is already pending; a norm must fold it in first")
        self.pending = delta
        self.activation_copy = None

    def settle(self) -> torch.Tensor:
        """Fold a pending delta into the residual (for a part that reads the residual itself); returns the residual."""
        if self.pending is not None:
            from torchinferno_b200.kernels import ops
            ops.add_pair(self.residual, self.pending)
            self.pending = None
        return self.residual


# --------------------------------------------------------------- interfaces
class Part:
    """Common to all parts: declared weights and their binding."""

    def __init__(self, *, dtype: torch.dtype, device: torch.device) -> None:
        self.dtype = dtype
        self.device = device

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def shared_weight_specs(self) -> list[WeightSpec]:
        """Tensors this part reads that are not its own: named in full (no prefix is put before them), declared
        alike by every part that reads them, loaded once and handed to each in :meth:`bind` under that name."""
        return []

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        """Take the tensors named by :meth:`weight_specs` (already on the device)."""


class Norm(Part):
    def forward(self, residual: torch.Tensor, out: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, delta: torch.Tensor, residual: torch.Tensor, out: torch.Tensor,
                    rows: torch.Tensor | None = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def encode_and_store(self, qkv: torch.Tensor, q_out: torch.Tensor, ctx: LayerContext, heads: int,
                         kv_heads: int, head_dim: int) -> torch.Tensor:
        """Encode positions into q (and k), and write k, v to ``ctx.kv`` if it writes."""
        raise NotImplementedError


class Mixer(Part):
    # ``capturable``: the forward only launches kernels on the current stream and reads the batch through its
    # device arrays, so a decode step that contains it may be captured in a CUDA graph.  Left unset, a mixer
    # without a StateSpec counts as capturable and one with a StateSpec does not (it is taken to walk
    # ``ctx.batch.entries`` on the host); a model with any mixer that is not runs its decode steps uncaptured.
    def cache_spec(self) -> CacheSpec | None:
        return None

    def side_cache_spec(self) -> CacheSpec | None:
        """A second cache beside the one of :meth:`cache_spec` (``ctx.side_kv``), e.g. one entry per run of tokens
        (``CacheSpec.stride``) holding a summary of the run."""
        return None

    def state_spec(self) -> StateSpec | None:
        return None

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, stream: ResidualStream, ctx: LayerContext) -> None:
        raise NotImplementedError

    def named_parts(self) -> list[tuple[str, Part]]:
        """(prefix relative to the block, part) for every part that owns weights."""
        raise NotImplementedError


class StreamStage(Part):
    """Something done to the residual stream once, after the embedding and before the first block: a learned
    absolute position table added to it, a multiplier, a norm.  ``ctx`` carries the batch (positions, slots)."""

    def forward(self, stream: ResidualStream, ctx: LayerContext) -> None:
        raise NotImplementedError


# ----------------------------------------------------------------- registry
_KINDS = ("mixer", "feed_forward", "norm", "position", "block", "stream_stage")
_REGISTRY: dict[str, dict[str, Callable[..., Part]]] = {kind: {} for kind in _KINDS}


def register_part(category: str, kind: str, factory: Callable[..., Part], *, replace: bool = False) -> None:
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r}; one of {_KINDS}")
    if kind in _REGISTRY[category] and not replace and _REGISTRY[category][kind] is not factory:
        raise ValueError(f"{category} kind {kind!r} is already registered")
    _REGISTRY[category][kind] = factory


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY.get(category, {}).pop(kind, None)


def build_part(category: str, spec: PartSpec, *, dtype: torch.dtype, device: torch.device, **extra: Any) -> Part:
    _ensure_builtin()
    table = _REGISTRY[category]
    if spec.kind not in table:
        raise ValueError(f"no {category} of kind {spec.kind!r}; registered: {sorted(table)}")
    return table[spec.kind](**dict(spec.params), **extra, dtype=dtype, device=device)


def registered_parts(category: str) -> tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(_REGISTRY[category]))


_loaded = False


def _ensure_builtin() -> None:
    global _loaded
    if _loaded:
        return
    _loaded = True
    from torchinferno_b200.parts import (attention, biased_attention, block, gated_recurrence, hyper_block,  # noqa: F401
                                         latent_attention, linear_attention, mlp, moe, norm, parallel_block,
                                         pooled_window_attention, rope, sandwich_block, sigmoid_attention, state_space,
                                         stream_stages)
