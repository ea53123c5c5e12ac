"""A model as data: parts by kind, a list of blocks and the order they run in.

``layers`` are the distinct blocks (each owns weights).  ``schedule`` is the
order of execution: a list of :class:`LayerCall` that may name a layer twice
and says which cache layer the call uses; a call with ``writes_cache=False``
reads what an earlier call stored there.  ``cache_layers`` is the number of
distinct cache layers the schedule addresses.  Between layer calls the schedule
may name a stage (:class:`StageCall`): a part of category ``stream_stage`` from
``stages`` that works on the residual stream, with an integer argument (the
number of a pass over a range of layers that runs several times, say).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from torchinferno_b200.parts.base import PartSpec


@dataclass(frozen=True)
class BlockSpec:
    block: PartSpec                 # category "block"; its params hold the PartSpecs of its parts
    prefix: str                     # weight-name prefix of the layer, e.g. "model.layers.3."


@dataclass(frozen=True)
class LayerCall:
    layer: int                      # index into ModelSpec.layers
    cache: int | None = None        # cache layer this call uses (None: the mixer keeps no keys)
    writes_cache: bool = True
    side_cache: int | None = None   # cache layer of the mixer's second cache (``Mixer.side_cache_spec``), which it writes


@dataclass(frozen=True)
class StageCall:
    stage: int                      # index into ModelSpec.stages
    arg: int = 0                    # handed to the stage as ``ctx.call_arg``


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding_name: str             # tensor name of the [vocab, hidden] table
    layers: tuple[BlockSpec, ...]
    schedule: tuple["LayerCall | StageCall", ...]
    final_norm: PartSpec            # prefix holds its full name prefix
    head_name: str | None           # tensor name of the [vocab, hidden] output matrix
    tie_head_to_embedding: bool = False
    after_embedding: PartSpec | None = None   # category "stream_stage"; prefix holds its full name prefix
    config: Mapping[str, Any] = field(default_factory=dict)  # the config.json this came from
    stages: tuple[PartSpec, ...] = ()         # category "stream_stage"; each prefix is a full name prefix
    logit_scale: float = 1.0                  # the head's output is multiplied by this
    keeps_embedding_output: bool = False      # stages read the embedding output (``ResidualStream.origin``)
    embedding_scale: float = 1.0              # the embedding output is multiplied by this
    logit_softcap: float | None = None        # c > 0: logits <- c * tanh(logits / c), after ``logit_scale``
    history_depth: int = 0                    # > 0: the residual stream lives in a [depth, tokens, hidden] tensor whose
                                              # slice 0 keeps the embedding output and whose later slices keep what
                                              # blocks leave there (``ResidualStream.history``); the stream starts in slice 1
    streams: int = 0                          # > 0: the residual is carried in this many streams [streams, tokens, hidden]
                                              # (``ResidualStream.streams``), each the embedding output at the start; blocks
                                              # of kind ``hyper_connection`` read and write them; the output is their sum

    def __post_init__(self) -> None:
        if self.streams and self.history_depth:
            raise ValueError("a residual in several streams and a history of layer outputs do not go together")
        for call in self.schedule:
            if isinstance(call, StageCall):
                if not 0 <= call.stage < len(self.stages):
                    raise ValueError(f"schedule names stage {call.stage}, but there are {len(self.stages)}")
            elif not 0 <= call.layer < len(self.layers):
                raise ValueError(f"schedule names layer {call.layer}, but there are {len(self.layers)}")
        written: set[int] = set()
        for call in self.schedule:
            if isinstance(call, LayerCall) and call.side_cache is not None:
                if call.side_cache in written or call.side_cache == call.cache:
                    raise ValueError(f"cache layer {call.side_cache} is written by two layer calls")
                written.add(call.side_cache)
            if isinstance(call, StageCall) or call.cache is None:
                continue
            if call.writes_cache:
                if call.cache in written:
                    raise ValueError(f"cache layer {call.cache} is written by two layer calls")
                written.add(call.cache)
            elif call.cache not in written:
                raise ValueError(f"cache layer {call.cache} is read before any call writes it")

    @property
    def cache_layers(self) -> int:
        calls = [call for call in self.schedule if isinstance(call, LayerCall)]
        ids = [c for call in calls for c in (call.cache, call.side_cache) if c is not None]
        return max(ids) + 1 if ids else 0
