"""The runnable model: parts built from a :class:`ModelSpec`, weights bound by name.

One forward pass serves every kind of step: it embeds the tokens of a ragged
batch, runs the schedule of layer calls against the cache, norms only the rows
whose logits are wanted and projects them to the vocabulary
(src/torchinferno/models/llama3/tensor_parallel.py:7088-7090 gathers before the
head likewise).  Logits are fp32.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import gemm, ops
from torchinferno_b200.kernels.gemm import linear
from torchinferno_b200.models.spec import ModelSpec, StageCall
from torchinferno_b200.parts.base import (Block, CacheSpec, KVBinding, LayerContext, ResidualStream,
                                          StateSpec, WeightSpec, build_part)


class CausalLM:
    def __init__(self, spec: ModelSpec, *, dtype: torch.dtype, device: torch.device | str) -> None:
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.blocks: list[Block] = [
            build_part("block", layer.block, dtype=dtype, device=self.device) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, dtype=dtype, device=self.device)
        self.after_embedding = None if spec.after_embedding is None else \
            build_part("stream_stage", spec.after_embedding, dtype=dtype, device=self.device)
        self.stages = [build_part("stream_stage", stage, dtype=dtype, device=self.device) for stage in spec.stages]
        self.embedding: torch.Tensor | None = None
        self.head: torch.Tensor | None = None

    def _owned_parts(self):
        """(full name prefix, part) of every part that owns weights, blocks first."""
        spec = self.spec
        for layer, block in zip(spec.layers, self.blocks):
            for prefix, part in block.named_parts():
                yield layer.prefix + prefix, part
        yield spec.final_norm.prefix, self.final_norm
        if self.after_embedding is not None:
            yield spec.after_embedding.prefix, self.after_embedding
        for stage_spec, stage in zip(spec.stages, self.stages):
            yield stage_spec.prefix, stage

    # ------------------------------------------------------------ weights
    def expected_tensors(self) -> dict[str, WeightSpec]:
        """Every tensor the model reads, by full checkpoint name."""
        spec = self.spec
        expected: dict[str, WeightSpec] = {
            spec.embedding_name: WeightSpec(spec.embedding_name, (spec.vocab_size, spec.hidden_size))}
        for prefix, part in self._owned_parts():
            for ws in part.weight_specs():
                name = prefix + ws.name
                expected[name] = WeightSpec(name, ws.shape, ws.init, ws.std, ws.role, ws.optional, ws.free_dims)
            for ws in part.shared_weight_specs():
                if ws.name in expected and tuple(expected[ws.name].shape) != tuple(ws.shape):
                    raise ValueError(f"{ws.name}: parts that share it declare shapes {expected[ws.name].shape} and {ws.shape}")
                expected[ws.name] = ws
        if spec.head_name is not None:
            expected[spec.head_name] = WeightSpec(
                spec.head_name, (spec.vocab_size, spec.hidden_size), optional=spec.tie_head_to_embedding)
        return expected

    def unused_optional_tensors(self) -> list[str]:
        """Optional tensors that are not read even when the file has them (a head tied to the embedding)."""
        spec = self.spec
        return [spec.head_name] if spec.tie_head_to_embedding and spec.head_name is not None else []

    def bind(self, tensors: Mapping[str, torch.Tensor], consume: bool = False) -> None:
        """Give every part its tensors.  ``consume``: ``tensors`` is a dict of the caller's that is emptied part
        by part, so that a part which repacks its weights (fused projections) does not leave the sources alive
        beside the packed copy until the whole model is bound."""
        spec = self.spec
        take = tensors.pop if consume else tensors.__getitem__
        self.embedding = take(spec.embedding_name)
        if spec.tie_head_to_embedding or spec.head_name is None:
            self.head = self.embedding
        elif spec.head_name in tensors:
            self.head = take(spec.head_name)
        else:
            # An untied model whose file has no head is refused on purpose: guessing that the embedding
            # doubles as the head would turn a truncated checkpoint into silently wrong logits.
            raise KeyError(f"{spec.head_name}: the model does not tie its head to the embedding, and no head was given")
        shared_names = {ws.name for _, part in self._owned_parts() for ws in part.shared_weight_specs()}
        shared = {name: take(name) for name in shared_names if name in tensors}
        for full, part in self._owned_parts():
            own = {ws.name: take(full + ws.name) for ws in part.weight_specs() if full + ws.name in tensors}
            own.update({ws.name: shared[ws.name] for ws in part.shared_weight_specs() if ws.name in shared})
            part.bind(own)
        if self.device.type == "cuda":
            gemm.tune_few_rows()      # weights that left the choice of their few-rows kernel open get it now

    def weight_bytes(self) -> int:
        """Bytes of distinct weight storage one step reads (a tied head counts once)."""
        seen: dict[int, int] = {}

        def note(t: torch.Tensor | None) -> None:
            if isinstance(t, torch.Tensor):
                seen[t.data_ptr()] = t.numel() * t.element_size()

        note(self.head)
        for _, part in self._owned_parts():
            for key, value in vars(part).items():
                if key.endswith("weight"):
                    note(getattr(value, "tensor", value) if not isinstance(value, torch.Tensor) else value)
        return sum(seen.values())

    # -------------------------------------------------------------- needs
    def cache_requirements(self) -> list[CacheSpec]:
        """CacheSpec of every cache layer, in cache-layer order."""
        needs: dict[int, CacheSpec] = {}
        for call in self.spec.schedule:
            if isinstance(call, StageCall) or call.cache is None:
                continue
            cs = self.blocks[call.layer].mixer.cache_spec()
            if cs is None:
                raise ValueError(f"layer {call.layer} is given cache layer {call.cache} but its mixer keeps no keys")
            if call.cache in needs and needs[call.cache] != cs:
                raise ValueError(f"cache layer {call.cache} is shared by mixers of different shapes")
            needs.setdefault(call.cache, cs)
        for call in self.spec.schedule:
            if isinstance(call, StageCall):
                continue
            side = self.blocks[call.layer].mixer.side_cache_spec()
            if (side is None) != (call.side_cache is None):
                raise ValueError(f"layer {call.layer}: the mixer's second cache and the schedule's side_cache do not agree")
            if side is not None:
                needs[call.side_cache] = side
        missing = [i for i in range(self.spec.cache_layers) if i not in needs]
        if missing:
            raise ValueError(f"cache layers {missing} are used by no layer call")
        return [needs[i] for i in range(self.spec.cache_layers)]

    def capturable(self) -> bool:
        """Whether a decode step of this model may be captured in a CUDA graph (see ``Mixer.capturable``)."""
        parts = [block.mixer for block in self.blocks] + ([self.after_embedding] if self.after_embedding is not None else []) \
            + list(self.stages)
        return all(getattr(part, "capturable", getattr(part, "state_spec", lambda: None)() is None) for part in parts)

    def state_requirements(self) -> list[StateSpec | None]:
        """StateSpec of every layer call of the schedule (None where the mixer has none)."""
        return [None if isinstance(call, StageCall) else self.blocks[call.layer].mixer.state_spec()
                for call in self.spec.schedule]

    # ------------------------------------------------------------ forward
    def forward(self, batch, cache) -> torch.Tensor:
        """Run the tokens of ``batch``; return fp32 logits [len(batch.logit_rows), vocab]."""
        n = batch.n_tokens
        depth = self.spec.history_depth
        history = None
        if depth:
            if depth < 2:
                raise ValueError("history_depth counts the embedding output and at least one slice to work in")
            history = torch.empty((depth, n, self.spec.hidden_size), dtype=torch.float32, device=self.device)
            residual = history[0]
        else:
            residual = torch.empty((n, self.spec.hidden_size), dtype=torch.float32, device=self.device)
        ops.embedding(batch.token_ids, self.embedding, residual)
        if self.spec.embedding_scale != 1.0:
            ops.scale_(residual, self.spec.embedding_scale)
        if depth:
            history[1].copy_(residual)
            residual = history[1]
        stream = ResidualStream(residual, self.dtype)
        stream.history = history
        if self.spec.streams:
            stream.streams = residual.unsqueeze(0).repeat(self.spec.streams, 1, 1)      # every stream starts as the embedding output
        if self.spec.keeps_embedding_output:
            stream.origin = residual.clone()
        if self.after_embedding is not None:
            self.after_embedding.forward(stream, LayerContext(batch=batch, error_word=cache.error_word, layer_index=-1))
        for index, call in enumerate(self.spec.schedule):
            if isinstance(call, StageCall):
                self.stages[call.stage].forward(stream, LayerContext(batch=batch, error_word=cache.error_word,
                                                                     layer_index=index, call_arg=call.arg))
                continue
            kv = None
            if call.cache is not None:
                kv = cache.kv_binding(call.cache)
                kv = KVBinding(kv.pool, kv.block_table, kv.page_size, kv.window, call.writes_cache, kv.keys, kv.values)
            side = None
            if call.side_cache is not None:
                b = cache.kv_binding(call.side_cache)
                side = KVBinding(b.pool, b.block_table, b.page_size, b.window, True, b.keys, b.values)
            ctx = LayerContext(batch=batch, kv=kv, state=cache.state(index),
                               error_word=cache.error_word, layer_index=index, side_kv=side)
            self.blocks[call.layer].forward(stream, ctx)
        if batch.n_logits == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        rows = stream.normed(self.final_norm, batch.logit_rows)
        logits = linear(rows, self.head, out_dtype=torch.float32)
        if self.spec.logit_scale != 1.0:
            ops.scale_(logits, self.spec.logit_scale)
        if self.spec.logit_softcap:
            ops.softcap_(logits, self.spec.logit_softcap)
        return logits
