"""A pre-norm block over a residual that is carried in several streams (hyper-connections).

Instead of one residual x there are S copies x_1 .. x_S, all equal to the embedding output at the start.  Sublayer q
(the mixer, then the feed-forward when there is one) has three tensors of its own: ``in`` [S], ``out`` [S] and ``mix``
[S, S], indexed [from, to]:

    u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] * y      (all t from the old x)

The model's output is the sum of the streams (``ModelSpec.streams``; the final norm reads it).  With S = 1, in = out = 1
and mix = [[1]] this is the ordinary pre-norm block.

The write is left pending on the stream and done by the launch that makes the next read, whoever asks for it: the
second sublayer, the next block or the final norm (csrc/hyper_streams.cu).  Sums and coefficients are fp32.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.parts.base import (Block, LayerContext, Part, PartSpec, ResidualStream, WeightSpec, build_part,
                                          register_part)


def _spec(value: PartSpec | Mapping | None) -> PartSpec | None:
    return value if value is None or isinstance(value, PartSpec) else PartSpec(**value)


class HyperConnectionBlock(Block):
    def __init__(self, *, streams: int, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: PartSpec | None = None,
                 feed_forward_norm: PartSpec | None = None, mixer_prefix: str = "hc1.", feed_forward_prefix: str = "hc2.",
                 in_name: str = "in", out_name: str = "out", mix_name: str = "mix", dtype: torch.dtype,
                 device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        if streams < 1:
            raise ValueError("a residual has at least one stream")
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.streams = int(streams)
        self.specs = {"mixer": _spec(mixer), "feed_forward": _spec(feed_forward), "mixer_norm": _spec(mixer_norm),
                      "feed_forward_norm": _spec(feed_forward_norm)}
        self.mixer = build_part("mixer", self.specs["mixer"], dtype=dtype, device=device)
        self.mixer_norm = build_part("norm", self.specs["mixer_norm"], dtype=dtype, device=device)
        self.feed_forward = None if feed_forward is None else \
            build_part("feed_forward", self.specs["feed_forward"], dtype=dtype, device=device)
        self.feed_forward_norm = None if feed_forward is None else \
            build_part("norm", self.specs["feed_forward_norm"], dtype=dtype, device=device)
        self.prefixes = (mixer_prefix, feed_forward_prefix)
        self.names = (in_name, out_name, mix_name)
        self.coefficients: list[tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = []

    def _sublayers(self) -> tuple[str, ...]:
        return self.prefixes if self.feed_forward is not None else self.prefixes[:1]

    # (the block owns the coefficients of its connections itself)
    def weight_specs(self) -> list[WeightSpec]:
        s, (into, out, mix) = self.streams, self.names
        specs = []
        for prefix in self._sublayers():
            specs += [WeightSpec(prefix + into, (s,), init="about_one", std=0.3, role="vector"),
                      WeightSpec(prefix + out, (s,), init="about_one", std=0.3, role="vector"),
                      WeightSpec(prefix + mix, (s, s), init="about_identity", std=0.2, role="vector")]
        return specs

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        into, out, mix = self.names

        def f32(name: str) -> torch.Tensor:
            return weights[name].to(torch.float32).contiguous()

        self.coefficients = [(f32(p + into), f32(p + out), f32(p + mix)) for p in self._sublayers()]

    def named_parts(self) -> list[tuple[str, Part]]:
        parts: list[tuple[str, Part]] = [(self.specs["mixer_norm"].prefix, self.mixer_norm),
                                         (self.specs["mixer"].prefix, self.mixer)]
        if self.feed_forward is not None:
            parts += [(self.specs["feed_forward_norm"].prefix, self.feed_forward_norm),
                      (self.specs["feed_forward"].prefix, self.feed_forward)]
        parts.append(("", self))
        return parts

    def forward(self, stream: ResidualStream, ctx: LayerContext) -> None:
        if stream.streams is None or stream.streams.shape[0] != self.streams:
            raise RuntimeError(f"this block works on a residual in {self.streams} streams (ModelSpec.streams)")
        into, out, mix = self.coefficients[0]
        stream.write_streams(self.mixer.forward(stream.read_streams(into, self.mixer_norm), ctx), mix, out)
        if self.feed_forward is not None:
            into, out, mix = self.coefficients[1]
            stream.write_streams(self.feed_forward.forward(stream.read_streams(into, self.feed_forward_norm), ctx), mix, out)


register_part("block", "hyper_connection", HyperConnectionBlock)
