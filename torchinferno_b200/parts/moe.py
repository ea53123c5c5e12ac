"""Routed feed-forward: every token goes through the ``top`` best of ``experts`` small feed-forwards.

Router logits z = W_router x in fp32; scores = softmax(z) over all experts (or sigmoid(z)); the ``top`` largest
are chosen (lowest index first among equals); their weights are the scores, divided by their sum plus
``norm_eps`` when ``normalize``.  An expert is W_down act(W_up x) with act = relu squared (or silu), no biases;
the output is the weighted sum of the chosen experts' outputs.  An optional shared expert of the same form
runs for every token and is added, multiplied by sigmoid(w_sg . x) when it has a gate row.

``activation="glu_clamp"`` makes an expert a clamped gated unit: g = min(W_gate x, limit), u = clamp(W_up x, -limit,
limit), y = g * sigmoid(alpha g) * (u + 1), output W_down y (``limit`` / ``shared_limit``, ``alpha``); gate and up run
as one product over row pairs (gate i, up i).  ``weight_on_input``: the router weight multiplies the expert's input
instead of its output, sum of expert(w x); it is applied to the 32-bit sums of the first product, ahead of the clamps
(W (w x) = w (W x)), so the input rows are not rounded a second time.

``activation="swiglu"``: an expert is the plain gated unit W_down (silu(W_gate x) * (W_up x)), gate and up again as row
pairs of one product.

``identity`` = n > 0: the router has ``experts`` + n outputs, and the last n stand for experts without tensors whose
output is their input (times the weight).  ``correction``: a tensor of one number per router output that is added to the
scores for the choice only; the weights are made from the scores themselves.  ``groups`` = (count, keep): the router's
outputs (identity ones included) are cut into ``count`` equal runs of adjacent ones, a run is ranked by the best corrected
score in it, and only members of the ``keep`` best runs are eligible.

The pairs (token, choice) are sorted by expert on the device and both products run over the sorted rows
(csrc/moe.cu); no count comes back to the host, so a step with this part may be captured.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.kernels.gemm import LinearWeight, linear
from torchinferno_b200.parts.base import FeedForward, LayerContext, WeightSpec, register_part


class RoutedExperts(FeedForward):
    def __init__(self, *, hidden_size: int, experts: int, top: int, expert_size: int, activation: str = "relu2",
                 scores: str = "softmax", normalize: bool = True, norm_eps: float = 0.0, shared_size: int = 0,
                 shared_gate: bool = False, router_name: str = "router", expert_prefix: str = "e", up_name: str = "up",
                 down_name: str = "down", shared_prefix: str = "shared.", shared_gate_name: str = "sg", gate_name: str = "gate",
                 limit: float = 0.0, shared_limit: float | None = None, alpha: float = 1.702, weight_on_input: bool = False,
                 identity: int = 0, correction: bool = False, correction_name: str = "correction",
                 groups: tuple[int, int] | None = None, dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.identity = int(identity)
        self.routed = experts + self.identity          # outputs of the router
        if experts < 1 or self.identity < 0 or not 1 <= top <= self.routed:
            raise ValueError("top must be between 1 and the number of experts (identity ones included)")
        if activation not in ("relu2", "silu", "glu_clamp", "swiglu") or scores not in ("softmax", "sigmoid"):
            raise ValueError(f"unknown activation {activation!r} or scores {scores!r}")
        self.groups = None if groups is None else (int(groups[0]), int(groups[1]))
        if self.groups is not None:
            count, keep = self.groups
            if count < 1 or not 1 <= keep <= count or self.routed % count or top > keep * (self.routed // count):
                raise ValueError("groups: equal groups, of which at least one and at most all are kept, with room for `top` choices")
        if self.identity and weight_on_input:
            raise ValueError("experts that hand their input through take their weight on the output")
        self.has_correction, self.correction_name = bool(correction), correction_name
        self.correction: torch.Tensor | None = None
        self.hidden_size, self.experts, self.top, self.expert_size = hidden_size, experts, top, expert_size
        self.activation, self.scores, self.normalize, self.norm_eps = activation, scores, bool(normalize), float(norm_eps)
        self.shared_size, self.shared_gate = int(shared_size or 0), bool(shared_gate and shared_size)
        self.names = (router_name, expert_prefix, up_name, down_name, shared_prefix, shared_gate_name)
        self.gate_name, self.glu = gate_name, activation in ("glu_clamp", "swiglu")       # (gate and up as row pairs)
        self.limit, self.alpha, self.weight_on_input = float(limit), float(alpha), bool(weight_on_input)
        self.shared_limit = self.limit if shared_limit is None else float(shared_limit)
        if activation == "glu_clamp" and not self.limit > 0:
            raise ValueError("the clamped gated unit needs a positive limit")

    def _expert(self, e: int, which: str) -> str:
        _, prefix, up, down, _, _ = self.names
        return f"{prefix}{e}.{ {'up': up, 'down': down, 'gate': self.gate_name}[which] }"

    def weight_specs(self) -> list[WeightSpec]:
        router, _, up, down, shared, gate = self.names
        std = self.hidden_size ** -0.5          # (random weights: rows of about unit size from normed input)
        specs = [WeightSpec(router, (self.routed, self.hidden_size), std=2 * std)]
        if self.has_correction:
            specs.append(WeightSpec(self.correction_name, (self.routed,), std=0.05, role="vector"))
        for e in range(self.experts):
            if self.glu:
                specs.append(WeightSpec(self._expert(e, "gate"), (self.expert_size, self.hidden_size), std=std))
            specs += [WeightSpec(self._expert(e, "up"), (self.expert_size, self.hidden_size), std=std),
                      WeightSpec(self._expert(e, "down"), (self.hidden_size, self.expert_size), std=self.expert_size ** -0.5)]
        if self.shared_size:
            if self.glu:
                specs.append(WeightSpec(shared + self.gate_name, (self.shared_size, self.hidden_size), std=std))
            specs += [WeightSpec(shared + up, (self.shared_size, self.hidden_size), std=std),
                      WeightSpec(shared + down, (self.hidden_size, self.shared_size), std=self.shared_size ** -0.5)]
            if self.shared_gate:
                specs.append(WeightSpec(shared + gate, (1, self.hidden_size), std=std))
        return specs

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        router, _, up, down, shared, gate = self.names
        rows = [weights[router]] + ([weights[shared + gate]] if self.shared_gate else [])
        self.router_weight = torch.cat(rows, dim=0).to(torch.float32).contiguous()      # (the router is fp32 in both modes)
        if self.has_correction:
            self.correction = weights[self.correction_name].to(torch.float32).contiguous()
        def first(name_of) -> torch.Tensor:
            """The first product's matrix: up, or (gate i, up i) row pairs for the gated unit."""
            if not self.glu:
                return name_of("up")
            g, u = name_of("gate"), name_of("up")
            return torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1])

        self.up_weight = torch.stack([first(lambda which, e=e: weights[self._expert(e, which)]) for e in range(self.experts)]).contiguous()
        self.down_weight = torch.stack([weights[self._expert(e, "down")] for e in range(self.experts)]).contiguous()
        if self.shared_size:
            self.shared_up_weight = LinearWeight(first(lambda which: weights[shared + {"up": up, "gate": self.gate_name}[which]]),
                                                 few_rows_tcgen05=None)
            self.shared_down_weight = LinearWeight(weights[shared + down], few_rows_tcgen05=None)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        n, dev, top = x.shape[0], x.device, self.top
        logits = torch.empty((n, self.router_weight.shape[0]), dtype=torch.float32, device=dev)
        ops.router_logits(x, self.router_weight, logits)
        ids = torch.empty((n, top), dtype=torch.int32, device=dev)
        weights = torch.empty((n, top), dtype=torch.float32, device=dev)
        count, keep = self.groups if self.groups is not None else (1, 1)
        ops.moe_route(logits, self.routed, top, ids, weights, sigmoid_scores=self.scores == "sigmoid",
                      normalize=self.normalize, norm_eps=self.norm_eps, correction=self.correction, groups=count, keep=keep)
        offsets = torch.empty(self.experts + 1, dtype=torch.int32, device=dev)
        order = torch.empty(n * top, dtype=torch.int32, device=dev)
        place = torch.empty(n * top, dtype=torch.int32, device=dev)
        ops.moe_group(ids, self.experts, offsets, order, place)
        inner = torch.empty((n * top, self.expert_size), dtype=x.dtype, device=dev)
        ops.moe_expert_product(x, self.up_weight, inner, offsets, order, top, x_by_pair=True, act=self.activation,
                               limit=self.limit, alpha=self.alpha, row_scale=weights.view(-1) if self.weight_on_input else None)
        outer = torch.empty((n * top, self.hidden_size), dtype=torch.float32, device=dev)
        ops.moe_expert_product(inner, self.down_weight, outer, offsets, order, top, x_by_pair=False)
        shared_rows = None
        if self.shared_size:
            hidden = linear(x, self.shared_up_weight)
            if self.activation == "relu2":
                ops.relu_squared(hidden, hidden)
            elif self.activation == "glu_clamp":
                hidden = ops.glu_clamp(hidden, torch.empty((n, self.shared_size), dtype=hidden.dtype, device=dev),
                                       self.shared_limit, self.alpha)
            else:
                raise NotImplementedError("a shared expert with silu")
            shared_rows = linear(hidden, self.shared_down_weight)
        out = torch.empty((n, self.hidden_size), dtype=x.dtype, device=dev)
        gate = logits[:, self.routed] if self.shared_gate else None
        # (a choice at or beyond `experts` found no place among the sorted rows: it adds the input itself)
        return ops.moe_combine(outer, place.view(n, top) if self.weight_on_input else place,
                               None if self.weight_on_input else weights, out, shared_rows, gate,
                               ids=ids if self.identity else None, identity_from=self.experts, x=x if self.identity else None)


register_part("feed_forward", "routed_experts", RoutedExperts)
