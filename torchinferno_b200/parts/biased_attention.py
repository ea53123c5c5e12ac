"""Grouped softmax attention without rotation: positions enter through a learned bias per head and distance and
through a query temperature.

q = W_q x, k = W_k x, v = W_v x (no biases); every q and k head is divided by its root mean square (``qk_norm_eps``)
and multiplied by a weight of ``dim`` numbers that all heads share (``q.norm`` / ``k.norm``, multiplied in as stored: no 1 is added);
with ``temp_every`` = E > 0 the query at position p is also multiplied by 1 + ``temp_coef`` * ln(floor((p + 1) / E) + 1);
score(i, j) = q_i . k_j * ``scale`` + rel[bucket(i - j), h], where ``rel`` is the layer's table of B rows (one number per
head in each; the checkpoint's tensor says how many, ``buckets`` is what random weights get) and, with ``bias_max`` = D
and half = B / 2,

    bucket(n) = n                                                            for n < half
              = min(B - 1, half + floor(ln(n / half) / ln(D / half) * (B - half)))   otherwise

(small distances have a row each, larger ones share rows on a logarithmic scale, everything from D on the last row);
the bias is added after the scaling.  Causal softmax (optionally inside a ``window``); query head h reads key/value
head h // (heads / kv_heads); keys may be wider or narrower than values; then the output projection.

When the model is bound the table is laid out by distance, [heads, D + 1] (distances from D on read the last entry),
so the kernels index it with min(i - j, D) and never take a logarithm.  All input projections are one product;
``qk_norm_append`` (csrc/sigmoid_attention.cu) norms, weighs, heats and stores; the attention itself is the kernel of
the windowed attention (csrc/pooled_window_attention.cu) with the table added to its scores.
"""
from __future__ import annotations

import math
from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.kernels.gemm import LinearWeight, linear
from torchinferno_b200.parts.base import CacheSpec, LayerContext, Mixer, WeightSpec, register_part

NO_WINDOW = 1 << 30        # what the kernel is told when every earlier token is visible


def distance_buckets(buckets: int, far: int) -> list[int]:
    """bucket(n) for n = 0 .. max(far, half): the row of the bias table that distance n reads (later distances read the last)."""
    half = buckets // 2
    table = []
    for n in range(max(far, half) + 1):
        if n < half:
            table.append(n)
        else:
            table.append(min(buckets - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (buckets - half)))))
    return table


class BiasedAttention(Mixer):
    capturable = True

    def __init__(self, *, hidden_size: int, heads: int, kv_heads: int, dim: int, value_dim: int, scale: float, buckets: int,
                 bias_max: int, qk_norm_eps: float | None = None, temp_coef: float = 0.0, temp_every: int = 0,
                 window: int | None = None, q_name: str = "q", k_name: str = "k", v_name: str = "v", o_name: str = "o",
                 rel_name: str = "rel", q_norm_name: str = "q.norm", k_norm_name: str = "k.norm",
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if buckets < 2 or bias_max <= buckets // 2:
            raise ValueError("the bias table needs at least two rows, and bias_max must lie beyond the first half of them")
        if temp_every < 0 or (window is not None and window < 1):
            raise ValueError("temp_every is not negative, and a window is positive when given")
        self.hidden_size, self.heads, self.kv_heads, self.dim, self.value_dim = hidden_size, heads, kv_heads, dim, value_dim
        self.scale, self.buckets, self.bias_max, self.qk_norm_eps = float(scale), int(buckets), int(bias_max), qk_norm_eps
        self.temp_coef, self.temp_every, self.window = float(temp_coef), int(temp_every), window
        self.names = {"q": q_name, "k": k_name, "v": v_name, "o": o_name, "rel": rel_name, "qn": q_norm_name, "kn": k_norm_name}
        qw, kw = heads * dim, kv_heads * dim
        self.k_off, self.v_off = qw, qw + kw
        self.in_weight: LinearWeight | None = None
        self.o_weight: LinearWeight | None = None
        self.q_norm_weight = self.k_norm_weight = self.bias_by_distance = None

    def weight_specs(self) -> list[WeightSpec]:
        n, w = self.names, self.hidden_size
        std = w ** -0.5                     # (random weights: rows of about unit size from normed input)
        specs = [WeightSpec(n["q"], (self.heads * self.dim, w), std=std),
                 WeightSpec(n["k"], (self.kv_heads * self.dim, w), std=std),
                 WeightSpec(n["v"], (self.kv_heads * self.value_dim, w), std=std)]
        if self.qk_norm_eps is not None:
            specs += [WeightSpec(n["qn"], (self.dim,), init="about_one", std=0.1, role="vector"),
                      WeightSpec(n["kn"], (self.dim,), init="about_one", std=0.1, role="vector")]
        # (how many rows the table has is the file's to say)
        specs += [WeightSpec(n["rel"], (self.buckets, self.heads), std=1.0, role="vector", free_dims=(0,)),
                  WeightSpec(n["o"], (w, self.heads * self.value_dim), std=(self.heads * self.value_dim) ** -0.5)]
        return specs

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        rows = [weights[n["q"]], weights[n["k"]], weights[n["v"]]]
        total = sum(r.shape[0] for r in rows)
        if total % 8:       # (rows of the product's output then start on 16-byte boundaries in bfloat16)
            rows.append(torch.zeros((8 - total % 8, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.in_weight = LinearWeight(torch.cat(rows, dim=0), few_rows_tcgen05=None)
        self.o_weight = LinearWeight(weights[n["o"]], few_rows_tcgen05=None)
        if self.qk_norm_eps is not None:
            self.q_norm_weight = weights[n["qn"]].to(torch.float32).contiguous()
            self.k_norm_weight = weights[n["kn"]].to(torch.float32).contiguous()
        rel = weights[n["rel"]].to(torch.float32)                                       # [buckets, heads]
        self.buckets = int(rel.shape[0])
        if self.buckets < 2 or self.bias_max <= self.buckets // 2:
            raise ValueError(f"a bias table of {self.buckets} rows does not go with bias_max = {self.bias_max}")
        index = torch.tensor(distance_buckets(self.buckets, self.bias_max), dtype=torch.long, device=rel.device)
        self.bias_by_distance = rel.index_select(0, index).t().contiguous()             # [heads, distances]

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.kv_heads, self.dim, self.window, None if self.value_dim == self.dim else self.value_dim)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        kv, batch = ctx.kv, ctx.batch
        if kv is None or kv.keys is None or kv.values is None or not kv.writes:
            raise RuntimeError("this attention needs a cache binding with keys and values that it writes")
        n, h, g = x.shape[0], self.heads, self.kv_heads
        proj = linear(x, self.in_weight)
        q = torch.empty((n, h * self.dim), dtype=x.dtype, device=x.device)
        ops.qk_norm_append(proj, 0, self.k_off, self.v_off, q, kv.keys, kv.values, batch.positions, batch.token_slot,
                           kv.block_table, None, h, g, self.dim, self.value_dim, rot_dim=0,
                           eps=-1.0 if self.qk_norm_eps is None else self.qk_norm_eps, error_word=ctx.error_word,
                           q_weight=self.q_norm_weight, k_weight=self.k_norm_weight, temp_coef=self.temp_coef,
                           temp_every=self.temp_every)
        out = torch.empty((n, h * self.value_dim), dtype=x.dtype, device=x.device)
        ops.pooled_window_attention(q, out, batch.q_start, batch.kv_start, batch.slots, kv.keys, kv.values, kv.block_table,
                                    None, None, None, batch.n_entries, batch.max_q_len, h, g,
                                    window=self.window or NO_WINDOW, pool=0, scale=self.scale,
                                    rel_bias=self.bias_by_distance, error_word=ctx.error_word, max_kv_len=batch.max_kv_len)
        return linear(out, self.o_weight)


register_part("mixer", "biased_attention", BiasedAttention)
