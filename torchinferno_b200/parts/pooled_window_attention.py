"""Attention over a sliding window plus pooled blocks, over two paged caches.

q = W_q x, k = W_k x, v = W_v x (with biases when ``bias``); q and k get the position encoding (``position``: a rotary
part, possibly on part of a head and under a frequency law with an amplitude); with ``value_rotation_base`` a value is
turned over its whole width by its own position (pair m with m + value_dim / 2, angle = position * base^(-2m / value_dim))
and cached so.  A query at position i sees the tokens j with 0 <= i - j < ``window`` and, with ``pool`` = P, one key and
one value for every block of P positions that lies wholly behind the window (b * P + P - 1 <= i - window): the means of
the block's keys and values as the cache holds them.  Tokens that have left the window and whose block is not yet
complete behind it are not seen.  score = q . k * ``scale`` (times a learned ``temp`` per head); tokens and blocks share
one softmax, whose denominator also holds exp(``sink``), a learned number per head without key or value.  The head's
sum is turned back by the query's own position (so that what it holds depends on distances only), multiplied element by
element by sigmoid(W_g x) (``gate``), and projected by W_o.  Query head h reads key/value head h // (heads / kv_heads).

The tokens' keys and values live in the mixer's cache (``cache_spec``, with a window: pages wholly behind it and behind
the running block go back to the pool), the blocks' means in its second cache (``side_cache_spec``: one entry per P
tokens), written when the last token of a block arrives.  All input projections are one product; the kernels are in
csrc/pooled_window_attention.cu.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.kernels.gemm import LinearWeight, linear
from torchinferno_b200.parts.base import (CacheSpec, LayerContext, Mixer, PartSpec, WeightSpec, build_part,
                                          register_part)


class PooledWindowAttention(Mixer):
    capturable = True

    def __init__(self, *, hidden_size: int, heads: int, kv_heads: int, dim: int, value_dim: int, scale: float,
                 position: PartSpec | Mapping, window: int, pool: int | None = None,
                 value_rotation_base: float | None = None, bias: bool = False, sink: bool = False, temperature: bool = False,
                 gate: bool = False, q_name: str = "q", k_name: str = "k", v_name: str = "v", o_name: str = "o",
                 gate_name: str = "g", sink_name: str = "sink", temp_name: str = "temp", bias_suffix: str = ".b",
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if window < 1 or (pool is not None and pool < 1):
            raise ValueError("window and pool are positive")
        if value_rotation_base is not None and value_dim % 2:
            raise ValueError("rotated values need an even width")
        self.hidden_size, self.heads, self.kv_heads, self.dim, self.value_dim = hidden_size, heads, kv_heads, dim, value_dim
        self.scale, self.window, self.pool = float(scale), int(window), (int(pool) if pool else 0)
        self.has_bias, self.has_sink, self.has_temp, self.has_gate = bool(bias), bool(sink), bool(temperature), bool(gate)
        self.names = {"q": q_name, "k": k_name, "v": v_name, "o": o_name, "g": gate_name, "sink": sink_name, "temp": temp_name}
        self.bias_suffix = bias_suffix
        if not isinstance(position, PartSpec):
            position = PartSpec(**position)
        self.position = build_part("position", position, dtype=dtype, device=device)
        self.value_freq: torch.Tensor | None = None
        if value_rotation_base is not None:
            m = torch.arange(value_dim // 2, dtype=torch.float64)
            self.value_freq = (torch.tensor(float(value_rotation_base), dtype=torch.float64) ** (-2.0 * m / value_dim)) \
                .to(torch.float32).to(device)
        qw, kw, vw = heads * dim, kv_heads * dim, kv_heads * value_dim
        self.k_off, self.v_off, self.g_off = qw, qw + kw, qw + kw + vw
        self.in_weight: LinearWeight | None = None
        self.o_weight: LinearWeight | None = None
        self.q_bias = self.k_bias = self.v_bias = self.sink = self.temp = None

    def weight_specs(self) -> list[WeightSpec]:
        n, w, b = self.names, self.hidden_size, self.bias_suffix
        std = w ** -0.5                     # (random weights: rows of about unit size from normed input)
        widths = {"q": self.heads * self.dim, "k": self.kv_heads * self.dim, "v": self.kv_heads * self.value_dim}
        specs = []
        for key in ("q", "k", "v"):
            specs.append(WeightSpec(n[key], (widths[key], w), std=std))
            if self.has_bias:
                specs.append(WeightSpec(n[key] + b, (widths[key],), std=0.5, role="vector"))
        if self.has_temp:
            specs.append(WeightSpec(n["temp"], (self.heads,), init="about_one", std=0.2, role="vector"))
        if self.has_sink:
            specs.append(WeightSpec(n["sink"], (self.heads,), std=1.0, role="vector"))
        if self.has_gate:
            specs.append(WeightSpec(n["g"], (self.heads * self.value_dim, w), std=std))
        specs.append(WeightSpec(n["o"], (w, self.heads * self.value_dim), std=(self.heads * self.value_dim) ** -0.5))
        return specs

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n, b = self.names, self.bias_suffix
        rows = [weights[n["q"]], weights[n["k"]], weights[n["v"]]] + ([weights[n["g"]]] if self.has_gate else [])
        total = sum(r.shape[0] for r in rows)
        if total % 8:       # (rows of the product's output then start on 16-byte boundaries in bfloat16)
            rows.append(torch.zeros((8 - total % 8, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.in_weight = LinearWeight(torch.cat(rows, dim=0), few_rows_tcgen05=None)
        self.o_weight = LinearWeight(weights[n["o"]], few_rows_tcgen05=None)

        def vector(name):
            return weights[name].to(torch.float32).contiguous()

        if self.has_bias:
            self.q_bias, self.k_bias, self.v_bias = vector(n["q"] + b), vector(n["k"] + b), vector(n["v"] + b)
        self.sink = vector(n["sink"]) if self.has_sink else None
        self.temp = vector(n["temp"]) if self.has_temp else None

    def cache_spec(self) -> CacheSpec:
        # a later query reads the last `window` tokens; the block that is still filling needs all of its own
        keep = max(self.window, self.pool)
        return CacheSpec(self.kv_heads, self.dim, keep, None if self.value_dim == self.dim else self.value_dim)

    def side_cache_spec(self) -> CacheSpec | None:
        if not self.pool:
            return None
        return CacheSpec(self.kv_heads, self.dim, None, None if self.value_dim == self.dim else self.value_dim, stride=self.pool)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        kv, side, batch = ctx.kv, ctx.side_kv, ctx.batch
        if kv is None or kv.keys is None or kv.values is None or not kv.writes:
            raise RuntimeError("this attention needs a cache binding with keys and values that it writes")
        if self.pool and (side is None or side.keys is None or side.values is None):
            raise RuntimeError("pooled blocks need the second cache")
        n, h, g = x.shape[0], self.heads, self.kv_heads
        proj = linear(x, self.in_weight)
        q = torch.empty((n, h * self.dim), dtype=x.dtype, device=x.device)
        freq, rot_dim, interleaved = self.position.rotary_table()
        if interleaved:
            raise RuntimeError("this attention's kernels pair element i with i + rot_dim / 2")
        ops.rotary_kv_append(proj, 0, self.k_off, self.v_off, q, kv.keys, kv.values, batch.positions, batch.token_slot,
                             kv.block_table, freq, self.value_freq, h, g, self.dim, self.value_dim, rot_dim=rot_dim,
                             amplitude=getattr(self.position, "amplitude", 1.0), q_bias=self.q_bias, k_bias=self.k_bias,
                             v_bias=self.v_bias, error_word=ctx.error_word)
        if self.pool:
            ops.pool_blocks(kv.keys, kv.values, kv.block_table, side.keys, side.values, side.block_table, batch.positions,
                            batch.token_slot, self.pool, error_word=ctx.error_word)
        out = torch.empty((n, h * self.value_dim), dtype=x.dtype, device=x.device)
        ops.pooled_window_attention(
            q, out, batch.q_start, batch.kv_start, batch.slots, kv.keys, kv.values, kv.block_table,
            side.keys if self.pool else None, side.values if self.pool else None, side.block_table if self.pool else None,
            batch.n_entries, batch.max_q_len, h, g, window=self.window, pool=self.pool, scale=self.scale, temp=self.temp,
            sink=self.sink, value_freq=self.value_freq,
            gate=proj[:, self.g_off:self.g_off + h * self.value_dim] if self.has_gate else None, error_word=ctx.error_word)
        return linear(out, self.o_weight)


register_part("mixer", "pooled_window_attention", PooledWindowAttention)
