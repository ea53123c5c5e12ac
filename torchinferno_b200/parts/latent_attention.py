"""Attention whose keys and values come from one low-rank latent per token.

From the layer input x: q = W_q x, laid out head by head as [``dim`` unrotated ; ``rot_dim`` rotated]; W_dkv x has
``kv_rank + rot_dim`` rows, the first kv_rank RMS-normed (plain weight) are the latent c, the last rot_dim, rotated,
are a key part r that all heads share.  Head j's key is [W_uk_j c ; r] and its value W_uv_j c; causal softmax with
the given scale; the heads' outputs are optionally multiplied by sigmoid(W_g x), element by element (``gate=True``) or
with one gate per head (``gate="head"``, W_g has ``heads`` rows), then projected by W_o.  With ``q_rank`` the queries are
made in two steps: the rows W_dq x of that width, RMS-normed and multiplied by a weight, then W_uq on the result.

Only c and r are cached (one row of kv_rank + rot_dim elements per token: a cache group with one key head and no
values).  The queries are folded through W_uk (a_j = W_uk_j^T q_j, one batched product), attention runs over the
latent rows with their first kv_rank elements as values, and W_uv is applied to the result (another batched
product): the same arithmetic regrouped, in which no per-head key or value is ever made.  Scores, softmax
weights, their sums and the folded queries are fp32.  Rotary pairs are (2i, 2i + 1) (``pairing="interleaved"``) or
(i, i + rot_dims / 2) (``pairing="half"``) over the first ``rot_dims`` elements of the rotated part, angle = position *
rot_base^(-2i / rot_dims).
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.kernels.gemm import LinearWeight, linear
from torchinferno_b200.parts.base import CacheSpec, LayerContext, Mixer, WeightSpec, register_part


class LatentAttention(Mixer):
    def __init__(self, *, hidden_size: int, heads: int, dim: int, rot_dim: int, value_dim: int, kv_rank: int, scale: float,
                 rot_base: float, rot_dims: int | None = None, eps: float = 1e-6, gate: bool | str = True,
                 q_rank: int | None = None, pairing: str = "interleaved",
                 q_name: str = "q", dkv_name: str = "dkv", latent_norm_name: str = "dkv.norm", uk_name: str = "uk",
                 uv_name: str = "uv", g_name: str = "g", o_name: str = "o", dq_name: str = "dq", q_norm_name: str = "dq.norm",
                 uq_name: str = "uq", dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        if gate not in (True, False, "element", "head") or pairing not in ("interleaved", "half"):
            raise ValueError(f"unknown gate {gate!r} or pairing {pairing!r}")
        self.hidden_size, self.heads, self.dim, self.rot_dim = hidden_size, heads, dim, rot_dim
        self.value_dim, self.kv_rank, self.scale, self.eps, self.gate = value_dim, kv_rank, float(scale), float(eps), bool(gate)
        self.gate_per_head = gate == "head"
        self.q_rank, self.half_pairs = (int(q_rank) if q_rank else 0), pairing == "half"
        self.rot_dims = rot_dim if rot_dims is None else int(rot_dims)
        if self.rot_dims % 2 or self.rot_dims > rot_dim:
            raise ValueError("rot_dims must be even and at most rot_dim")
        i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
        self.inv_freq = (torch.tensor(float(rot_base), dtype=torch.float64) ** (-2.0 * i / max(self.rot_dims, 1))) \
            .to(torch.float32).to(device)
        self.names = {"q": q_name, "dkv": dkv_name, "norm": latent_norm_name, "uk": uk_name, "uv": uv_name, "g": g_name,
                      "o": o_name, "dq": dq_name, "q_norm": q_norm_name, "uq": uq_name}
        self.in_weight: LinearWeight | None = None
        self.uq_weight: LinearWeight | None = None
        self.o_weight: LinearWeight | None = None

    def weight_specs(self) -> list[WeightSpec]:
        n, h, w = self.names, self.heads, self.hidden_size
        std, rank_std = w ** -0.5, self.kv_rank ** -0.5      # (random weights: rows of about unit size)
        if self.q_rank:
            specs = [WeightSpec(n["dq"], (self.q_rank, w), std=std),
                     WeightSpec(n["q_norm"], (self.q_rank,), init="about_one", std=0.1, role="vector"),
                     WeightSpec(n["uq"], (h * (self.dim + self.rot_dim), self.q_rank), std=self.q_rank ** -0.5)]
        else:
            specs = [WeightSpec(n["q"], (h * (self.dim + self.rot_dim), w), std=std)]
        specs += [WeightSpec(n["dkv"], (self.kv_rank + self.rot_dim, w), std=std),
                 WeightSpec(n["norm"], (self.kv_rank,), init="ones", role="vector"),
                 WeightSpec(n["uk"], (h * self.dim, self.kv_rank), std=rank_std),
                 WeightSpec(n["uv"], (h * self.value_dim, self.kv_rank), std=rank_std)]
        if self.gate:
            specs.append(WeightSpec(n["g"], (h if self.gate_per_head else h * self.value_dim, w), std=std))
        specs.append(WeightSpec(n["o"], (w, h * self.value_dim), std=(h * self.value_dim) ** -0.5))
        return specs

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n, h = self.names, self.heads
        rows = [weights[n["dq"] if self.q_rank else n["q"]], weights[n["dkv"]]] + ([weights[n["g"]]] if self.gate else [])
        total = sum(r.shape[0] for r in rows)
        if total % 8:       # (rows of the product's output then start on 16-byte boundaries in bfloat16)
            rows.append(torch.zeros((8 - total % 8, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.in_weight = LinearWeight(torch.cat(rows, dim=0), few_rows_tcgen05=None)
        if self.q_rank:
            self.uq_weight = LinearWeight(weights[n["uq"]], few_rows_tcgen05=None)
            self.q_norm_weight = weights[n["q_norm"]].to(torch.float32).contiguous()
        self.o_weight = LinearWeight(weights[n["o"]], few_rows_tcgen05=None)
        self.latent_norm_weight = weights[n["norm"]].to(torch.float32).contiguous()
        uk = weights[n["uk"]].view(h, self.dim, self.kv_rank)              # per head [in = dim, out = kv_rank]
        self.uv_weight = weights[n["uv"]].view(h, self.value_dim, self.kv_rank).contiguous()   # per head [out, in]
        if uk.dtype == torch.float32:
            self.uk_weight = uk.transpose(1, 2).contiguous()               # the fp32 product wants [out, in]
        else:
            self.uk_weight = uk.contiguous()

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(1, self.kv_rank + self.rot_dim, None, value_dim=0)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        kv, batch = ctx.kv, ctx.batch
        if kv is None or kv.keys is None:
            raise RuntimeError("latent attention needs a cache binding with key pages")
        n, h, c, r = x.shape[0], self.heads, self.kv_rank, self.rot_dim
        width = c + r
        q_width = self.q_rank if self.q_rank else h * (self.dim + r)      # columns of the first projection's q part
        proj = linear(x, self.in_weight)
        q, dkv = proj[:, :q_width], proj[:, q_width:q_width + width]
        if self.q_rank:
            latent_q = ops.rmsnorm(q, self.q_norm_weight, self.eps, torch.empty((n, self.q_rank), dtype=x.dtype, device=x.device))
            q = linear(latent_q, self.uq_weight)
        folded = torch.empty((n, h, width), dtype=torch.float32, device=x.device)
        ops.latent_append(dkv, q, folded, kv.keys if kv.writes else None, batch.positions, batch.token_slot, kv.block_table,
                          self.latent_norm_weight, self.eps, self.inv_freq, h, self.dim, c, r, ctx.error_word,
                          half_pairs=self.half_pairs)
        q_plain = q.as_strided((n, h, self.dim), (q.stride(0), self.dim + r, 1))
        if x.dtype == torch.float32:
            for j in range(h):
                ops.gemm_f32(q_plain[:, j], self.uk_weight[j], folded[:, j, :c])
        else:
            ops.library_gemm_batched(q_plain, self.uk_weight, folded[:, :, :c], w_kn=True)
        latent_out = torch.empty((n, h, c), dtype=torch.float32, device=x.device)
        ops.latent_attention(folded, kv.keys, latent_out, batch.q_start, batch.kv_start, batch.slots, kv.block_table,
                             batch.n_entries, batch.max_q_len, h, c, r, self.scale, ctx.error_word, max_kv_len=batch.max_kv_len)
        heads_out = torch.empty((n, h, self.value_dim), dtype=x.dtype, device=x.device)
        if x.dtype == torch.float32:
            for j in range(h):
                ops.gemm_f32(latent_out[:, j], self.uv_weight[j], heads_out[:, j])
        else:
            rows = ops.cast(latent_out, torch.empty((n, h, c), dtype=x.dtype, device=x.device))
            ops.library_gemm_batched(rows, self.uv_weight, heads_out, w_kn=False)
        heads_out = heads_out.view(n, h * self.value_dim)
        if self.gate:
            gates = h if self.gate_per_head else h * self.value_dim
            ops.sigmoid_gate(heads_out, proj[:, q_width + width:q_width + width + gates], heads_out,
                             group=self.value_dim if self.gate_per_head else 1)
        return linear(heads_out, self.o_weight)


register_part("mixer", "latent_attention", LatentAttention)
