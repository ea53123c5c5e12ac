"""A state-space mixer of the Mamba-2 kind (state-space duality), over state kept per request.

One product makes [z | x | B | C | dt] from the input, with inner = heads * head_dim, N = state_dim, G = groups:
z and x are inner wide, B and C are G * N wide, dt has one number per head.  x, B and C together pass a causal
convolution per channel over ``taps`` tokens (weight [channels, taps] whose last column is the current token's, a bias,
zeros before the start of a sequence) and silu.  Per head h, with its group g = h // (heads / G) and S an N x head_dim
matrix that starts at zero:

    dt_t = softplus(dt_t + dt_bias[h]);   S_t = exp(-exp(A_log[h]) dt_t) S_(t-1) + dt_t B_t x_t^T;   y_t = S_t^T C_t + D[h] x_t

The heads' outputs side by side are multiplied by silu(z), divided by their root mean square in ``norm_groups`` equal
parts (each part by its own), multiplied by a weight, and projected by W_o.  S (fp32) and the convolution's last
taps - 1 inputs live in the cache manager's state slots, one row per request: first S [heads, N, head_dim], then the
inputs [taps - 1, channels]; a new request finds zeros.  The mixer keeps no keys.  The kernels (csrc/state_space.cu)
take the step's whole ragged batch and read it through its device arrays only.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.kernels.gemm import LinearWeight, linear
from torchinferno_b200.parts.base import LayerContext, Mixer, StateSpec, WeightSpec, register_part


class StateSpaceDuality(Mixer):
    capturable = True       # (state is read and written by the kernels through the slots array)

    def __init__(self, *, hidden_size: int, heads: int, head_dim: int, state_dim: int, groups: int = 1, taps: int = 4,
                 norm_groups: int = 1, eps: float = 1e-6, in_name: str = "in", conv_name: str = "conv", dt_bias_name: str = "dt_bias",
                 a_name: str = "A_log", d_name: str = "D", norm_name: str = "norm", o_name: str = "o", bias_suffix: str = ".b",
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        if heads % groups:
            raise ValueError("heads must be a multiple of groups")
        if (heads * head_dim) % norm_groups:
            raise ValueError("norm_groups must divide heads * head_dim")
        if taps < 1:
            raise ValueError("the convolution has at least one tap")
        self.hidden_size, self.heads, self.head_dim, self.state_dim = hidden_size, heads, head_dim, state_dim
        self.groups, self.taps, self.norm_groups, self.eps = groups, taps, norm_groups, float(eps)
        self.inner = heads * head_dim
        self.channels = self.inner + 2 * groups * state_dim
        self.in_width = 2 * self.inner + 2 * groups * state_dim + heads
        self.names = {"in": in_name, "conv": conv_name, "conv_b": conv_name + bias_suffix, "dt_bias": dt_bias_name, "a": a_name,
                      "d": d_name, "norm": norm_name, "o": o_name}
        self.in_weight: LinearWeight | None = None
        self.o_weight: LinearWeight | None = None

    def weight_specs(self) -> list[WeightSpec]:
        n, w = self.names, self.hidden_size
        return [WeightSpec(n["in"], (self.in_width, w), std=w ** -0.5),
                WeightSpec(n["conv"], (self.channels, self.taps), std=self.taps ** -0.5, role="vector"),
                WeightSpec(n["conv_b"], (self.channels,), std=0.1, role="vector"),
                WeightSpec(n["dt_bias"], (self.heads,), std=1.0, role="vector"),
                WeightSpec(n["a"], (self.heads,), std=0.5, role="vector"),
                WeightSpec(n["d"], (self.heads,), init="about_one", std=0.3, role="vector"),
                WeightSpec(n["norm"], (self.inner,), init="about_one", std=0.1, role="vector"),
                WeightSpec(n["o"], (w, self.inner), std=self.inner ** -0.5)]

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        rows = weights[n["in"]]
        if self.in_width % 8:       # (rows of the product's output then start on 16-byte boundaries in bfloat16)
            pad = torch.zeros((8 - self.in_width % 8, self.hidden_size), dtype=rows.dtype, device=rows.device)
            rows = torch.cat([rows, pad], dim=0)
        self.in_weight = LinearWeight(rows, few_rows_tcgen05=None)
        self.o_weight = LinearWeight(weights[n["o"]], few_rows_tcgen05=None)

        def vector(name):
            return weights[name].to(torch.float32).contiguous()

        self.conv_weight, self.conv_bias = vector(n["conv"]), vector(n["conv_b"])
        self.dt_bias, self.a_log, self.d_skip, self.norm_weight = vector(n["dt_bias"]), vector(n["a"]), vector(n["d"]), vector(n["norm"])
        if weights[n["in"]].is_cuda and self.state_dim > ops.ssd_scan_max_state():
            raise ValueError(f"a state of {self.state_dim} per head does not fit the scan kernel (at most {ops.ssd_scan_max_state()})")

    def state_spec(self) -> StateSpec:
        return StateSpec((self.heads * self.state_dim * self.head_dim + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        if ctx.state is None:
            raise RuntimeError("the state-space mixer needs a state tensor")
        batch, n, inner = ctx.batch, x.shape[0], self.inner
        proj = linear(x, self.in_weight)                        # [z | x | B | C | dt]
        xbc = torch.empty((n, self.channels), dtype=x.dtype, device=x.device)
        ops.short_conv(proj, inner, self.conv_weight, self.conv_bias, ctx.state, self.heads * self.state_dim * self.head_dim,
                       batch.q_start, batch.slots, xbc, batch.n_entries, batch.max_q_len, silu=True)
        y = torch.empty((n, inner), dtype=torch.float32, device=x.device)
        ops.ssd_scan(xbc, proj, inner + self.channels, self.dt_bias, self.a_log, self.d_skip, ctx.state, batch.q_start, batch.slots,
                     y, batch.n_entries, heads=self.heads, groups=self.groups, state_dim=self.state_dim, head_dim=self.head_dim,
                     max_q_len=batch.max_q_len)
        rows = torch.empty((n, inner), dtype=x.dtype, device=x.device)
        ops.gated_group_norm(y, proj, 0, self.norm_weight, self.eps, rows, self.norm_groups)
        return linear(rows, self.o_weight)


register_part("mixer", "state_space_duality", StateSpaceDuality)
