"""RMSNorm, plain and fused with the residual add; layer norm with weight and bias; the tanh norm.

y = x * rsqrt(mean(x^2) + eps) * w with the statistics, the product and the
residual sum in fp32 (src/torchinferno/models/llama3/raw_ops.py:9-11,
src/torchinferno/kernels/triton_ops.py:2044-2048, 2088-2096).  The weight
multiplies after normalisation; there is no bias and no ``1 + w`` form.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.parts.base import Norm, WeightSpec, register_part


class RMSNorm(Norm):
    def __init__(self, *, width: int, eps: float, weight_name: str = "weight",
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.width, self.eps, self.weight_name = int(width), float(eps), weight_name
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.width,), init="ones", role="vector")]

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self.weight = weights[self.weight_name].to(torch.float32).contiguous()

    def forward(self, residual, out, rows=None):
        return ops.add_rmsnorm(None, residual, self.weight, self.eps, out, rows)

    def add_forward(self, delta, residual, out, rows=None):
        return ops.add_rmsnorm(delta, residual, self.weight, self.eps, out, rows)

    def forward_rows(self, x: torch.Tensor) -> torch.Tensor:
        """Norm rows held in the activation type (not the residual stream)."""
        return ops.rmsnorm(x, self.weight, self.eps, torch.empty_like(x))


class LayerNorm(Norm):
    """y = (x - mean) / sqrt(mean of squared deviations + eps) * w + b, statistics and scaling in fp32
    (csrc/layernorm.cu).  ``bias_name`` defaults to the weight's name with ``.b`` added."""

    def __init__(self, *, width: int, eps: float, weight_name: str = "weight", bias_name: str | None = None,
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.width, self.eps, self.weight_name = int(width), float(eps), weight_name
        self.bias_name = weight_name + ".b" if bias_name is None else bias_name
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.width,), init="about_one", std=0.1, role="vector"),
                WeightSpec(self.bias_name, (self.width,), std=0.1, role="vector")]

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self.weight = weights[self.weight_name].to(torch.float32).contiguous()
        self.bias = weights[self.bias_name].to(torch.float32).contiguous()

    def forward(self, residual, out, rows=None):
        return ops.layernorm(residual, self.weight, self.bias, self.eps, out, rows)

    def add_forward(self, delta, residual, out, rows=None):
        if rows is None:
            # (one launch: the sum into the 32-bit residual, then the norm of the new row)
            ops.layernorm_tail(residual, self.eps, y=delta, y_norm=None, out=out, out_norm=(self.weight, self.bias))
            return out
        # (with rows the delta is only looked at and stays pending)
        index = rows.long()
        picked = residual.index_select(0, index) + delta.index_select(0, index).to(torch.float32)
        return ops.layernorm(picked, self.weight, self.bias, self.eps, out)

    def forward_rows(self, x: torch.Tensor) -> torch.Tensor:
        """Norm rows held in the activation type (not the residual stream)."""
        return ops.layernorm(x, self.weight, self.bias, self.eps, torch.empty_like(x))


class TanhNorm(Norm):
    """y = tanh(alpha * x) * w + b: a norm that takes no statistic of the row ("dynamic tanh"); ``alpha`` is a learned scalar,
    stored as a tensor without dimensions.  All of it in fp32 (csrc/hyper_streams.cu: it is the read of a residual in
    streams, with one stream here).  ``bias_name`` / ``alpha_name`` default to the weight's name with ``.b`` / ``.alpha``."""

    def __init__(self, *, width: int, weight_name: str = "weight", bias_name: str | None = None, alpha_name: str | None = None,
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.width, self.weight_name = int(width), weight_name
        self.bias_name = weight_name + ".b" if bias_name is None else bias_name
        self.alpha_name = weight_name + ".alpha" if alpha_name is None else alpha_name
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None
        self.alpha = 1.0
        self._one = self._one_by_one = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.width,), init="about_one", std=0.1, role="vector"),
                WeightSpec(self.bias_name, (self.width,), std=0.1, role="vector"),
                WeightSpec(self.alpha_name, (), init="about_one", std=0.2, role="vector")]

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self.weight = weights[self.weight_name].to(torch.float32).contiguous()
        self.bias = weights[self.bias_name].to(torch.float32).contiguous()
        self.alpha = float(weights[self.alpha_name].to(torch.float32).item())    # (read once, when the model is bound)
        self._one = torch.ones(1, dtype=torch.float32, device=self.weight.device)
        self._one_by_one = self._one.view(1, 1)

    def tanh_params(self) -> tuple[float, torch.Tensor, torch.Tensor]:
        return self.alpha, self.weight, self.bias

    def forward(self, residual, out, rows=None):
        return ops.hyper_step(residual.unsqueeze(0), in_weights=self._one, out=out, rows=rows, tanh_norm=self.tanh_params())

    def add_forward(self, delta, residual, out, rows=None):
        # (one launch: the sum into the 32-bit residual, then the norm of the new row; with rows the delta is only looked at)
        return ops.hyper_step(residual.unsqueeze(0), y=delta, mix=self._one_by_one, out_weights=self._one, in_weights=self._one,
                              out=out, rows=rows, tanh_norm=self.tanh_params())


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
register_part("norm", "tanh", TanhNorm)
