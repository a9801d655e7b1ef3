"""RMSNorm as a part: sizes and eps are parameters; statistics are fp32.

  ms = sum(x^2) / H;  r = 1 / sqrt(ms + eps);  y_j = (x_j * r) * w_j
(crates/ferrisinfer-kernel/src/cpu/reduction.rs:35-41).

``DynamicTanh``: no statistics at all: y_j = tanh(alpha x_j) * w_j + b_j with one learned number alpha; the tensors are
``weight_name``, ``<weight_name>.<alpha_name>`` and ``<weight_name>.<bias_name>`` under the part's prefix.

``GroupedRMSNorm``: the row in ``groups`` equal consecutive parts, each divided by its own root mean square; the
weight spans the whole row.  The tensor is named by ``weight_name`` under the part's prefix ("" = the prefix itself).
``unit_offset``: the folder stores the weight around zero and the norm multiplies by 1 + w; the sum is formed once, in
fp32, when the tensor arrives, so every kernel sees a plain weight.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm, TensorSpec
from .plan import register_part


class RMSNorm(Norm):
    def __init__(self, hidden_size: int, eps: float):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.weight = None

    def tensor_specs(self, prefix):
        return [TensorSpec(f"{prefix}.weight", (self.hidden_size,), "norm")]

    def bind(self, tensors, prefix):
        self.weight = tensors[f"{prefix}.weight"]

    def forward(self, h, out, row_index=None):
        ops.rmsnorm(h, self.weight, self.eps, out, row_index)

    def lazy(self, h, out):
        return ops.LazyRMSNorm(h, self.weight, self.eps, out)


class GroupedRMSNorm(Norm):
    def __init__(self, hidden_size: int, eps: float, groups: int = 1, weight_name: str = "weight",
                 unit_offset: bool = False):
        self.hidden_size, self.eps, self.groups = int(hidden_size), float(eps), int(groups)
        self.unit_offset = bool(unit_offset)
        if self.groups < 1 or self.hidden_size % self.groups:
            raise ValueError(f"{self.hidden_size} columns cannot be normed in {self.groups} equal groups")
        self.weight_name = weight_name
        self.weight = None

    def _name(self, prefix):
        return f"{prefix}.{self.weight_name}" if self.weight_name else prefix

    def tensor_specs(self, prefix):
        # a weight stored around zero is drawn like a bias in random folders
        return [TensorSpec(self._name(prefix), (self.hidden_size,), "bias" if self.unit_offset else "norm")]

    def bind(self, tensors, prefix):
        self.weight = tensors[self._name(prefix)]
        if self.unit_offset:
            self.weight = (self.weight.to(torch.float32) + 1.0).contiguous()

    def forward(self, h, out, row_index=None):
        ops.grouped_rmsnorm(h, self.weight, self.eps, self.groups, out, row_index)

    def lazy(self, h, out):
        if self.groups == 1:
            return ops.LazyRMSNorm(h, self.weight, self.eps, out)
        self.forward(h, out)
        return out

    def forward_pair(self, other, h, out, other_out) -> bool:
        """This norm and ``other`` of the same rows in one launch; False (nothing done) if ``other`` is not the same
        norm with another weight."""
        if not isinstance(other, GroupedRMSNorm) or (other.hidden_size, other.eps, other.groups) != (
                self.hidden_size, self.eps, self.groups):  # (either may store its weight around zero: both hold 1 + w)
            return False
        ops.grouped_rmsnorm_pair(h, self.weight, other.weight, self.eps, self.groups, out, other_out)
        return True


class DynamicTanh(Norm):
    """tanh(alpha * x) * weight + bias, element by element in fp32; ``eps`` is accepted and unused (the norm divides by
    nothing)."""

    def __init__(self, hidden_size: int, eps: float = 0.0, weight_name: str = "weight", alpha_name: str = "alpha",
                 bias_name: str = "b"):
        self.hidden_size = int(hidden_size)
        self.weight_name, self.alpha_name, self.bias_name = weight_name, alpha_name, bias_name
        self.weight = self.bias = self.alpha = None

    def _names(self, prefix):
        w = f"{prefix}.{self.weight_name}" if self.weight_name else prefix
        return w, f"{w}.{self.alpha_name}", f"{w}.{self.bias_name}"

    def tensor_specs(self, prefix):
        w, a, b = self._names(prefix)
        return [TensorSpec(w, (self.hidden_size,), "norm"), TensorSpec(b, (self.hidden_size,), "bias"),
                TensorSpec(a, (), "norm")]

    def bind(self, tensors, prefix):
        w, a, b = self._names(prefix)
        self.weight, self.bias, self.alpha = tensors[w], tensors[b], tensors[a].reshape(1)

    def forward(self, h, out, row_index=None):
        ops.dynamic_tanh(h, self.weight, self.bias, self.alpha, out, row_index)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
register_part("norm", "grouped_rmsnorm", GroupedRMSNorm)
