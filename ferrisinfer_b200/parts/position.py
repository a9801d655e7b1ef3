"""Position encodings as parts.

``RotaryEncoding``: rotate-half rotary positions over the first ``rotary_dim``
dims of each head.  Frequencies as the reference forms them, a running product
in f32 (crates/ferrisinfer-kernel/src/cpu/attention.rs:1254-1276):
``step = theta ** (-2 / head_dim)``, ``inv_freq[0] = 1``,
``inv_freq[i + 1] = inv_freq[i] * step`` (the exponent uses head_dim, not
rotary_dim).  The angle ``float(pos) * inv_freq[i]`` and its sine and cosine
are fp32, formed in the kernel that also writes the cache.

``ScaledRotary``: a rotation of the first ``rotary_dim`` elements of a head with frequencies
``base ** (-2 i / rotary_dim)`` (formed in 64-bit on the host, rounded once), pairs laid out (i, i + rotary_dim / 2)
("half") or (2i, 2i + 1) ("interleaved"), optionally with YaRN scaling: with c(r) = rotary_dim ln(original / (2 pi r)) /
(2 ln base), lo = max(floor(c(fast)), 0), hi = min(ceil(c(slow)), rotary_dim - 1) and ramp_i = clamp((i - lo) /
max(hi - lo, 0.001), 0, 1), frequency i becomes f_i / factor * ramp_i + f_i (1 - ramp_i), and every cosine and sine is
multiplied by 0.1 ln(factor) + 1.  It is applied by the kernel that prepares a mixer's queries and keys.

``NoPosition``: nothing is encoded (the keys go to the cache as they are).

``DistanceSlopes``: nothing is rotated; the score of the key at position j for the query at position P loses
slope_h * (P - j), with slope_h = 2^(-span (h + 1) / heads) for head h = 0 .. heads - 1 (span 8 by default).
"""

from __future__ import annotations

import math

import numpy as np
import torch

from ..kernels import ops
from .base import PositionEncoding, TensorSpec
from .plan import register_part


def rotary_inverse_frequencies(head_dim: int, rotary_dim: int, theta: float) -> np.ndarray:
    step = np.float32(np.power(np.float32(theta), np.float32(-2.0) / np.float32(head_dim), dtype=np.float32))
    out = np.empty(rotary_dim // 2, dtype=np.float32)
    f = np.float32(1.0)
    for i in range(rotary_dim // 2):
        out[i] = f
        f = np.float32(f * step)
    return out


class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def __init__(self, head_dim: int, rotary_dim: int, theta: float):
        if rotary_dim % 2 or not (0 <= rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.head_dim, self.rotary_dim, self.theta = int(head_dim), int(rotary_dim), float(theta)
        self._host = rotary_inverse_frequencies(self.head_dim, self.rotary_dim, self.theta)
        self._device = {}

    def rotary_table(self, device=None):
        if self.rotary_dim == 0:
            return None, 0
        device = torch.device(device if device is not None else "cuda")
        key = str(device)
        if key not in self._device:
            self._device[key] = torch.from_numpy(self._host.copy()).to(device)
        return self._device[key], self.rotary_dim

    def angles(self, ctx):
        """(cos, sin) of position x frequency for the tokens of the step, fp32 [T, rotary_dim / 2, 2]: computed by
        the first layer of a pass that asks, shared with the other layers of the same frequencies."""
        key = ("rotary_angles", self.head_dim, self.rotary_dim, self.theta)
        angles = ctx.shared.get(key)
        if angles is None:
            inv_freq, _ = self.rotary_table(ctx.positions.device)
            angles = ctx.workspace.get(f"rotary_angles_{len(ctx.shared)}", (ctx.positions.numel(), inv_freq.numel(), 2),
                                       torch.float32)
            ops.rotary_angles(ctx.positions, inv_freq, angles)
            ctx.shared[key] = angles
        return angles


class ScaledRotary(PositionEncoding):
    graph_safe = True

    def __init__(self, rotary_dim: int, base: float, layout: str = "half", scaling: dict = None):
        """``scaling``: None, or the four numbers ``factor``, ``original``, ``fast``, ``slow`` of a YaRN scaling."""
        if layout not in ("half", "interleaved"):
            raise ValueError(f"rotary layout '{layout}' is not known (half, interleaved)")
        if rotary_dim < 0 or rotary_dim % 2:
            raise ValueError(f"{rotary_dim} rotated elements: an even count is needed")
        self.rotary_dim, self.base, self.layout = int(rotary_dim), float(base), layout
        self.scaling = dict(scaling) if scaling else None
        R = self.rotary_dim
        freq = [self.base ** (-2.0 * i / R) for i in range(R // 2)]
        self.magnitude = 1.0
        if self.scaling and R:
            factor, original = float(self.scaling["factor"]), float(self.scaling["original"])
            fast, slow = float(self.scaling["fast"]), float(self.scaling["slow"])
            if factor <= 0 or original <= 0 or fast <= 0 or slow <= 0 or self.base <= 1.0:
                raise ValueError(f"rotary scaling {self.scaling} with base {self.base}: positive numbers and a base above one")

            def crossing(r):
                return R * math.log(original / (2.0 * math.pi * r)) / (2.0 * math.log(self.base))

            lo = max(math.floor(crossing(fast)), 0)
            hi = min(math.ceil(crossing(slow)), R - 1)
            for i, f in enumerate(freq):
                ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                freq[i] = f / factor * ramp + f * (1.0 - ramp)
            self.magnitude = 0.1 * math.log(factor) + 1.0
        exact = np.asarray(freq, dtype=np.float64)
        self._host = exact.astype(np.float32)
        # what the 32-bit frequencies lack of the 64-bit ones, for kernels that form their angles beyond 32-bit rounding
        self._host_lo = (exact - self._host.astype(np.float64)).astype(np.float32)
        self._device = {}

    def rotary_table(self, device=None):
        return None  # not the plain layer's rotation: the mixer asks for ``table`` instead

    def table(self, device=None) -> "ops.RotaryTable":
        """What the kernels take: frequencies on ``device``, layout, the factor on cosines and sines."""
        device = torch.device(device if device is not None else "cuda")
        key = str(device)
        if key not in self._device:
            self._device[key] = ops.RotaryTable(torch.from_numpy(self._host.copy()).to(device), self.rotary_dim,
                                                self.layout == "interleaved", self.magnitude,
                                                freq_lo=torch.from_numpy(self._host_lo.copy()).to(device))
        return self._device[key]


class NoPosition(PositionEncoding):
    graph_safe = True

    def rotary_table(self, device=None):
        return None, 0


class DistanceSlopes(PositionEncoding):
    graph_safe = True

    def __init__(self, span: float = 8.0):
        self.span = float(span)
        self._device = {}

    def rotary_table(self, device=None):
        return None, 0

    def score_slopes(self, num_heads, device=None):
        device = torch.device(device if device is not None else "cuda")
        key = (str(device), int(num_heads))
        if key not in self._device:
            slopes = [2.0 ** (-self.span * (h + 1) / num_heads) for h in range(num_heads)]
            self._device[key] = torch.tensor(slopes, dtype=torch.float64).to(torch.float32).to(device)
        return self._device[key]


class LogDistancePenalty(PositionEncoding):
    """Nothing is rotated; the score of the key at position j for the query at position P loses
    r1_h * ln(1 + r2_h * (P - j)), with two learned numbers per head, named ``r1_name`` and ``r2_name`` under the
    mixer's prefix."""

    graph_safe = True
    learned_scores = True  # its numbers come from the folder: the mixer asks for its tensors and attends the general way

    def __init__(self, num_heads: int, r1_name: str = "r1", r2_name: str = "r2"):
        self.num_heads, self.r1_name, self.r2_name = int(num_heads), r1_name, r2_name
        self.r1 = self.r2 = None

    def rotary_table(self, device=None):
        return None, 0

    def tensor_specs(self, prefix):
        # role "norm": positive numbers of order one (a random folder draws them around one)
        return [TensorSpec(f"{prefix}.{self.r1_name}", (self.num_heads,), "norm"),
                TensorSpec(f"{prefix}.{self.r2_name}", (self.num_heads,), "norm")]

    def bind(self, tensors, prefix):
        self.r1, self.r2 = tensors[f"{prefix}.{self.r1_name}"], tensors[f"{prefix}.{self.r2_name}"]

    def score_log_penalty(self, num_heads, device=None):
        if num_heads != self.num_heads:
            raise ValueError(f"a distance penalty for {self.num_heads} heads, asked for {num_heads}")
        return self.r1, self.r2


register_part("position", "rotary", RotaryEncoding)
register_part("position", "scaled_rotary", ScaledRotary)
register_part("position", "log_distance_penalty", LogDistancePenalty)
register_part("position", "distance_slopes", DistanceSlopes)
register_part("position", "none", NoPosition)
