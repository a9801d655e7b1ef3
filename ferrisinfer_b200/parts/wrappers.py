"""Mixers that wrap other mixers: a token shift in front of one, and several side by side.

``TokenShiftInput``: the wrapped mixer reads y_t + (y_(t-1) - y_t) * shift instead of y_t, y_(t-1) being the row of the
token before as it was BEFORE its own shift (zeros for a sequence's first token).  The request's last unshifted row
is its state (a slot of [H], fp32, zero at admission), beside whatever the wrapped mixer keeps.  The weight is named
``weight_name`` under the part's prefix and the wrapped mixer's tensors live under ``inner_prefix`` there.

``ParallelMixers``: every branch reads the same input; h += coef * sum_b rmsnorm(branch_b(y)) * w_b, the norm over the
model width with a plain weight per branch (``<prefix>.<name>.out``); coef is 1 / branches unless given.  With
``norm=False`` the branches' results are simply added, h += sum_b branch_b(y): every branch then adds into the residual
rows itself (a factor on a branch's result is that branch's own parameter), and there are no tensors beside the
branches'.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import CombinedNeed, FixedState, LayerCache, Mixer, TensorSpec
from .plan import PartSpec, build_part, register_part


class TokenShiftInput(Mixer):
    accepts_lazy_norm = False

    def __init__(self, hidden_size: int, inner, weight_name: str = "shift", inner_prefix: str = "mix"):
        self.hidden_size = int(hidden_size)
        self.inner = build_part("mixer", inner) if isinstance(inner, PartSpec) else inner
        self.weight_name, self.inner_prefix = weight_name, inner_prefix
        self.weight = None

    @property
    def graph_safe(self):
        return bool(getattr(self.inner, "graph_safe", False))

    @property
    def can_overwrite(self):
        return bool(getattr(self.inner, "can_overwrite", False))

    def tensor_specs(self, prefix):
        return [TensorSpec(f"{prefix}.{self.weight_name}", (self.hidden_size,), "vector")] + \
            self.inner.tensor_specs(f"{prefix}.{self.inner_prefix}")

    def bind(self, tensors, prefix):
        self.weight = tensors[f"{prefix}.{self.weight_name}"]
        self.inner.bind(tensors, f"{prefix}.{self.inner_prefix}")

    def cache_need(self):
        return CombinedNeed((FixedState((self.hidden_size,), torch.float32), self.inner.cache_need()))

    def shift_in_read(self, ctx, cache: LayerCache, owns_cache: bool):
        """(weights, state) if the caller's kernel that forms this mixer's input can shift it on its way (a step in which
        every request brings one token, the state moved on as well), else None.  A caller that does so hands the rows to
        ``forward`` with ``shifted=True``."""
        if owns_cache and ctx.max_q_len == 1 and ctx.num_tokens == ctx.num_seqs:
            return self.weight, cache.parts[0].state
        return None

    def forward(self, x, h, ctx, cache: LayerCache, owns_cache: bool, accumulate: bool = True, shifted: bool = False):
        last, inner_cache = cache.parts
        if shifted:
            u = x
        else:
            u = ctx.workspace.get("token_shift_out", (x.shape[0], self.hidden_size), x.dtype)
            ops.token_shift(x, u, self.weight, last.state, ctx, advance=owns_cache)
        if accumulate:
            self.inner.forward(u, h, ctx, inner_cache, owns_cache)
        else:
            self.inner.forward(u, h, ctx, inner_cache, owns_cache, accumulate=False)


class ParallelMixers(Mixer):
    accepts_lazy_norm = False
    can_overwrite = True

    def __init__(self, hidden_size: int, branches: dict, norm_eps: float = 0.0, coef: float = None, out_name: str = "out",
                 norm: bool = True):
        """``branches``: name -> PartSpec of a mixer (one to four), in order."""
        if not 1 <= len(branches) <= 4:
            raise ValueError(f"{len(branches)} mixers side by side (one to four)")
        self.hidden_size, self.norm_eps = int(hidden_size), float(norm_eps)
        self.names = list(branches)
        self.mixers = [build_part("mixer", b) if isinstance(b, PartSpec) else b for b in branches.values()]
        self.coef = 1.0 / len(self.mixers) if coef is None else float(coef)
        self.out_name, self.norm = out_name, bool(norm)
        if not self.norm and coef is not None:
            raise ValueError("branches that are simply added take their factors themselves")
        self.out_weights = None

    @property
    def graph_safe(self):
        return all(getattr(m, "graph_safe", False) for m in self.mixers)

    def tensor_specs(self, prefix):
        specs = []
        for name, m in zip(self.names, self.mixers):
            specs += m.tensor_specs(f"{prefix}.{name}")
        if not self.norm:
            return specs
        return specs + [TensorSpec(f"{prefix}.{name}.{self.out_name}", (self.hidden_size,), "norm") for name in self.names]

    def bind(self, tensors, prefix):
        for name, m in zip(self.names, self.mixers):
            m.bind(tensors, f"{prefix}.{name}")
        if not self.norm:
            return
        self.out_weights = [tensors[f"{prefix}.{name}.{self.out_name}"] for name in self.names]

    def cache_need(self):
        return CombinedNeed(tuple(m.cache_need() for m in self.mixers))

    def forward(self, x, h, ctx, cache: LayerCache, owns_cache: bool, accumulate: bool = True):
        if not self.norm:  # every branch adds into h; the first replaces it where the caller wants the result alone
            for i, m in enumerate(self.mixers):
                if i == 0 and not accumulate:
                    if getattr(m, "can_overwrite", False):
                        m.forward(x, h, ctx, cache.parts[i], owns_cache, accumulate=False)
                        continue
                    h.zero_()
                m.forward(x, h, ctx, cache.parts[i], owns_cache)
            return
        T = x.shape[0]
        results = ctx.workspace.get("parallel_mixers_out", (len(self.mixers), T, self.hidden_size), torch.float32)
        for i, m in enumerate(self.mixers):
            if getattr(m, "can_overwrite", False):
                m.forward(x, results[i], ctx, cache.parts[i], owns_cache, accumulate=False)
            else:  # a mixer that only adds: into zeroed rows
                results[i].zero_()
                m.forward(x, results[i], ctx, cache.parts[i], owns_cache)
        ops.branch_norm_sum(h, [(results[i], w) for i, w in enumerate(self.out_weights)], self.coef, self.norm_eps,
                            accumulate=accumulate)


register_part("mixer", "token_shift_input", TokenShiftInput)
register_part("mixer", "parallel_mixers", ParallelMixers)
