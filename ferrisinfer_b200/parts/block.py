"""How a layer's parts are arranged.

The pre-norm residual block, one branch after the other:
  h += mixer(norm_1(h));  h += feed_forward(norm_2(h))          (a layer may have no feed-forward: the first half alone)
(crates/ferrisinfer-runtime/src/reference.rs:244-249, 331-344, 362-368).

The parallel block, both branches from the same h:
  h += mixer(norm_1(h)) + feed_forward(norm_2(h))
Both norms are taken before either branch adds, into buffers of their own.  A layer may have no feed-forward.

The sums are made in the fp32 residual stream by the last matrix product of each branch.
"""

from __future__ import annotations

from .base import Block, TensorSpec
from .plan import build_part, register_part


class PreNormResidualBlock(Block):
    def __init__(self, hidden_size: int, mixer, feed_forward, mixer_norm, feed_forward_norm,
                 mixer_prefix: str = "self_attn", feed_forward_prefix: str = "mlp",
                 mixer_norm_prefix: str = "input_layernorm",
                 feed_forward_norm_prefix: str = "post_attention_layernorm"):
        self.hidden_size = int(hidden_size)
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self._names = (mixer_prefix, feed_forward_prefix, mixer_norm_prefix, feed_forward_norm_prefix)

    def _children(self, prefix):
        m, f, n1, n2 = self._names
        return [(part, p) for part, p in (
            (self.mixer_norm, f"{prefix}.{n1}"),
            (self.mixer, f"{prefix}.{m}"),
            (self.feed_forward_norm, f"{prefix}.{n2}"),
            (self.feed_forward, f"{prefix}.{f}"),
        ) if part is not None]

    def tensor_specs(self, prefix):
        out = []
        for part, p in self._children(prefix):
            specs = part.tensor_specs(p)
            if part is self.feed_forward_norm and self.feed_forward is None:  # read if the folder has it, and not used
                specs = [TensorSpec(s.name, s.shape, s.role, required=False) for s in specs]
            out += specs
        return out

    def bind(self, tensors, prefix):
        for part, p in self._children(prefix):
            if part is self.feed_forward_norm and self.feed_forward is None:
                continue
            part.bind(tensors, p)

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_safe(self):
        return bool(getattr(self.mixer, "graph_safe", False)
                    and (self.feed_forward is None or getattr(self.feed_forward, "graph_safe", False)))

    def forward(self, h, ctx, cache, owns_cache):
        buf = ctx.workspace.get("block_normed", (h.shape[0], self.hidden_size), ctx.act_dtype)
        x = self.mixer_norm.lazy(h, buf)
        if not getattr(self.mixer, "accepts_lazy_norm", False) and hasattr(x, "materialize"):
            x = x.materialize()
        self.mixer.forward(x, h, ctx, cache, owns_cache)
        if self.feed_forward is None:  # a layer of the mixer's branch alone
            return
        x = self.feed_forward_norm.lazy(h, buf)
        if not getattr(self.feed_forward, "accepts_lazy_norm", False) and hasattr(x, "materialize"):
            x = x.materialize()
        self.feed_forward.forward(x, h, ctx)


class ParallelResidualBlock(PreNormResidualBlock):
    """h += mixer(norm_1(h)) + feed_forward(norm_2(h)); ``feed_forward`` None: the mixer's branch alone (the
    second norm's tensor is then read if the folder has it, and not used)."""

    def __init__(self, hidden_size: int, mixer, feed_forward, mixer_norm, feed_forward_norm,
                 mixer_prefix: str = "mix", feed_forward_prefix: str = "mlp", mixer_norm_prefix: str = "norm1",
                 feed_forward_norm_prefix: str = "norm2"):
        super().__init__(hidden_size, mixer, feed_forward, mixer_norm, feed_forward_norm, mixer_prefix,
                         feed_forward_prefix, mixer_norm_prefix, feed_forward_norm_prefix)

    def _children(self, prefix):
        # an empty name stands for the layer's own prefix (a mixer that names its tensors itself)
        return [(part, f"{prefix}.{name}" if name else prefix) for part, name in zip(
            (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward),
            (self._names[2], self._names[0], self._names[3], self._names[1])) if part is not None]

    def tensor_specs(self, prefix):
        out = []
        for part, p in self._children(prefix):
            specs = part.tensor_specs(p)
            if part is self.feed_forward_norm and self.feed_forward is None:
                specs = [TensorSpec(s.name, s.shape, s.role, required=False) for s in specs]
            out += specs
        return out

    def bind(self, tensors, prefix):
        for part, p in self._children(prefix):
            if part is self.feed_forward_norm and self.feed_forward is None:
                continue
            part.bind(tensors, p)

    @property
    def graph_safe(self):
        return bool(getattr(self.mixer, "graph_safe", False)
                    and (self.feed_forward is None or getattr(self.feed_forward, "graph_safe", False)))

    def forward(self, h, ctx, cache, owns_cache):
        T = h.shape[0]
        x1 = ctx.workspace.get("block_normed", (T, self.hidden_size), ctx.act_dtype)
        if self.feed_forward is None:
            self.mixer_norm.forward(h, x1)
        else:
            x2 = ctx.workspace.get("block_normed_2", (T, self.hidden_size), ctx.act_dtype)
            pair = getattr(self.mixer_norm, "forward_pair", None)
            if pair is None or not pair(self.feed_forward_norm, h, x1, x2):  # both norms in one launch where they can be
                self.mixer_norm.forward(h, x1)
                self.feed_forward_norm.forward(h, x2)
        self.mixer.forward(x1, h, ctx, cache, owns_cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(x2, h, ctx)


register_part("block", "pre_norm_residual", PreNormResidualBlock)
register_part("block", "parallel_residual", ParallelResidualBlock)
