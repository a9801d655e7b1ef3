"""Feed-forwards as parts: the gated SiLU one (SwiGLU), a plain one with a choice of activation, and a mixture of
gated SiLU experts of which every token uses a few.

  u = y W_up^T;  g = y W_gate^T;  m = u * (g * sigmoid(g));  h += m W_down^T
(crates/ferrisinfer-runtime/src/reference.rs:346-368; the reference's w1 is up_proj and w3 is
gate_proj: crates/ferrisinfer-io/src/hf.rs:437-457).  No bias.  Gate and up are held as one
[2I, H] matrix (gate rows first) so that one matrix product feeds the activation.

``GatedFeedForward`` is the same layer with the gate's function as a parameter (``ops.GATED_ACTIVATIONS``: "silu",
"gelu_tanh", "clamped_swish" with its limit) and the three tensors' names under the prefix.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, TensorSpec
from .plan import register_part


class SwiGLU(FeedForward):
    accepts_lazy_norm = True  # x goes to ops.gemm_swiglu and nowhere else
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.gate_up = None
        self.down = None

    def tensor_specs(self, prefix):
        H, I = self.hidden_size, self.intermediate_size
        return [
            TensorSpec(f"{prefix}.gate_proj.weight", (I, H), "matrix"),
            TensorSpec(f"{prefix}.up_proj.weight", (I, H), "matrix"),
            TensorSpec(f"{prefix}.down_proj.weight", (H, I), "matrix"),
        ]

    def bind(self, tensors, prefix):
        self.gate_up = torch.cat(
            [tensors.pop(f"{prefix}.gate_proj.weight"), tensors.pop(f"{prefix}.up_proj.weight")], dim=0
        ).contiguous()
        self.down = tensors[f"{prefix}.down_proj.weight"]

    def forward(self, x, h, ctx):
        T, I = x.shape[0], self.intermediate_size
        act = ctx.workspace.get("ffn_act", (T, I), x.dtype)
        ops.gemm_swiglu(x, self.gate_up, act, ctx.workspace)
        ops.gemm(act, self.down, None, h, accumulate=True)


class GatedFeedForward(FeedForward):
    """h += W_down f(W_gate y, W_up y), f a gated activation: silu(g) u, gelu_tanh(g) u, or, with a ``limit`` L,
    min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1)."""

    accepts_lazy_norm = True
    graph_safe = True
    can_overwrite = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", limit: float = 0.0,
                 gate_name: str = "gate", up_name: str = "up", down_name: str = "down"):
        if activation not in ops.GATED_ACTIVATIONS:
            raise ValueError(f"gated activation '{activation}' is not known ({', '.join(ops.GATED_ACTIVATIONS)})")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.activation, self.limit = activation, float(limit)
        self._names = (gate_name, up_name, down_name)
        self.gate_up = self.down = None

    def tensor_specs(self, prefix):
        H, I = self.hidden_size, self.intermediate_size
        g, u, d = self._names
        return [TensorSpec(f"{prefix}.{g}", (I, H), "matrix"), TensorSpec(f"{prefix}.{u}", (I, H), "matrix"),
                TensorSpec(f"{prefix}.{d}", (H, I), "matrix")]

    def bind(self, tensors, prefix):
        g, u, d = self._names
        self.gate_up = torch.cat([tensors.pop(f"{prefix}.{g}"), tensors.pop(f"{prefix}.{u}")], dim=0).contiguous()
        self.down = tensors[f"{prefix}.{d}"]

    def forward(self, x, h, ctx, accumulate: bool = True):
        T, I = x.shape[0], self.intermediate_size
        act = ctx.workspace.get("ffn_act", (T, I), ctx.act_dtype)
        ops.gemm_gated(x, self.gate_up, act, self.activation, self.limit, ctx.workspace)
        ops.gemm(act, self.down, None, h, accumulate=accumulate)


class DenseActivation(FeedForward):
    """h += W_down a(W_up y), no gate, no bias.  ``activation``: "xielu" (two learned numbers p, q in the tensor
    ``act``: softplus(p) z^2 + z / 2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise), "silu" or
    "relu2" (the square of max(z, 0)).
    The activation is evaluated in fp32: in the up product's epilogue on the accumulator where a tensor-core or
    weight-stationary kernel runs the product (bf16), in a kernel of its own otherwise."""

    accepts_lazy_norm = True
    graph_safe = True
    can_overwrite = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "xielu",
                 up_name: str = "up", down_name: str = "down", act_name: str = "act"):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not known ({', '.join(ops.ACTIVATIONS)})")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.activation = activation
        self._names = (up_name, down_name, act_name)
        self.up = self.down = self.act = None

    def tensor_specs(self, prefix):
        H, I = self.hidden_size, self.intermediate_size
        up, down, act = self._names
        specs = [TensorSpec(f"{prefix}.{up}", (I, H), "matrix"), TensorSpec(f"{prefix}.{down}", (H, I), "matrix")]
        if self.activation == "xielu":
            specs.append(TensorSpec(f"{prefix}.{act}", (2,), "vector"))
        return specs

    def bind(self, tensors, prefix):
        up, down, act = self._names
        self.up, self.down = tensors[f"{prefix}.{up}"], tensors[f"{prefix}.{down}"]
        self.act = tensors.get(f"{prefix}.{act}")
        self.coefficients = (0.0, 0.0)
        if self.act is not None:
            # what the product's epilogue needs of the two learned numbers, formed once: softplus(p), 1/2 + softplus(q)
            sp = torch.nn.functional.softplus(self.act.detach().to("cpu", torch.float32), threshold=20.0)
            self.coefficients = (float(sp[0]), 0.5 + float(sp[1]))

    def forward(self, x, h, ctx, accumulate: bool = True):
        T, I = x.shape[0], self.intermediate_size
        z = ctx.workspace.get("ffn_act", (T, I), ctx.act_dtype)
        ops.gemm_activation(x, self.up, z, self.activation, self.coefficients, self.act)
        ops.gemm(z, self.down, None, h, accumulate=accumulate)


class MixtureOfExperts(FeedForward):
    """h += sum over the token's ``top`` experts of weight_e W_down_e (silu(W_gate_e y) * (W_up_e y)).

    Router: z = W_r y + b_r in fp32 sums; the ``top`` largest z (the lowest index among equals); the weights are the
    softmax over those alone.  Experts have no biases.  Tensors under the prefix: ``router`` [experts, H],
    ``router.b`` [experts], and for expert i ``e<i>.gate`` / ``e<i>.up`` [ff, H], ``e<i>.down`` [H, ff]; on the device
    the experts' matrices are stacked ([experts, 2 ff, H], an expert's gate rows before its up rows, and
    [experts, H, ff]) so that kernels address an expert by its index.

    ``scored`` = {"correction": tensor name, "groups": n, "keep": n} selects the other kind of router: scores s =
    softmax(z) over ALL router outputs (no bias), the choice made by s + correction (a learned number per output)
    among the outputs of the ``keep`` best of ``groups`` equal groups of neighbours (a group's score is its largest
    choice score), the weights s_e / (sum of the chosen s + 1e-20).  ``identity``: that many router outputs after the
    experts stand for experts without tensors whose result is the token's row itself.  ``activation``, ``limit``: the
    experts' gated activation (``ops.GATED_ACTIVATIONS``)."""

    graph_safe = True
    can_overwrite = True

    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int, router_name: str = "router",
                 router_bias_name: str = "router.b", expert_prefix: str = "e", gate_name: str = "gate",
                 up_name: str = "up", down_name: str = "down", scored: dict = None, identity: int = 0,
                 activation: str = "silu", limit: float = 0.0):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.experts, self.top, self.identity = int(experts), int(top), int(identity)
        self.outputs = self.experts + self.identity  # of the router
        if not (1 <= self.top <= self.outputs) or self.identity < 0:
            raise ValueError(f"{self.top} of {self.experts} + {self.identity} experts cannot be chosen")
        if activation not in ops.GATED_ACTIVATIONS:
            raise ValueError(f"gated activation '{activation}' is not known ({', '.join(ops.GATED_ACTIVATIONS)})")
        self.activation, self.limit = activation, float(limit)
        self.scored = None
        if scored is not None:
            groups, keep = int(scored.get("groups", 1)), int(scored.get("keep", 1))
            if groups < 1 or self.outputs % groups or not (1 <= keep <= groups) or self.top > keep * (self.outputs // groups):
                raise ValueError(f"{self.outputs} router outputs in {groups} groups of which {keep} stay, {self.top} chosen")
            self.scored = (scored.get("correction"), groups, keep)
        elif self.identity:
            raise ValueError("identity experts go with the scored kind of router")
        self.correction = None
        self._names = (router_name, router_bias_name, expert_prefix, gate_name, up_name, down_name)
        self.router = self.router_bias = self.gate_up = self.down = None

    def _expert(self, prefix, e, which):
        return f"{prefix}.{self._names[2]}{e}.{which}"

    def tensor_specs(self, prefix):
        H, I = self.hidden_size, self.intermediate_size
        r, rb, _, g, u, d = self._names
        specs = []
        for e in range(self.experts):
            specs += [TensorSpec(self._expert(prefix, e, g), (I, H), "matrix"),
                      TensorSpec(self._expert(prefix, e, u), (I, H), "matrix"),
                      TensorSpec(self._expert(prefix, e, d), (H, I), "matrix")]
        if self.scored is not None:
            specs.append(TensorSpec(f"{prefix}.{r}", (self.outputs, H), "matrix"))
            if self.scored[0]:
                specs.append(TensorSpec(f"{prefix}.{self.scored[0]}", (self.outputs,), "bias"))
            return specs
        return specs + [TensorSpec(f"{prefix}.{r}", (self.experts, H), "matrix"),
                        TensorSpec(f"{prefix}.{rb}", (self.experts,), "bias")]

    def bind(self, tensors, prefix):
        r, rb, _, g, u, d = self._names
        if self.experts:
            self.gate_up = torch.stack([torch.cat([tensors.pop(self._expert(prefix, e, g)), tensors.pop(self._expert(prefix, e, u))])
                                        for e in range(self.experts)]).contiguous()
            self.down = torch.stack([tensors.pop(self._expert(prefix, e, d)) for e in range(self.experts)]).contiguous()
        self.router = tensors[f"{prefix}.{r}"]
        if self.scored is not None:
            self.router_bias = None
            self.correction = tensors[f"{prefix}.{self.scored[0]}"] if self.scored[0] else None
        else:
            self.router_bias = tensors[f"{prefix}.{rb}"]
        if self.experts == 0:  # identity experts only: the kernels still want matrices to point at
            W, I = self.hidden_size, self.intermediate_size
            self.gate_up = self.router.new_zeros(1, 2 * I, W)
            self.down = self.router.new_zeros(1, W, I)

    def forward(self, x, h, ctx, accumulate: bool = True):
        T = x.shape[0]
        ids = ctx.workspace.get("moe_ids", (T, self.top), torch.int32)
        weights = ctx.workspace.get("moe_weights", (T, self.top), torch.float32)
        identity_w = ctx.workspace.get("moe_identity_w", (T,), torch.float32) if self.identity else None
        scored = None
        if self.scored is not None:
            scored = {"correction": self.correction, "groups": self.scored[1], "keep": self.scored[2],
                      "with_weights": self.experts, "identity_w": identity_w}
        ops.moe_router(x, self.router, self.router_bias, ids, weights, self.top, scored=scored)
        ops.moe_experts(x, self.gate_up, self.down, ids, weights, h, ctx.workspace, accumulate=accumulate,
                        activation=self.activation, limit=self.limit, identity_w=identity_w)


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "gated", GatedFeedForward)
register_part("feed_forward", "mixture_of_experts", MixtureOfExperts)
register_part("feed_forward", "dense_activation", DenseActivation)
