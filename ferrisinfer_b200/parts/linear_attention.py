"""Linear attention with a fixed decay per head, as a part: a state of fixed size per request instead of keys.

  q, k, v = a(y Wq^T), a(y Wk^T), a(y Wv^T)      heads x dim, heads x dim, heads x vdim; a = SiLU (or nothing)
  S_t = decay_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t          per head, fp32, S zero when the request is admitted
  h += (rmsnorm(concat_h o_t) * n * sigmoid(y Wg^T)) Wo^T       one norm over all heads, a plain weight n

Options, each a parameter: ``position`` (a ``scaled_rotary`` encoding: q and k are rotated by their positions on their
way into the recurrence), ``k_scale`` (k is multiplied by it after the rotation), ``head_norm`` (every head's o is
divided by its own sqrt(mean(o^2) + eps) and there is no weight n, instead of one norm over all heads), ``gate``
("sigmoid" or "silu": the function of y Wg^T that multiplies the normed output).

The four input matrices are held as one [2 heads dim + 2 heads vdim, H] matrix so that one product feeds the
recurrence and the gate.  The state is carried from step to step in the request's slot, so prompts may be cut
anywhere; the recurrence, the norm and the gate are fp32 whatever the activations' type.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FixedState, LayerCache, Mixer, TensorSpec
from .plan import PartSpec, build_part, register_part


class DecayedLinearAttention(Mixer):
    accepts_lazy_norm = True
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, decay, norm_eps: float,
                 activation: str = "silu", tensor_names: dict = None, position: PartSpec = None, k_scale: float = 1.0,
                 head_norm: bool = False, gate: str = "sigmoid"):
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.decay = [float(d) for d in decay]
        if len(self.decay) != self.num_heads:
            raise ValueError(f"{len(self.decay)} decays for {self.num_heads} heads")
        if activation not in ("silu", "none"):
            raise ValueError(f"activation '{activation}' of q, k, v is not known (silu, none)")
        if self.head_dim > 256:
            raise ValueError(f"heads of {self.head_dim} are larger than the recurrence kernel takes (256)")
        if gate not in ("sigmoid", "silu"):
            raise ValueError(f"gate '{gate}' of the output is not known (sigmoid, silu)")
        self.norm_eps, self.activation = float(norm_eps), activation
        self.position = build_part("position", position) if isinstance(position, PartSpec) else position
        if self.position is not None and not hasattr(self.position, "table"):
            raise ValueError("the recurrence rotates q and k only by a position encoding that gives a rotary table")
        self.k_scale, self.head_norm, self.gate = float(k_scale), bool(head_norm), gate
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}
        self.names.update(tensor_names or {})
        self.qk_size = self.num_heads * self.head_dim
        self.v_size = self.num_heads * self.v_head_dim
        self.in_weight = self.o_weight = self.norm_weight = None
        self._decay = {}

    def tensor_specs(self, prefix):
        H, n = self.hidden_size, self.names
        specs = [
            TensorSpec(f"{prefix}.{n['q']}", (self.qk_size, H), "matrix"),
            TensorSpec(f"{prefix}.{n['k']}", (self.qk_size, H), "matrix"),
            TensorSpec(f"{prefix}.{n['v']}", (self.v_size, H), "matrix"),
            TensorSpec(f"{prefix}.{n['g']}", (self.v_size, H), "matrix"),
            TensorSpec(f"{prefix}.{n['o']}", (H, self.v_size), "matrix"),
        ]
        if not self.head_norm:
            specs.append(TensorSpec(f"{prefix}.{n['norm']}", (self.v_size,), "norm"))
        return specs

    def bind(self, tensors, prefix):
        n = self.names
        self.in_weight = torch.cat([tensors.pop(f"{prefix}.{n[w]}") for w in "qkvg"], dim=0).contiguous()
        self.o_weight = tensors[f"{prefix}.{n['o']}"]
        if self.head_norm:  # no learned weight: one 1 that the norm kernel repeats over the columns
            self.norm_weight = torch.ones(1, dtype=torch.float32, device=self.o_weight.device)
        else:
            self.norm_weight = tensors[f"{prefix}.{n['norm']}"]

    def cache_need(self):
        # transposed: a column of S (one value dim) is a row of the slot
        return FixedState((self.num_heads, self.v_head_dim, self.head_dim), torch.float32)

    def _decays(self, device):
        key = str(device)
        if key not in self._decay:
            self._decay[key] = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(device)
        return self._decay[key]

    def forward(self, x, h, ctx, cache: LayerCache, owns_cache: bool):
        T = x.shape[0]
        nh, d, dv = self.num_heads, self.head_dim, self.v_head_dim
        proj = ctx.workspace.get("linear_attn_in", (T, 2 * self.qk_size + 2 * self.v_size), ctx.act_dtype)
        ops.gemm(x, self.in_weight, None, proj)
        o = ctx.workspace.get("linear_attn_out", (T, self.v_size), torch.float32)
        ops.linear_attention(proj, (0, self.qk_size, 2 * self.qk_size), o, cache.state, self._decays(o.device), ctx,
                             nh, d, dv, silu=self.activation == "silu", write_state=owns_cache,
                             rotary=None if self.position is None else self.position.table(o.device), k_scale=self.k_scale)
        y = ctx.workspace.get("linear_attn_gated", (T, self.v_size), ctx.act_dtype)
        g = proj[:, 2 * self.qk_size + self.v_size:]
        if self.head_norm or self.gate != "sigmoid":
            ops.gated_group_norm(o, g, self.norm_weight, self.norm_eps, y, dv if self.head_norm else self.v_size,
                                 gate_kind=self.gate)
        else:
            ops.gated_rmsnorm(o, g, self.norm_weight, self.norm_eps, y)
        ops.gemm(y, self.o_weight, None, h, accumulate=True)


register_part("mixer", "decayed_linear_attention", DecayedLinearAttention)
