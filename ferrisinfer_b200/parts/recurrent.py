"""Mixers that keep a state of fixed size per request and a decay that changes from token to token.

``GatedDeltaRule``:
  q, k (qk_heads x dim) and v (heads x vdim) = SiLU(conv(y W^T)), a short causal convolution per channel; q and k are
  made unit vectors per head (1 / sqrt(sum x^2 + 1e-6)), q also times dim^(-1/2); per value head (which reads q/k head
  h / (heads / qk_heads)): beta = sigmoid(y Wb^T), g = exp(-exp(A_log) softplus(y Wa^T + dt_bias));
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q          (the read-out sees the token's own write)
  h += (rmsnorm_per_head(o) * n * SiLU(y Wg^T)) Wo^T,   n of size vdim, shared by the heads.

``StateSpaceDuality`` (a selective state-space layer in its attention-like reading):
  y W_in^T = [z: inner | x: inner | B: groups x N | C: groups x N | dt: heads], inner = heads x vdim;
  x, B, C = SiLU(conv(.) + bias);  dt = softplus(dt + dt_bias);  per head (group h / (heads / groups)):
    S <- exp(-exp(A_log) dt) S + dt B x^T;  o = S^T C + D x
  h += (rmsnorm_in_groups(o * SiLU(z)) * n) Wo^T       the gate before the norm, ``norm_groups`` equal parts.

``GatedLinearUnit`` (a recurrent block in the manner of Griffin: a linear recurrence per channel whose two gates are real numbers):
  b = a(y Wy^T + by), a the tanh form of GELU;  u = conv(y Wx^T + bx) + cb, a short causal convolution per channel, no
  activation;  per block n of the C channels (C / blocks neighbours): r = sigmoid(Ra[n] u_n + ra), i = sigmoid(Ri[n] u_n + ri);
    log a = -decay_factor r softplus(lam);  s_t = exp(log a) s_(t-1) + sqrt(1 - exp(2 log a)) i u_t
  h += (s_t * b) Wo^T.   State: s [C] fp32 and the convolution's last taps - 1 inputs.

``GatedLinearAttention`` (linear attention with a decay per key channel that the token sets):
  q = y Wq^T dim^(-1/2), k = y Wk^T, v = y Wv^T;  alpha = sigmoid((y Wa1^T) Wa2^T + ba2)^(1 / tau), heads x dim;
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t         per head
  h += scale (rmsnorm_per_head(o) * n * SiLU(y Wg^T)) Wo^T,   n of size vdim, shared by the heads.

All hold their input matrices as one, so that one product feeds the convolution, the gates and the recurrence; the
state (S transposed, [heads, vdim, dim] fp32) and the convolution's last taps - 1 inputs are carried in the request's slot, so a
sequence may be cut anywhere.  Decays, step sizes, unit norms, the recurrence and the norms are fp32 whatever the
activations' type.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import CombinedNeed, FixedState, LayerCache, Mixer, TensorSpec
from .plan import register_part


def _fused_rows(parts: list) -> torch.Tensor:
    """The matrices one below the other, with zero rows added up to a multiple of eight (rows of the product's
    output then start on 16 bytes in either type)."""
    w = torch.cat(parts, dim=0)
    pad = (-w.shape[0]) % 8
    if pad:
        w = torch.cat([w, torch.zeros(pad, w.shape[1], dtype=w.dtype, device=w.device)], dim=0)
    return w.contiguous()


class GatedDeltaRule(Mixer):
    accepts_lazy_norm = True
    graph_safe = True
    can_overwrite = True

    def __init__(self, hidden_size: int, num_heads: int, num_qk_heads: int, head_dim: int, v_head_dim: int,
                 conv_taps: int, norm_eps: float, unit_norm_eps: float = 1e-6):
        if num_heads % num_qk_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_qk_heads} q/k heads")
        if head_dim > 256:
            raise ValueError(f"heads of {head_dim} are larger than the recurrence kernel takes (256)")
        self.hidden_size, self.num_heads, self.num_qk_heads = int(hidden_size), int(num_heads), int(num_qk_heads)
        self.head_dim, self.v_head_dim, self.taps = int(head_dim), int(v_head_dim), int(conv_taps)
        self.norm_eps, self.unit_norm_eps = float(norm_eps), float(unit_norm_eps)
        self.qk_size = self.num_qk_heads * self.head_dim
        self.v_size = self.num_heads * self.v_head_dim
        self.conv_size = 2 * self.qk_size + self.v_size

    def tensor_specs(self, prefix):
        H, nh = self.hidden_size, self.num_heads
        return [
            TensorSpec(f"{prefix}.q", (self.qk_size, H), "matrix"),
            TensorSpec(f"{prefix}.q.conv", (self.qk_size, self.taps), "vector"),
            TensorSpec(f"{prefix}.k", (self.qk_size, H), "matrix"),
            TensorSpec(f"{prefix}.k.conv", (self.qk_size, self.taps), "vector"),
            TensorSpec(f"{prefix}.v", (self.v_size, H), "matrix"),
            TensorSpec(f"{prefix}.v.conv", (self.v_size, self.taps), "vector"),
            TensorSpec(f"{prefix}.b", (nh, H), "matrix"),
            TensorSpec(f"{prefix}.A_log", (nh,), "vector"),
            TensorSpec(f"{prefix}.norm", (self.v_head_dim,), "norm"),
            TensorSpec(f"{prefix}.a", (nh, H), "matrix"),
            TensorSpec(f"{prefix}.dt_bias", (nh,), "vector"),
            TensorSpec(f"{prefix}.g", (self.v_size, H), "matrix"),
            TensorSpec(f"{prefix}.o", (H, self.v_size), "matrix"),
        ]

    def bind(self, tensors, prefix):
        # one product: [q | k | v | gate | b | a]
        self.in_weight = _fused_rows([tensors.pop(f"{prefix}.{n}") for n in ("q", "k", "v", "g", "b", "a")])
        self.conv_weight = torch.cat([tensors.pop(f"{prefix}.{n}.conv") for n in "qkv"], dim=0).contiguous()
        self.A_log, self.dt_bias = tensors[f"{prefix}.A_log"], tensors[f"{prefix}.dt_bias"]
        self.norm_weight, self.o_weight = tensors[f"{prefix}.norm"], tensors[f"{prefix}.o"]

    def cache_need(self):
        history = FixedState((self.taps - 1, self.conv_size), torch.float32) if self.taps > 1 else None
        return CombinedNeed((history, FixedState((self.num_heads, self.v_head_dim, self.head_dim), torch.float32)))

    def forward(self, x, h, ctx, cache: LayerCache, owns_cache: bool, accumulate: bool = True):
        T = x.shape[0]
        nh, g, d, dv = self.num_heads, self.num_qk_heads, self.head_dim, self.v_head_dim
        QK, V, C = self.qk_size, self.v_size, self.conv_size
        history, state = cache.parts
        ws = ctx.workspace
        proj = ws.get("recurrent_in", (T, self.in_weight.shape[0]), ctx.act_dtype)
        ops.gemm(x, self.in_weight, None, proj)
        conv = ws.get("recurrent_conv", (T, C), ctx.act_dtype)
        ops.short_conv(proj[:, :C], conv, self.conv_weight, None if history is None else history.state, ctx,
                       advance=owns_cache, residual=False, silu=True)
        decay, beta = ws.get("recurrent_decay", (T, nh), torch.float32), ws.get("recurrent_beta", (T, nh), torch.float32)
        qscale, kscale = ws.get("recurrent_qscale", (T, g), torch.float32), ws.get("recurrent_kscale", (T, g), torch.float32)
        ops.recurrence_gates(proj, C + V + nh, C + V, self.A_log, self.dt_bias, decay, beta, nh,
                             unit_norm=(conv, 0, QK, g, d, self.unit_norm_eps, d ** -0.5, qscale, kscale))
        o = ws.get("recurrent_out", (T, V), torch.float32)
        ops.gated_recurrence(conv[:, :QK], conv[:, QK:2 * QK], conv[:, 2 * QK:], decay, beta, o, state.state, ctx, nh, g, d, dv,
                             delta_rule=True, qscale=qscale, kscale=kscale, write_state=owns_cache)
        y = ws.get("recurrent_gated", (T, V), ctx.act_dtype)
        ops.gated_group_norm(o, proj[:, C:C + V], self.norm_weight, self.norm_eps, y, group=dv, gate_kind="silu")
        ops.gemm(y, self.o_weight, None, h, accumulate=accumulate)


class StateSpaceDuality(Mixer):
    accepts_lazy_norm = True
    graph_safe = True
    can_overwrite = True

    def __init__(self, hidden_size: int, num_heads: int, v_head_dim: int, state_size: int, groups: int, norm_groups: int,
                 conv_taps: int, norm_eps: float):
        if num_heads % groups:
            raise ValueError(f"{num_heads} heads cannot share {groups} groups")
        if (num_heads * v_head_dim) % norm_groups:
            raise ValueError(f"{num_heads * v_head_dim} columns cannot be normed in {norm_groups} equal parts")
        if state_size > 256:
            raise ValueError(f"a state of {state_size} rows is larger than the recurrence kernel takes (256)")
        self.hidden_size, self.num_heads, self.v_head_dim = int(hidden_size), int(num_heads), int(v_head_dim)
        self.state_size, self.groups, self.norm_groups = int(state_size), int(groups), int(norm_groups)
        self.taps, self.norm_eps = int(conv_taps), float(norm_eps)
        self.inner = self.num_heads * self.v_head_dim
        self.bc_size = self.groups * self.state_size
        self.conv_size = self.inner + 2 * self.bc_size

    def tensor_specs(self, prefix):
        H, nh = self.hidden_size, self.num_heads
        return [
            TensorSpec(f"{prefix}.in", (2 * self.inner + 2 * self.bc_size + nh, H), "matrix"),
            TensorSpec(f"{prefix}.conv", (self.conv_size, self.taps), "vector"),
            TensorSpec(f"{prefix}.conv.b", (self.conv_size,), "bias"),
            TensorSpec(f"{prefix}.dt_bias", (nh,), "vector"),
            TensorSpec(f"{prefix}.A_log", (nh,), "vector"),
            TensorSpec(f"{prefix}.D", (nh,), "vector"),
            TensorSpec(f"{prefix}.norm", (self.inner,), "norm"),
            TensorSpec(f"{prefix}.o", (H, self.inner), "matrix"),
        ]

    def bind(self, tensors, prefix):
        self.in_weight = _fused_rows([tensors.pop(f"{prefix}.in")])
        self.conv_weight, self.conv_bias = tensors[f"{prefix}.conv"], tensors[f"{prefix}.conv.b"]
        self.dt_bias, self.A_log, self.skip = tensors[f"{prefix}.dt_bias"], tensors[f"{prefix}.A_log"], tensors[f"{prefix}.D"]
        self.norm_weight, self.o_weight = tensors[f"{prefix}.norm"], tensors[f"{prefix}.o"]

    def cache_need(self):
        history = FixedState((self.taps - 1, self.conv_size), torch.float32) if self.taps > 1 else None
        return CombinedNeed((history, FixedState((self.num_heads, self.v_head_dim, self.state_size), torch.float32)))

    def forward(self, x, h, ctx, cache: LayerCache, owns_cache: bool, accumulate: bool = True):
        T = x.shape[0]
        nh, dv, N, G = self.num_heads, self.v_head_dim, self.state_size, self.groups
        inner, BC, C = self.inner, self.bc_size, self.conv_size
        history, state = cache.parts
        ws = ctx.workspace
        proj = ws.get("recurrent_in", (T, self.in_weight.shape[0]), ctx.act_dtype)
        ops.gemm(x, self.in_weight, None, proj)
        conv = ws.get("recurrent_conv", (T, C), ctx.act_dtype)
        ops.short_conv(proj[:, inner:inner + C], conv, self.conv_weight, None if history is None else history.state, ctx,
                       advance=owns_cache, bias=self.conv_bias, residual=False, silu=True)
        decay, step = ws.get("recurrent_decay", (T, nh), torch.float32), ws.get("recurrent_beta", (T, nh), torch.float32)
        ops.recurrence_gates(proj, inner + C, None, self.A_log, self.dt_bias, decay, step, nh)
        o = ws.get("recurrent_out", (T, inner), torch.float32)
        # q = C, k = B, v = x; the step size multiplies the write
        ops.gated_recurrence(conv[:, inner + BC:], conv[:, inner:inner + BC], conv[:, :inner], decay, step, o, state.state, ctx,
                             nh, G, N, dv, delta_rule=False, skip=self.skip, write_state=owns_cache)
        y = ws.get("recurrent_gated", (T, inner), ctx.act_dtype)
        ops.gated_group_norm(o, proj[:, :inner], self.norm_weight, self.norm_eps, y, group=inner // self.norm_groups,
                             gate_kind="silu", gate_first=True)
        ops.gemm(y, self.o_weight, None, h, accumulate=accumulate)


class GatedLinearUnit(Mixer):
    accepts_lazy_norm = True
    graph_safe = True
    can_overwrite = True

    def __init__(self, hidden_size: int, width: int, blocks: int, conv_taps: int, decay_factor: float = 8.0,
                 activation: str = "gelu_tanh", tensor_names: dict = None):
        if width <= 0 or blocks <= 0 or width % blocks:
            raise ValueError(f"{width} channels cannot stand in {blocks} equal blocks")
        if conv_taps < 1:
            raise ValueError(f"a convolution of {conv_taps} taps")
        if activation not in ("gelu_tanh", "none"):
            raise ValueError(f"activation '{activation}' of the gate branch is not known (gelu_tanh, none)")
        self.hidden_size, self.width, self.blocks, self.taps = int(hidden_size), int(width), int(blocks), int(conv_taps)
        self.decay_factor, self.activation = float(decay_factor), activation
        self.names = {"y": "y", "x": "x", "conv": "conv", "ra": "ra", "ri": "ri", "lam": "lam", "o": "o"}
        self.names.update(tensor_names or {})

    def tensor_specs(self, prefix):
        H, C, n, bs = self.hidden_size, self.width, self.names, self.width // self.blocks
        return [
            TensorSpec(f"{prefix}.{n['y']}", (C, H), "matrix"), TensorSpec(f"{prefix}.{n['y']}.b", (C,), "bias"),
            TensorSpec(f"{prefix}.{n['x']}", (C, H), "matrix"), TensorSpec(f"{prefix}.{n['x']}.b", (C,), "bias"),
            TensorSpec(f"{prefix}.{n['conv']}", (C, self.taps), "vector"), TensorSpec(f"{prefix}.{n['conv']}.b", (C,), "bias"),
            TensorSpec(f"{prefix}.{n['ra']}", (self.blocks, bs, bs), "matrix"),
            TensorSpec(f"{prefix}.{n['ra']}.b", (self.blocks, bs), "bias"),
            TensorSpec(f"{prefix}.{n['ri']}", (self.blocks, bs, bs), "matrix"),
            TensorSpec(f"{prefix}.{n['ri']}.b", (self.blocks, bs), "bias"),
            TensorSpec(f"{prefix}.{n['lam']}", (C,), "vector"),
            TensorSpec(f"{prefix}.{n['o']}", (H, C), "matrix"),
        ]

    def bind(self, tensors, prefix):
        n = self.names
        # one product: [gate branch | recurrent branch]
        self.in_weight = _fused_rows([tensors.pop(f"{prefix}.{n['y']}"), tensors.pop(f"{prefix}.{n['x']}")])
        bias = torch.cat([tensors[f"{prefix}.{n['y']}.b"], tensors[f"{prefix}.{n['x']}.b"]])
        pad = self.in_weight.shape[0] - bias.numel()
        self.in_bias = torch.cat([bias, bias.new_zeros(pad)]).contiguous() if pad else bias.contiguous()
        self.conv_weight, self.conv_bias = tensors[f"{prefix}.{n['conv']}"], tensors[f"{prefix}.{n['conv']}.b"]
        # the gates' matrices transposed ([block, in, out]): the threads of the gates kernel read consecutive weights
        # (and as they are stored, for the tensor-core form of long bf16 steps, whose B operand that layout is)
        self.ra, self.ri = tensors.pop(f"{prefix}.{n['ra']}").contiguous(), tensors.pop(f"{prefix}.{n['ri']}").contiguous()
        self.ra_t, self.ri_t = self.ra.transpose(1, 2).contiguous(), self.ri.transpose(1, 2).contiguous()
        self.ra_bias = tensors[f"{prefix}.{n['ra']}.b"].reshape(-1).contiguous()
        self.ri_bias = tensors[f"{prefix}.{n['ri']}.b"].reshape(-1).contiguous()
        # softplus of the decay's parameter, formed once in 64-bit and rounded once
        lam = tensors[f"{prefix}.{n['lam']}"]
        self.rate = torch.nn.functional.softplus(lam.to(torch.float64)).to(torch.float32).contiguous()
        self.o_weight = tensors[f"{prefix}.{n['o']}"]

    def cache_need(self):
        history = FixedState((self.taps - 1, self.width), torch.float32) if self.taps > 1 else None
        return CombinedNeed((history, FixedState((self.width,), torch.float32)))

    def forward(self, x, h, ctx, cache: LayerCache, owns_cache: bool, accumulate: bool = True):
        T, C = x.shape[0], self.width
        history, state = cache.parts
        ws = ctx.workspace
        proj = ws.get("recurrent_in", (T, self.in_weight.shape[0]), ctx.act_dtype)
        ops.gemm(x, self.in_weight, self.in_bias, proj)
        u = ws.get("recurrent_conv", (T, C), ctx.act_dtype)
        ops.short_conv(proj[:, C:2 * C], u, self.conv_weight, None if history is None else history.state, ctx,
                       advance=owns_cache, bias=self.conv_bias, residual=False, silu=False)
        y = ws.get("recurrent_gated", (T, C), ctx.act_dtype)
        gelu = self.activation == "gelu_tanh"
        if ctx.max_q_len == 1 and T == ctx.num_seqs:  # single tokens: the gates kernel moves the state on itself
            ops.rglru_gates(u, self.ra_t, self.ri_t, self.ra_bias, self.ri_bias, self.rate, None, None, self.decay_factor,
                            step=(state.state, ctx, proj[:, :C], y, gelu, owns_cache))
        else:
            a, b = ws.get("recurrent_unit_a", (T, C), torch.float32), ws.get("recurrent_unit_b", (T, C), torch.float32)
            ops.rglru_gates(u, self.ra_t, self.ri_t, self.ra_bias, self.ri_bias, self.rate, a, b, self.decay_factor,
                            stored=(self.ra, self.ri))
            ops.rglru_scan(a, b, proj[:, :C], y, state.state, ctx, gelu=gelu, write_state=owns_cache)
        ops.gemm(y, self.o_weight, None, h, accumulate=accumulate)


class GatedLinearAttention(Mixer):
    accepts_lazy_norm = True
    graph_safe = True
    can_overwrite = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, tau: float, norm_eps: float,
                 decay_rank: int = None, output_scale: float = 1.0, tensor_names: dict = None):
        """``decay_rank``: inner size of the decay's low-rank projection; None = whatever the folder's tensors have (a
        random folder then draws 16)."""
        if head_dim > 256:
            raise ValueError(f"heads of {head_dim} are larger than the recurrence kernel takes (256)")
        if not (tau > 0.0):
            raise ValueError(f"a decay root of {tau}: a positive number is needed")
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.decay_rank = None if decay_rank is None else int(decay_rank)
        self.tau, self.norm_eps, self.output_scale = float(tau), float(norm_eps), float(output_scale)
        self.qk_size, self.v_size = self.num_heads * self.head_dim, self.num_heads * self.v_head_dim
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2"}
        self.names.update(tensor_names or {})

    def tensor_specs(self, prefix):
        H, n = self.hidden_size, self.names
        rank = -16 if self.decay_rank is None else self.decay_rank  # negative: the folder decides
        return [
            TensorSpec(f"{prefix}.{n['q']}", (self.qk_size, H), "matrix"),
            TensorSpec(f"{prefix}.{n['k']}", (self.qk_size, H), "matrix"),
            TensorSpec(f"{prefix}.{n['v']}", (self.v_size, H), "matrix"),
            TensorSpec(f"{prefix}.{n['g']}", (self.v_size, H), "matrix"),
            TensorSpec(f"{prefix}.{n['o']}", (H, self.v_size), "matrix"),
            TensorSpec(f"{prefix}.{n['norm']}", (self.v_head_dim,), "norm"),
            TensorSpec(f"{prefix}.{n['a1']}", (rank, H), "matrix"),
            TensorSpec(f"{prefix}.{n['a2']}", (self.qk_size, rank), "matrix"),
            TensorSpec(f"{prefix}.{n['a2']}.b", (self.qk_size,), "bias"),
        ]

    def bind(self, tensors, prefix):
        n = self.names
        # one product: [q | k | v | gate | the decay's low-rank input], every part starting on a multiple of eight columns
        a1, a2 = tensors.pop(f"{prefix}.{n['a1']}"), tensors.pop(f"{prefix}.{n['a2']}")
        if a1.shape[0] != a2.shape[1]:
            raise ValueError(f"{prefix}: the decay's two matrices do not meet ({tuple(a1.shape)} and {tuple(a2.shape)})")
        self.decay_rank = int(a1.shape[0])
        self.rank_cols = (self.decay_rank + 7) // 8 * 8
        if self.rank_cols != self.decay_rank:
            a1 = torch.cat([a1, a1.new_zeros(self.rank_cols - self.decay_rank, a1.shape[1])], dim=0)
        self.in_weight = _fused_rows([tensors.pop(f"{prefix}.{n[w]}") for w in "qkvg"] + [a1])
        self.a_off = 2 * self.qk_size + 2 * self.v_size
        if self.rank_cols != self.decay_rank:  # zero columns meet the zero rows that fill the input matrix up
            a2 = torch.cat([a2, a2.new_zeros(a2.shape[0], self.rank_cols - self.decay_rank)], dim=1)
        self.a2_weight, self.a2_bias = a2.contiguous(), tensors[f"{prefix}.{n['a2']}.b"]
        # the factor on the mixer's result rides in the norm's weight (fp32)
        self.norm_weight = (tensors[f"{prefix}.{n['norm']}"].to(torch.float32) * self.output_scale).contiguous()
        self.o_weight = tensors[f"{prefix}.{n['o']}"]

    def cache_need(self):
        # transposed: a column of S (one value dim) is a row of the slot
        return FixedState((self.num_heads, self.v_head_dim, self.head_dim), torch.float32)

    def forward(self, x, h, ctx, cache: LayerCache, owns_cache: bool, accumulate: bool = True):
        T = x.shape[0]
        nh, d, dv, QK, V = self.num_heads, self.head_dim, self.v_head_dim, self.qk_size, self.v_size
        ws = ctx.workspace
        proj = ws.get("linear_attn_in", (T, self.in_weight.shape[0]), ctx.act_dtype)
        ops.gemm(x, self.in_weight, None, proj)
        z = ws.get("linear_attn_decay", (T, QK), torch.float32)
        ops.gemm(proj[:, self.a_off:self.a_off + self.rank_cols], self.a2_weight, self.a2_bias, z)
        o = ws.get("linear_attn_out", (T, V), torch.float32)
        ops.row_decay_recurrence(proj[:, :QK], proj[:, QK:2 * QK], proj[:, 2 * QK:2 * QK + V], z, 1.0 / self.tau, o,
                                 cache.state, ctx, nh, d, dv, q_scale=d ** -0.5, write_state=owns_cache)
        y = ws.get("linear_attn_gated", (T, V), ctx.act_dtype)
        ops.gated_group_norm(o, proj[:, 2 * QK + V:2 * QK + 2 * V], self.norm_weight, self.norm_eps, y, group=dv,
                             gate_kind="silu")
        ops.gemm(y, self.o_weight, None, h, accumulate=accumulate)


register_part("mixer", "gated_linear_unit", GatedLinearUnit)
register_part("mixer", "gated_linear_attention", GatedLinearAttention)
register_part("mixer", "gated_delta_rule", GatedDeltaRule)
register_part("mixer", "state_space_duality", StateSpaceDuality)
