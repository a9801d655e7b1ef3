"""Grouped-query attention over the paged cache, as a part.

  q = y Wq^T + bq, k = y Wk^T + bk, v = y Wv^T + bv       (reference.rs:251-268)
  q, k <- position encoding (rotary here)                  (reference.rs:291-297)
  k (after rotation) and v go to the cache                 (reference.rs:311-316)
  head hq reads kv head hq / (nh / nkv); s = (q . k) * scale; causal; softmax; sum w v
                                                           (kernel/cpu/attention.rs:729-781)
  h += o Wo^T                                              (reference.rs:331-337)
(paths under crates/ferrisinfer-runtime/src and crates/ferrisinfer-kernel/src).  The biases are
used iff the folder has them (crates/ferrisinfer-io/src/hf.rs:458-478); there is no output bias.

Unlike the reference, the step's keys and values are written to the cache BEFORE the
attention kernel runs, so one kernel serves whole prompts, portions and decoded tokens alike,
and q, k, v come from one fused [Q + 2 KV, H] matrix product.  ``window`` (keys the query sees,
itself included; None = all) is a parameter, as are the scale and every size.

Options beyond the reference's layer, each a parameter of its own:
  ``v_head_dim``        value heads of another size than query and key heads
  ``qk_unit_norm_eps``  q and k heads divided by their own sqrt(mean(.^2) + eps), no weight
  ``query_temperature`` (coef, every): q at position p times 1 + coef * ln(floor((p + 1) / every) + 1)
  ``tensor_names``      the folder's names of the four matrices under the prefix (then no biases are read, unless
                        ``bias_names`` names those of q, k and v)
  ``sink_name``         a learned number per head under that name: the softmax's denominator also holds its
                        exponential, a weight that belongs to no key and no value (unscaled, unbiased, counted once)
  ``values_from_keys``  there is no value matrix: a token's values are its keys as projected (before any norm or rotation)
  ``qk_norm``           {"eps", "q", "k"}: q and k each divided by sqrt(mean(.^2) + eps) over their WHOLE projection (all
                        heads at once) and multiplied by the weights named ``q`` and ``k`` under the prefix (one number
                        per element of the projection), before the rotation; with "per_head": True every head is
                        divided by the root mean square of its OWN elements instead, and the two weights hold
                        ``head_dim`` numbers that all heads share
  ``output_gate``       {"name", "kind"}: a matrix [heads x v_head_dim, H] named ``name`` under the prefix, held as further
                        rows of the fused input matrix; the heads side by side are multiplied element by element by
                        sigmoid ("sigmoid") or SiLU ("silu") of that projection of the mixer's input before the output
                        product
  ``output_scale``      a factor on the mixer's result (applied to the rows that enter the output product)
  ``chunk``             instead of a window: positions are counted off in chunks of that many from 0, and a token
                        sees the keys of its own chunk up to itself
  ``fp32_weights``      the softmax's weights and the weighted sum of values stay in 32-bit (the general kernel)
  a ``scaled_rotary`` position encoding (either pair layout, part of a head, scaled frequencies) rotates in the kernel
  that also norms and writes the cache; it goes with ``qk_norm``, ``values_from_keys``, ``chunk`` and value heads of
  their own size, not with the unit norm or the temperature
With any of these but the names the step runs product -> norm / temperature / cache write -> attention -> product;
the position encoding must then be one that rotates nothing (it may add slopes or a logarithmic distance penalty to
the scores; one with learned numbers names them under the mixer's prefix).
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, PagedKV, TensorSpec
from .plan import PartSpec, build_part, register_part


class GroupedQueryAttention(Mixer):
    accepts_lazy_norm = True  # x goes to ops.gemm and nowhere else
    can_overwrite = True

    @property
    def graph_safe(self):
        # its own work is kernels on device-resident metadata; the position encoding's ``apply`` may be anything
        return bool(getattr(self.position, "graph_safe", False))

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, window: Optional[int] = None, scale: Optional[float] = None,
                 v_head_dim: Optional[int] = None, qk_unit_norm_eps: Optional[float] = None,
                 query_temperature: Optional[tuple] = None, tensor_names: Optional[dict] = None,
                 bias_names: Optional[dict] = None, sink_name: Optional[str] = None,
                 values_from_keys: bool = False, qk_norm: Optional[dict] = None, chunk: Optional[int] = None,
                 fp32_weights: bool = False, output_gate: Optional[dict] = None, output_scale: float = 1.0):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} kv heads")
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.num_kv_heads, self.head_dim = int(num_kv_heads), int(head_dim)
        self.v_head_dim = self.head_dim if v_head_dim is None else int(v_head_dim)
        self.window = None if window is None else int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = build_part("position", position) if isinstance(position, PartSpec) else position
        self.qk_unit_norm_eps = None if qk_unit_norm_eps is None else float(qk_unit_norm_eps)
        self.query_temperature = None
        if query_temperature is not None:
            coef, every = query_temperature
            if int(every) <= 0:
                raise ValueError(f"the query temperature grows every {every} positions: a positive count is needed")
            self.query_temperature = (float(coef), int(every))
        self.values_from_keys, self.fp32_weights = bool(values_from_keys), bool(fp32_weights)
        self.chunk = None if chunk is None else int(chunk)
        if self.chunk is not None and (self.chunk <= 0 or self.window is not None):
            raise ValueError(f"a chunk of {chunk} keys (a positive count, and no window beside it)")
        if self.values_from_keys and self.v_head_dim != self.head_dim:
            raise ValueError(f"keys of {self.head_dim} cannot serve as values of {self.v_head_dim}")
        self.qk_norm = None
        if qk_norm is not None:
            self.qk_norm = (float(qk_norm["eps"]), qk_norm.get("q", "q.norm"), qk_norm.get("k", "k.norm"))
        self.qk_norm_per_head = bool(qk_norm and qk_norm.get("per_head", False))
        if self.qk_norm_per_head and self.values_from_keys:
            raise ValueError("a norm per head does not go with values taken from the keys")
        self.output_gate = None
        if output_gate is not None:
            self.output_gate = (output_gate["name"], output_gate.get("kind", "sigmoid"))
            if self.output_gate[1] not in ("sigmoid", "silu"):
                raise ValueError(f"output gate '{self.output_gate[1]}' is not known (sigmoid, silu)")
        self.output_scale = float(output_scale)
        if self.output_scale != 1.0 and self.output_gate is None:
            raise ValueError("a factor on the attention's result rides in the kernel of its output gate: it needs one")
        self.q_norm_weight = self.k_norm_weight = None
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.v_size = 0 if self.values_from_keys else self.num_kv_heads * self.v_head_dim
        self.o_size = self.num_heads * self.v_head_dim
        # the plain layer (the reference's) keeps its fused kernels; any option sends the step the general way
        self.sink_name, self.sink = sink_name, None
        # norm over the whole projection, rotation of either layout and the cache write are one kernel of their own
        self.rotary_prepare = hasattr(self.position, "table") or self.qk_norm is not None or self.values_from_keys
        if self.rotary_prepare and (self.qk_unit_norm_eps is not None or self.query_temperature is not None):
            raise ValueError("a norm over the whole projection, a scaled rotation or values taken from the keys do not "
                             "go with unit-normed heads or a query temperature")
        self.plain = (self.v_head_dim == self.head_dim and self.qk_unit_norm_eps is None
                      and self.output_gate is None and self.output_scale == 1.0
                      and self.query_temperature is None and sink_name is None and not self.rotary_prepare
                      and self.chunk is None and not self.fp32_weights
                      and not getattr(self.position, "learned_scores", False))
        if not self.plain and not hasattr(self.position, "table") and getattr(self.position, "rotary_dim", 0):
            raise ValueError("unit-norm keys, a query temperature or value heads of their own size go with a "
                             "position encoding that rotates nothing")
        self.tensor_names = dict(tensor_names) if tensor_names else None
        self.bias_names = dict(bias_names) if bias_names else None
        self.qkv_weight = self.qkv_bias = self.o_weight = None

    # ------------------------------------------------------------------ weights
    def _matrix_name(self, prefix, which):
        if self.tensor_names:
            return f"{prefix}.{self.tensor_names[which]}"
        return f"{prefix}.{which}_proj.weight"

    def tensor_specs(self, prefix):
        H, Q, KV = self.hidden_size, self.q_size, self.kv_size
        specs = [
            TensorSpec(self._matrix_name(prefix, "q"), (Q, H), "matrix"),
            TensorSpec(self._matrix_name(prefix, "k"), (KV, H), "matrix"),
        ]
        if not self.values_from_keys:
            specs.append(TensorSpec(self._matrix_name(prefix, "v"), (self.v_size, H), "matrix"))
        if self.qk_norm is not None:
            nq, nk = (self.head_dim, self.head_dim) if self.qk_norm_per_head else (Q, KV)
            specs += [TensorSpec(f"{prefix}.{self.qk_norm[1]}", (nq,), "norm"),
                      TensorSpec(f"{prefix}.{self.qk_norm[2]}", (nk,), "norm")]
        if self.output_gate is not None:
            specs.append(TensorSpec(f"{prefix}.{self.output_gate[0]}", (self.o_size, H), "matrix"))
        if self.bias_names:
            specs += [TensorSpec(f"{prefix}.{self.bias_names[n]}", (size,), "bias")
                      for n, size in zip(self._inputs, (Q, KV, self.v_size))]
        elif not self.tensor_names:
            specs += [
                TensorSpec(f"{prefix}.q_proj.bias", (Q,), "bias", required=False),
                TensorSpec(f"{prefix}.k_proj.bias", (KV,), "bias", required=False),
                TensorSpec(f"{prefix}.v_proj.bias", (self.v_size,), "bias", required=False),
            ][:len(self._inputs)]
        specs += self.position.tensor_specs(prefix)  # learned numbers of the position encoding, if it has any
        if self.sink_name:
            specs.append(TensorSpec(f"{prefix}.{self.sink_name}", (self.num_heads,), "vector"))
        return specs + [TensorSpec(self._matrix_name(prefix, "o"), (H, self.o_size), "matrix")]

    @property
    def _inputs(self) -> str:
        """The projections the folder holds, one letter each."""
        return "qk" if self.values_from_keys else "qkv"

    def bind(self, tensors, prefix):
        w = [tensors.pop(self._matrix_name(prefix, n)) for n in self._inputs]
        if self.output_gate is not None:  # the gate's projection rides in the same product
            w.append(tensors.pop(f"{prefix}.{self.output_gate[0]}"))
        self.qkv_weight = torch.cat(w, dim=0).contiguous()
        if self.bias_names:
            biases = [tensors.pop(f"{prefix}.{self.bias_names[n]}") for n in self._inputs]
        else:
            biases = [None if self.tensor_names else tensors.pop(f"{prefix}.{n}_proj.bias", None) for n in self._inputs]
        if self.qk_norm is not None:
            self.q_norm_weight = tensors[f"{prefix}.{self.qk_norm[1]}"]
            self.k_norm_weight = tensors[f"{prefix}.{self.qk_norm[2]}"]
        self.position.bind(tensors, prefix)
        if self.sink_name:
            self.sink = tensors[f"{prefix}.{self.sink_name}"]
        if any(b is not None for b in biases):
            sizes = (self.q_size, self.kv_size, self.v_size)[:len(biases)]
            if self.output_gate is not None:
                biases, sizes = biases + [None], sizes + (self.o_size,)
            parts = [
                b if b is not None else torch.zeros(n, dtype=torch.float32, device=self.qkv_weight.device)
                for b, n in zip(biases, sizes)
            ]
            self.qkv_bias = torch.cat(parts).contiguous()
        else:
            self.qkv_bias = None
        self.o_weight = tensors[self._matrix_name(prefix, "o")]

    # -------------------------------------------------------------------- cache
    def cache_need(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.window,
                       None if self.v_head_dim == self.head_dim else self.v_head_dim, chunk=self.chunk)

    # ------------------------------------------------------------------ forward
    def forward(self, x, h, ctx, cache: LayerCache, owns_cache: bool, accumulate: bool = True):
        T = x.shape[0]
        nh, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        meta = ctx.paged[cache.group]
        n_qkv = self.q_size + self.kv_size + self.v_size
        qkv = ctx.workspace.get("attn_qkv", (T, self.qkv_weight.shape[0]), x.dtype)
        if not self.plain:
            dv = self.v_head_dim
            ops.gemm(x, self.qkv_weight, self.qkv_bias, qkv)
            gate = None
            if self.output_gate is not None:
                qkv, gate = qkv[:, :n_qkv], qkv[:, n_qkv:]
            if self.rotary_prepare:
                rotary = self.position.table(qkv.device) if hasattr(self.position, "table") else None
                ops.qk_norm_rotary_cache_write(qkv, ctx, meta.slot_mapping, cache.k, cache.v, nh, nkv, d, dv,
                                               self.q_norm_weight, self.k_norm_weight,
                                               self.qk_norm[0] if self.qk_norm else 0.0, rotary,
                                               values_from_keys=self.values_from_keys, write_kv=owns_cache,
                                               per_head=self.qk_norm_per_head)
            else:
                ops.qk_prepare_cache_write(qkv, ctx.positions, meta.slot_mapping, cache.k, cache.v, nh, nkv, d, dv,
                                           self.qk_unit_norm_eps, self.query_temperature, write_kv=owns_cache)
            out = ctx.workspace.get("attn_out", (T, self.o_size), x.dtype)
            log = self.position.score_log_penalty(nh, qkv.device)
            terms = ops.ScoreTerms(slopes=self.position.score_slopes(nh, qkv.device), sink=self.sink,
                                   log_r1=None if log is None else log[0], log_r2=None if log is None else log[1])
            ops.paged_attention(qkv, out, cache.k, cache.v, meta.block_tables, ctx, nh, nkv, d, self.window or 0,
                                self.scale, score_slopes=terms, v_head_dim=dv, chunk=self.chunk or 0,
                                fp32_weights=self.fp32_weights)
            if gate is not None:
                ops.gate_mul(out, gate, out, self.output_gate[1], self.output_scale)
            ops.gemm(out, self.o_weight, None, h, accumulate=accumulate)
            return
        table = self.position.rotary_table(qkv.device)
        inv_freq, rotary = table if table is not None else (None, 0)
        slopes = self.position.score_slopes(nh, qkv.device)
        # a long step of prompt portions: rotation and cache write ride in the product's epilogue
        fused = False
        if (inv_freq is not None and ctx.max_q_len > 1 and T >= ops.QKV_ROPE_MIN_TOKENS
                and hasattr(self.position, "angles")):
            x = x.materialize() if hasattr(x, "materialize") else x
            fused = ops.qkv_rope_gemm_takes(x, self.qkv_weight, qkv, nh, nkv, d, rotary, cache.k)
        if fused:
            ops.qkv_rope_gemm(x, self.qkv_weight, self.qkv_bias, qkv, self.position.angles(ctx),
                              meta.slot_mapping if owns_cache else None, cache.k, cache.v, nh, nkv, d)
        else:
            ops.gemm(x, self.qkv_weight, self.qkv_bias, qkv)
            if table is None:
                self.position.apply(qkv, ctx.positions, nh, nkv, d)
        out = ctx.workspace.get("attn_out", (T, self.q_size), x.dtype)
        attended = ops.attention_step(qkv, out, cache.k, cache.v, meta, ctx, nh, nkv, d, inv_freq, rotary,
                                      self.window or 0, self.scale, write_kv=owns_cache, lazy_merge=True,
                                      rotated=fused, score_slopes=slopes)
        ops.gemm(attended, self.o_weight, None, h, accumulate=accumulate)


register_part("mixer", "gqa_attention", GroupedQueryAttention)
