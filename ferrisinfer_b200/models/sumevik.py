"""The Sumevik decoder as a plan.

A plain token embedding whose table is also the output matrix; pre-norm residual layers whose RMS norms store their
weight around zero (the row is multiplied by 1 + w); two kinds of mixer, chosen per layer by the configuration: a
recurrent block with a gated linear recurrent unit over channels (a GELU branch beside a short convolution and
block-diagonal gates), and two mixers side by side that read the same input and whose results are added with a factor
each, a grouped-query softmax attention (biases, a norm per head on queries and keys, part of every head rotated in
neighbouring pairs, a token seeing the keys of its own chunk of positions, a sigmoid gate on the heads' outputs)
beside a gated linear attention whose decay per key channel is set by every token; a feed-forward that is either a
gated one with the tanh form of GELU or a mixture of experts (scores by a softmax over all router outputs, a learned
correction that only steers the choice, groups of experts of which the best stay, identity experts without tensors,
a clamped gate); the norm once more and logits through the embedding table times a factor.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sumevik import SumevikConfig, SumevikDense
from ..parts.plan import LayerPlan, ModelPlan, PartSpec, RunStep

MAX_POSITIONS = 1 << 20  # the design sets no limit; the step function wants one
DECAY_FACTOR = 8.0  # log a = -8 r softplus(lam) in the recurrent unit


def _recurrent(m, width: int) -> PartSpec:
    return PartSpec("gated_linear_unit", {"hidden_size": width, "width": m.width, "blocks": m.blocks, "conv_taps": m.conv,
                                          "decay_factor": DECAY_FACTOR, "activation": "gelu_tanh"})


def _side_by_side(m, width: int, eps: float) -> PartSpec:
    a, g = m.left, m.right
    rotation = PartSpec("none")
    if a.rot_dims:
        # neighbouring elements rotate together
        rotation = PartSpec("scaled_rotary", {"rotary_dim": a.rot_dims, "base": a.rot_base, "layout": "interleaved",
                                              "scaling": None})
    attention = PartSpec("gqa_attention", {
        "hidden_size": width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
        "scale": a.scale, "chunk": a.chunk, "position": rotation,
        "qk_norm": {"eps": eps, "q": "q.norm", "k": "k.norm", "per_head": True}, "fp32_weights": True,
        "tensor_names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "bias_names": {"q": "q.b", "k": "k.b", "v": "v.b"},
        "output_gate": {"name": "g", "kind": "sigmoid"}, "output_scale": m.left_scale})
    linear = PartSpec("gated_linear_attention", {
        "hidden_size": width, "num_heads": g.heads, "head_dim": g.dim, "v_head_dim": g.vdim, "tau": g.tau,
        # the inner size of the decay's projection stands in no configuration key: the tensors' shapes give it
        "decay_rank": None, "norm_eps": eps, "output_scale": m.right_scale})
    return PartSpec("parallel_mixers", {"hidden_size": width, "norm": False, "branches": {"left": attention, "right": linear}})


def _feed_forward(mlp, width: int):
    if mlp is None:
        return None
    if isinstance(mlp, SumevikDense):
        return PartSpec("gated", {"hidden_size": width, "intermediate_size": mlp.ff, "activation": "gelu_tanh"})
    return PartSpec("mixture_of_experts", {
        "hidden_size": width, "intermediate_size": mlp.ff, "experts": mlp.experts, "top": mlp.top, "identity": mlp.identity,
        "scored": {"correction": "correction", "groups": mlp.group_count, "keep": mlp.group_keep},
        "activation": "clamped_swish", "limit": mlp.limit})


def plan_sumevik(cfg: SumevikConfig) -> ModelPlan:
    cfg.validate()
    W = cfg.width
    norm = PartSpec("grouped_rmsnorm", {"hidden_size": W, "eps": cfg.norm_eps, "groups": 1, "weight_name": "",
                                        "unit_offset": True})
    layers = []
    for i, layer in enumerate(cfg.layers):
        if layer.type == "rglru":
            mixer = _recurrent(layer.mixer, W)
        else:
            mixer = _side_by_side(layer.mixer, W, cfg.norm_eps)
        layers.append(LayerPlan(prefix=f"l{i}", mixer=mixer, feed_forward=_feed_forward(layer.mlp, W), mixer_norm=norm,
                                feed_forward_norm=norm,
                                block=PartSpec("pre_norm_residual", {
                                    "mixer_prefix": "mix", "feed_forward_prefix": "mlp", "mixer_norm_prefix": "norm1",
                                    "feed_forward_norm_prefix": "norm2"})))
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "weight_name": ""}),
        embedding_prefix="embed",
        layers=tuple(layers),
        run_order=tuple(RunStep(i) for i in range(len(layers))),
        final_norm=norm,
        final_norm_prefix="final.norm",
        output=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied_to": "embed",
                                        "logit_scale": cfg.logit_scale}),
        output_prefix="head",
        max_positions=MAX_POSITIONS,
    )


register_architecture("Sumevik", SumevikConfig, plan_sumevik, replace=True)
