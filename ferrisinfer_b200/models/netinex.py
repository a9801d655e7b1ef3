"""The Netinex decoder as a plan.

A plain token embedding whose table is also the output matrix; pre-norm residual layers whose norm is a dynamic tanh
(no statistics: tanh(alpha x) w + b); two kinds of mixer, chosen per layer by the configuration: a retention (linear
attention with a fixed decay per head, rotated queries and keys, every head's output divided by its own root mean
square and gated by a SiLU branch) and a grouped-query attention whose queries and keys are RMS-normed over their
whole projection and rotated with scaled frequencies, whose values are the keys as projected, and in which a token
sees the keys of its own chunk of positions only; a mixture of gated SiLU experts as the feed-forward; the dynamic
tanh once more and soft-capped logits at the end.

Tensor names: ``embed``, ``l<i>.norm1[.alpha|.b]``, ``l<i>.norm2[.alpha|.b]``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm[.alpha|.b]``.
"""

from __future__ import annotations

from ..config.netinex import NetinexConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerPlan, ModelPlan, PartSpec, RunStep

MAX_POSITIONS = 1 << 20  # the design sets no limit; the step function wants one


def _rotation(rot, layout: str):
    if rot is None or rot.dims == 0:
        return None
    return PartSpec("scaled_rotary", {"rotary_dim": rot.dims, "base": rot.base, "layout": layout,
                                      "scaling": rot.scaling_dict()})


def plan_netinex(cfg: NetinexConfig) -> ModelPlan:
    cfg.validate()
    W = cfg.width
    norm = PartSpec("dynamic_tanh", {"hidden_size": W, "eps": cfg.norm_eps, "weight_name": ""})
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if m.type == "attention":
            # pairs of neighbouring elements rotate together here
            rotation = _rotation(m.rot, "interleaved")
            mixer = PartSpec("gqa_attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "v_head_dim": m.vdim, "scale": m.scale, "chunk": m.chunk,
                "position": rotation if rotation is not None else PartSpec("none"),
                "values_from_keys": True, "qk_norm": {"eps": cfg.norm_eps, "q": "q.norm", "k": "k.norm"},
                "fp32_weights": True, "tensor_names": {"q": "q", "k": "k", "o": "o"},
            })
        else:
            # element i rotates with element i + dims / 2; the keys are divided by sqrt(dim) after the rotation
            mixer = PartSpec("decayed_linear_attention", {
                "hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim, "decay": m.decay,
                "norm_eps": cfg.norm_eps, "activation": "none", "position": _rotation(m.rot, "half"),
                "k_scale": m.dim ** -0.5, "head_norm": True, "gate": "silu",
            })
        ff = None if layer.mlp is None else PartSpec("mixture_of_experts", {
            "hidden_size": W, "intermediate_size": layer.mlp.ff, "experts": layer.mlp.experts, "top": layer.mlp.top})
        layers.append(LayerPlan(prefix=f"l{i}", mixer=mixer, feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm,
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
                                        "softcap": cfg.logit_softcap}),
        output_prefix="head",
        max_positions=MAX_POSITIONS,
    )


register_architecture("Netinex", NetinexConfig, plan_netinex, replace=True)
