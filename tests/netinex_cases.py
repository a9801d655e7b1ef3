"""Small Netinex configurations and weights for the tests, and how a step function's logits are compared with the
plain implementation (``plain_netinex``).

The weights are not N(0, 0.02): projections are drawn with a standard deviation of 1 / sqrt(inputs), norm weights
around one, the dynamic tanh's alpha between 0.5 and 1.5, router matrices so that the experts' logits spread over a few
units, so that every mechanism moves the logits by far more than a tolerance (queries and keys are normed by the
design, so attention scores spread over several units whatever the projections' scale).

Sequences are drawn token by token so that no router's choice is a close call anywhere (``safe_sequence``): in
bfloat16 the router sees rounded inputs, and a choice that a rounding can turn is no fault of the engine.
"""

from __future__ import annotations

import math
import random

import torch

import plain_netinex as plain


def rotation(dims, base=10000.0, scaling=None):
    d = {"dims": dims, "base": base}
    if scaling is not None:
        factor, original, fast, slow = scaling
        d["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return d


def experts(ff, n, top):
    return None if ff is None else {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": n, "top": top}}


def retention_layer(heads, dim, vdim, mlp, rot="full", decay=None, seed=0):
    rng = random.Random(seed)
    mixer = {"heads": heads, "dim": dim, "vdim": vdim,
             "decay": decay or [round(rng.uniform(0.6, 0.999), 4) for _ in range(heads)]}
    if rot is not None:
        mixer["rot"] = rotation(dim, 10000.0) if rot == "full" else rot
    return {"type": "retention", "mixer": mixer, "mlp": mlp}


def attention_layer(heads, kv_heads, dim, chunk, mlp, rot="full", scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
             "scale": scale if scale is not None else 2.0 / math.sqrt(dim)}
    if chunk is not None:
        mixer["mask"] = {"size": chunk}
    if rot is not None:
        mixer["rot"] = rotation(dim, 10000.0, (4.0, 64, 8.0, 2.0)) if rot == "full" else rot
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def config(layers, width=64, vocab=97, eps=1e-6, softcap=10.0):
    d = {"architecture": "Netinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if softcap is not None:
        d["logit_softcap"] = softcap
    return d


# A: both mixers, a chunk of three pages, scaled frequencies, two of six experts
CASE_A = config([attention_layer(4, 2, 32, 48, experts(64, 6, 2)), retention_layer(2, 32, 32, experts(64, 6, 2), seed=1),
                 attention_layer(4, 2, 32, 48, experts(64, 6, 2))], width=64)
# B: what the usual model makes equal or one: value heads of another size than the keys', a part of a head rotating,
# one kv head, one expert of five chosen, a layer without a feed-forward, a chunk that is no multiple of a page, head
# sizes that are no multiple of 32, no cap on the logits, a scaling whose ramp starts above the first frequency
CASE_B = config([retention_layer(3, 24, 40, None, rot=rotation(16, 500.0), seed=2),
                 attention_layer(3, 1, 40, 21, experts(72, 5, 1), rot=rotation(24, 100.0, (8.0, 32, 4.0, 1.0))),
                 attention_layer(2, 2, 16, 37, experts(56, 7, 3), rot=rotation(16, 1000000.0), scale=0.4)],
                width=48, vocab=131, eps=1e-5, softcap=None)
# C: as many kv heads as heads, a chunk of one page exactly, all experts chosen, decays of one and of nothing, a
# retention without rotation, an attention that sees every earlier key, a factor of one (nothing scaled)
CASE_C = config([attention_layer(6, 6, 16, 16, experts(80, 3, 3), rot=rotation(16, 10000.0, (1.0, 128, 16.0, 1.0))),
                 retention_layer(4, 16, 16, experts(40, 9, 4), rot=None, decay=[1.0, 0.9, 0.5, 0.0]),
                 attention_layer(2, 1, 64, None, experts(40, 9, 4), rot=None)], width=72, vocab=64, softcap=30.0)
# D: retentions only (no pages at all), a width that is no multiple of eight, heads of 64 with 24 of them rotating
CASE_D = config([retention_layer(2, 64, 64, experts(36, 4, 2), rot=rotation(24, 50000.0, (2.0, 16, 4.0, 0.5)), seed=4),
                 retention_layer(1, 32, 96, experts(36, 4, 2), seed=5)], width=44, vocab=50, softcap=5.0)
# E: attentions only, heads of 128, a chunk of 100
CASE_E = config([attention_layer(2, 2, 128, 100, experts(64, 2, 1)), attention_layer(4, 1, 32, 25, None)], width=32,
                vocab=75)
CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D, "E": CASE_E}


def tensor_shapes(cfg: dict) -> dict:
    """name -> shape of every tensor of a folder of this configuration."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W)}

    def norm(name):
        out[name], out[name + ".b"], out[name + ".alpha"] = (W,), (W,), ()

    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        norm(p + ".norm1")
        q = p + ".mix"
        if layer["type"] == "retention":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out[q + ".q"] = out[q + ".k"] = (H * d, W)
            out[q + ".v"] = out[q + ".g"] = (H * dv, W)
            out[q + ".o"] = (W, H * dv)
        else:
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            out[q + ".q"], out[q + ".k"] = (H * d, W), (G * d, W)
            out[q + ".q.norm"], out[q + ".k.norm"] = (H * d,), (G * d,)
            out[q + ".o"] = (W, H * d)
        if layer["mlp"] is not None:
            norm(p + ".norm2")
            ff, E = layer["mlp"]["expert"]["ff"], layer["mlp"]["router"]["experts"]
            for e in range(E):
                out[f"{p}.mlp.e{e}.gate"] = out[f"{p}.mlp.e{e}.up"] = (ff, W)
                out[f"{p}.mlp.e{e}.down"] = (W, ff)
            out[p + ".mlp.router"], out[p + ".mlp.router.b"] = (E, W), (E,)
    norm("final.norm")
    return out


def make_weights(cfg: dict, seed: int) -> dict:
    """bfloat16 tensors (as a folder stores them) for ``cfg``."""
    g = torch.Generator().manual_seed(seed)
    randn = lambda shape: torch.randn(shape, generator=g)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            t = 0.5 + torch.rand(shape, generator=g)
        elif last in ("norm1", "norm2", "norm"):
            t = 1.0 + 0.1 * randn(shape)
        elif last == "b":
            t = 0.2 * randn(shape)
        elif last == "router":
            t = 3.0 * randn(shape) / math.sqrt(shape[-1])
        elif name == "embed":
            t = randn(shape)
        else:
            t = randn(shape) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out


def random_ids(vocab: int, n: int, seed: int) -> list:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


CLOSE_CALL = 0.02  # of the spread of a router's logits


def safe_sequence(cfg: dict, weights: dict, n: int, seed: int):
    """(ids, float64 logits [n, vocab]) of a random sequence in which no router's choice is a close call: token by
    token, a token whose choice at some layer lies within ``CLOSE_CALL`` of turning is drawn again."""
    rng = random.Random(seed)
    w64 = {k: v.to(torch.float64) for k, v in weights.items()}
    ids, rows, state = [], [], None
    for t in range(n):
        for attempt in range(200):
            tok = rng.randrange(cfg["vocab"])
            margin = [math.inf]
            logits, new_state = plain.forward(cfg, w64, [tok], start=t, state=state, margins=margin)
            if margin[0] >= CLOSE_CALL:
                break
        else:
            raise AssertionError(f"no token without a close call at position {t}")
        ids.append(tok)
        rows.append(logits[0])
        state = new_state
    return ids, torch.stack(rows)


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: root mean square of the difference (its mean taken off) over the standard deviation of the wanted row."""
    d = got.double() - want.double()
    d = d - d.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / want.double().std(dim=-1)


TOLERANCE = {"float32": 3e-5, "bfloat16": 5e-2}


def random_config(rng: random.Random) -> dict:
    """A configuration drawn at random: sizes, head counts, groupings, rotations, chunks, experts, the order of the layers."""
    divisor = lambda n: rng.choice([d for d in range(1, n + 1) if n % d == 0])
    size = lambda: rng.choice([8, 16, 24, 32, 40, 64])
    width = rng.choice([40, 48, 52, 64, 72, 96])

    def rot(dim):
        if rng.random() < 0.15:
            return None
        dims = rng.choice([dim, dim, 2 * rng.randint(1, dim // 2)])
        scaling = None if rng.random() < 0.4 else (rng.choice([1.0, 2.0, 4.0, 16.0]), rng.choice([16, 64, 2048]),
                                                   rng.choice([4.0, 8.0, 32.0]), rng.choice([0.5, 1.0, 2.0]))
        return rotation(dims, rng.choice([100.0, 10000.0, 1000000.0]), scaling)

    layers = []
    for _ in range(rng.randint(2, 5)):
        n = rng.randint(2, 9)
        mlp = None if rng.random() < 0.2 else experts(rng.choice([24, 40, 56, 64, 96]), n, rng.randint(1, n))
        if rng.random() < 0.5:
            heads = rng.choice([1, 2, 3, 4, 6])
            dim = size()
            layers.append(retention_layer(heads, dim, size(), mlp, rot=rot(dim), seed=rng.randint(0, 99)))
        else:
            heads = rng.choice([1, 2, 3, 4, 6, 8])
            dim = size()
            layers.append(attention_layer(heads, divisor(heads), dim, rng.choice([None, 5, 16, 23, 32, 64, 100]), mlp,
                                          rot=rot(dim), scale=rng.choice([None, 0.3])))
    return config(layers, width=width, vocab=rng.randint(40, 200), eps=rng.choice([1e-6, 1e-5]),
                  softcap=rng.choice([None, 8.0, 30.0]))
