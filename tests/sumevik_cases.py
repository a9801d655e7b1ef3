"""Small Sumevik configurations and weights for the tests, and how a step function's logits are compared with the
plain implementation (``plain_sumevik``).

The weights are not N(0, 0.02): projections are drawn with a standard deviation of 1 / sqrt(inputs), norm weights
around zero (the layers' norms, which multiply by 1 + w) or around one (the norms inside the mixers), the recurrent
unit's decay parameters so that its decays spread from 0.3 to 0.999, the decay bias of the gated linear attention so that
its decays lie near one, router matrices so that the scores spread, corrections of the size of a score, so that every
mechanism moves the logits by far more than a tolerance.

Sequences are drawn token by token so that no router's choice (of a group or of an expert) is a close call anywhere
(``safe_sequence``): in bfloat16 the router sees rounded inputs, and a choice that a rounding can turn is no fault of
the engine.
"""

from __future__ import annotations

import math
import random

import torch

import plain_sumevik as plain


def dense(ff):
    return {"kind": "dense", "ff": ff}


def experts(ff, n, top, identity=0, groups=(1, 1), limit=1.0):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": n, "identity": identity, "top": top, "groups": {"count": groups[0], "keep": groups[1]}}}


def recurrent_layer(width, blocks, conv, mlp):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, chunk=None, rot=None, scale=None):
    """``rot``: (dims, base) or None."""
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if chunk is not None:
        d["mask"] = {"size": chunk}
    if rot is not None:
        d["rot"] = {"dims": rot[0], "base": rot[1]}
    return d


def linear(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def parallel_layer(left, right, mlp, scales=(1.0, 1.0)):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "right": right, "left_scale": scales[0], "right_scale": scales[1]}}


def config(layers, width=64, vocab=97, eps=1e-6, logit_scale=None, ranks=None):
    """``ranks``: layer index -> inner size of that layer's decay projection (a size that only the tensors state); it is
    kept beside the configuration under a key that the reader of config.json does not know and ignores."""
    d = {"architecture": "Sumevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if logit_scale is not None:
        d["logit_scale"] = logit_scale
    d["_ranks"] = dict(ranks or {})
    return d


def folder_config(cfg: dict) -> dict:
    """What goes into config.json."""
    return {k: v for k, v in cfg.items() if not k.startswith("_")}


# A: both mixers and both feed-forwards; a chunk of three pages; half of every head rotating; two of six experts and two
# identity experts in four groups of which two stay; factors on the two mixers
CASE_A = config([
    recurrent_layer(48, 3, 4, dense(96)),
    parallel_layer(attention(4, 2, 32, 48, chunk=48, rot=(16, 10000.0)), linear(2, 16, 32, 8.0),
                   experts(40, 6, 2, identity=2, groups=(4, 2), limit=0.7), scales=(0.7, 1.3)),
    recurrent_layer(64, 1, 2, experts(40, 6, 2, identity=2, groups=(4, 2), limit=0.7)),
], width=64, logit_scale=0.6, ranks={1: 8})
# B: what a usual model makes equal or one: a width that is no multiple of eight, a convolution of one tap (no inputs
# kept), blocks of eight channels, one kv head, value heads of another size than the keys', whole heads rotating, a
# chunk that is no multiple of a page, heads that are no multiple of 32, a decay root of one, one expert of five
# chosen without groups or identity experts, a layer without a feed-forward, no factor on the logits, a rank of five
CASE_B = config([
    parallel_layer(attention(3, 1, 24, 40, chunk=21, rot=(24, 100.0), scale=0.3), linear(3, 8, 24, 1.0), None),
    recurrent_layer(40, 5, 1, experts(72, 5, 1)),
    parallel_layer(attention(2, 2, 16, 8, chunk=37, rot=(2, 1000000.0)), linear(1, 40, 8, 3.0), dense(56), scales=(1.5, 0.5)),
], width=44, vocab=131, eps=1e-5, ranks={0: 5, 2: 16})
# C: side-by-side layers only; as many kv heads as heads; a chunk of one page exactly; an attention that sees every
# earlier key and rotates nothing; all five router outputs chosen, three of them identity experts; key heads of 64
CASE_C = config([
    parallel_layer(attention(6, 6, 16, 16, chunk=16, rot=(16, 10000.0)), linear(2, 64, 16, 16.0),
                   experts(80, 2, 5, identity=3, groups=(5, 5), limit=2.0)),
    parallel_layer(attention(2, 1, 64, 32), linear(4, 16, 16, 4.0), experts(40, 9, 4, identity=1, groups=(2, 1), limit=0.5),
                   scales=(1.0, 2.0)),
], width=72, vocab=64, logit_scale=3.0, ranks={0: 3, 1: 24})
# D: recurrent layers only (no pages at all); five taps; blocks of one channel and one block of all; dense feed-forwards
CASE_D = config([recurrent_layer(36, 36, 5, dense(40)), recurrent_layer(80, 1, 3, None), recurrent_layer(24, 2, 2, dense(24))],
                width=40, vocab=50, logit_scale=0.25)
# E: heads of 128 in the attention, key heads of 128 and of 136 in the linear attention, a chunk of 100
CASE_E = config([
    parallel_layer(attention(2, 2, 128, 64, chunk=100, rot=(64, 500000.0)), linear(1, 128, 24, 16.0), dense(64)),
    parallel_layer(attention(4, 1, 32, 32, chunk=25, rot=(32, 50.0)), linear(1, 136, 16, 32.0), None, scales=(0.5, 0.5)),
], width=32, vocab=75, ranks={0: 16, 1: 4})
CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D, "E": CASE_E}


def tensor_shapes(cfg: dict) -> dict:
    """name -> shape of every tensor of a folder of this configuration."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        out[p + ".norm1"] = (W,)
        q = p + ".mix"
        if layer["type"] == "rglru":
            C, n, taps = m["width"], m["blocks"], m["conv"]
            out[q + ".y"] = out[q + ".x"] = (C, W)
            out[q + ".y.b"] = out[q + ".x.b"] = out[q + ".conv.b"] = out[q + ".lam"] = (C,)
            out[q + ".conv"] = (C, taps)
            out[q + ".ra"] = out[q + ".ri"] = (n, C // n, C // n)
            out[q + ".ra.b"] = out[q + ".ri.b"] = (n, C // n)
            out[q + ".o"] = (W, C)
        else:
            a, g = m["left"], m["right"]
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            l, r = q + ".left", q + ".right"
            out[l + ".q"], out[l + ".q.b"] = (H * d, W), (H * d,)
            out[l + ".k"], out[l + ".k.b"] = (G * d, W), (G * d,)
            out[l + ".v"], out[l + ".v.b"] = (G * dv, W), (G * dv,)
            out[l + ".q.norm"] = out[l + ".k.norm"] = (d,)
            out[l + ".g"], out[l + ".o"] = (H * dv, W), (W, H * dv)
            H, d, dv = g["heads"], g["dim"], g["vdim"]
            rank = cfg["_ranks"].get(i, 16)
            out[r + ".q"] = out[r + ".k"] = (H * d, W)
            out[r + ".v"] = out[r + ".g"] = (H * dv, W)
            out[r + ".o"], out[r + ".norm"] = (W, H * dv), (dv,)
            out[r + ".a1"], out[r + ".a2"], out[r + ".a2.b"] = (rank, W), (H * d, rank), (H * d,)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        out[p + ".norm2"] = (W,)
        if mlp["kind"] == "dense":
            out[p + ".mlp.gate"] = out[p + ".mlp.up"] = (mlp["ff"], W)
            out[p + ".mlp.down"] = (W, mlp["ff"])
        else:
            ff, E, I = mlp["expert"]["ff"], mlp["router"]["experts"], mlp["router"].get("identity", 0)
            for e in range(E):
                out[f"{p}.mlp.e{e}.gate"] = out[f"{p}.mlp.e{e}.up"] = (ff, W)
                out[f"{p}.mlp.e{e}.down"] = (W, ff)
            out[p + ".mlp.router"], out[p + ".mlp.correction"] = (E + I, W), (E + I,)
    return out


def make_weights(cfg: dict, seed: int) -> dict:
    """bfloat16 tensors (as a folder stores them) for ``cfg``."""
    g = torch.Generator().manual_seed(seed)
    randn = lambda shape: torch.randn(shape, generator=g)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2") or name == "final.norm":
            t = 0.1 * randn(shape)  # the norm multiplies by 1 + w
        elif last == "norm":
            t = 1.0 + 0.1 * randn(shape)
        elif last == "lam":
            t = -6.0 + 5.0 * torch.rand(shape, generator=g)
        elif name.endswith(".a2.b"):
            t = 2.0 + randn(shape)
        elif last == "b":
            t = 0.2 * randn(shape)
        elif last == "router":
            t = 3.0 * randn(shape) / math.sqrt(shape[-1])
        elif last == "correction":
            t = 0.3 * randn(shape) / shape[0]
        elif name == "embed":
            t = randn(shape)
        elif last in ("ra", "ri"):
            t = 2.0 * randn(shape) / math.sqrt(shape[-1])
        else:
            t = randn(shape) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out


def random_ids(vocab: int, n: int, seed: int) -> list:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


CLOSE_CALL = 0.03  # of a router's scores, which add up to one (bfloat16 inputs move a score of 0.5 by some 0.02)


def safe_sequence(cfg: dict, weights: dict, n: int, seed: int, close_call: float = None):
    """(ids, float64 logits [n, vocab]) of a random sequence in which no router's choice is a close call: token by
    token, a token whose choice at some layer lies within ``close_call`` (``CLOSE_CALL`` unless given: with many router
    outputs the scores and their gaps are smaller, and so is what rounding moves them by) of turning is drawn again."""
    close_call = CLOSE_CALL if close_call is None else close_call
    rng = random.Random(seed)
    w64 = {k: v.to(torch.float64) for k, v in weights.items()}
    plain_cfg = folder_config(cfg)
    ids, rows, state = [], [], None
    for t in range(n):
        for attempt in range(200):
            tok = rng.randrange(cfg["vocab"])
            margins = []
            logits, new_state = plain.forward(plain_cfg, w64, [tok], start=t, state=state, margins=margins)
            if not margins or min(margins) >= close_call:
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

    def feed_forward():
        r = rng.random()
        if r < 0.15:
            return None
        if r < 0.45:
            return dense(rng.choice([24, 40, 56, 64, 96]))
        count = rng.choice([1, 1, 2, 3, 4])
        per = rng.randint(1, 4)
        n = count * per
        identity = rng.randint(0, min(3, n - 1)) if rng.random() < 0.6 else 0
        keep = rng.randint(1, count)
        return experts(rng.choice([24, 40, 56, 64]), n - identity, rng.randint(1, keep * per), identity=identity,
                       groups=(count, keep), limit=rng.choice([0.5, 1.0, 7.0]))

    layers, ranks = [], {}
    for i in range(rng.randint(2, 5)):
        if rng.random() < 0.5:
            blocks = rng.choice([1, 2, 3, 4, 8])
            layers.append(recurrent_layer(blocks * rng.choice([1, 4, 8, 12, 16]), blocks, rng.randint(1, 5), feed_forward()))
        else:
            heads, dim = rng.choice([1, 2, 3, 4, 6, 8]), size()
            rot = None if rng.random() < 0.15 else (rng.choice([dim, 2 * rng.randint(1, dim // 2)]),
                                                    rng.choice([100.0, 10000.0, 1000000.0]))
            left = attention(heads, divisor(heads), dim, size(), chunk=rng.choice([None, 5, 16, 23, 32, 64, 100]), rot=rot,
                             scale=rng.choice([None, 0.3]))
            right = linear(rng.choice([1, 2, 3, 4]), size(), size(), rng.choice([1.0, 4.0, 16.0]))
            ranks[i] = rng.choice([1, 4, 7, 16])
            layers.append(parallel_layer(left, right, feed_forward(),
                                         scales=(rng.choice([1.0, 0.75, 1.5]), rng.choice([1.0, 1.25, 0.4]))))
    return config(layers, width=width, vocab=rng.randint(40, 200), eps=rng.choice([1e-6, 1e-5]),
                  logit_scale=rng.choice([None, 0.5, 2.0]), ranks=ranks)
