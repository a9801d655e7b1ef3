"""A plain, slow restatement of the Netinex decoder, one function per mechanism, in one precision throughout
(float64 by default).  It shares no code with the package: it takes the dict of config.json and a dict of
tensors by name, loops over tokens where that is the clearest way to say what is computed, and continues a
sequence from an explicit state, so that the plain implementation itself can be checked cut anywhere.

Notation: W is the model width, t a position counted from 0 in its sequence, R the rotated dimensions of a head.

  embedding        x_t = E[id_t]
  dynamic tanh     y = tanh(alpha x) * w + b, alpha one learned number; no statistics of x
  frequencies      f_i = base^(-2i / R), i < R / 2.  With a scaling (factor, original, fast, slow):
                   c(r) = R ln(original / (2 pi r)) / (2 ln base); lo = max(floor(c(fast)), 0);
                   hi = min(ceil(c(slow)), R - 1); ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1);
                   f_i <- f_i / factor * ramp_i + f_i (1 - ramp_i); cosines and sines times 0.1 ln(factor) + 1
  rotation         the pair (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = t f_i; pairs are the elements
                   (i, i + R / 2) ("half") or (2i, 2i + 1) ("interleaved") of a head's first R elements
  retention        q, k rotated (half); k / sqrt(dim); S_t = decay_h S_(t-1) + k_t v_t^T; o_t = S_t^T q_t;
                   out = Wo (concat_h(o_h / sqrt(mean(o_h^2) + eps)) * silu(Wg y))
  attention        q <- q / sqrt(mean(q^2) + eps) * nq over the WHOLE projection (all heads at once), k likewise;
                   the values are the keys as projected (before norm and rotation); q, k rotated (interleaved);
                   s_tj = (q_t . k_j) * scale for j <= t with floor(j / chunk) = floor(t / chunk); softmax; Wo
  mixture          z = Wr y + br; the `top` largest z; weights = softmax over those alone;
                   out = sum_e weight_e Wdown_e (silu(Wgate_e y) * (Wup_e y))
  layer            x <- x + mixer(norm1(x));  x <- x + mixture(norm2(x))
  output           logits = cap * tanh((E norm(x)) / cap)
"""

from __future__ import annotations

import math

import torch


def dynamic_tanh(x, w, b, alpha):
    return torch.tanh(x * alpha) * w + b


def silu(z):
    return z * torch.sigmoid(z)


def frequencies(rot):
    """(list of R / 2 frequencies, factor on cosines and sines) of a rotation's configuration (None: nothing rotates)."""
    if not rot or not rot.get("dims"):
        return [], 1.0
    R, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / R) for i in range(R // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def c(r):
        return R * math.log(original / (2.0 * math.pi * r)) / (2.0 * math.log(base))

    lo = max(math.floor(c(float(sc["fast"]))), 0)
    hi = min(math.ceil(c(float(sc["slow"]))), R - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot, layout):
    """x [T, heads, dim]; the first rot.dims elements of every head are rotated by the token's position."""
    f, mag = frequencies(rot)
    if not f:
        return x
    R = 2 * len(f)
    out = x.clone()
    for n, p in enumerate(positions):
        for i, fi in enumerate(f):
            a = p * fi
            c, s = math.cos(a) * mag, math.sin(a) * mag
            iu, iv = (i, i + R // 2) if layout == "half" else (2 * i, 2 * i + 1)
            u, v = x[n, :, iu], x[n, :, iv]
            out[n, :, iu] = u * c - v * s
            out[n, :, iv] = v * c + u * s
    return out


def retention(y, w, prefix, mixer, eps, start=0, state=None):
    """y [T, W] from position ``start``; ``state`` [heads, dim, vdim] or None (zero).  Returns (out [T, W], state)."""
    H, d, dv = mixer["heads"], mixer["dim"], mixer["vdim"]
    T = y.shape[0]
    pos = range(start, start + T)
    q = rotate((y @ w[prefix + ".q"].T).reshape(T, H, d), pos, mixer.get("rot"), "half")
    k = rotate((y @ w[prefix + ".k"].T).reshape(T, H, d), pos, mixer.get("rot"), "half") / math.sqrt(d)
    v = (y @ w[prefix + ".v"].T).reshape(T, H, dv)
    S = torch.zeros(H, d, dv, dtype=y.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=y.dtype)
    for t in range(T):
        for h in range(H):
            S[h] = mixer["decay"][h] * S[h] + torch.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    o = o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps)
    gated = o.reshape(T, H * dv) * silu(y @ w[prefix + ".g"].T)
    return gated @ w[prefix + ".o"].T, S


def chunk_attention(y, w, prefix, mixer, eps, start=0, past=None):
    """``past`` = (keys [start, G, d] as cached, values [start, G, d]) or None.  Returns (out, (keys, values))."""
    H, G, d = mixer["heads"], mixer["kv_heads"], mixer["dim"]
    T = y.shape[0]
    pos = list(range(start, start + T))
    q = y @ w[prefix + ".q"].T
    k = y @ w[prefix + ".k"].T
    v = k.reshape(T, G, d)
    q = q / torch.sqrt((q * q).mean(dim=-1, keepdim=True) + eps) * w[prefix + ".q.norm"]
    kn = k / torch.sqrt((k * k).mean(dim=-1, keepdim=True) + eps) * w[prefix + ".k.norm"]
    q = rotate(q.reshape(T, H, d), pos, mixer.get("rot"), "interleaved")
    kn = rotate(kn.reshape(T, G, d), pos, mixer.get("rot"), "interleaved")
    if past is not None:
        kn, v = torch.cat([past[0], kn]), torch.cat([past[1], v])
    chunk = (mixer.get("mask") or {}).get("size")
    o = torch.zeros(T, H, d, dtype=y.dtype)
    for n, t in enumerate(pos):
        first = 0 if not chunk else (t // chunk) * chunk
        for h in range(H):
            g = h // (H // G)
            s = (kn[first:t + 1, g] @ q[n, h]) * mixer["scale"]
            p = torch.softmax(s, dim=0)
            o[n, h] = p @ v[first:t + 1, g]
    return o.reshape(T, H * d) @ w[prefix + ".o"].T, (kn, v)


def mixture(y, w, prefix, mlp, margins=None):
    """``margins`` (a list with one entry per token, or None): lowered to the gap between the last chosen logit and the
    first that is not, over the logits' spread, where that is smaller: how close the choice was."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = y @ w[prefix + ".router"].T + w[prefix + ".router.b"]
    if margins is not None and top < E:
        ordered = torch.sort(z, dim=-1, descending=True).values
        gap = (ordered[:, top - 1] - ordered[:, top]) / (ordered[:, 0] - ordered[:, -1])
        for t in range(y.shape[0]):
            margins[t] = min(margins[t], float(gap[t]))
    out = torch.zeros(y.shape[0], w[prefix + ".e0.down"].shape[0], dtype=y.dtype)
    for t in range(y.shape[0]):
        chosen = sorted(range(E), key=lambda e: -float(z[t, e]))[:top]
        zs = torch.stack([z[t, e] for e in chosen])
        p = torch.exp(zs - zs.max())
        p = p / p.sum()
        for weight, e in zip(p, chosen):
            a = silu(w[f"{prefix}.e{e}.gate"] @ y[t]) * (w[f"{prefix}.e{e}.up"] @ y[t])
            out[t] += weight * (w[f"{prefix}.e{e}.down"] @ a)
    return out


def norm_of(x, w, name):
    return dynamic_tanh(x, w[name], w[name + ".b"], w[name + ".alpha"])


def forward(cfg, w, ids, start=0, state=None, dtype=torch.float64, after_layer=None, margins=None):
    """Logits [len(ids), vocab] of the tokens ``ids`` at positions start .. and the state to continue from.
    ``state``: what an earlier call returned (one entry per layer), or None at position 0.  ``after_layer(i, x)`` sees
    the residual stream after every layer; ``margins``: see ``mixture`` (one entry per token, initially large)."""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(list(ids), dtype=torch.long)]
    new_state = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        y = norm_of(x, w, p + ".norm1")
        old = None if state is None else state[i]
        if layer["type"] == "retention":
            m, s = retention(y, w, p + ".mix", layer["mixer"], eps, start, old)
        elif layer["type"] == "attention":
            m, s = chunk_attention(y, w, p + ".mix", layer["mixer"], eps, start, old)
        else:
            raise ValueError(layer["type"])
        new_state.append(s)
        x = x + m
        if layer.get("mlp") is not None:
            x = x + mixture(norm_of(x, w, p + ".norm2"), w, p + ".mlp", layer["mlp"], margins)
        if after_layer is not None:
            after_layer(i, x)
    logits = norm_of(x, w, "final.norm") @ w["embed"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, new_state
