"""A plain, slow restatement of the Sumevik decoder, one function per mechanism, in one precision throughout
(float64 by default).  It shares no code with the package: it takes the dict of config.json and a dict of tensors
by name, loops over tokens where that is the clearest way to say what is computed, and continues a sequence from
an explicit state, so that the plain implementation itself can be checked cut anywhere.

Notation: W the model width, t a position counted from 0 in its sequence, R the rotated dimensions of a head,
ms(x) = mean(x^2).

  embedding     x_t = E[id_t]
  norm          y = x / sqrt(ms(x) + eps) * (1 + w)              (the stored weight lies around zero)
  gelu          g(z) = z / 2 * (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))
  recurrent     b_t = g(Wy y_t + by);  u_t = cb + sum_j C[:, j] p_(t - taps + 1 + j),  p = Wx y + bx, zeros before t = 0;
  unit          per block n of the channels: r = sigmoid(Ra[n] u_n + ra[n]), i = sigmoid(Ri[n] u_n + ri[n]);
                a = exp(-8 r softplus(lam));  s_t = a s_(t-1) + sqrt(1 - a^2) i u_t,  s_(-1) = 0;  out = Wo (s_t * b_t)
  attention     q, k, v with biases; q and k heads normed (x / sqrt(ms + eps) * n, n shared by the heads), then the
                pairs (2i, 2i + 1), i < R / 2, rotated by t * base^(-2i / R); s_tj = (q_t . k_j) * scale for j <= t
                with floor(j / chunk) = floor(t / chunk); softmax; heads side by side times sigmoid(Wg y); Wo
  gated linear  q = Wq y / sqrt(dim), k = Wk y, v = Wv y;  alpha_t = sigmoid(Wa2 (Wa1 y) + ba2)^(1 / tau) per key
  attention     channel;  S_t = diag(alpha_t) S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t;
                out = Wo (concat_h(o_h / sqrt(ms(o_h) + eps) * n) * silu(Wg y))
  side by side  left_scale * attention + right_scale * gated linear attention, both of the same input
  dense         Wdown (g(Wgate y) * (Wup y))
  mixture       z = Wr y;  s = softmax(z) over experts and identity experts;  c = s + correction;  experts in
                ``count`` equal groups of neighbours, a group's score its largest c, the ``keep`` best groups stay
                (the others' c count as -inf);  the ``top`` largest c are chosen;  weights s_e / (sum of the chosen s
                + 1e-20);  expert: a = min(Wgate y, L), b = clamp(Wup y, -L, L), Wdown (a sigmoid(1.702 a) (b + 1));
                the last ``identity`` router outputs stand for experts that return y itself
  layer         x <- x + mixer(norm1(x));  x <- x + ff(norm2(x))   (a layer may have no feed-forward)
  output        logits = E norm(x) * logit_scale
"""

from __future__ import annotations

import math

import torch


def norm_one_plus(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(p, taps_weight, bias, history):
    """p [T, C] inputs, taps_weight [C, taps] (last column = the current token), history [taps - 1, C] the inputs
    before p (zeros at a sequence's start).  Returns (u [T, C], the new history)."""
    taps = taps_weight.shape[1]
    full = torch.cat([history, p], dim=0)
    u = torch.zeros_like(p)
    for t in range(p.shape[0]):
        for j in range(taps):
            u[t] += taps_weight[:, j] * full[t + j]
        u[t] += bias
    return u, full[full.shape[0] - (taps - 1):]


def recurrent_unit(y, w, prefix, mixer, state=None):
    """The recurrent mixer over y [T, W] from ``state`` = (history [taps - 1, C], s [C]) or None.  Returns (out, state)."""
    C, blocks, taps = mixer["width"], mixer["blocks"], mixer["conv"]
    n = C // blocks
    if state is None:
        state = (torch.zeros(taps - 1, C, dtype=y.dtype), torch.zeros(C, dtype=y.dtype))
    history, s = state
    branch = gelu_tanh(y @ w[prefix + ".y"].T + w[prefix + ".y.b"])
    p = y @ w[prefix + ".x"].T + w[prefix + ".x.b"]
    u, history = causal_conv(p, w[prefix + ".conv"], w[prefix + ".conv.b"], history)
    sp = torch.nn.functional.softplus(w[prefix + ".lam"])
    rows = []
    s = s.clone()
    for t in range(y.shape[0]):
        r = torch.empty(C, dtype=y.dtype)
        i = torch.empty(C, dtype=y.dtype)
        for b in range(blocks):
            ub = u[t, b * n:(b + 1) * n]
            r[b * n:(b + 1) * n] = torch.sigmoid(w[prefix + ".ra"][b] @ ub + w[prefix + ".ra.b"][b])
            i[b * n:(b + 1) * n] = torch.sigmoid(w[prefix + ".ri"][b] @ ub + w[prefix + ".ri.b"][b])
        a = torch.exp(-8.0 * r * sp)
        s = a * s + torch.sqrt(1.0 - a * a) * i * u[t]
        rows.append(s * branch[t])
    return torch.stack(rows) @ w[prefix + ".o"].T, (history, s)


def rotate_pairs(x, positions, rot):
    """x [T, heads, dim]: the pairs (2i, 2i + 1) of the first ``dims`` elements of every head turn by t * f_i."""
    if not rot or not rot.get("dims"):
        return x
    R, base = int(rot["dims"]), float(rot["base"])
    out = x.clone()
    for i in range(R // 2):
        f = base ** (-2.0 * i / R)
        ang = torch.tensor([p * f for p in positions], dtype=x.dtype)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = a * c - b * s
        out[:, :, 2 * i + 1] = b * c + a * s
    return out


def chunk_attention(y, w, prefix, m, eps, start=0, past=None):
    """The softmax attention over y [T, W] at positions start..; ``past`` = (keys [start, G, dim], values) or None."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = y.shape[0]
    positions = list(range(start, start + T))
    q = (y @ w[prefix + ".q"].T + w[prefix + ".q.b"]).reshape(T, H, d)
    k = (y @ w[prefix + ".k"].T + w[prefix + ".k.b"]).reshape(T, G, d)
    v = (y @ w[prefix + ".v"].T + w[prefix + ".v.b"]).reshape(T, G, dv)
    q = rotate_pairs(norm_plain(q, w[prefix + ".q.norm"], eps), positions, m.get("rot"))
    k = rotate_pairs(norm_plain(k, w[prefix + ".k.norm"], eps), positions, m.get("rot"))
    if past is not None:
        k, v = torch.cat([past[0], k]), torch.cat([past[1], v])
    chunk = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, dv, dtype=y.dtype)
    for t in range(T):
        p = start + t
        first = 0 if chunk is None else p - p % chunk
        for h in range(H):
            g = h // (H // G)
            s = (k[first:p + 1, g] @ q[t, h]) * m["scale"]
            out[t, h] = torch.softmax(s, 0) @ v[first:p + 1, g]
    gate = torch.sigmoid(y @ w[prefix + ".g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[prefix + ".o"].T, (k, v)


def gated_linear_attention(y, w, prefix, m, eps, state=None):
    """The linear attention with a decay per key channel over y [T, W]; ``state`` [heads, dim, vdim] or None."""
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    T = y.shape[0]
    q = (y @ w[prefix + ".q"].T).reshape(T, H, d) * d ** -0.5
    k = (y @ w[prefix + ".k"].T).reshape(T, H, d)
    v = (y @ w[prefix + ".v"].T).reshape(T, H, dv)
    z = (y @ w[prefix + ".a1"].T) @ w[prefix + ".a2"].T + w[prefix + ".a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).reshape(T, H, d)
    S = torch.zeros(H, d, dv, dtype=y.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=y.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = norm_plain(o, w[prefix + ".norm"], eps).reshape(T, H * dv)
    return (o * silu(y @ w[prefix + ".g"].T)) @ w[prefix + ".o"].T, S


def side_by_side(y, w, prefix, m, eps, start=0, state=None):
    left_state, right_state = state if state is not None else (None, None)
    left, left_state = chunk_attention(y, w, prefix + ".left", m["left"], eps, start, left_state)
    right, right_state = gated_linear_attention(y, w, prefix + ".right", m["right"], eps, right_state)
    return m["left_scale"] * left + m["right_scale"] * right, (left_state, right_state)


def dense(y, w, prefix):
    return (gelu_tanh(y @ w[prefix + ".gate"].T) * (y @ w[prefix + ".up"].T)) @ w[prefix + ".down"].T


def route(y_row, w, prefix, router):
    """(chosen expert indices in the order they are found, their weights, the margin of the closest decision)."""
    E, I, top = router["experts"], router.get("identity", 0), router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    n = E + I
    s = torch.softmax(w[prefix + ".router"] @ y_row, 0)
    c = s + w[prefix + ".correction"]
    size = n // groups["count"]
    best = [max(float(c[g * size + j]) for j in range(size)) for g in range(groups["count"])]
    order = sorted(range(groups["count"]), key=lambda g: (-best[g], g))
    kept = set(order[:groups["keep"]])
    margin = math.inf
    if groups["keep"] < groups["count"]:
        margin = best[order[groups["keep"] - 1]] - best[order[groups["keep"]]]
    allowed = [e for e in range(n) if e // size in kept]
    ranked = sorted(allowed, key=lambda e: (-float(c[e]), e))
    chosen = ranked[:top]
    if len(ranked) > top:
        margin = min(margin, float(c[ranked[top - 1]]) - float(c[ranked[top]]))
    total = sum(s[e] for e in chosen) + 1e-20
    return chosen, [s[e] / total for e in chosen], margin


def expert(y_row, w, prefix, limit):
    a = torch.clamp(w[prefix + ".gate"] @ y_row, max=limit)
    b = torch.clamp(w[prefix + ".up"] @ y_row, min=-limit, max=limit)
    return w[prefix + ".down"] @ (a * torch.sigmoid(1.702 * a) * (b + 1.0))


def mixture(y, w, prefix, mlp, margins=None):
    router, limit = mlp["router"], float(mlp["expert"]["limit"])
    out = torch.zeros_like(y)
    for t in range(y.shape[0]):
        chosen, weights, margin = route(y[t], w, prefix, router)
        if margins is not None:
            margins.append(margin)
        for e, g in zip(chosen, weights):
            out[t] += g * (y[t] if e >= router["experts"] else expert(y[t], w, f"{prefix}.e{e}", limit))
    return out


def forward(cfg, w, ids, start=0, state=None, dtype=torch.float64, after_layer=None, margins=None):
    """Logits [T, vocab] of ``ids`` at positions start.., and the state after them.  ``state``: None (a new sequence)
    or what an earlier call returned.  ``after_layer(i, x)`` sees the residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    state = list(state) if state is not None else [None] * len(cfg["layers"])
    x = w["embed"][torch.tensor(ids, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        y = norm_one_plus(x, w[f"l{i}.norm1"], eps)
        if layer["type"] == "rglru":
            mixed, state[i] = recurrent_unit(y, w, f"l{i}.mix", layer["mixer"], state[i])
        elif layer["type"] == "parallel":
            mixed, state[i] = side_by_side(y, w, f"l{i}.mix", layer["mixer"], eps, start, state[i])
        else:
            raise ValueError(layer["type"])
        x = x + mixed
        mlp = layer.get("mlp")
        if mlp is not None:
            y = norm_one_plus(x, w[f"l{i}.norm2"], eps)
            x = x + (dense(y, w, f"l{i}.mlp") if mlp["kind"] == "dense" else mixture(y, w, f"l{i}.mlp", mlp, margins))
        if after_layer is not None:
            after_layer(i, x)
    y = norm_one_plus(x, w["final.norm"], eps)
    return (y @ w["embed"].T) * float(cfg.get("logit_scale", 1.0)), state
