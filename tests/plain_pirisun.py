"""Plain implementation of the Pirisun design: NumPy, float64, whole sequences, no cache, one function per
mechanism, loops over tokens, heads and keys.  Shares nothing with the library; slow on purpose.

Notation: n tokens, D width, H heads, G key/value heads, d head width, e value width, r latent width,
p rotated width.  A weight W [out, in] is applied as W x."""
from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def layer_norm(x, w, b, eps):
    mu = np.mean(x, axis=-1, keepdims=True)
    var = np.mean((x - mu) ** 2, axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rotate(vec, pos, base, dims, interleaved):
    """Rotates the first `dims` entries of one vector by position `pos`.  Pairs are (2i, 2i + 1) when `interleaved`,
    else (i, i + dims/2); pair i turns by pos * base^(-2i/dims)."""
    out = np.array(vec, dtype=np.float64)
    half = dims // 2
    for i in range(half):
        a = pos * base ** (-2.0 * i / dims)
        ia, ib = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        u, v = vec[ia], vec[ib]
        out[ia] = u * math.cos(a) - v * math.sin(a)
        out[ib] = v * math.cos(a) + u * math.sin(a)
    return out


def softmax_list(scores, sink=None):
    """Softmax over a list of scores; `sink` is one more term of the denominator, without a value."""
    m = max(scores) if sink is None else max(max(scores), sink)
    e = [math.exp(s - m) for s in scores]
    z = sum(e) + (0.0 if sink is None else math.exp(sink - m))
    return [x / z for x in e]


def latent_attention(h, W, m, eps):
    """Causal attention whose keys and values are expanded from one latent per token; one rotated key part for all
    heads (interleaved pairs); a sink per head in the softmax; a sigmoid gate on every output value.
    W: q, dkv, dkv.norm, uk, uv, sink, g, o."""
    n = h.shape[0]
    H, d, p, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base = m["rot"]["base"]
    q = (h @ W["q"].T).reshape(n, H, d + p)
    low = h @ W["dkv"].T
    c = rms(low[:, :r], eps) * W["dkv.norm"]
    k_rot = np.stack([rotate(low[t, r:], t, base, p, True) for t in range(n)])
    k = (c @ W["uk"].T).reshape(n, H, d)
    v = (c @ W["uv"].T).reshape(n, H, e)
    gate = sigmoid(h @ W["g"].T).reshape(n, H, e) if "g" in W else None
    out = np.zeros((n, H, e))
    for t in range(n):
        for a in range(H):
            q_rot = rotate(q[t, a, d:], t, base, p, True)
            sc = [(float(q[t, a, :d] @ k[j, a]) + float(q_rot @ k_rot[j])) * m["scale"] for j in range(t + 1)]
            w = softmax_list(sc, None if "sink" not in W else float(W["sink"][a]))
            for j in range(t + 1):
                out[t, a] += w[j] * v[j, a]
    if gate is not None:
        out = out * gate
    return out.reshape(n, H * e) @ W["o"].T


def capped_attention(h, W, m):
    """Grouped-query softmax attention without a rotation: the query at position p is multiplied by
    1 + coef * ln(floor((p + 1) / every) + 1); a score s becomes cap * tanh(s / cap).  W: q, k, v, o."""
    n = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W["q"].T).reshape(n, H, d).copy()
    k = (h @ W["k"].T).reshape(n, G, d)
    v = (h @ W["v"].T).reshape(n, G, e)
    qt = m.get("q_temp")
    if qt:
        for t in range(n):
            q[t] *= 1.0 + qt["coef"] * math.log(math.floor((t + 1) / qt["every"]) + 1.0)
    cap = m.get("softcap")
    out = np.zeros((n, H, e))
    for t in range(n):
        for a in range(H):
            g = a // (H // G)
            sc = [float(q[t, a] @ k[j, g]) * m["scale"] for j in range(t + 1)]
            if cap:
                sc = [cap * math.tanh(s / cap) for s in sc]
            w = softmax_list(sc)
            for j in range(t + 1):
                out[t, a] += w[j] * v[j, g]
    return out.reshape(n, H * e) @ W["o"].T


def retention(h, W, m, eps):
    """Linear attention with one fixed decay per head: S_t = decay * S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, state from
    zero; q and k rotated (half-split pairs), k then multiplied by d^(-1/2); every head's o divided by its root mean
    square; times silu(W_g h); W_o.  W: q, k, v, g, o."""
    n = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    rot = m.get("rot")
    q = (h @ W["q"].T).reshape(n, H, d).copy()
    k = (h @ W["k"].T).reshape(n, H, d).copy()
    v = (h @ W["v"].T).reshape(n, H, e)
    out = np.zeros((n, H, e))
    for a in range(H):
        S = np.zeros((d, e))
        for t in range(n):
            qt, kt = q[t, a], k[t, a]
            if rot:
                qt = rotate(qt, t, rot["base"], rot["dims"], False)
                kt = rotate(kt, t, rot["base"], rot["dims"], False)
            kt = kt * d ** -0.5
            S = m["decay"][a] * S + np.outer(kt, v[t, a])
            out[t, a] = S.T @ qt
    out = rms(out, eps).reshape(n, H * e) * silu(h @ W["g"].T)
    return out @ W["o"].T


def mixer_pair(h, W, m, eps):
    """Two mixers read the same rows; half the sum of their results, each RMS-normalised over the width with a
    weight of its own.  W: left.*, right.*, left.out, right.out."""
    sub = lambda side: {k[len(side) + 1:]: v for k, v in W.items() if k.startswith(side + ".") and k != side + ".out"}
    left = capped_attention(h, sub("left"), m["left"])
    right = retention(h, sub("right"), m["right"], eps)
    return 0.5 * (rms(left, eps) * W["left.out"] + rms(right, eps) * W["right.out"])


def gated_unit(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(z, correction, top):
    """Softmax scores of the logits z [experts]; the `top` experts with the largest score + correction, their
    weights (the scores without the correction, over their sum), and the margin of the choice: how far the last chosen
    expert's score + correction lies above the best one that was not chosen (inf when all are chosen)."""
    s = np.exp(z - z.max())
    s = s / s.sum()
    pick = s + correction if correction is not None else s
    ranked = sorted(range(len(z)), key=lambda i: (-pick[i], i))
    chosen = ranked[:top]
    total = sum(s[i] for i in chosen) + 1e-20
    margin = pick[ranked[top - 1]] - pick[ranked[top]] if top < len(z) else np.inf
    return chosen, [s[i] / total for i in chosen], margin


def experts(h, W, ml, margins=None):
    """Routed experts; the last `identity` outputs of the router stand for experts that return their input; a shared
    expert every token takes.  W: router, correction, e<i>.gate/up/down, shared.gate/up/down.  `margins`: a list with
    one entry per token that is lowered to the token's margin of choice (see `route`)."""
    n = h.shape[0]
    ro = ml["router"]
    E, ident, top = ro["experts"], ro.get("identity", 0), ro["top"]
    out = np.zeros_like(h)
    z = h @ W["router"].T
    for t in range(n):
        chosen, wts, margin = route(z[t], W.get("correction"), top)
        if margins is not None:
            margins[t] = min(margins[t], margin)
        for i, w in zip(chosen, wts):
            if i >= E:
                out[t] += w * h[t]
            else:
                out[t] += w * gated_unit(h[t], W[f"e{i}.gate"], W[f"e{i}.up"], W[f"e{i}.down"])
    if "shared.gate" in W:
        out += gated_unit(h, W["shared.gate"], W["shared.up"], W["shared.down"])
    return out


def layer_runs(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    return (list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n)))


def forward(cfg, W, tokens, taps=None, margins=None):
    """Logits [n, vocab] of one sequence.  W: name -> float64 array.  `taps`: a list that receives the rows after
    every layer run.  `margins`: a list with one entry per token, lowered to the smallest margin of any expert choice
    made for that token."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)].astype(np.float64)
    for i in layer_runs(cfg):
        L, pre = cfg["layers"][i], f"l{i}."
        h = layer_norm(x, W[pre + "norm1"], W[pre + "norm1.b"], eps)
        mw = {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mix.")}
        if L["type"] == "latent_attention":
            y = latent_attention(h, mw, L["mixer"], eps)
        elif L["type"] == "parallel":
            y = mixer_pair(h, mw, L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            fw = {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mlp.")}
            y = y + experts(h, fw, L["mlp"], margins)
        x = x + y
        if taps is not None:
            taps.append(x.copy())
    xn = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return (xn @ W["head"].T) * cfg.get("logit_scale", 1.0)
