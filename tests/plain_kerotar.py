"""Plain implementation of the Kerotar design: NumPy, float64, whole sequences, no cache, one function per
mechanism, loops over tokens, heads and keys.  Shares nothing with the library; slow on purpose.

Notation: n tokens, D width, H heads, G key/value heads, d head width, e value width, r latent width,
p rotated width.  A weight W [out, in] is applied as W x."""
from __future__ import annotations

import math

import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rmsnorm(x, w, eps):
    return rms(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rotate_half(vec, pos, base, dims):
    """Rotates the first `dims` entries of one vector: entry i pairs with entry i + dims/2."""
    out = np.array(vec, dtype=np.float64)
    half = dims // 2
    for i in range(half):
        a = pos * base ** (-2.0 * i / dims)
        u, v = vec[i], vec[i + half]
        out[i] = u * math.cos(a) - v * math.sin(a)
        out[i + half] = v * math.cos(a) + u * math.sin(a)
    return out


def visible(i, j, size, keep_first):
    """Whether query position i sees key position j: causal, inside a window of `size` (0 = no window)
    or among the first `keep_first` tokens."""
    if j > i:
        return False
    if size <= 0:
        return True
    return i - j < size or j < keep_first


def softmax_rows(scores, sink=None):
    """Softmax over a list of scores; `sink` is one more term of the denominator without a value."""
    m = max(scores) if sink is None else max(max(scores), sink)
    e = [math.exp(s - m) for s in scores]
    z = sum(e) + (0.0 if sink is None else math.exp(sink - m))
    return [x / z for x in e]


def window_attention(h, W, m, eps, pos0=0):
    """Grouped-query attention with q/k norms over the whole projection, a partial rotation, a window that keeps
    the first tokens, and a sink per head.  h [n, D]; W: q, k, v, o, q.norm, k.norm, sink; m: heads, kv_heads,
    dim, vdim, scale, rot (base, dims) or None, mask (size, keep_first) or None."""
    n = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot, mask = m.get("rot"), m.get("mask")
    q = rmsnorm(h @ W["q"].T, W["q.norm"], eps)
    k = rmsnorm(h @ W["k"].T, W["k.norm"], eps)
    v = h @ W["v"].T
    q = q.reshape(n, H, d).copy()
    k = k.reshape(n, G, d).copy()
    v = v.reshape(n, G, e)
    if rot:
        for t in range(n):
            for a in range(H):
                q[t, a] = rotate_half(q[t, a], pos0 + t, rot["base"], rot["dims"])
            for a in range(G):
                k[t, a] = rotate_half(k[t, a], pos0 + t, rot["base"], rot["dims"])
    size, keep = (mask["size"], mask.get("keep_first", 0)) if mask else (0, 0)
    out = np.zeros((n, H, e))
    for t in range(n):
        for a in range(H):
            g = a // (H // G)
            js = [j for j in range(t + 1) if visible(t, j, size, keep)]
            sc = [float(q[t, a] @ k[j, g]) * m["scale"] for j in js]
            w = softmax_rows(sc, float(W["sink"][a]) if "sink" in W else None)
            for wj, j in zip(w, js):
                out[t, a] += wj * v[j, g]
    return out.reshape(n, H * e) @ W["o"].T


def latent_attention(h, W, m, eps, pos0=0):
    """Attention whose keys and values are expanded from one latent vector per token, with one rotated key part
    shared by all heads and a sigmoid gate per head on the output.  W: dq, dq.norm, uq, dkv, dkv.norm, uk, uv,
    g, o; m: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot.base."""
    n = h.shape[0]
    H, d, p, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base = m["rot"]["base"]
    cq = rmsnorm(h @ W["dq"].T, W["dq.norm"], eps)
    q = (cq @ W["uq"].T).reshape(n, H, d + p)
    dkv = h @ W["dkv"].T
    c = rmsnorm(dkv[:, :r], W["dkv.norm"], eps)
    kr = np.stack([rotate_half(dkv[t, r:], pos0 + t, base, p) for t in range(n)])
    ku = (c @ W["uk"].T).reshape(n, H, d)
    v = (c @ W["uv"].T).reshape(n, H, e)
    gate = sigmoid(h @ W["g"].T)
    out = np.zeros((n, H, e))
    for t in range(n):
        for a in range(H):
            qu, qr = q[t, a, :d], rotate_half(q[t, a, d:], pos0 + t, base, p)
            sc = [(float(qu @ ku[j, a]) + float(qr @ kr[j])) * m["scale"] for j in range(t + 1)]
            w = softmax_rows(sc)
            for j, wj in enumerate(w):
                out[t, a] += wj * v[j, a]
            out[t, a] *= gate[t, a]
    return out.reshape(n, H * e) @ W["o"].T


def clamped_glu(h, W, limit):
    """Dense feed-forward: gate capped from above, up clamped on both sides, sigmoid-1.702 gate, (up + 1)."""
    g = np.minimum(h @ W["gate"].T, limit)
    u = np.clip(h @ W["up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W["down"].T


def routed_experts(h, W, experts, top, margins=None):
    """Softmax router over all experts, the `top` largest taken, their scores renormalised.  `margins` (a list of
    n numbers, or None) is lowered, per token, to the gap between the last chosen logit and the first one left out,
    relative to the largest |logit|: how close the choice came to falling the other way."""
    n = h.shape[0]
    out = np.zeros((n, W["e0.down"].shape[0]))
    for t in range(n):
        z = W["router"] @ h[t]
        s = np.exp(z - z.max())
        s = s / s.sum()
        order = sorted(range(experts), key=lambda i: (-s[i], i))
        chosen = order[:top]
        if margins is not None and top < experts:
            margins[t] = min(margins[t], float(z[order[top - 1]] - z[order[top]]) / float(np.abs(z).max()))
        total = sum(s[i] for i in chosen) + 1e-20
        for i in chosen:
            g, u = W[f"e{i}.gate"] @ h[t], W[f"e{i}.up"] @ h[t]
            out[t] += (s[i] / total) * (W[f"e{i}.down"] @ (g * sigmoid(g) * u))
    return out


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def layer(x, weights, i, L, eps, pos0=0, margins=None):
    """One parallel layer: both sublayers read the same normalised rows, x + mixer + feed-forward."""
    h = rmsnorm(x, weights[f"l{i}.norm1"], eps)
    Wm = sub(weights, f"l{i}.mix.")
    if L["type"] == "attention":
        y = window_attention(h, Wm, L["mixer"], eps, pos0)
    elif L["type"] == "latent_attention":
        y = latent_attention(h, Wm, L["mixer"], eps, pos0)
    else:
        raise ValueError(L["type"])
    mlp = L.get("mlp")
    if mlp is not None:
        Wf = sub(weights, f"l{i}.mlp.")
        if mlp["kind"] == "dense":
            y = y + clamped_glu(h, Wf, mlp["limit"])
        elif mlp["kind"] == "moe":
            y = y + routed_experts(h, Wf, mlp["router"]["experts"], mlp["router"]["top"], margins)
        else:
            raise ValueError(mlp["kind"])
    return x + y


def run_order(cfg):
    """[(layer, pass number or None)]: pass number set on the run that opens a pass of the loop."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], n)]


def forward(cfg, weights, tokens, taps=None, margins=None):
    """Logits [n, vocab] of one whole sequence; `taps` (a list) receives the rows after every layer run; `margins`
    (a list of n numbers) is lowered to every token's closest expert choice (see routed_experts)."""
    weights = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x0 = weights["embed"][np.asarray(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    x = x0.copy()
    for i, t in run_order(cfg):
        if t is not None:
            x = np.concatenate([x, x0], axis=1) @ weights["loop.in"].T + weights["loop.step"][t]
        x = layer(x, weights, i, cfg["layers"][i], eps, margins=margins)
        if taps is not None:
            taps.append(x.copy())
    return rmsnorm(x, weights["final.norm"], eps) @ weights["head"].T
