"""Plain, slow restatement of the Tosevik design in numpy float64: one function per mechanism, written from the equations and
not from the kernels; recurrences and attention walk whole sequences. Test infrastructure only: nothing here is shared
with the CUDA path (the safetensors writer of stack_oracle.py, also test infrastructure, is reused for the model files).

Notation: a mechanism gets the whole sequence h [T, width] and returns [T, width]; matrices are stored [out, in], so a
projection is h @ M.T; positions count from 0.

Design in short. Norms are element-wise: dyt(x) = tanh(a x) w + b. x_0 = dyt(embed[token]). Layer i: y = z + mix(dyt1(z)),
y = y + ff(dyt2(y)) when the layer has a feed-forward; y is kept as x_(i+1), and the next layer (or the head) reads
z = sum_(j <= i+1) c_i[j] x_j. Mixers: retention (matrix state with a constant decay per head, rotated queries and keys),
parallel (the mean of two normed branches: a sigmoid attention with a linear distance penalty and a retention). The
feed-forward is a routed mixture of gated units with group-limited choice plus a gated shared unit.
"""
from __future__ import annotations

import numpy as np

import stack_oracle as so

F = np.float64


def sigm(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigm(x)


def unit_rms(x, eps):
    """x over the root of (mean square + eps), along the last axis"""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def dyt(x, W, name):
    """element-wise norm without statistics: tanh(alpha x) w + b"""
    return np.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def rotate_front(x, pos, rot):
    """x [T, heads, dim]: entries i and i + n/2 of the first n = rot.dims form a pair turned by pos * base^(-2i/n)"""
    n = int(rot["dims"])
    half = n // 2
    f = float(rot["base"]) ** (-2.0 * np.arange(half) / n)
    ang = np.asarray(pos, F)[:, None] * f[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    y = x.copy()
    a, b = x[..., :half], x[..., half:n]
    y[..., :half] = a * c - b * s
    y[..., half:n] = b * c + a * s
    return y


def mix_retention(h, W, mx, eps):
    """S <- decay_h S + k v^T, o = S^T q per head: a plain decayed sum, nothing divides the read-out"""
    T = h.shape[0]
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    pos = np.arange(T)
    q = rotate_front((h @ W["q"].T).reshape(T, H, D), pos, mx["rot"])
    k = rotate_front((h @ W["k"].T).reshape(T, H, D), pos, mx["rot"]) * D ** -0.5
    v = (h @ W["v"].T).reshape(T, H, V)
    out = np.zeros((T, H, V))
    for hd in range(H):
        S = np.zeros((D, V))
        for t in range(T):
            S = float(mx["decay"][hd]) * S + np.outer(k[t, hd], v[t, hd])
            out[t, hd] = q[t, hd] @ S
    out = unit_rms(out, eps).reshape(T, H * V) * silu(h @ W["g"].T)
    return out @ W["o"].T


def mix_sigmoid_attention(h, W, mx, eps):
    """grouped heads; queries and keys normed over their whole projection; each key weighs in by a sigmoid of its own"""
    T = h.shape[0]
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    pos = np.arange(T)
    q = unit_rms(h @ W["q"].T, eps) * W["q.norm"]
    k = unit_rms(h @ W["k"].T, eps) * W["k.norm"]
    qt = mx["q_temp"]
    q = q * (1.0 + qt["coef"] * np.log(np.floor((pos + 1) / qt["every"]) + 1.0))[:, None]
    q, k = q.reshape(T, H, D), k.reshape(T, G, D)
    v = unit_rms((h @ W["v"].T).reshape(T, G, V), eps)
    out = np.zeros((T, H, V))
    dist = pos[:, None] - pos[None, :]
    for hd in range(H):
        g = hd // (H // G)
        slope = 2.0 ** (-8.0 * (hd + 1) / H)
        s = (q[:, hd] @ k[:, g].T) * mx["scale"] - slope * dist + W["pb"][hd]
        w = np.where(dist >= 0, sigm(s), 0.0)
        out[:, hd] = w @ v[:, g]
    return out.reshape(T, H * V) @ W["o"].T


def mix_parallel(h, W, mx, eps):
    a = mix_sigmoid_attention(h, sub(W, "left."), mx["left"], eps)
    b = mix_retention(h, sub(W, "right."), mx["right"], eps)
    return 0.5 * (unit_rms(a, eps) * W["left.out"] + unit_rms(b, eps) * W["right.out"])


def gated_unit(h, W):
    return (silu(h @ W["gate"].T) * (h @ W["up"].T)) @ W["down"].T


def route(h, W, r):
    """-> chosen [T, top] expert indices and their weights: soft-max over all experts, the choice confined to the best-ranked blocks of experts"""
    z = h @ W["router"].T
    e = np.exp(z - z.max(-1, keepdims=True))
    s = e / e.sum(-1, keepdims=True)
    n, top = r["experts"], r["top"]
    gr = r.get("groups") or {"count": 1, "keep": 1}
    per = n // gr["count"]
    best = s.reshape(-1, gr["count"], per).max(-1)
    chosen, weight = [], []
    for t in range(h.shape[0]):
        keep = np.argsort(-best[t], kind="stable")[:gr["keep"]]
        ok = np.zeros(n, bool)
        for g in keep:
            ok[g * per:(g + 1) * per] = True
        idx = np.argsort(-np.where(ok, s[t], -1.0), kind="stable")[:top]
        chosen.append(idx)
        weight.append(s[t, idx] * r["scale"])
    return np.array(chosen), np.array(weight)


def mixture(h, W, mlp):
    chosen, weight = route(h, W, mlp["router"])
    y = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weight[t]):
            y[t] += w * gated_unit(h[t:t + 1], sub(W, f"e{e}."))[0]
    if mlp.get("shared"):
        y += sigm(h @ W["shared.sg"].T) * gated_unit(h, sub(W, "shared."))
    return y


def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


MIXERS = {"retention": mix_retention, "parallel": mix_parallel}


def forward(cfg, W, tokens, residuals=None):
    """logits [T, vocab]; residuals (a list) receives what each layer hands on, [T, width]"""
    W = {k: np.asarray(v, F) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    z = dyt(W["embed"][np.asarray(tokens)], W, "embed.norm")
    kept = [z]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = z + MIXERS[L["type"]](dyt(z, W, p + "norm1"), sub(W, p + "mix."), L["mixer"], eps)
        if L.get("mlp"):
            y = y + mixture(dyt(y, W, p + "norm2"), sub(W, p + "mlp."), L["mlp"])
        kept.append(y)
        z = sum(c * x for c, x in zip(W[p + "dwa"], kept))
        if residuals is not None:
            residuals.append(z)
    return dyt(z, W, "final.norm") @ W["head"].T


def norm_shapes(t, name, n):
    t[name] = [n]; t[name + ".b"] = [n]; t[name + ".alpha"] = []


def retention_shapes(t, p, mx, E):
    H, D, V = mx["heads"], mx["dim"], mx["vdim"]
    t.update({p + "q": [H * D, E], p + "k": [H * D, E], p + "v": [H * V, E], p + "g": [H * V, E], p + "o": [E, H * V]})


def tensor_shapes(cfg):
    E, V = cfg["width"], cfg["vocab"]
    t = {"embed": [V, E]}
    norm_shapes(t, "embed.norm", E)
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        norm_shapes(t, p + "norm1", E)
        if L["type"] == "retention":
            retention_shapes(t, p + "mix.", mx, E)
        else:
            a = mx["left"]
            H, G, D, Vd = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            t.update({p + "mix.left.q": [H * D, E], p + "mix.left.k": [G * D, E], p + "mix.left.v": [G * Vd, E], p + "mix.left.q.norm": [H * D],
                      p + "mix.left.k.norm": [G * D], p + "mix.left.pb": [H], p + "mix.left.o": [E, H * Vd], p + "mix.left.out": [E], p + "mix.right.out": [E]})
            retention_shapes(t, p + "mix.right.", mx["right"], E)
        if L.get("mlp"):
            m = L["mlp"]
            norm_shapes(t, p + "norm2", E)
            units = [(f"e{e}.", m["expert"]["ff"]) for e in range(m["router"]["experts"])]
            if m.get("shared"):
                units.append(("shared.", m["shared"]["ff"]))
                t[p + "mlp.shared.sg"] = [1, E]
            for u, ff in units:
                t.update({p + "mlp." + u + "gate": [ff, E], p + "mlp." + u + "up": [ff, E], p + "mlp." + u + "down": [E, ff]})
            t[p + "mlp.router"] = [m["router"]["experts"], E]
        t[p + "dwa"] = [i + 2]
    norm_shapes(t, "final.norm", E)
    t["head"] = [V, E]
    return t


def random_model(cfg, seed=0):
    """random weights rounded to bfloat16 (what a model file holds): matrices ~ N(0, 1/in), norm weights near 1, router rows
    spread so that the choice of experts is never a close call, depth coefficients that weigh every earlier layer"""
    rng = np.random.default_rng(seed)
    W = {}
    for name, shp in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if name.endswith(".alpha"):
            x = np.asarray(0.6 + 0.3 * rng.random())
        elif leaf == "router":
            x = rng.standard_normal(shp) * (3.0 / np.sqrt(shp[1]))
        elif leaf == "dwa":
            x = 0.3 * rng.standard_normal(shp)
            x[-1] += 1.0
        elif leaf == "pb":
            x = rng.standard_normal(shp) - 1.0
        elif leaf == "b":
            x = 0.1 * rng.standard_normal(shp)
        elif len(shp) == 2:
            x = rng.standard_normal(shp) / np.sqrt(shp[1])
        else:
            x = 1.0 + 0.1 * rng.standard_normal(shp)
        W[name] = so.round_bf16(np.asarray(x, np.float32)).astype(F)
    return W


def write_model(d, cfg, W):
    import json
    import os
    os.makedirs(d, exist_ok=True)
    so.save_safetensors(os.path.join(d, "model.safetensors"), {k: np.asarray(v, np.float32) for k, v in W.items()})
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return d
