"""Plain numpy restatement (float64) of the Rumurax design, one function per mechanism, whole sequences only.

It shares no code with the engine. A model is a configuration dict (the content of config.json) and a dict of tensors by
name. Notation: T tokens, E width, S streams, H query heads, G key/value heads, D key size, V value size, p / j positions.

    streams      x_1 .. x_S start as the embedding row. Sub-layer q of a layer (1 mixer, 2 feed-forward):
                 u = sum_s a_q[s] x_s;  y = f_q(u / rms(u) * g_q);  x_t <- sum_s M_q[s, t] x_s + b_q[t] y
                 (g_q one number). The residual after a layer and the head's input are sum_s x_s.
    attention    grouped heads, q and k RMS-normed per head with a weight, optional rotation of neighbouring pairs,
                 score (q.k) scale, optional cap c tanh(. / c), optional distance penalty r1 ln(1 + r2 (p - j)),
                 a chunk mask (same floor(p / n)) or a sliding window of n tokens with means of blocks of P cached
                 keys / values standing in for what lies wholly before the window, optional sink in the denominator,
                 optional value mixing with the first mixing layer's values, optional per-head sigmoid gate.
    latent       keys and values through a normed latent plus one rotated key part for all heads, causal, gated
                 element by element.
    mixture      sigmoid router, the `top` best experts, each run on (score x input), plus a shared gated unit.
"""
import numpy as np


def scalar(x):
    return float(np.asarray(x).reshape(-1)[0])


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rotate_pairs(x, pos, base, dims):
    """x [T, heads, D]: entries (2i, 2i + 1), i < dims / 2, turned by pos * base^(-2i / dims); the rest unchanged."""
    out = np.array(x, dtype=np.float64)
    i = np.arange(dims // 2)
    ang = np.asarray(pos, dtype=np.float64)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def gated_unit(h, Wg, Wu, Wd):
    return (silu(h @ Wg.T) * (h @ Wu.T)) @ Wd.T


def visible_chunk(p, n):
    """positions j that p sees under a chunk mask of n"""
    return np.arange((p // n) * n, p + 1)


def visible_window(p, n, P):
    """(token positions, block indices) that p sees: the last n tokens and every block of P tokens that ends at or before p - n"""
    toks = np.arange(max(0, p - n + 1), p + 1)
    nb = 0
    if P and p - n >= 0:
        nb = (p - n + 1) // P                    # blocks b with b P + P - 1 <= p - n
    return toks, np.arange(nb)


def softmax_sink(s, sink):
    m = np.max(s) if sink is None else max(np.max(s), sink)
    e = np.exp(s - m)
    den = e.sum() + (0.0 if sink is None else np.exp(sink - m))
    return e / den


def attention(h, mx, W, pre, eps, kind, v_first):
    """kind 'chunk' | 'window'. Returns (output [T, E], values as cached [T, G, V])."""
    T = h.shape[0]
    H, G, D, V = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, D)
    k = (h @ W[pre + "k"].T).reshape(T, G, D)
    v = (h @ W[pre + "v"].T).reshape(T, G, V)
    q = rms_unit(q, eps) * W[pre + "q.norm"]
    k = rms_unit(k, eps) * W[pre + "k.norm"]
    pos = np.arange(T)
    if "rot" in mx:
        q = rotate_pairs(q, pos, mx["rot"]["base"], mx["rot"]["dims"])
        k = rotate_pairs(k, pos, mx["rot"]["base"], mx["rot"]["dims"])
    if mx.get("v_mix") and v_first is not None:
        lam = scalar(W[pre + "vmix"])
        v = (1.0 - lam) * v + lam * v_first
    n = mx["mask"]["size"]
    P = mx["mask"].get("pool", 0) if kind == "window" else 0
    cap = mx.get("softcap", 0.0)
    r1, r2 = W.get(pre + "r1"), W.get(pre + "r2")
    sink = W.get(pre + "sink")
    nblk = T // P if P else 0                   # whole blocks of the sequence: means of the keys and values as cached
    kb = np.stack([k[b * P:(b + 1) * P].mean(axis=0) for b in range(nblk)]) if nblk else None
    vb = np.stack([v[b * P:(b + 1) * P].mean(axis=0) for b in range(nblk)]) if nblk else None
    out = np.zeros((T, H, V))
    for p in range(T):
        if kind == "chunk":
            toks, blocks = visible_chunk(p, n), np.arange(0)
        else:
            toks, blocks = visible_window(p, n, P)
        for hh in range(H):
            g = hh // (H // G)
            keys, vals = [k[toks, g]], [v[toks, g]]
            dist = [(p - toks).astype(np.float64)]
            if len(blocks):
                keys.append(kb[blocks, g])
                vals.append(vb[blocks, g])
                dist.append(np.zeros(len(blocks)))
            keys, vals, dist = np.concatenate(keys), np.concatenate(vals), np.concatenate(dist)
            s = (keys @ q[p, hh]) * mx["scale"]
            if cap:
                s = cap * np.tanh(s / cap)
            if r1 is not None:
                s = s - r1[hh] * np.log1p(r2[hh] * dist)
            w = softmax_sink(s, None if sink is None else float(sink[hh]))
            out[p, hh] = w @ vals
    if pre + "g" in W:
        out = out * sigmoid(h @ W[pre + "g"].T)[:, :, None]
    return out.reshape(T, H * V) @ W[pre + "o"].T, v


def latent_attention(h, mx, W, pre, eps):
    T = h.shape[0]
    H, D, R, V, rank = mx["heads"], mx["dim"], mx.get("rot_dim", 0), mx["vdim"], mx["kv_rank"]
    q = (h @ W[pre + "q"].T).reshape(T, H, D + R)
    dkv = h @ W[pre + "dkv"].T
    c = rms_unit(dkv[:, :rank], eps) * W[pre + "dkv.norm"]
    ku = (c @ W[pre + "uk"].T).reshape(T, H, D)
    vv = (c @ W[pre + "uv"].T).reshape(T, H, V)
    qu, qr, kr = q[..., :D], q[..., D:], dkv[:, None, rank:]
    if R and "rot" in mx:
        pos = np.arange(T)
        qr = rotate_pairs(qr, pos, mx["rot"]["base"], mx["rot"]["dims"])
        kr = rotate_pairs(kr, pos, mx["rot"]["base"], mx["rot"]["dims"])
    out = np.zeros((T, H, V))
    for p in range(T):
        for hh in range(H):
            s = (ku[:p + 1, hh] @ qu[p, hh] + kr[:p + 1, 0] @ qr[p, hh]) * mx["scale"]
            out[p, hh] = softmax_sink(s, None) @ vv[:p + 1, hh]
    out = out.reshape(T, H * V)
    if pre + "g" in W:
        out = out * sigmoid(h @ W[pre + "g"].T)
    return out @ W[pre + "o"].T


def route(h, Wr, top):
    """experts [T, top] (best first; the lower index among equals) and their scores"""
    s = sigmoid(h @ Wr.T)
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=-1)


def mixture(h, mj, W, pre):
    T = h.shape[0]
    sel, wt = route(h, W[pre + "router"], mj["router"]["top"])
    y = np.zeros_like(h)
    for t in range(T):
        for e, w in zip(sel[t], wt[t]):
            ep = pre + "e%d." % e
            y[t] += gated_unit(w * h[t], W[ep + "gate"], W[ep + "up"], W[ep + "down"])
    if mj.get("shared"):
        y += gated_unit(h, W[pre + "shared.gate"], W[pre + "shared.up"], W[pre + "shared.down"])
    return y


def forward(cfg, W, tokens):
    """logits [T, vocab] and the residual (sum of the streams) after every layer [layers, T, E]"""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    S = cfg.get("streams", 1)
    x0 = W["embed"][np.asarray(tokens)]
    xs = np.stack([x0] * S)
    v_first = None
    taps = []
    for i, lj in enumerate(cfg["layers"]):
        p = "l%d." % i
        for q in (1, 2):
            if q == 2 and not lj.get("mlp"):
                continue
            hp = p + "hc%d." % q
            if hp + "in" in W:
                a, M, b = W[hp + "in"], W[hp + "mix"], W[hp + "out"]
            else:
                a, M, b = np.ones(1), np.ones((1, 1)), np.ones(1)
            u = np.tensordot(a, xs, axes=(0, 0))
            hn = rms_unit(u, eps) * scalar(W[p + "norm%d" % q])
            if q == 2:
                y = mixture(hn, lj["mlp"], W, p + "mlp.")
            elif lj["type"] == "latent_attention":
                y = latent_attention(hn, lj["mixer"], W, p + "mix.", eps)
            else:
                kind = "chunk" if lj["type"] == "attention" else "window"
                y, v = attention(hn, lj["mixer"], W, p + "mix.", eps, kind, v_first)
                if lj["mixer"].get("v_mix") and v_first is None:
                    v_first = v
            xs = np.tensordot(M.T, xs, axes=(1, 0)) + b[:, None, None] * y[None]
        taps.append(xs.sum(axis=0))
    x = xs.sum(axis=0)
    logits = (rms_unit(x, eps) * scalar(W["final.norm"])) @ W["head"].T
    return logits, np.stack(taps)


def tensor_shapes(cfg):
    """tensor name -> shape of a model file of this design"""
    E, Vc, S = cfg["width"], cfg["vocab"], cfg.get("streams", 1)
    t = {"embed": [Vc, E]}
    for i, lj in enumerate(cfg["layers"]):
        p, mx = "l%d." % i, lj["mixer"]
        subs = (1, 2) if lj.get("mlp") else (1,)
        for q in subs:
            t[p + "norm%d" % q] = []
            t[p + "hc%d.in" % q] = [S]
            t[p + "hc%d.out" % q] = [S]
            t[p + "hc%d.mix" % q] = [S, S]
        m = p + "mix."
        H, D, V = mx["heads"], mx["dim"], mx["vdim"]
        if lj["type"] == "latent_attention":
            R, rank = mx.get("rot_dim", 0), mx["kv_rank"]
            t.update({m + "q": [H * (D + R), E], m + "dkv": [rank + R, E], m + "dkv.norm": [rank], m + "uk": [H * D, rank], m + "uv": [H * V, rank],
                      m + "g": [H * V, E], m + "o": [E, H * V]})
        else:
            G = mx.get("kv_heads", H)
            t.update({m + "q": [H * D, E], m + "k": [G * D, E], m + "v": [G * V, E], m + "q.norm": [D], m + "k.norm": [D], m + "o": [E, H * V]})
            if mx.get("v_mix"):
                t[m + "vmix"] = []
            if lj["type"] == "attention":
                t.update({m + "r1": [H], m + "r2": [H], m + "sink": [H], m + "g": [H, E]})
        if lj.get("mlp"):
            mj, f = lj["mlp"], p + "mlp."
            units = [("e%d." % e, mj["expert"]["ff"]) for e in range(mj["router"]["experts"])]
            if mj.get("shared"):
                units.append(("shared.", mj["shared"]["ff"]))
            for u, ff in units:
                t.update({f + u + "gate": [ff, E], f + u + "up": [ff, E], f + u + "down": [E, ff]})
            t[f + "router"] = [mj["router"]["experts"], E]
    t["final.norm"] = []
    t["head"] = [Vc, E]
    return t


def random_model(cfg, seed=0):
    """random weights rounded to bfloat16 (what a model file holds): matrices ~ N(0, 1/in), norm weights near 1, router rows spread
    so that the choice of experts is never a close call, stream weights near (read the mean, keep every stream, write to all)"""
    import stack_oracle as so
    rng = np.random.default_rng(seed)
    S = cfg.get("streams", 1)
    W = {}
    for name, shp in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if ".hc" in name:
            if leaf == "in":
                x = 1.0 / S + 0.2 * rng.standard_normal(shp)
            elif leaf == "out":
                x = 1.0 + 0.3 * rng.standard_normal(shp)
            else:
                x = np.eye(S) + 0.2 * rng.standard_normal(shp)
        elif leaf == "router":
            x = rng.standard_normal(shp) * (3.0 / np.sqrt(shp[1]))
        elif leaf == "r1":
            x = 0.3 + 0.5 * rng.random(shp)
        elif leaf == "r2":
            x = 0.2 + 1.5 * rng.random(shp)
        elif leaf == "sink":
            x = rng.standard_normal(shp)
        elif leaf == "vmix":
            x = np.asarray(0.25 + 0.5 * rng.random())
        elif len(shp) == 2:
            x = rng.standard_normal(shp) / np.sqrt(shp[1])
        elif len(shp) == 0:
            x = np.asarray(1.0 + 0.1 * rng.standard_normal())
        else:
            x = 1.0 + 0.1 * rng.standard_normal(shp)
        W[name] = so.round_bf16(np.asarray(x, np.float32)).astype(np.float64).reshape(shp)
    return W


def write_model(d, cfg, W):
    import json
    import os
    import stack_oracle as so
    os.makedirs(d, exist_ok=True)
    so.save_safetensors(os.path.join(d, "model.safetensors"), {k: np.asarray(v, np.float32) for k, v in W.items()})
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return d
