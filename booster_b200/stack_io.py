"""Synthetic models of the layer-stack family (Matulorn, Dopilorn, Tosevik and Rumurax designs; config.json + model.safetensors) for benchmarks and smoke runs: random
bfloat16 weights of the right shapes, the counterpart of gguf_io.synth_llama for the GGUF path. Pure host code."""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List

import numpy as np


def matulorn_config(width: int, n_layer: int, ff: int, heads: int, vocab: int = 32000, head_dim: int = 128, rot_dim: int = 64,
                    kv_rank: int = 512, window: int = 1024, groups: int = 8, pattern=("mingru", "latent_attention", "delta", "latent_attention")) -> dict:
    """a configuration whose layers resemble a real model's: mixers in `pattern` order, a feed-forward on every layer"""
    layers = []
    for i in range(n_layer):
        kind = pattern[i % len(pattern)]
        if kind == "mingru":
            mx = {"width": width}
        elif kind == "latent_attention":
            mx = {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "kv_rank": kv_rank, "scale": (head_dim + rot_dim) ** -0.5,
                  "mask": {"size": window},
                  "rot": {"base": 500000.0, "dims": rot_dim, "scaling": {"factor": 8.0, "fast": 32.0, "slow": 1.0, "original": 4096}}}
        else:
            mx = {"heads": heads, "kv_heads": max(1, heads // 2), "dim": head_dim, "vdim": head_dim, "conv": 4}
        layers.append({"type": kind, "mixer": mx, "mlp": {"ff": ff, "kind": "dense", "limit": 7.0}})
    return {"architecture": "Matulorn", "layers": layers, "norm": {"eps": 1e-6, "groups": groups}, "vocab": vocab, "width": width}


def dopilorn_config(width: int, n_layer: int, ff: int, heads: int, vocab: int = 32000, head_dim: int = 128, q_rank: int = 768, kv_rank: int = 512,
                    window: int = 1024, kv_heads: int = 0, decay_rank: int = 64, taps: int = 4, loop=(2, 5, 2),
                    pattern=("latent_attention", "general_delta", "attention")) -> dict:
    """a Dopilorn configuration whose layers resemble a real model's: mixers in `pattern` order, a polynomial feed-forward on every
    layer, layers loop[0] .. loop[1] - 1 run loop[2] times. `decay_rank` is not a key the loader reads (it takes the rank from the
    tensor's shape); tensor_shapes() does."""
    layers = []
    for i in range(n_layer):
        kind = pattern[i % len(pattern)]
        if kind == "latent_attention":
            mx = {"heads": heads, "dim": head_dim, "vdim": head_dim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": head_dim ** -0.5}
        elif kind == "general_delta":
            mx = {"heads": heads, "dim": head_dim, "decay_rank": decay_rank}
        else:
            mx = {"heads": heads, "kv_heads": kv_heads or max(1, heads // 4), "dim": head_dim // 2, "vdim": head_dim, "conv": 4, "diff": 0.5,
                  "scale": (head_dim // 2) ** -0.5, "mask": {"size": window}}
        layers.append({"type": kind, "mixer": mx, "mlp": {"ff": ff, "kind": "dense"}})
    if loop and loop[1] > n_layer:                       # few layers: the span ends with the last one
        loop = (min(loop[0], n_layer - 1), n_layer, loop[2])
    cfg = {"architecture": "Dopilorn", "canon": {"taps": taps}, "layers": layers, "logit_softcap": 50.0, "norm": {"eps": 1e-6}, "vocab": vocab, "width": width}
    if loop and loop[1] > loop[0] and loop[1] <= n_layer:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def tosevik_config(width: int, n_layer: int, ff: int, heads: int, vocab: int = 32000, head_dim: int = 128, kv_heads: int = 0, experts: int = 16, top: int = 4,
                   groups=(4, 2), pattern=("retention", "parallel")) -> dict:
    """a Tosevik configuration whose layers resemble a real model's: mixers in `pattern` order, a routed mixture on every layer whose
    chosen experts plus the shared unit are as wide together as a dense feed-forward of `ff` (top x 3 ff / 16 + ff / 4)"""
    def ret(h, dim, vdim):
        return {"heads": h, "dim": dim, "vdim": vdim, "rot": {"base": 500000.0, "dims": dim // 2},
                "decay": [1.0 - 2.0 ** (-5.0 - 3.0 * i / h) for i in range(h)]}
    e_ff = max(8, ff * 3 // (4 * top) // 8 * 8)
    layers = []
    for i in range(n_layer):
        kind = pattern[i % len(pattern)]
        if kind == "retention":
            mx = ret(heads, head_dim, head_dim)
        else:
            mx = {"left": {"heads": heads, "kv_heads": kv_heads or max(1, heads // 4), "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5,
                           "q_temp": {"coef": 0.1, "every": 1024}},
                  "right": ret(heads, head_dim // 2, head_dim)}
        mlp = {"kind": "moe", "expert": {"ff": e_ff}, "shared": {"ff": ff - top * e_ff},
               "router": {"experts": experts, "top": top, "scale": 2.5, "groups": {"count": groups[0], "keep": groups[1]}}}
        layers.append({"type": kind, "mixer": mx, "mlp": mlp})
    return {"architecture": "Tosevik", "layers": layers, "norm": {"eps": 1e-6}, "vocab": vocab, "width": width}


def rumurax_config(width: int, n_layer: int, ff: int, heads: int, vocab: int = 32000, head_dim: int = 128, kv_heads: int = 0, experts: int = 16, top: int = 4,
                   streams: int = 4, window: int = 1024, pool: int = 32, chunk: int = 1024, kv_rank: int = 512, rot_dim: int = 64,
                   pattern=("attention", "attention_2", "attention", "latent_attention")) -> dict:
    """a Rumurax configuration whose layers resemble a real model's: mixers in `pattern` order, a routed mixture on every layer whose
    chosen experts plus the shared unit are as wide together as a dense feed-forward of `ff` (top x 3 ff / 16 + ff / 4)"""
    e_ff = max(8, ff * 3 // (4 * top) // 8 * 8)
    G = kv_heads or max(1, heads // 4)
    layers = []
    for i in range(n_layer):
        kind = pattern[i % len(pattern)]
        if kind == "attention_2":
            mx = {"heads": heads, "kv_heads": G, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "mask": {"size": window, "pool": pool},
                  "rot": {"base": 500000.0, "dims": head_dim // 2}, "v_mix": True}
        elif kind == "attention":
            mx = {"heads": heads, "kv_heads": G, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "mask": {"size": chunk}, "softcap": 50.0, "v_mix": True}
        else:
            mx = {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "kv_rank": kv_rank, "scale": (head_dim + rot_dim) ** -0.5,
                  "rot": {"base": 500000.0, "dims": rot_dim}}
        mlp = {"kind": "moe", "expert": {"ff": e_ff}, "shared": {"ff": ff - top * e_ff}, "router": {"experts": experts, "top": top}}
        layers.append({"type": kind, "mixer": mx, "mlp": mlp})
    return {"architecture": "Rumurax", "layers": layers, "norm": {"eps": 1e-6}, "streams": streams, "vocab": vocab, "width": width}


def rumurax_shapes(cfg: dict) -> Dict[str, List[int]]:
    E, V, S = cfg["width"], cfg["vocab"], cfg.get("streams", 1)
    t: Dict[str, List[int]] = {"embed": [V, E]}
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        for q in ((1, 2) if L.get("mlp") else (1,)):
            t.update({f"{p}norm{q}": [], f"{p}hc{q}.in": [S], f"{p}hc{q}.out": [S], f"{p}hc{q}.mix": [S, S]})
        H, D, Vd, m = mx["heads"], mx["dim"], mx["vdim"], p + "mix."
        if L["type"] == "latent_attention":
            R, rank = mx.get("rot_dim", 0), mx["kv_rank"]
            t.update({m + "q": [H * (D + R), E], m + "dkv": [rank + R, E], m + "dkv.norm": [rank], m + "uk": [H * D, rank], m + "uv": [H * Vd, rank],
                      m + "g": [H * Vd, E], m + "o": [E, H * Vd]})
        elif L["type"] in ("attention", "attention_2"):
            G = mx.get("kv_heads", H)
            t.update({m + "q": [H * D, E], m + "k": [G * D, E], m + "v": [G * Vd, E], m + "q.norm": [D], m + "k.norm": [D], m + "o": [E, H * Vd]})
            if mx.get("v_mix"):
                t[m + "vmix"] = []
            if L["type"] == "attention":
                t.update({m + "r1": [H], m + "r2": [H], m + "sink": [H], m + "g": [H, E]})
        else:
            raise ValueError(L["type"])
        mj = L.get("mlp")
        if mj:
            units = [(f"e{e}.", mj["expert"]["ff"]) for e in range(mj["router"]["experts"])]
            if mj.get("shared"):
                units.append(("shared.", mj["shared"]["ff"]))
            for u, f in units:
                t.update({p + "mlp." + u + "gate": [f, E], p + "mlp." + u + "up": [f, E], p + "mlp." + u + "down": [E, f]})
            t[p + "mlp.router"] = [mj["router"]["experts"], E]
    t["final.norm"] = []
    t["head"] = [V, E]
    return t


def tosevik_shapes(cfg: dict) -> Dict[str, List[int]]:
    E, V = cfg["width"], cfg["vocab"]
    t: Dict[str, List[int]] = {"embed": [V, E]}

    def norm(name):
        t[name] = [E]; t[name + ".b"] = [E]; t[name + ".alpha"] = []

    def ret(p, mx):
        H, D, Vd = mx["heads"], mx["dim"], mx["vdim"]
        t.update({p + "q": [H * D, E], p + "k": [H * D, E], p + "v": [H * Vd, E], p + "g": [H * Vd, E], p + "o": [E, H * Vd]})
    norm("embed.norm")
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        norm(p + "norm1")
        if L["type"] == "retention":
            ret(p + "mix.", mx)
        elif L["type"] == "parallel":
            a = mx["left"]
            H, G, D, Vd = a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a["vdim"]
            q = p + "mix.left."
            t.update({q + "q": [H * D, E], q + "k": [G * D, E], q + "v": [G * Vd, E], q + "q.norm": [H * D], q + "k.norm": [G * D], q + "pb": [H], q + "o": [E, H * Vd],
                      q + "out": [E], p + "mix.right.out": [E]})
            ret(p + "mix.right.", mx["right"])
        else:
            raise ValueError(L["type"])
        m = L.get("mlp")
        if m:
            norm(p + "norm2")
            units = [(f"e{e}.", m["expert"]["ff"]) for e in range(m["router"]["experts"])]
            if m.get("shared"):
                units.append(("shared.", m["shared"]["ff"]))
                t[p + "mlp.shared.sg"] = [1, E]
            for u, f in units:
                t.update({p + "mlp." + u + "gate": [f, E], p + "mlp." + u + "up": [f, E], p + "mlp." + u + "down": [E, f]})
            t[p + "mlp.router"] = [m["router"]["experts"], E]
        t[p + "dwa"] = [i + 2]
    norm("final.norm")
    t["head"] = [V, E]
    return t


def n_layer_runs(cfg: dict) -> int:
    lp = cfg.get("loop")
    return len(cfg["layers"]) + ((lp["stop"] - lp["start"]) * (lp["times"] - 1) if lp else 0)


def dopilorn_shapes(cfg: dict) -> Dict[str, List[int]]:
    E, V = cfg["width"], cfg["vocab"]
    t = {"embed": [V, E]}
    lp, ct = cfg.get("loop"), (cfg.get("canon") or {}).get("taps", 0)
    if lp:
        t["loop.in"] = [E, 2 * E]; t["loop.step"] = [lp["times"], E]
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        t[p + "norm1"] = [E]
        if ct:
            t[p + "canon1"] = [E, ct]
        if L["type"] == "latent_attention":
            H, D, Vd, qr, kr = mx["heads"], mx["dim"], mx["vdim"], mx["q_rank"], mx["kv_rank"]
            t.update({p + "mix.dq": [qr, E], p + "mix.dq.norm": [qr], p + "mix.uq": [H * D, qr], p + "mix.dkv": [kr, E], p + "mix.dkv.norm": [kr],
                      p + "mix.uk": [H * D, kr], p + "mix.uv": [H * Vd, kr], p + "mix.g": [H, E], p + "mix.o": [E, H * Vd]})
        elif L["type"] == "general_delta":
            n, r = mx["heads"] * mx["dim"], mx.get("decay_rank", 64)
            t.update({p + "mix.r": [n, E], p + "mix.k": [n, E], p + "mix.v": [n, E], p + "mix.g": [n, E], p + "mix.a": [n, E], p + "mix.a.b": [n],
                      p + "mix.w1": [r, E], p + "mix.w2": [n, r], p + "mix.w0": [n], p + "mix.norm": [n], p + "mix.o": [E, n]})
        elif L["type"] == "attention":
            H, G, D, Vd = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx["vdim"]
            for k, n in (("q", H * 2 * D), ("k", G * 2 * D), ("v", G * Vd)):
                t[p + "mix." + k] = [n, E]; t[p + "mix." + k + ".b"] = [n]
                if mx.get("conv"):
                    t[p + "mix." + k + ".conv"] = [n, mx["conv"]]
            for k in ("lq1", "lk1", "lq2", "lk2"):
                t[p + "mix." + k] = [D]
            t[p + "mix.o"] = [E, H * Vd]
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            t.update({p + "norm2": [E], p + "mlp.up": [ff, E], p + "mlp.down": [E, ff], p + "mlp.act": [4]})
            if ct:
                t[p + "canon2"] = [E, ct]
    t["final.norm"] = [E]
    t["head"] = [V, E]
    return t


def tensor_shapes(cfg: dict) -> Dict[str, List[int]]:
    if cfg.get("architecture") == "Dopilorn":
        return dopilorn_shapes(cfg)
    if cfg.get("architecture") == "Tosevik":
        return tosevik_shapes(cfg)
    if cfg.get("architecture") == "Rumurax":
        return rumurax_shapes(cfg)
    E, V = cfg["width"], cfg["vocab"]
    t = {"embed": [V, E]}
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        t[p + "norm1"] = [E]; t[p + "norm1b"] = [E]
        if L["type"] == "mingru":
            w = mx["width"]
            t.update({p + "mix.z": [w, E], p + "mix.z.b": [w], p + "mix.x": [w, E], p + "mix.x.b": [w], p + "mix.g": [w, E], p + "mix.o": [E, w]})
        elif L["type"] == "latent_attention":
            H, D, R, Vd, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
            t.update({p + "mix.q": [H * (D + R), E], p + "mix.dkv": [rank + R, E], p + "mix.dkv.norm": [rank], p + "mix.uk": [H * D, rank],
                      p + "mix.uv": [H * Vd, rank], p + "mix.sink": [H], p + "mix.o": [E, H * Vd]})
        elif L["type"] == "delta":
            H, KH, D, Vd, taps = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["conv"]
            t.update({p + "mix.q": [KH * D, E], p + "mix.q.conv": [KH * D, taps], p + "mix.k": [KH * D, E], p + "mix.k.conv": [KH * D, taps],
                      p + "mix.v": [H * Vd, E], p + "mix.v.conv": [H * Vd, taps], p + "mix.b": [H, E], p + "mix.A_log": [H], p + "mix.norm": [Vd],
                      p + "mix.a": [H, E], p + "mix.dt_bias": [H], p + "mix.g": [H * Vd, E], p + "mix.o": [E, H * Vd]})
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            t.update({p + "norm2": [E], p + "norm2b": [E], p + "mlp.gate": [ff, E], p + "mlp.gate.b": [ff], p + "mlp.up": [ff, E],
                      p + "mlp.up.b": [ff], p + "mlp.down": [E, ff], p + "mlp.down.b": [E]})
    t["final.norm"] = [E]
    t["head"] = [V, E]
    return t


def synth_stack(d: str, cfg: dict, seed: int = 1234) -> str:
    """write config.json + model.safetensors with random bfloat16 weights: matrices ~ N(0, 1/fan_in), norm weights ~ 1"""
    os.makedirs(d, exist_ok=True)
    shapes = tensor_shapes(cfg)
    head, off = {}, 0
    for name, shp in shapes.items():
        n = int(np.prod(shp)) * 2
        head[name] = {"dtype": "BF16", "shape": shp, "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(head).encode()
    hj += b" " * (-len(hj) % 8)
    rng = np.random.default_rng(seed)
    tmp = os.path.join(d, f"model.safetensors.tmp{os.getpid()}")
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for name, shp in shapes.items():
            n = int(np.prod(shp))
            zero_centred = cfg.get("architecture") == "Dopilorn" and name.rsplit(".", 1)[-1] in ("norm1", "norm2") or name == "final.norm" and cfg.get("architecture") == "Dopilorn"
            leaf = name.rsplit(".", 1)[-1]
            if cfg.get("architecture") == "Tosevik" and leaf in ("b", "alpha", "dwa", "pb"):
                if leaf == "dwa":                                # mostly the layer's own result, a little of every earlier one
                    x = (0.3 / math.sqrt(n)) * rng.standard_normal(n, dtype=np.float32)
                    x[-1] += 1.0
                elif leaf == "alpha":
                    x = np.full(1, 0.75, np.float32)
                else:
                    x = 0.1 * rng.standard_normal(n, dtype=np.float32) - (1.0 if leaf == "pb" else 0.0)
            elif cfg.get("architecture") == "Rumurax" and (".hc" in name or leaf in ("r1", "r2", "vmix")):
                if leaf == "mix":                                # keep every stream, leak a little into the others
                    x = (np.eye(shp[0], dtype=np.float32) + 0.05 * rng.standard_normal(shp, dtype=np.float32)).reshape(-1)
                elif leaf == "in":                               # read the streams' mean
                    x = np.full(n, 1.0 / n, np.float32) + 0.02 * rng.standard_normal(n, dtype=np.float32)
                elif leaf == "out":
                    x = 0.5 + 0.1 * rng.standard_normal(n, dtype=np.float32)
                elif leaf == "vmix":
                    x = np.full(1, 0.5, np.float32)
                else:                                            # positive: the penalty is r1 ln(1 + r2 distance)
                    x = 0.1 + rng.random(n, dtype=np.float32)
            elif name.endswith("mlp.act"):
                x = np.array([1.0, 0.5, 0.25, 0.0], np.float32)
            elif "canon" in name or zero_centred or name == "loop.step":
                x = 0.1 * rng.standard_normal(n, dtype=np.float32)
            elif len(shp) == 2 and not name.endswith(".conv"):
                x = rng.standard_normal(n, dtype=np.float32) * (1.0 / math.sqrt(shp[1]))
            elif "norm" in name:
                x = 1.0 + 0.1 * rng.standard_normal(n, dtype=np.float32)
            elif name.endswith("A_log"):
                x = -1.0 + 0.5 * rng.standard_normal(n, dtype=np.float32)
            else:
                x = 0.3 * rng.standard_normal(n, dtype=np.float32)
            f.write((x.view(np.uint32) >> 16).astype(np.uint16).tobytes())        # truncation to bfloat16: random data
    os.replace(tmp, os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return d


def n_params(cfg: dict) -> int:
    return sum(int(np.prod(s)) for s in tensor_shapes(cfg).values())
