"""The Rumurax design on the GPU against the plain numpy restatement in tests/rumurax_oracle.py: every mechanism alone (with and
without a mixture, with the residual after the layer), whole prompts against token-by-token decoding and portions down to two
tokens, contexts that are cleared and used again, several live contexts stepping in turn, what every position sees under
each mask (by changing one token and looking at who notices), far keys and the first tokens of a sequence, long decoding
through the replayed graph, other sizes (scalar and vector load paths, one to four streams, grouped and ungrouped heads, partial
and no rotation, one expert, all experts, no shared unit, no feed-forward), bfloat16, greedy generation through the bridge's job
loop and the trace runner. Small random models in a temporary folder; float32 is the sharp comparison."""
import copy

import numpy as np
import pytest

import rumurax_oracle as ro
import stack_oracle as so
from booster_b200 import _lib, engine

pytestmark = pytest.mark.gpu

TOL32 = 2e-4


def err(got, want):
    """root mean square of the difference with its mean taken off, over the root mean square of the expected row; worst row"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return float((np.sqrt((d * d).mean(-1)) / (np.sqrt((w * w).mean(-1)) + 1e-30)).max())


def moe(experts=6, top=2, ff=20, shared=12):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def chunk(heads=4, kv_heads=2, dim=8, vdim=6, size=9, scale=0.4, cap=5.0, v_mix=False, mlp=None):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}
    if cap:
        mx["softcap"] = cap
    if v_mix:
        mx["v_mix"] = True
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def window(heads=4, kv_heads=2, dim=8, vdim=6, size=9, pool=4, rot=8, base=100.0, scale=0.4, v_mix=False, mlp=None):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}
    if pool:
        mx["mask"]["pool"] = pool
    if rot:
        mx["rot"] = {"base": base, "dims": rot}
    if v_mix:
        mx["v_mix"] = True
    return {"type": "attention_2", "mixer": mx, "mlp": mlp}


def latent(heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=16, base=100.0, scale=0.3, mlp=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if rot_dim:
        mx["rot"] = {"base": base, "dims": rot_dim}
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def config(layers, width=48, vocab=61, eps=1e-5, streams=2):
    return {"architecture": "Rumurax", "layers": layers, "norm": {"eps": eps}, "streams": streams, "vocab": vocab, "width": width}


class Pair:
    """the same random model in the framework and in the oracle"""

    def __init__(self, tmp_path, cfg, seed=0, dtype="float32", n_ctx=512, edit=None):
        self.cfg = cfg
        self.w = ro.random_model(cfg, seed)
        if edit:
            edit(self.w)
        self.dir = ro.write_model(str(tmp_path / f"r{seed}_{dtype}_{abs(hash(str(cfg))) % 10**8}"), cfg, self.w)
        self.model = engine.Model(self.dir, dtype=dtype)
        self.ctx = engine.Context(self.model, n_ctx)

    def close(self):
        self.ctx.close()
        self.model.close()

    def tokens(self, n, seed=1):
        return np.random.default_rng(seed).integers(0, self.cfg["vocab"], size=n).tolist()

    def expected(self, toks, cfg=None, w=None, residuals=False):
        lg, taps = ro.forward(cfg or self.cfg, w or self.w, toks)
        return (lg, taps) if residuals else lg

    def run(self, toks, cuts=None, ctx=None):
        """logits of every position, the token stream cut into steps of the given sizes (None: one step)"""
        ctx = ctx or self.ctx
        ctx.kv_clear()
        out, pos, i = [], 0, 0
        cuts = list(cuts) if cuts else [len(toks)]
        while pos < len(toks):
            n = min(cuts[i % len(cuts)], len(toks) - pos)
            out.append(ctx.decode_rows(toks[pos:pos + n], pos, list(range(n))))
            pos += n
            i += 1
        return np.concatenate(out)


@pytest.mark.parametrize("layer", [chunk(), chunk(heads=3, kv_heads=3, dim=5, vdim=7, size=4, cap=0.0, mlp=moe()), window(), window(heads=6, kv_heads=2, dim=12, vdim=5, size=5, pool=3, rot=6, mlp=moe(experts=4, top=3, shared=0)),
                                   window(pool=0, rot=0, size=7), latent(), latent(heads=2, dim=5, rot_dim=6, vdim=9, kv_rank=11, mlp=moe(experts=8, top=1, ff=9, shared=5))],
                         ids=["chunks", "chunks-ungrouped-uncapped+moe", "window+means", "window-odd+moe-unshared", "window-plain", "latent", "latent-odd+moe"])
def test_each_mixer_alone_with_the_residual_after_the_layer(tmp_path, layer):
    p = Pair(tmp_path, config([layer]))
    toks = p.tokens(29)
    want, res = p.expected(toks, residuals=True)
    p.ctx.set_taps(True)
    got = p.ctx.decode_rows(toks, 0, list(range(len(toks))))
    taps = p.ctx.layer_taps(len(toks))
    p.ctx.set_taps(False)
    assert taps.shape[0] == 1 and np.abs(taps[0] - res[0]).max() < 1e-4 * max(1.0, np.abs(res[0]).max())
    assert err(got, want) < TOL32
    assert err(p.run(toks, [1]), want) < TOL32
    assert err(p.run(toks, [3]), want) < TOL32
    p.close()


def test_small_mechanisms_matter(tmp_path):
    """the oracle without one of the small mechanisms is far from the framework: none of them is a no-op in these models"""
    cfg = config([window(v_mix=True, mlp=moe()), chunk(v_mix=True, mlp=moe(top=1)), latent(mlp=moe()), window(size=6, pool=2, rot=4, v_mix=True)], streams=3)
    p = Pair(tmp_path, cfg)
    toks = p.tokens(37)
    got = p.run(toks)
    assert err(got, p.expected(toks)) < TOL32
    for key in ("l1.mix.sink", "l1.mix.r1", "l1.mix.g", "l1.mix.vmix", "l3.mix.vmix", "l0.hc1.in", "l0.hc2.out", "l1.hc1.mix", "l2.hc2.mix", "l1.mlp.router", "l2.mix.g"):
        w2 = dict(p.w); w2[key] = np.zeros_like(p.w[key])
        assert err(got, p.expected(toks, w=w2)) > 20 * TOL32, key
    for key in ("l0.mix.q.norm", "l1.mix.k.norm", "l2.mix.dkv.norm", "l1.mix.r2"):
        w2 = dict(p.w); w2[key] = p.w[key] * np.linspace(0.5, 1.5, p.w[key].size)
        assert err(got, p.expected(toks, w=w2)) > 20 * TOL32, key
    w2 = dict(p.w); w2["l0.mix.vmix"] = np.asarray(0.9)              # the first mixing layer's own weight is not used
    assert err(got, p.expected(toks, w=w2)) < TOL32
    w2 = dict(p.w)
    for e in range(6):
        w2["l0.mlp.e%d.gate" % e] = p.w["l0.mlp.e%d.gate" % e] * 1.5
    assert err(got, p.expected(toks, w=w2)) > 20 * TOL32
    for edit in (lambda c: c["layers"][0]["mixer"]["rot"].update(base=50.0), lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6),
                 lambda c: c["layers"][0]["mixer"]["mask"].update(pool=3), lambda c: c["layers"][0]["mixer"]["mask"].update(size=10),
                 lambda c: c["layers"][0]["mixer"]["mask"].pop("pool"), lambda c: c["layers"][1]["mixer"]["mask"].update(size=8),
                 lambda c: c["layers"][1]["mixer"].update(softcap=2.0), lambda c: c["layers"][1]["mixer"].pop("softcap"), lambda c: c["layers"][1]["mixer"].update(scale=0.3),
                 lambda c: c["layers"][2]["mixer"]["rot"].update(base=10.0), lambda c: c["layers"][1]["mlp"]["router"].update(top=2), lambda c: c["norm"].update(eps=1e-2),
                 lambda c: c["layers"][3]["mixer"].pop("v_mix")):
        c2 = copy.deepcopy(cfg); edit(c2)
        assert err(got, p.expected(toks, cfg=c2)) > 20 * TOL32, c2
    p.close()


def test_weight_on_the_experts_input_is_not_a_weight_on_the_output(tmp_path):
    cfg = config([latent(mlp=moe(experts=4, top=2, shared=0))])
    p = Pair(tmp_path, cfg, seed=3)
    toks = p.tokens(20)
    want = p.expected(toks)
    assert err(p.run(toks), want) < TOL32 and err(p.run(toks, [1]), want) < TOL32

    def output_weighted(h, mj, W, pre):
        sel, wt = ro.route(h, W[pre + "router"], mj["router"]["top"])
        y = np.zeros_like(h)
        for t in range(h.shape[0]):
            for e, w in zip(sel[t], wt[t]):
                ep = pre + "e%d." % e
                y[t] += w * ro.gated_unit(h[t], W[ep + "gate"], W[ep + "up"], W[ep + "down"])
        return y
    keep = ro.mixture
    ro.mixture = output_weighted
    try:
        assert err(p.run(toks), p.expected(toks)) > 20 * TOL32
    finally:
        ro.mixture = keep
    p.close()


FULL = [window(v_mix=True, mlp=moe()), chunk(v_mix=True, mlp=moe(experts=4, top=1, ff=16, shared=24)), latent(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24),
        chunk(heads=2, kv_heads=1, dim=8, vdim=16, size=16, cap=20.0, mlp=moe(experts=5, top=2, ff=32)), window(size=13, pool=5, rot=4, v_mix=True, mlp=moe(experts=9, top=3, shared=0)),
        latent(mlp=moe(experts=3, top=3))]


def test_whole_prompt_token_by_token_and_portions_agree(tmp_path):
    p = Pair(tmp_path, config(FULL))
    toks = p.tokens(75)
    want, res = p.expected(toks, residuals=True)
    p.ctx.set_taps(True)
    p.ctx.kv_clear()
    p.ctx.decode_rows(toks, 0, [])
    taps = p.ctx.layer_taps(len(toks))
    p.ctx.set_taps(False)
    assert taps.shape[0] == len(res) == len(FULL)
    for a, b in zip(taps, res):
        assert np.abs(a - b).max() < 1e-4 * max(1.0, np.abs(b).max())
    assert err(p.run(toks), want) < TOL32
    assert err(p.run(toks, [1]), want) < TOL32        # every token through the replayed one-token graph
    for cuts in ([2], [3, 2, 7, 1, 5], [37, 2, 2, 30], [6, 1, 1, 11], [4], [9, 8]):
        assert err(p.run(toks, cuts), want) < TOL32, cuts
    p.close()


def test_cleared_context_is_as_good_as_new_and_contexts_do_not_meet(tmp_path):
    p = Pair(tmp_path, config(FULL))
    a, b = p.tokens(60, seed=3), p.tokens(29, seed=4)
    fresh = engine.Context(p.model, 512)
    ref_b = p.run(b, [5, 1, 1, 9], ctx=fresh)
    p.run(a, [7, 1])                                  # fills cache rows and block means
    again = p.run(b, [5, 1, 1, 9])                    # run() clears first: the same context, used again
    assert np.array_equal(again, ref_b)
    assert err(again, p.expected(b)) < TOL32
    # two live sequences of unequal length stepping in turn, each as if alone
    p.ctx.kv_clear(); fresh.kv_clear()
    ga, gb, pa, pb = [], [], 0, 0
    for na, nb in ((9, 3), (1, 1), (4, 13), (1, 2), (45, 10)):
        ga.append(p.ctx.decode_rows(a[pa:pa + na], pa, list(range(na)))); pa += na
        gb.append(fresh.decode_rows(b[pb:pb + nb], pb, list(range(nb)))); pb += nb
    assert err(np.concatenate(ga), p.expected(a)) < TOL32
    assert err(np.concatenate(gb), p.expected(b)) < TOL32
    fresh.close()
    p.close()


def sees(layer, p, j):
    """position p sees token j under the layer's mask, restated from the masks' definitions"""
    mk = layer["mixer"]["mask"]
    n, P = mk["size"], mk.get("pool", 0)
    if j > p:
        return False
    if layer["type"] == "attention":
        return p // n == j // n
    if p - j < n:
        return True
    return P > 0 and (j // P) * P + P - 1 <= p - n


@pytest.mark.parametrize("layer", [chunk(size=9), chunk(size=16, heads=2, kv_heads=2), chunk(size=1), window(size=9, pool=4), window(size=16, pool=16), window(size=5, pool=7, rot=0),
                                   window(size=1, pool=1), window(size=11, pool=0), window(size=2, pool=3, heads=2, kv_heads=1), chunk(size=33), window(size=40, pool=12)],
                         ids=["chunks-9", "chunks-16", "chunks-1", "window-9-means-4", "window-16-means-16", "window-5-means-7", "window-1-means-1", "window-11", "window-2-means-3",
                              "chunks-33", "window-40-means-12"])
def test_who_notices_a_changed_token(tmp_path, layer):
    """a model whose only path between positions is one attention layer: when token j changes, exactly the positions that see j
    under the mask change (a token that left the window and whose block is not complete yet is seen by nobody), in a whole
    prompt, in decoding and in portions that start anywhere"""
    cfg = config([layer], width=32, vocab=40)
    p = Pair(tmp_path, cfg, seed=2)
    n = 70
    toks = p.tokens(n, seed=5)
    for cuts in (None, [40, 1], [2, 3, 5, 1, 7, 11]):
        base = p.run(toks, cuts)
        for j in (0, 3, 17, 32, 44):
            other = list(toks); other[j] = (toks[j] + 1) % 40
            got = p.run(other, cuts)
            for q in range(n):
                same = np.array_equal(got[q], base[q])
                assert same != sees(layer, q, j), (cuts, j, q)
    assert err(p.run(toks), p.expected(toks)) < TOL32
    p.close()


def sharpen(names, gain=6.0):
    def edit(w):
        for k in list(w):
            if any(k.endswith(n) for n in names):
                w[k] = so.round_bf16(np.asarray(w[k] * gain, np.float32)).astype(np.float64)
    return edit


@pytest.mark.parametrize("size,pool", [(1, 2), (2, 1), (9, 4), (33, 5)])
def test_mask_edges_with_sharpened_queries(tmp_path, size, pool):
    """peaked attention: an oracle whose window or chunk is one token off, or whose blocks are one token shorter, is far away"""
    cfg = config([window(size=size, pool=pool, dim=8, rot=8, mlp=moe()), chunk(size=size, cap=50.0)], width=32, vocab=40)
    p = Pair(tmp_path, cfg, seed=size, edit=sharpen(["q.norm"], 5.0))
    toks = p.tokens(150, seed=size)
    want = p.expected(toks)
    edits = [lambda c: c["layers"][1]["mixer"]["mask"].update(size=size + 1), lambda c: c["layers"][0]["mixer"]["mask"].update(pool=pool + 1)]
    if pool > 1:                                          # blocks of one token: every older token is seen whatever the window
        edits.append(lambda c: c["layers"][0]["mixer"]["mask"].update(size=size + 1))
    for edit in edits:
        c2 = copy.deepcopy(cfg); edit(c2)
        assert err(p.expected(toks, cfg=c2), want) > 50 * TOL32
    for cuts in (None, [110, 1], [size, 1, size + 1, 2, 31], [7, 2]):
        assert err(p.run(toks, cuts), want) < TOL32, cuts
    p.close()


def test_far_keys_and_first_tokens(tmp_path):
    """a token hundreds of positions back reaches a late position through the latent attention (every key) and through the mean of
    its block (the window layer): one early token is changed and the late logits move, in a prompt and in decoding"""
    for layer in (latent(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=12, scale=1.5), window(heads=2, kv_heads=1, dim=8, vdim=8, size=8, pool=4, scale=1.5)):
        cfg = config([layer], width=32, vocab=40)
        p = Pair(tmp_path, cfg, seed=5, n_ctx=400)
        toks = p.tokens(330, seed=9)
        want = p.expected(toks)
        other = list(toks); other[3] = (toks[3] + 1) % 40
        assert err(p.expected(other)[300:], want[300:]) > 20 * TOL32          # position 3 is seen from 300 on
        got = p.run(toks, [300, 1])
        assert err(got, want) < TOL32
        assert err(got[:4], want[:4]) < TOL32             # the first tokens of a sequence: one key, no block
        assert err(p.run(toks[:40], [1]), want[:40]) < TOL32
        assert err(p.run(toks, [2, 129, 3, 64]), want) < TOL32
        assert err(p.run(other, [31, 32, 33, 1]), p.expected(other)) < TOL32
        p.close()


def test_one_far_key_among_hundreds_stands_out(tmp_path):
    """all tokens but one have nearly the same embedding row, so all keys but one are nearly equal; the odd token sits at position 5
    and the scores are steep: the late positions must find its key among 300 (latent attention), or the mean of its block (window)"""
    for layer in (latent(heads=1, dim=8, rot_dim=0, vdim=8, kv_rank=8, scale=3.0), window(heads=1, kv_heads=1, dim=8, vdim=8, size=8, pool=2, rot=0, scale=3.0)):
        cfg = config([layer], width=16, vocab=12, streams=1)
        toks = [int(t) for t in np.random.default_rng(3).integers(0, 7, size=320)]
        with_key = list(toks); with_key[5] = 7

        def edit(w):
            e = np.asarray(w["embed"])
            e[:7] = e[0] + 0.02 * e[:7]                      # tokens 0 .. 6: one direction; token 7 keeps its own
            w["embed"] = so.round_bf16(e.astype(np.float32)).astype(np.float64)
        for seed in range(40):                               # a model in which the odd key wins the late soft-max
            w = ro.random_model(cfg, seed); edit(w)
            want, plain = ro.forward(cfg, w, with_key)[0], ro.forward(cfg, w, toks)[0]
            if err(want[300:], plain[300:]) > 50 * TOL32:
                break
        else:
            raise AssertionError("no seed makes the far key matter")
        p = Pair(tmp_path, cfg, seed=seed, n_ctx=340, edit=edit)
        for cuts in (None, [290, 1], [5, 1, 2, 250, 3]):
            assert err(p.run(with_key, cuts), want) < TOL32, cuts
        p.close()


def test_long_decoding_through_the_graph(tmp_path):
    p = Pair(tmp_path, config(FULL[:5]))
    toks = p.tokens(300, seed=11)
    want = p.expected(toks)
    got = p.run(toks, [4, 1])
    assert err(got, want) < 2 * TOL32
    assert err(got[-1:], want[-1:]) < 2 * TOL32
    p.close()


@pytest.mark.parametrize("width,vocab,streams", [(36, 50, 1), (40, 77, 3), (64, 130, 4), (37, 53, 2)], ids=["scalar-loads-one-stream", "width-40-three-streams", "vector-loads-four-streams", "odd-width"])
def test_other_sizes(tmp_path, width, vocab, streams):
    layers = [latent(heads=5, dim=9, rot_dim=2, vdim=5, kv_rank=7, mlp=moe(experts=3, top=3, ff=7, shared=3)),
              chunk(heads=6, kv_heads=2, dim=9, vdim=5, size=3, v_mix=True),
              window(heads=4, kv_heads=4, dim=16, vdim=40, size=40, pool=3, rot=6, mlp=moe(experts=16, top=4, ff=64, shared=64)),
              window(heads=3, kv_heads=1, dim=6, vdim=20, size=4, pool=1, rot=0, v_mix=False),
              chunk(heads=2, kv_heads=2, dim=4, vdim=5, size=100, cap=0.0, v_mix=True, mlp=moe(experts=1, top=1, ff=24)),
              latent(heads=1, dim=4, rot_dim=0, vdim=36, kv_rank=40, mlp=moe(experts=2, top=1, shared=0)),
              window(heads=4, kv_heads=2, dim=64, vdim=5, size=7, pool=2, rot=64, v_mix=True)]
    p = Pair(tmp_path, config(layers, width=width, vocab=vocab, eps=1e-6, streams=streams), seed=width)
    toks = p.tokens(70, seed=width)
    want = p.expected(toks)
    assert err(p.run(toks), want) < TOL32
    assert err(p.run(toks, [13, 2, 1]), want) < TOL32
    p.close()


def test_a_model_without_stream_weights_is_the_plain_residual(tmp_path):
    """one stream and no connection tensors in the file: x <- x + f(norm(x))"""
    cfg = config([chunk(mlp=moe()), latent()], streams=1)
    w = {k: v for k, v in ro.random_model(cfg, 4).items() if ".hc" not in k}
    d = ro.write_model(str(tmp_path / "plain"), cfg, w)
    model = engine.Model(d, dtype="float32")
    ctx = engine.Context(model, 64)
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], size=33).tolist()
    want = ro.forward(cfg, w, toks)[0]
    assert err(ctx.decode_rows(toks, 0, list(range(33))), want) < TOL32
    ctx.close(); model.close()


def test_latent_attention_over_large_tiles(tmp_path):
    """enough heads and keys for the 128 x 128 float32 tile product of the prompt path (whole and ragged tiles in both products), beside
    a layer that stays on the small tiles"""
    cfg = config([latent(heads=9, dim=16, rot_dim=8, vdim=12, kv_rank=136, mlp=moe()), latent(heads=8, dim=8, rot_dim=4, vdim=8, kv_rank=128), latent(heads=3, dim=8, rot_dim=4, vdim=8, kv_rank=20)],
                 width=64, vocab=80)
    p = Pair(tmp_path, cfg, seed=6, n_ctx=420)
    toks = p.tokens(410, seed=6)
    want = p.expected(toks)
    for cuts in (None, [128, 256, 26], [131, 1, 200, 9, 69]):
        assert err(p.run(toks, cuts), want) < TOL32, cuts
    p.close()


def random_config(rng):
    """a random arrangement of the mixers with random sizes: nothing may rest on one model's values"""
    pick = lambda values: int(rng.choice(values))

    def rnd_moe():
        if rng.random() < 0.25:
            return None
        n = pick([1, 2, 5, 8, 12])
        return moe(experts=n, top=pick(range(1, min(n, 4) + 1)), ff=pick([8, 24, 64, 100]), shared=pick([0, 8, 40, 136]))
    layers = []
    for _ in range(pick([2, 3, 4, 6])):
        kind = pick([0, 1, 2])
        kv = pick([1, 2, 3])
        d = pick([4, 6, 16, 32, 64, 128])
        if kind == 0:
            layers.append(chunk(heads=kv * pick([1, 2, 4]), kv_heads=kv, dim=d, vdim=pick([4, 8, 48, 128, 200]), size=pick([1, 3, 16, 50, 128, 1000]), scale=float(rng.choice([0.1, 0.3])),
                                cap=float(rng.choice([0.0, 3.0, 30.0])), v_mix=bool(rng.random() < 0.6), mlp=rnd_moe()))
        elif kind == 1:
            layers.append(window(heads=kv * pick([1, 2, 4]), kv_heads=kv, dim=d, vdim=pick([4, 8, 48, 128, 200]), size=pick([1, 3, 16, 50, 128]), pool=pick([0, 1, 2, 7, 16, 40]),
                                 rot=pick([r for r in (0, 2, 4, 16, 32, 64, 128) if r <= d]), base=float(rng.choice([100.0, 1e4, 5e5])), scale=float(rng.choice([0.1, 0.3])),
                                 v_mix=bool(rng.random() < 0.6), mlp=rnd_moe()))
        else:
            r = pick([0, 2, 8, 32])
            layers.append(latent(heads=pick([1, 2, 3, 6]), dim=d, rot_dim=r, vdim=pick([4, 8, 48, 128]), kv_rank=pick([8, 24, 64, 136]), base=float(rng.choice([100.0, 5e5])),
                                 scale=float(rng.choice([0.1, 0.3])), mlp=rnd_moe()))
    # value-mixing layers must agree in kv_heads x vdim: later ones take the first one's
    first = None
    for L in layers:
        if L["mixer"].get("v_mix"):
            if first is None:
                first = L["mixer"]
            else:
                ratio = L["mixer"]["heads"] // L["mixer"]["kv_heads"]
                L["mixer"].update(kv_heads=first["kv_heads"], heads=first["kv_heads"] * ratio, vdim=first["vdim"])
    return config(layers, width=pick([24, 36, 64, 100, 136]), vocab=pick([37, 100, 257, 513]), eps=float(rng.choice([1e-6, 1e-5])), streams=pick([1, 2, 3, 4]))


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(tmp_path, seed):
    rng = np.random.default_rng(700 + seed)
    cfg = random_config(rng)
    n = int(rng.choice([70, 150, 330]))
    p = Pair(tmp_path, cfg, seed=seed, n_ctx=n + 4)
    toks = p.tokens(n, seed=seed)
    want = p.expected(toks)
    assert err(p.run(toks), want) < 2 * TOL32, cfg
    assert err(p.run(toks, [n - 20] + [1] * 20), want) < 2 * TOL32, cfg
    assert err(p.run(toks, [2, 67, 3, 129, 1, 5]), want) < 2 * TOL32, cfg
    p.close()


def test_a_step_longer_than_one_pass(tmp_path):
    """a 700-token step runs as two passes of the layers: cached keys, block means and the first mixing layer's values cross the pass's edge"""
    p = Pair(tmp_path, config(FULL[:5]), n_ctx=704)
    toks = p.tokens(700, seed=5)
    want = p.expected(toks)
    assert err(p.run(toks), want) < 2 * TOL32
    assert err(p.run(toks, [509, 2, 3, 186]), want) < 2 * TOL32
    p.close()


def row_errs(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / (np.sqrt((w * w).mean(-1)) + 1e-30)


def test_bfloat16_prompt_kernels_and_decode(tmp_path):
    """wide enough for the tensor-core products, also the segmented ones of the routed mixture"""
    layers = [window(heads=4, kv_heads=2, dim=32, vdim=32, size=40, pool=8, rot=16, v_mix=True, mlp=moe(experts=4, top=2, ff=64, shared=64)),
              chunk(heads=4, kv_heads=2, dim=16, vdim=32, size=64, v_mix=True, mlp=moe(experts=3, top=1, ff=128, shared=0)),
              latent(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, mlp=moe(experts=4, top=2, ff=64, shared=128))]
    cfg = config(layers, width=128, vocab=160)
    p = Pair(tmp_path, cfg, dtype="bfloat16")
    toks = p.tokens(300, seed=2)
    want = p.expected(toks)
    # token by token: mat-vec kernels with float32 activations on the stored bfloat16 weights: as sharp as float32
    assert err(p.run(toks[:60], [1]), want[:60]) < TOL32
    assert err(p.run(toks[:60], [3, 4, 2]), want[:60]) < TOL32
    # longer portions: tensor-core products round the activation operand to bfloat16
    for cuts in (None, [280, 1], [5, 17, 133]):
        e = row_errs(p.run(toks, cuts), want)
        assert np.median(e) < 3e-2 and e.max() < 0.25, (cuts, float(np.median(e)), float(e.max()))
    p.close()


def test_greedy_generation_through_the_bridge(tmp_path, monkeypatch):
    """initContext / doInference on a folder model: decimal-id prompt, standard chain at temperature 0 (arg-max on the device),
    prompt through the prompt kernels, generation through the one-token graph: the ids the oracle generates greedily"""
    monkeypatch.setenv("BOOSTER_B200_DTYPE", "float32")
    p = Pair(tmp_path, config(FULL[:4]))
    prompt, n_gen = p.tokens(21, seed=6), 10
    seq, ids = list(prompt), []
    for _ in range(n_gen):
        lg = p.expected(seq)[-1]
        srt = np.sort(lg)
        assert srt[-1] - srt[-2] > 1e-3               # no near-tie: float32 must pick the same id
        ids.append(int(np.argmax(lg)))
        seq.append(ids[-1])
    L = _lib.lib()
    L.init(b"", b"")
    ctx = L.initContext(6, p.dir.encode(), 1, 0, 100, 0, 0, 0, 64, n_gen, 0, 0.0, 0.0, 0.0, 1, 1.0, 1.0, 1.0, 0, 0, 200, 1.0, 1.0, 1.0, 42, b"")
    assert ctx, _lib.last_error()
    n = L.doInference(6, ctx, b"rumurax-job", b"", " ".join(map(str, prompt)).encode())
    out = [int(x) for x in L.status(b"rumurax-job").decode().split()]
    assert out[:len(prompt)] == prompt and out[len(prompt):] == ids
    assert n == len(prompt) + n_gen - 1 and L.getPromptTokenCount(b"rumurax-job") == len(prompt)
    # the device-resident loop of the token-level interface gives the same ids
    p.ctx.kv_clear()
    first = int(np.argmax(p.ctx.decode(prompt, 0)))
    dev = p.ctx.generate_greedy(first, len(prompt), n_gen - 1).tolist()
    assert [first] + dev == ids
    after = p.ctx.decode([ids[-1]], len(prompt) + n_gen - 1)
    assert err(after[None], p.expected(seq)[-1][None]) < TOL32
    assert p.ctx.L.b200_kernel_launches(p.ctx.h) > 0
    p.close()


def test_trace_runner_replays_steps(tmp_path):
    """bin/trace_run on a folder model of this design: wanted rows per step, a finished request's context used again"""
    import json
    import os
    import subprocess
    import sys
    cfg = config(FULL[:3])
    w = ro.random_model(cfg, 5)
    d = ro.write_model(str(tmp_path / "m"), cfg, w)
    rng = np.random.default_rng(3)
    a, b = rng.integers(0, cfg["vocab"], size=40).tolist(), rng.integers(0, cfg["vocab"], size=23).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:31], "want": [0, 7, 30]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[31:33], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[33:40], "want": [6, 1]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b[:22], "want": [21]}], "end": []},
             {"step": 4, "entries": [{"id": "b", "tokens": b[22:], "want": [0]}], "end": ["b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(out), "--max-tokens", "64"],
                       input="".join(json.dumps(x) + "\n" for x in steps).encode(), stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=600)
    assert r.returncode == 0, r.stderr.decode()[-2000:]
    assert [l for l in r.stdout.decode().split("\n") if l.startswith("done")] == ["done %d" % i for i in range(5)]
    assert not (out / "1.f32").exists()
    wa, wb = ro.forward(cfg, w, a)[0], ro.forward(cfg, w, b)[0]
    for n, want in ((0, wa[[0, 7, 30]]), (2, wa[[39, 34]]), (3, wb[[21]]), (4, wb[[22]])):
        got = np.fromfile(str(out / ("%d.f32" % n)), "<f4").reshape(len(want), cfg["vocab"])
        assert err(got, want) < TOL32, n


def test_bad_models_fail_loudly(tmp_path):
    cfg = config([chunk(v_mix=True, mlp=moe()), window(v_mix=True), latent()])
    w = ro.random_model(cfg)
    c2 = copy.deepcopy(cfg); c2["layers"][0]["type"] = "mingru"
    with pytest.raises(_lib.B200Error, match="not part of the Rumurax design"):
        engine.Model(ro.write_model(str(tmp_path / "mixer"), c2, w))
    w2 = dict(w); del w2["l1.hc1.mix"]
    with pytest.raises(_lib.B200Error, match="missing"):
        engine.Model(ro.write_model(str(tmp_path / "missing"), cfg, w2))
    c3 = copy.deepcopy(cfg); c3["streams"] = 9
    with pytest.raises(_lib.B200Error, match="streams"):
        engine.Model(ro.write_model(str(tmp_path / "streams"), c3, w))
    c4 = copy.deepcopy(cfg); c4["layers"][1]["mixer"]["kv_heads"] = 3
    with pytest.raises(_lib.B200Error, match="multiple of kv_heads"):
        engine.Model(ro.write_model(str(tmp_path / "heads"), c4, w))
    c5 = copy.deepcopy(cfg); c5["layers"][0]["mlp"]["router"]["top"] = 7
    with pytest.raises(_lib.B200Error, match="exceeds the experts"):
        engine.Model(ro.write_model(str(tmp_path / "top"), c5, w))
    c6 = copy.deepcopy(cfg); c6["layers"][1]["mixer"].update(kv_heads=1, vdim=12)      # as many value entries, another shape
    with pytest.raises(_lib.B200Error, match="agree in kv_heads and vdim"):
        engine.Model(ro.write_model(str(tmp_path / "vmix"), c6, ro.random_model(c6)))
