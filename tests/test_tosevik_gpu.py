"""The Tosevik design on the GPU against the plain numpy restatement in tests/tosevik_oracle.py: every mechanism alone (with and
without a feed-forward, with the residual stream after the layer), whole prompts against token-by-token decoding and portions
down to two tokens, contexts that are cleared and used again, several live contexts stepping in turn, far keys and the first
tokens of a sequence with sharpened attention in prompts and in decoding, long decoding through the replayed graph, other
sizes (scalar and vector load paths, grouped and ungrouped key heads, partial rotation, one group, one expert, no shared unit),
bfloat16, and greedy generation through the bridge's job loop. Small random models in a temporary folder; float32 is the
sharp comparison."""
import copy

import numpy as np
import pytest

import stack_oracle as so
import tosevik_oracle as to
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


def moe(experts=6, top=2, groups=(3, 2), ff=20, shared=12, scale=1.3):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if groups:
        m["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def ret_mixer(heads=3, dim=8, vdim=6, rot=8, base=100.0, decay=None):
    return {"heads": heads, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot},
            "decay": decay or [1.0 - 2.0 ** (-2 - 1.5 * h) for h in range(heads)]}


def retention(mlp=None, **kw):
    return {"type": "retention", "mixer": ret_mixer(**kw), "mlp": mlp}


def parallel(heads=4, kv_heads=2, dim=6, vdim=10, scale=0.4, coef=0.4, every=5, right=None, mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "q_temp": {"coef": coef, "every": every}}
    return {"type": "parallel", "mixer": {"left": left, "right": right or ret_mixer(heads=2, dim=4, vdim=12, rot=2)}, "mlp": mlp}


def config(layers, width=48, vocab=61, eps=1e-5):
    return {"architecture": "Tosevik", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


class Pair:
    """the same random model in the framework and in the oracle"""

    def __init__(self, tmp_path, cfg, seed=0, dtype="float32", n_ctx=512, edit=None):
        self.cfg = cfg
        self.w = to.random_model(cfg, seed)
        if edit:
            edit(self.w)
        self.dir = to.write_model(str(tmp_path / f"t{seed}_{dtype}_{abs(hash(str(cfg))) % 10**8}"), cfg, self.w)
        self.model = engine.Model(self.dir, dtype=dtype)
        self.ctx = engine.Context(self.model, n_ctx)

    def close(self):
        self.ctx.close()
        self.model.close()

    def tokens(self, n, seed=1):
        return np.random.default_rng(seed).integers(0, self.cfg["vocab"], size=n).tolist()

    def expected(self, toks, residuals=None, cfg=None, w=None):
        return to.forward(cfg or self.cfg, w or self.w, toks, residuals)

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


@pytest.mark.parametrize("layer", [retention(), retention(heads=2, dim=5, vdim=7, rot=4, mlp=moe()), parallel(), parallel(heads=3, kv_heads=3, dim=5, vdim=7, mlp=moe(experts=4, top=3, groups=None, shared=0)),
                                   retention(heads=1, dim=16, vdim=3, rot=16, mlp=moe(experts=8, top=2, groups=(4, 1), ff=9, shared=5))],
                         ids=["retention", "retention-odd+moe", "parallel-grouped", "parallel-ungrouped+moe-plain", "retention-one-head+moe-one-group-kept"])
def test_each_mixer_alone_with_the_residual_after_the_layer(tmp_path, layer):
    p = Pair(tmp_path, config([layer]))
    toks = p.tokens(23)
    res = []
    want = p.expected(toks, res)
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
    cfg = config([parallel(mlp=moe()), retention(mlp=moe(groups=(2, 1)))])
    p = Pair(tmp_path, cfg)
    toks = p.tokens(31)
    got = p.run(toks)
    assert err(got, p.expected(toks)) < TOL32
    for key in ("l0.mix.left.pb", "l0.mix.left.out", "l0.mix.right.out", "l0.norm1.b", "l0.norm2.b", "embed.norm.b", "final.norm.b", "l0.mlp.shared.sg", "l1.mlp.router",
                "l0.mix.left.q.norm", "l0.mix.left.k.norm"):
        w2 = dict(p.w); w2[key] = np.zeros_like(p.w[key])
        assert err(got, p.expected(toks, w=w2)) > 20 * TOL32, key
    for key in ("l0.norm1.alpha", "embed.norm.alpha", "final.norm.alpha"):
        w2 = dict(p.w); w2[key] = p.w[key] * 0.5
        assert err(got, p.expected(toks, w=w2)) > 20 * TOL32, key
    w2 = dict(p.w); w2["l0.dwa"] = np.array([0.0, 1.0]); w2["l1.dwa"] = np.array([0.0, 0.0, 1.0])
    assert err(got, p.expected(toks, w=w2)) > 20 * TOL32        # the depth average
    for edit in (lambda c: c["layers"][0]["mixer"]["left"]["q_temp"].update(coef=0.0), lambda c: c["layers"][0]["mixer"]["left"]["q_temp"].update(every=6),
                 lambda c: c["layers"][1]["mixer"]["rot"].update(base=50.0), lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6),
                 lambda c: c["layers"][0]["mlp"]["router"].update(scale=1.0), lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=2),
                 lambda c: c["layers"][1]["mixer"]["decay"].__setitem__(0, 0.5), lambda c: c["layers"][0]["mlp"]["router"].update(top=3)):
        c2 = copy.deepcopy(cfg); edit(c2)
        assert err(got, p.expected(toks, cfg=c2)) > 20 * TOL32, c2
    p.close()


FULL = [retention(mlp=moe()), parallel(mlp=moe(experts=4, top=1, groups=(2, 2), ff=16, shared=24)), retention(heads=2, dim=16, vdim=16, rot=8),
        parallel(heads=2, kv_heads=1, dim=8, vdim=16, right=ret_mixer(heads=3, dim=8, vdim=4, rot=8), mlp=moe(experts=5, top=2, groups=None, ff=32)),
        retention(heads=4, dim=4, vdim=12, rot=2, mlp=moe(experts=9, top=3, groups=(3, 1), shared=0))]


def test_whole_prompt_token_by_token_and_portions_agree(tmp_path):
    p = Pair(tmp_path, config(FULL))
    toks = p.tokens(75)
    res = []
    want = p.expected(toks, res)
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
    for cuts in ([2], [3, 2, 7, 1, 5], [37, 2, 2, 30], [6, 1, 1, 11], [4]):
        assert err(p.run(toks, cuts), want) < TOL32, cuts
    p.close()


def test_cleared_context_is_as_good_as_new_and_contexts_do_not_meet(tmp_path):
    p = Pair(tmp_path, config(FULL))
    a, b = p.tokens(40, seed=3), p.tokens(29, seed=4)
    fresh = engine.Context(p.model, 512)
    ref_b = p.run(b, [5, 1, 1, 9], ctx=fresh)
    p.run(a, [7, 1])                                  # fills cache rows and recurrent state
    again = p.run(b, [5, 1, 1, 9])                    # run() clears first: the same context, used again
    assert np.array_equal(again, ref_b)
    assert err(again, p.expected(b)) < TOL32
    # two live sequences of unequal length stepping in turn, each as if alone
    p.ctx.kv_clear(); fresh.kv_clear()
    ga, gb, pa, pb = [], [], 0, 0
    for na, nb in ((9, 3), (1, 1), (4, 13), (1, 2), (25, 10)):
        ga.append(p.ctx.decode_rows(a[pa:pa + na], pa, list(range(na)))); pa += na
        gb.append(fresh.decode_rows(b[pb:pb + nb], pb, list(range(nb)))); pb += nb
    assert err(np.concatenate(ga), p.expected(a)) < TOL32
    assert err(np.concatenate(gb), p.expected(b)) < TOL32
    fresh.close()
    p.close()


def sharpen(names, gain=6.0):
    def edit(w):
        for k in list(w):
            if any(k.endswith(n) for n in names):
                w[k] = so.round_bf16(np.asarray(w[k] * gain, np.float32)).astype(np.float64)
    return edit


def test_far_keys_through_the_attention_and_first_tokens(tmp_path):
    """the retention branch forgets within a few tokens (decay 1/16), so only the attention's flattest head carries a token
    hundreds of positions back: one early token is changed and the late logits move, in a prompt and in decoding"""
    right = ret_mixer(heads=2, dim=4, vdim=4, rot=4, decay=[0.0625, 0.03125])
    cfg = config([parallel(heads=2, kv_heads=1, dim=8, vdim=8, scale=1.0, coef=0.3, every=64, right=right)], width=32, vocab=40)

    def edit(w):
        sharpen(["left.q.norm"], 3.0)(w)
        w["l0.mix.left.pb"] = np.array([0.5, 1.0])
    p = Pair(tmp_path, cfg, seed=5, edit=edit, n_ctx=400)
    toks = p.tokens(330, seed=9)
    want = p.expected(toks)
    other = list(toks); other[3] = (toks[3] + 1) % 40
    assert err(p.expected(other)[300:], want[300:]) > 20 * TOL32          # position 3 is seen from 300 on
    got = p.run(toks, [300, 1])
    assert err(got, want) < TOL32
    assert err(got[:4], want[:4]) < TOL32             # the first tokens of a sequence: zero state, one key
    assert err(p.run(toks[:40], [1]), want[:40]) < TOL32
    assert err(p.run(toks, [2, 129, 3, 64]), want) < TOL32
    assert err(p.run(other, [31, 32, 33, 1]), p.expected(other)) < TOL32
    p.close()


def test_far_tokens_through_the_retention_state(tmp_path):
    """a slow decay keeps a token for hundreds of positions; the rotation's fast pairs turn many times on the way"""
    cfg = config([retention(heads=2, dim=8, vdim=8, rot=8, base=10.0, decay=[0.998, 0.9995])], width=32, vocab=40)
    p = Pair(tmp_path, cfg, seed=2, n_ctx=600)
    toks = p.tokens(520, seed=4)
    want = p.expected(toks)
    other = list(toks); other[2] = (toks[2] + 1) % 40
    assert err(p.expected(other)[500:], want[500:]) > 20 * TOL32
    assert err(p.run(toks), want) < TOL32             # two passes: the state crosses the pass's edge
    assert err(p.run(toks, [490, 1]), want) < TOL32
    assert err(p.run(toks, [7, 250, 2, 1]), want) < TOL32
    p.close()


def test_long_portions_run_the_retention_chunk_by_chunk(tmp_path):
    """portions of 128 tokens and more take the chunked form of the recurrence (32-token chunks, ragged last chunk), shorter ones
    the token walk: both against the oracle, with head sizes that are no multiple of 4, more than 128 value channels (two column
    tiles) and a decay so fast that its powers vanish within a chunk"""
    layers = [retention(heads=2, dim=6, vdim=130, rot=4, decay=[0.05, 0.999]), retention(heads=3, dim=64, vdim=8, rot=64, decay=[0.9, 0.5, 0.99], mlp=moe()),
              parallel(right=ret_mixer(heads=1, dim=9, vdim=5, rot=8, decay=[0.97]))]
    p = Pair(tmp_path, config(layers), seed=4, n_ctx=420)
    toks = p.tokens(400, seed=8)
    want = p.expected(toks)
    for cuts in (None, [128, 129, 143], [127, 1, 160, 112], [131, 5, 264], [200, 1]):
        assert err(p.run(toks, cuts), want) < TOL32, cuts
    p.close()


def test_query_temperature_steps_at_multiples_of_every(tmp_path):
    """the temperature changes exactly where (p + 1) / every crosses an integer: an oracle whose step is one position off differs
    there and only there"""
    cfg = config([parallel(heads=2, kv_heads=2, dim=8, vdim=8, scale=1.0, coef=2.0, every=7)], width=32)
    p = Pair(tmp_path, cfg, seed=7)
    toks = p.tokens(40, seed=7)
    want = p.expected(toks)
    c2 = copy.deepcopy(cfg); c2["layers"][0]["mixer"]["left"]["q_temp"]["every"] = 8
    off = p.expected(toks, cfg=c2)
    assert err(off[:6], want[:6]) < 1e-9 and err(off[6:7], want[6:7]) > 20 * TOL32
    for cuts in (None, [1], [6, 1], [7, 1], [5, 2, 1]):
        assert err(p.run(toks, cuts), want) < TOL32, cuts
    p.close()


def test_router_choices_follow_the_groups(tmp_path):
    """router rows far apart: the chosen experts are never a close call, and an expert outside the kept groups is never used even
    when its own score is among the largest"""
    cfg = config([retention(mlp=moe(experts=8, top=2, groups=(4, 1), ff=8, shared=0))], width=32)
    p = Pair(tmp_path, cfg, seed=11, edit=sharpen(["mlp.router"], 3.0))
    toks = p.tokens(64, seed=3)
    want = p.expected(toks)
    c2 = copy.deepcopy(cfg); c2["layers"][0]["mlp"]["router"]["groups"] = {"count": 1, "keep": 1}
    assert err(p.expected(toks, cfg=c2), want) > 20 * TOL32
    for cuts in (None, [1], [3], [9, 2]):
        assert err(p.run(toks, cuts), want) < TOL32, cuts
    p.close()


def test_long_decoding_through_the_graph(tmp_path):
    p = Pair(tmp_path, config(FULL[:4]))
    toks = p.tokens(300, seed=11)
    want = p.expected(toks)
    got = p.run(toks, [4, 1])
    assert err(got, want) < 2 * TOL32
    assert err(got[-1:], want[-1:]) < 2 * TOL32
    p.close()


@pytest.mark.parametrize("width,vocab", [(36, 50), (40, 77), (64, 130), (37, 53)], ids=["scalar-loads", "width-40", "vector-loads", "odd-width"])
def test_other_sizes(tmp_path, width, vocab):
    layers = [parallel(heads=6, kv_heads=2, dim=9, vdim=5, coef=0.1, every=1, right=ret_mixer(heads=1, dim=64, vdim=3, rot=10), mlp=moe(experts=3, top=3, groups=None, ff=7, shared=3)),
              retention(heads=1, dim=6, vdim=40, rot=0),
              parallel(heads=4, kv_heads=4, dim=16, vdim=40, every=1000, right=ret_mixer(heads=5, dim=12, vdim=16, rot=12)),
              retention(heads=5, dim=3, vdim=3, rot=2, mlp=moe(experts=16, top=4, groups=(4, 2), ff=64, shared=64)),
              parallel(heads=1, kv_heads=1, dim=4, vdim=36, right=ret_mixer(heads=2, dim=32, vdim=32, rot=32), mlp=moe(experts=1, top=1, groups=(1, 1), ff=24))]
    p = Pair(tmp_path, config(layers, width=width, vocab=vocab, eps=1e-6), seed=width)
    toks = p.tokens(70, seed=width)
    want = p.expected(toks)
    assert err(p.run(toks), want) < TOL32
    assert err(p.run(toks, [13, 2, 1]), want) < TOL32
    p.close()


def random_config(rng):
    """a random arrangement of the mixers with random sizes: nothing may rest on one model's values"""
    pick = lambda values: int(rng.choice(values))

    def rnd_ret():
        d = pick([2, 4, 16, 32, 48, 128])
        h = pick([1, 2, 3, 6])
        return ret_mixer(heads=h, dim=d, vdim=pick([4, 8, 48, 128, 200]), rot=pick([r for r in (0, 2, 4, 16, 32, 48, 128) if r <= d]), base=float(rng.choice([100.0, 1e4, 5e5])),
                         decay=[float(x) for x in 1.0 - 2.0 ** -rng.uniform(1, 9, size=h)])

    def rnd_moe():
        if rng.random() < 0.3:
            return None
        g = pick([1, 2, 4])
        per = pick([1, 2, 3])
        keep = pick(range(1, g + 1))
        return moe(experts=g * per, top=pick(range(1, keep * per + 1)), groups=(g, keep) if rng.random() < 0.8 or g > 1 else None, ff=pick([8, 24, 64, 100]),
                   shared=pick([0, 8, 40, 136]), scale=float(rng.choice([1.0, 2.5])))
    layers = []
    for _ in range(pick([2, 3, 4, 5])):
        if rng.random() < 0.5:
            layers.append({"type": "retention", "mixer": rnd_ret(), "mlp": rnd_moe()})
        else:
            kv = pick([1, 2, 3])
            layers.append(parallel(heads=kv * pick([1, 2, 4]), kv_heads=kv, dim=pick([4, 16, 32, 128]), vdim=pick([4, 8, 48, 128, 200]), scale=float(rng.choice([0.1, 0.3])),
                                   coef=float(rng.choice([0.0, 0.5, 1.5])), every=pick([1, 3, 16, 128]), right=rnd_ret(), mlp=rnd_moe()))
    return config(layers, width=pick([24, 36, 64, 100, 136]), vocab=pick([37, 100, 257, 513]), eps=float(rng.choice([1e-6, 1e-5])))


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(tmp_path, seed):
    rng = np.random.default_rng(900 + seed)
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
    """a 700-token step runs as two passes of the layers: cached keys, recurrent state and the depth history cross the pass's edge"""
    p = Pair(tmp_path, config(FULL[:3]), n_ctx=704)
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
    layers = [retention(heads=2, dim=32, vdim=32, rot=16, mlp=moe(experts=4, top=2, groups=(2, 1), ff=64, shared=64)),
              parallel(heads=4, kv_heads=2, dim=16, vdim=32, right=ret_mixer(heads=2, dim=32, vdim=32, rot=32), mlp=moe(experts=3, top=1, groups=None, ff=128, shared=0))]
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
    ctx = L.initContext(7, p.dir.encode(), 1, 0, 100, 0, 0, 0, 64, n_gen, 0, 0.0, 0.0, 0.0, 1, 1.0, 1.0, 1.0, 0, 0, 200, 1.0, 1.0, 1.0, 42, b"")
    assert ctx, _lib.last_error()
    n = L.doInference(7, ctx, b"tosevik-job", b"", " ".join(map(str, prompt)).encode())
    out = [int(x) for x in L.status(b"tosevik-job").decode().split()]
    assert out[:len(prompt)] == prompt and out[len(prompt):] == ids
    assert n == len(prompt) + n_gen - 1 and L.getPromptTokenCount(b"tosevik-job") == len(prompt)
    # the device-resident loop of the token-level interface gives the same ids
    p.ctx.kv_clear()
    first = int(np.argmax(p.ctx.decode(prompt, 0)))
    dev = p.ctx.generate_greedy(first, len(prompt), n_gen - 1).tolist()
    assert [first] + dev == ids
    after = p.ctx.decode([ids[-1]], len(prompt) + n_gen - 1)
    assert err(after[None], p.expected(seq)[-1][None]) < TOL32
    assert p.ctx.L.b200_kernel_launches(p.ctx.h) > 0
    p.close()


def test_trace_runner_replays_steps_and_reuses_a_finished_requests_context(tmp_path):
    """bin/trace_run on a folder model: steps arrive as JSON lines, the wanted rows of each step come back as a float32 file, a
    request that ends gives its context back and the next request starts from a clean one"""
    import json
    import os
    import subprocess
    import sys
    cfg = config(FULL[:3])
    w = to.random_model(cfg, 5)
    d = to.write_model(str(tmp_path / "m"), cfg, w)
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
    wa, wb = to.forward(cfg, w, a), to.forward(cfg, w, b)
    for n, want in ((0, wa[[0, 7, 30]]), (2, wa[[39, 34]]), (3, wb[[21]]), (4, wb[[22]])):
        got = np.fromfile(str(out / ("%d.f32" % n)), "<f4").reshape(len(want), cfg["vocab"])
        assert err(got, want) < TOL32, n


def test_bad_models_fail_loudly(tmp_path):
    cfg = config([retention(mlp=moe()), parallel()])
    w = to.random_model(cfg)
    c2 = copy.deepcopy(cfg); c2["layers"][0]["type"] = "mingru"
    with pytest.raises(_lib.B200Error, match="not part of the Tosevik design"):
        engine.Model(to.write_model(str(tmp_path / "mixer"), c2, w))
    w2 = dict(w); del w2["l1.mix.left.pb"]
    with pytest.raises(_lib.B200Error, match="missing tensor"):
        engine.Model(to.write_model(str(tmp_path / "missing"), cfg, w2))
    c3 = copy.deepcopy(cfg); c3["layers"][0]["mixer"]["decay"] = [0.5]
    with pytest.raises(_lib.B200Error, match="one number per head"):
        engine.Model(to.write_model(str(tmp_path / "decay"), c3, w))
    c4 = copy.deepcopy(cfg); c4["layers"][1]["mixer"]["left"]["kv_heads"] = 3
    with pytest.raises(_lib.B200Error, match="multiple of kv_heads"):
        engine.Model(to.write_model(str(tmp_path / "heads"), c4, w))
    c5 = copy.deepcopy(cfg); c5["layers"][0]["mlp"]["router"]["top"] = 5
    with pytest.raises(_lib.B200Error, match="exceeds the experts of the kept groups"):
        engine.Model(to.write_model(str(tmp_path / "top"), c5, w))
