"""The numpy restatement of the Tosevik design checked against itself on the CPU: properties that follow from the equations
(causality, the retention state against its closed forms, the rotation's relative-position property, the router's choice under
groups, the depth average, the sigmoid attention's distance penalty) hold for the oracle the GPU tests compare with; the
synthetic-model writer of the package produces what the oracle reads."""
import numpy as np

import stack_oracle as so
import tosevik_oracle as to

RET = {"type": "retention", "mixer": {"heads": 2, "dim": 6, "vdim": 4, "rot": {"base": 50.0, "dims": 4}, "decay": [0.9, 0.5]}, "mlp": None}
MOE = {"kind": "moe", "expert": {"ff": 10}, "shared": {"ff": 6}, "router": {"experts": 6, "top": 2, "scale": 1.4, "groups": {"count": 3, "keep": 2}}}
PAR = {"type": "parallel", "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 4, "vdim": 6, "scale": 0.5, "q_temp": {"coef": 0.7, "every": 4}},
                                     "right": {"heads": 2, "dim": 4, "vdim": 4, "rot": {"base": 10.0, "dims": 2}, "decay": [0.8, 0.95]}}, "mlp": MOE}


def cfg_of(layers):
    return {"architecture": "Tosevik", "layers": layers, "norm": {"eps": 1e-5}, "vocab": 41, "width": 24}


def f64(W):
    return {k: np.asarray(v, np.float64) for k, v in W.items()}


def test_later_tokens_do_not_reach_back_and_every_layer_reports_what_it_hands_on():
    c = cfg_of([RET, PAR, dict(RET, mlp=MOE)])
    W = to.random_model(c, 1)
    toks = np.random.default_rng(0).integers(0, 41, size=30).tolist()
    res = []
    full = to.forward(c, W, toks, res)
    assert len(res) == 3 and res[0].shape == (30, 24) and full.shape == (30, 41)
    other = toks[:20] + [(t + 1) % 41 for t in toks[20:]]
    assert np.allclose(to.forward(c, W, other)[:20], full[:20], atol=1e-12)


def test_retention_after_one_token_and_as_a_decayed_sum():
    mx = RET["mixer"]
    W = f64(to.sub(to.random_model(cfg_of([RET]), 3), "l0.mix."))
    h = np.random.default_rng(2).standard_normal((7, 24))
    got = to.mix_retention(h, W, mx, 1e-5)
    pos = np.arange(7)
    q = to.rotate_front((h @ W["q"].T).reshape(7, 2, 6), pos, mx["rot"])
    k = to.rotate_front((h @ W["k"].T).reshape(7, 2, 6), pos, mx["rot"]) / np.sqrt(6.0)
    v = (h @ W["v"].T).reshape(7, 2, 4)
    o = np.zeros((7, 2, 4))
    for hd in range(2):
        for t in range(7):
            for j in range(t + 1):                      # o_t = sum_(j <= t) decay^(t - j) (q_t . k_j) v_j
                o[t, hd] += mx["decay"][hd] ** (t - j) * (q[t, hd] @ k[j, hd]) * v[j, hd]
    want = (to.unit_rms(o, 1e-5).reshape(7, 8) * to.silu(h @ W["g"].T)) @ W["o"].T
    assert np.allclose(got, want, atol=1e-12)
    assert np.allclose(o[0, 0], (q[0, 0] @ k[0, 0]) * v[0, 0])            # S_1 = k v^T from a zero state


def test_rotation_makes_scores_depend_on_the_distance_only_and_leaves_the_tail_alone():
    rot = {"base": 100.0, "dims": 4}
    rng = np.random.default_rng(5)
    a, b = rng.standard_normal((1, 1, 6)), rng.standard_normal((1, 1, 6))
    def score(p, j):
        return float(to.rotate_front(a, [p], rot)[0, 0] @ to.rotate_front(b, [j], rot)[0, 0])
    assert abs(score(9, 4) - score(105, 100)) < 1e-9 and abs(score(9, 4) - score(9, 5)) > 1e-6
    assert np.array_equal(to.rotate_front(a, [17], rot)[..., 4:], a[..., 4:])
    # pairs are (i, i + dims / 2): turning position 0 is the identity, and a quarter turn of pair 0 swaps its two entries
    assert np.allclose(to.rotate_front(a, [0], rot), a)
    x = np.zeros((1, 1, 6)); x[0, 0, 0] = 1.0
    y = to.rotate_front(x, [np.pi / 2], rot)[0, 0]
    assert abs(y[0]) < 1e-12 and abs(y[2] - 1.0) < 1e-12


def test_router_chooses_inside_the_best_groups_only():
    r = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    z = np.array([[0.0, 0.1, 3.0, 0.2, 2.9, 2.5]])       # groups (0,1) (2,3) (4,5): best single expert 2, so group 1 is kept
    W = {"router": np.eye(6)}
    chosen, weight = to.route(z, W, r)
    s = np.exp(z[0]) / np.exp(z[0]).sum()
    assert chosen.tolist() == [[2, 3]] and np.allclose(weight[0], 2.0 * s[[2, 3]])
    r2 = dict(r, groups={"count": 3, "keep": 2})
    assert to.route(z, W, r2)[0].tolist() == [[2, 4]]
    assert to.route(z, W, dict(r, groups=None))[0].tolist() == [[2, 4]]
    assert to.route(z, W, dict(r, top=3, groups={"count": 1, "keep": 1}))[0].tolist() == [[2, 4, 5]]


def test_depth_average_with_unit_coefficients_is_the_plain_stack():
    c = cfg_of([RET, dict(RET, mlp=MOE)])
    W = f64(to.random_model(c, 4))
    W["l0.dwa"] = np.array([0.0, 1.0]); W["l1.dwa"] = np.array([0.0, 0.0, 1.0])
    toks = [3, 9, 27, 1, 5]
    res = []
    to.forward(c, W, toks, res)
    x = to.dyt(W["embed"][toks], W, "embed.norm")
    x = x + to.mix_retention(to.dyt(x, W, "l0.norm1"), to.sub(W, "l0.mix."), RET["mixer"], 1e-5)
    assert np.allclose(res[0], x, atol=1e-12)
    W["l1.dwa"] = np.array([0.5, 0.0, 1.0])
    res2 = []
    to.forward(c, W, toks, res2)
    assert np.allclose(res2[1] - res[1], 0.5 * to.dyt(W["embed"][toks], W, "embed.norm"), atol=1e-12)


def test_sigmoid_attention_weights_fall_with_distance_by_the_head_slope():
    mx = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 3, "scale": 0.0, "q_temp": {"coef": 0.0, "every": 1}}     # scale 0: only the penalty and the offset are left
    W = {"q": np.zeros((8, 5)), "k": np.zeros((4, 5)), "v": np.zeros((3, 5)), "q.norm": np.ones(8), "k.norm": np.ones(4), "pb": np.array([0.3, -0.2]), "o": np.eye(6)}
    W["v"][:, 0] = [1.0, 2.0, 3.0]
    h = np.zeros((6, 5)); h[2, 0] = 1.0                   # one token carries a value
    out = to.mix_sigmoid_attention(h, W, mx, 1e-12).reshape(6, 2, 3)
    unit = np.array([1.0, 2.0, 3.0]) / np.sqrt(np.mean(np.array([1.0, 4.0, 9.0])))
    for hd, slope in ((0, 2.0 ** -4), (1, 2.0 ** -8)):
        for p in range(6):
            w = to.sigm(W["pb"][hd] - slope * (p - 2)) if p >= 2 else 0.0
            assert np.allclose(out[p, hd], w * unit, atol=1e-9)


def test_the_package_writes_synthetic_models_the_oracle_reads(tmp_path):
    from booster_b200 import stack_io
    c = stack_io.tosevik_config(64, 3, 64, 2, vocab=100, head_dim=16, experts=4, top=2, groups=(2, 1))
    d = stack_io.synth_stack(str(tmp_path / "m"), c)
    W = so.load_safetensors(d + "/model.safetensors")
    assert sorted(W) == sorted(to.tensor_shapes(c)) and stack_io.n_params(c) == sum(int(np.prod(v.shape)) for v in W.values())
    assert np.isfinite(to.forward(c, W, [1, 2, 3, 4, 5])).all()
