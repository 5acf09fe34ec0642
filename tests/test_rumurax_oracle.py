"""The numpy restatement of the Rumurax design checked against itself and by hand (CPU): causality, the exact reach of both masks,
block means that appear only when a block is complete and wholly before the window, the sink and the cap on a hand-made input,
streams that reduce to the plain residual, the router's choice, the rotation's relative-position property, the model writer."""
import numpy as np

import rumurax_oracle as ro
import stack_oracle as so
from test_rumurax_gpu import chunk, config, latent, moe, sees, window


def test_later_tokens_do_not_reach_back():
    cfg = config([window(v_mix=True, mlp=moe()), chunk(v_mix=True), latent(mlp=moe(top=1))])
    w = ro.random_model(cfg, 1)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], size=40).tolist()
    full = ro.forward(cfg, w, toks)[0]
    for n in (1, 2, 17, 39):
        assert np.allclose(ro.forward(cfg, w, toks[:n])[0], full[:n], rtol=0, atol=1e-9)


def test_masks_by_hand():
    assert ro.visible_chunk(10, 4).tolist() == [8, 9, 10] and ro.visible_chunk(8, 4).tolist() == [8] and ro.visible_chunk(3, 4).tolist() == [0, 1, 2, 3]
    t, b = ro.visible_window(9, 4, 3)
    assert t.tolist() == [6, 7, 8, 9] and b.tolist() == [0, 1]       # block 1 = 3..5 ends at 5 <= 9 - 4
    t, b = ro.visible_window(11, 4, 3)
    assert t.tolist() == [8, 9, 10, 11] and b.tolist() == [0, 1]     # block 2 = 6..8 ends at 8 > 11 - 4: tokens 6 and 7 are seen by nobody
    t, b = ro.visible_window(12, 4, 3)
    assert t.tolist() == [9, 10, 11, 12] and b.tolist() == [0, 1, 2]
    t, b = ro.visible_window(3, 4, 3)
    assert t.tolist() == [0, 1, 2, 3] and len(b) == 0
    t, b = ro.visible_window(20, 4, 0)
    assert t.tolist() == [17, 18, 19, 20] and len(b) == 0
    for layer in (chunk(size=5), window(size=4, pool=3), window(size=6, pool=0)):
        for p in range(30):
            if layer["type"] == "attention":
                toks, blocks, P = ro.visible_chunk(p, 5), [], 0
            else:
                P = layer["mixer"]["mask"].get("pool", 0)
                toks, blocks = ro.visible_window(p, layer["mixer"]["mask"]["size"], P)
            seen = set(toks.tolist()) | {b * P + i for b in blocks for i in range(P)}
            assert seen == {j for j in range(30) if sees(layer, p, j)}


def test_soft_max_with_a_sink_by_hand():
    w = ro.softmax_sink(np.array([0.0, np.log(2.0)]), np.log(3.0))
    assert np.allclose(w, [1 / 6, 2 / 6])
    assert np.allclose(ro.softmax_sink(np.array([1.0, 1.0]), None), [0.5, 0.5])


def test_one_stream_with_unit_weights_is_the_plain_residual():
    cfg = config([chunk(mlp=moe())], streams=1)
    w = ro.random_model(cfg, 2)
    for k in list(w):
        if ".hc" in k:
            w[k] = np.ones_like(w[k])
    stripped = {k: v for k, v in w.items() if ".hc" not in k}
    toks = [3, 1, 4, 1, 5, 9, 2, 6]
    assert np.allclose(ro.forward(cfg, w, toks)[0], ro.forward(cfg, stripped, toks)[0])


def test_router_takes_the_largest_scores_lowest_index_first():
    Wr = np.array([[1.0, 0.0], [0.0, 1.0], [1.0, 0.0], [-1.0, 0.0]])
    sel, wt = ro.route(np.array([[2.0, 1.0]]), Wr, 3)
    assert sel.tolist() == [[0, 2, 1]] and np.allclose(wt, ro.sigmoid(np.array([[2.0, 2.0, 1.0]])))


def test_rotation_depends_on_the_distance_only():
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((1, 1, 8)), rng.standard_normal((1, 1, 8))
    dots = [float((ro.rotate_pairs(q, [p + 3], 100.0, 6) * ro.rotate_pairs(k, [p], 100.0, 6)).sum()) for p in (0, 5, 40)]
    assert np.allclose(dots, dots[0])
    assert np.allclose(ro.rotate_pairs(q, [7], 100.0, 6)[..., 6:], q[..., 6:])           # entries past rot.dims pass unchanged
    r = ro.rotate_pairs(np.array([[[1.0, 0.0]]]), [1], 100.0, 2)
    assert np.allclose(r, [[[np.cos(1.0), np.sin(1.0)]]])                                  # neighbours (2i, 2i + 1) form a pair


def test_model_writer_round_trips(tmp_path):
    cfg = config([window(v_mix=True, mlp=moe()), latent()])
    w = ro.random_model(cfg, 3)
    d = ro.write_model(str(tmp_path / "m"), cfg, w)
    back = so.load_safetensors(d + "/model.safetensors")
    assert set(back) == set(w) == set(ro.tensor_shapes(cfg))
    for k in w:
        assert list(np.shape(back[k])) == ro.tensor_shapes(cfg)[k] and np.array_equal(np.asarray(back[k], np.float64), w[k])
