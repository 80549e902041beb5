"""Host-side pieces of the Nafelix family (no GPU): config -> layer descriptors (one per run of a layer), the tensor set, the
registry, and sanity properties of the float64 oracle's mechanisms."""
import copy

import numpy as np
import pytest

import nafelix_util as nu
from oracle import nafelix_ref as ref


def f64(w):
    return {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}


def test_config_to_descriptors():
    from llama_cpp import _cabi, nafelix
    cfg = nu.config([nu.parallel(mlp=nu.dense(44), left=nu.attn(heads=6, kv_heads=3, dim=10, vdim=14, window=21, rot=4, base=777.0, scale=0.3),
                                 right=nu.delta(heads=4, kv_heads=2, dim=8, vdim=6, conv=5)),
                     nu.attention(mlp=nu.moe(experts=7, top=3, ff=16, limit=2.5)), nu.attention(), nu.parallel(mlp=nu.moe())],
                    streams=5, taps=2, loop=(1, 3, 2))
    d = nafelix.read_dims(cfg)
    assert d.block_style == _cabi.B2_BLOCK_HYPER_RMS and d.n_streams == 5 and d.canon_taps == 2
    assert [x.weights_of for x in d.layers] == [1, 2, 3, 2, 3, 4] and d.n_layer == 6
    a, b, c = d.layers[0], d.layers[1], d.layers[2]
    assert (a.mixer, a.n_head, a.n_head_kv, a.head_dim, a.attn_vdim, a.window, a.rot_dims, a.rope_base, a.attn_scale) == (_cabi.B2_MIX_SINK_DELTA, 6, 3, 10, 14, 21, 4, 777.0, 0.3)
    assert a.attn_flags == _cabi.B2_ATTN_TALK | _cabi.B2_ATTN_HEAD_GATE
    assert (a.mm_heads, a.key_heads, a.mm_dim, a.mm_vdim, a.conv_taps) == (4, 2, 8, 6, 5)
    assert (a.ff_kind, a.n_ff) == (_cabi.B2_FF_PIECEWISE, 44)
    assert (b.mixer, b.attn_flags) == (_cabi.B2_MIX_SINK_ATTN, _cabi.B2_ATTN_BIAS | _cabi.B2_ATTN_UNIT_QK)
    assert (b.ff_kind, b.n_ff, b.moe_experts, b.moe_top, b.moe_route, b.moe_renorm, b.moe_expert, b.moe_limit) == (
        _cabi.B2_FF_MOE, 16, 7, 3, _cabi.B2_ROUTE_SOFTMAX_ALL, 1, _cabi.B2_EXPERT_CLAMPED, 2.5)
    assert c.n_ff == 0
    shapes = nafelix.tensor_shapes(cfg)
    assert shapes["l0.mix.left.g"] == (6, 72) and shapes["l0.mix.left.talk"] == (6, 6) and shapes["l0.mix.left.o"] == (72, 84)
    assert shapes["l0.mix.right.a"] == (4, 72) and shapes["l0.mix.right.q.conv"] == (16, 5) and shapes["l0.mix.right.norm"] == (6,)
    assert shapes["l1.mix.g"] == (96, 72) and shapes["l1.mix.q.b"] == (96,) and "l1.mix.talk" not in shapes
    assert shapes["l1.hc2.mix"] == (5, 5) and shapes["l1.canon2"] == (72, 2) and "l2.norm2" not in shapes and "l2.hc2.in" not in shapes
    plain = nu.config([nu.attention()], streams=0, taps=0)
    assert nafelix.read_dims(plain).n_streams == 1 and not any(".hc" in n or "canon" in n for n in nafelix.tensor_shapes(plain))


def test_registry_and_folder(tmp_path):
    from llama_cpp import models, nafelix
    cfg = nu.config([nu.parallel(mlp=nu.moe())])
    path = nu.write_model(str(tmp_path / "m"), cfg, nu.random_weights(cfg))
    assert models.open_model(path).family.name == "Nafelix" and "Nafelix" in models.architectures()
    with pytest.raises(ValueError):
        nafelix.layer_desc(0, {"type": "nope", "mixer": {}})
    with pytest.raises(ValueError):
        nafelix.layer_runs({"layers": [1, 2], "loop": {"start": 1, "stop": 3, "times": 2}})
    assert nafelix.layer_runs({"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}) == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert ref.layer_runs({"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}) == [0, 1, 2, 1, 2, 1, 2, 3, 4]


def test_window_and_sink():
    """A changed token moves the attention output of the positions whose window holds it and of no other; a sink far above the
    scores silences a head."""
    cfg = nu.config([nu.attention(m=nu.attn(heads=2, kv_heads=1, dim=8, vdim=8, window=5, rot=4))])
    w = f64(nu.random_weights(cfg, seed=1))
    h = np.random.default_rng(2).standard_normal((17, cfg["width"]))
    h2 = h.copy()
    h2[6] += 1.0
    m = cfg["layers"][0]["mixer"]
    w["l0.mix.g"] = w["l0.mix.g"] * 0           # a gate of one half everywhere: it reads h too and would move row 6 alone
    moved = np.abs(ref.attention_mixer(h, w, "l0.mix.", m, 1e-6) - ref.attention_mixer(h2, w, "l0.mix.", m, 1e-6)).max(-1) > 1e-12
    assert moved.tolist() == [6 <= i <= 10 for i in range(17)]
    w["l0.mix.sink"] = np.array([60.0, 60.0])
    assert np.abs(ref.attention_mixer(h, w, "l0.mix.", m, 1e-6)).max() < 1e-12


def test_sink_softmax_denominator():
    s = np.array([[0.3, -np.inf], [1.0, 2.0]])
    p = ref.sink_softmax(s, np.array([[True, False], [True, True]]), 0.5)
    assert np.allclose(p[0], [np.exp(0.3) / (np.exp(0.3) + np.exp(0.5)), 0.0])
    assert np.allclose(p[1].sum(), (np.exp(1.0) + np.exp(2.0)) / (np.exp(1.0) + np.exp(2.0) + np.exp(0.5)))


def test_mixed_heads_use_their_own_values():
    """With a mixing matrix that hands head 0 the weights of head 3, head 0 applies head 3's weights to the values of ITS OWN
    key/value head."""
    cfg = nu.config([nu.parallel(left=nu.attn(heads=4, kv_heads=2, dim=8, vdim=6, window=50, rot=0))])
    w = f64(nu.random_weights(cfg, seed=3))
    p, m = "l0.mix.left.", cfg["layers"][0]["mixer"]["left"]
    T = 9
    h = np.random.default_rng(4).standard_normal((T, cfg["width"]))
    talk = np.zeros((4, 4))
    talk[0, 3] = 1.0
    w[p + "talk"] = talk
    w[p + "o"] = np.eye(cfg["width"], 24)
    w[p + "g"] = w[p + "g"] * 0
    out = ref.window_attention(h, w, p, m, 1e-6, biases=False, unit_qk=False, talk=True)[:, :24].reshape(T, 4, 6) * 2.0
    q, k, v = (h @ w[p + n].T for n in "qkv")
    t = T - 1
    s = (q[t, 24:32] @ k[:, 8:16].T) * m["scale"]           # head 3 scores against key head 1
    pr = np.exp(s) / (np.exp(s).sum() + np.exp(w[p + "sink"][3]))
    assert np.allclose(out[t, 0], pr @ v[:, 0:6])            # ... applied to the values of key/value head 0
    assert np.allclose(out[t, 1:], 0.0)


def test_delta_rule_returns_what_it_stored():
    """With beta = 1 and no decay the memory returns the value just written for its key: o = (k . q) v."""
    cfg = nu.config([nu.parallel(right=nu.delta(heads=2, kv_heads=1, dim=6, vdim=5, conv=1))])
    w = f64(nu.random_weights(cfg, seed=5))
    p, m = "l0.mix.right.", cfg["layers"][0]["mixer"]["right"]
    h = np.random.default_rng(6).standard_normal((1, cfg["width"]))
    w[p + "b"] = np.outer(np.ones(2), h[0]) * 10.0          # beta -> 1 for this input
    w[p + "A_log"] = np.array([-30.0, -30.0])
    w[p + "o"] = np.eye(cfg["width"], 10)
    w[p + "norm"] = np.ones(5)
    got = ref.head_delta(h, w, p, m, 0.0)[0, :10].reshape(2, 5)
    q = ref.silu(h @ w[p + "q"].T * w[p + "q.conv"][:, -1])[0]
    k = ref.silu(h @ w[p + "k"].T * w[p + "k.conv"][:, -1])[0]
    v = ref.silu(h @ w[p + "v"].T * w[p + "v.conv"][:, -1])[0].reshape(2, 5)
    q, k = q / np.sqrt(q @ q + 1e-6) * 6 ** -0.5, k / np.sqrt(k @ k + 1e-6)
    o = (k @ q) * v
    want = o / np.sqrt((o * o).mean(-1, keepdims=True)) * ref.silu(h @ w[p + "g"].T).reshape(2, 5)
    assert np.allclose(got, want, rtol=1e-6)


def test_routing_renormalises_the_chosen_scores():
    w = {"p.router": np.array([[1.0, 0], [0, 1.0], [0.5, 0.5], [0, 0]])}
    chosen, weight = ref.route(np.array([[1.0, 0.2]]), w, "p.", {"experts": 4, "top": 2})
    assert chosen.tolist() == [[0, 2]]
    z = np.exp(np.array([1.0, 0.6]))
    assert np.allclose(weight, z / z.sum()) and np.allclose(weight.sum(), 1.0)


def test_clamped_expert_and_piecewise_activation():
    w = {"e.gate": np.array([[3.0], [-3.0]]), "e.up": np.array([[5.0], [-5.0]]), "e.down": np.eye(2)}
    out = ref.clamped_expert(np.array([1.0]), w, "e.", 2.0)
    assert np.allclose(out, [2.0 * ref.sigmoid(1.702 * 2.0) * 3.0, -3.0 * ref.sigmoid(1.702 * -3.0) * -1.0])
    z = np.array([-2.0, 0.0, 1.5])
    a = ref.piecewise_act(z, 0.3, -0.2)
    sp = lambda x: np.log1p(np.exp(x))
    assert np.allclose(a, [(0.5 + sp(-0.2)) * (np.exp(-2.0) - 1 + 2.0) - 1.0, 0.0, sp(0.3) * 2.25 + 0.75])


def test_stream_copies_and_plain_residual():
    """Identity mixing with unit write weights and a read of copy 0 alone is the plain residual stream."""
    cfg = nu.config([nu.attention(mlp=nu.dense(20)), nu.parallel(mlp=nu.moe())], streams=3, taps=0)
    w = nu.random_weights(cfg, seed=7)
    for i in range(2):
        for q in "12":
            w[f"l{i}.hc{q}.mix"] = np.eye(3, dtype=np.float32)
            w[f"l{i}.hc{q}.out"] = np.array([1.0, 0.0, 0.0], dtype=np.float32)
            w[f"l{i}.hc{q}.in"] = np.array([1.0, 0.0, 0.0], dtype=np.float32)
    plain_cfg = copy.deepcopy(cfg)
    del plain_cfg["streams"]
    plain_w = {k: v for k, v in w.items() if ".hc" not in k}
    toks = [int(t) for t in np.random.default_rng(8).integers(0, cfg["vocab"], size=20)]
    _, la = ref.forward(cfg, w, toks, return_layers=True)
    _, lb = ref.forward(plain_cfg, plain_w, toks, return_layers=True)
    x0 = f64(w)["embed"][toks]
    assert np.allclose(la - 2 * x0[None], lb)        # copies 1 and 2 never change; copy 0 is the plain stream


def test_repeated_layers_share_weights_not_state():
    cfg = nu.config([nu.parallel(mlp=nu.dense(16)), nu.attention()], loop=(0, 2, 2))
    unrolled = nu.config([nu.parallel(mlp=nu.dense(16)), nu.attention(), nu.parallel(mlp=nu.dense(16)), nu.attention()])
    w = nu.random_weights(cfg, seed=9)
    w2 = dict(w)
    for k, v in w.items():
        if k.startswith("l0."):
            w2["l2." + k[3:]] = v
        if k.startswith("l1."):
            w2["l3." + k[3:]] = v
    toks = [int(t) for t in np.random.default_rng(10).integers(0, cfg["vocab"], size=25)]
    assert np.allclose(ref.forward(cfg, w, toks), ref.forward(unrolled, w2, toks))


def test_oracle_is_causal():
    cfg = nu.config([nu.parallel(mlp=nu.moe()), nu.attention(mlp=nu.dense())], loop=(0, 1, 2))
    w = nu.random_weights(cfg, seed=4)
    toks = [int(t) for t in np.random.default_rng(5).integers(0, cfg["vocab"], size=30)]
    full = ref.forward(cfg, w, toks)
    assert np.allclose(ref.forward(cfg, w, toks[:17]), full[:17], atol=1e-10)
