"""Host-side pieces of the Dibesun family (no GPU): config -> layer descriptors, the tensor set, the registry, and sanity
properties of the float64 oracle's mechanisms."""
import copy

import numpy as np
import pytest

import dibesun_util as du
from oracle import dibesun_ref as ref


def test_config_to_descriptors():
    from llama_cpp import _cabi, dibesun
    cfg = du.config([du.layer(mlp=du.dense(44), l=du.left(heads=6, kv_heads=3, dim=10, vdim=14, chunk=21, scale=0.3, softcap=7.5),
                              r=du.right(heads=2, dim=8, vdim=6, decay=[0.5, 0.9]), left_scale=0.25, right_scale=2.0),
                     du.layer(mlp=du.moe(experts=7, top=3, ff=16, shared=12)), du.layer(mlp=du.moe(shared=0)), du.layer()],
                    groups=4, embed_scale=3.5)
    d = dibesun.read_dims(cfg)
    assert d.block_style == _cabi.B2_BLOCK_OUTNORM_RMS and d.norm_groups == 4 and d.embed_scale == 3.5 and d.tie_head
    a, b, c, e = d.layers
    assert (a.mixer, a.n_head, a.n_head_kv, a.head_dim, a.attn_vdim, a.window, a.attn_scale, a.softcap) == (_cabi.B2_MIX_CHUNK_LINEAR, 6, 3, 10, 14, 21, 0.3, 7.5)
    assert (a.mm_heads, a.mm_dim, a.mm_vdim, a.branch_scale[0], a.branch_scale[1]) == (2, 8, 6, 0.25, 2.0)
    assert (a.ff_kind, a.n_ff) == (_cabi.B2_FF_GLU, 44)
    assert (b.ff_kind, b.n_ff, b.moe_experts, b.moe_top, b.moe_route, b.moe_shared_ff, b.moe_identity) == (_cabi.B2_FF_MOE, 16, 7, 3, _cabi.B2_ROUTE_TOPK_SOFTMAX, 12, 0)
    assert c.moe_shared_ff == 0 and e.n_ff == 0
    shapes = dibesun.tensor_shapes(cfg)
    assert shapes["l0.mix.left.q.norm"] == (60,) and shapes["l0.mix.left.v"] == (42, 72) and shapes["l0.mix.left.o"] == (72, 84)
    assert shapes["l1.mlp.router.b"] == (7,) and shapes["l1.mlp.shared.down"] == (72, 12) and "l2.mlp.shared.up" not in shapes
    assert "head" not in shapes and "l3.norm2" not in shapes
    decays = dibesun.config_tensors(cfg)
    assert decays["l0.mix.right.decay"].data.tolist() == [0.5, np.float32(0.9)]


def test_registry_and_folder(tmp_path):
    from llama_cpp import dibesun, models
    cfg = du.config([du.layer(mlp=du.moe())])
    path = du.write_model(str(tmp_path / "m"), cfg, du.random_weights(cfg))
    assert models.open_model(path).family.name == "Dibesun" and "Dibesun" in models.architectures()
    with pytest.raises(ValueError):
        dibesun.layer_desc(0, {"type": "nope", "mixer": {}})
    bad = copy.deepcopy(cfg["layers"][0])
    bad["mixer"]["right"]["decay"] = [0.5]
    with pytest.raises(ValueError):
        dibesun.layer_desc(0, bad)


def test_chunks_start_at_position_zero():
    """Changing a token changes the attention output of the later positions of its own chunk and of no other."""
    cfg = du.config([du.layer(l=du.left(chunk=5))])
    w = {k: np.asarray(v, dtype=np.float64) for k, v in du.random_weights(cfg, seed=1).items()}
    h = np.random.default_rng(2).standard_normal((17, cfg["width"]))
    h2 = h.copy()
    h2[6] += 1.0
    m = cfg["layers"][0]["mixer"]["left"]
    moved = np.abs(ref.chunk_sigmoid_attention(h, w, "l0.mix.left.", m, 1e-6) - ref.chunk_sigmoid_attention(h2, w, "l0.mix.left.", m, 1e-6)).max(-1) > 1e-9
    assert moved.tolist() == [5 <= i <= 9 and i >= 6 for i in range(17)]


def test_key_weights_are_not_normalised():
    """A second copy of a key doubles its share: the sigmoid weights are summed as they are."""
    cfg = du.config([du.layer(l=du.left(chunk=64))])
    w = {k: np.asarray(v, dtype=np.float64) for k, v in du.random_weights(cfg, seed=3).items()}
    m = cfg["layers"][0]["mixer"]["left"]
    row = np.random.default_rng(4).standard_normal(cfg["width"])
    one = ref.chunk_sigmoid_attention(np.stack([row]), w, "l0.mix.left.", m, 1e-6)[0]
    three = ref.chunk_sigmoid_attention(np.stack([row] * 3), w, "l0.mix.left.", m, 1e-6)[2]
    assert np.allclose(three, 3 * one)


def test_linear_attention_is_a_decayed_sum():
    cfg = du.config([du.layer(r=du.right(heads=2, dim=4, vdim=3, decay=[0.5, 1.0]))])
    w = {k: np.asarray(v, dtype=np.float64) for k, v in du.random_weights(cfg, seed=5).items()}
    m, p = cfg["layers"][0]["mixer"]["right"], "l0.mix.right."
    h = np.random.default_rng(6).standard_normal((9, cfg["width"]))
    q, k, v = (ref.silu(h @ w[p + n].T) for n in "qkv")
    t = 8
    o = np.zeros(6)
    for hd, dec in enumerate(m["decay"]):
        for j in range(t + 1):
            o[3 * hd:3 * hd + 3] += dec ** (t - j) * (q[t, 4 * hd:4 * hd + 4] @ k[j, 4 * hd:4 * hd + 4]) * v[j, 3 * hd:3 * hd + 3]
    want = (ref.unit_rms(o[None], 1e-6) * w[p + "norm"] * ref.sigmoid(h[t:t + 1] @ w[p + "g"].T)) @ w[p + "o"].T
    assert np.allclose(ref.decayed_linear_attention(h, w, p, m, 1e-6)[t], want[0])


def test_routing_weights_and_bias():
    w = {"p.router": np.array([[1.0, 0], [0, 1.0], [0.5, 0.5], [0, 0]]), "p.router.b": np.array([0.0, 0.0, 0.0, 1.2])}
    chosen, weight = ref.route(np.array([[1.0, 0.2]]), w, "p.", {"experts": 4, "top": 2})
    assert chosen.tolist() == [[3, 0]]                         # the bias lifts a slot whose product is zero
    z = np.array([1.2, 1.0])
    assert np.allclose(weight, np.exp(z) / np.exp(z).sum())    # softmax over the chosen (biased) logits alone


def test_part_norm_parts_are_independent():
    x = np.random.default_rng(7).standard_normal((2, 12))
    y = x.copy()
    y[:, :4] *= 100.0
    a, b = ref.part_norm(x, np.ones(12), 3, 0.0), ref.part_norm(y, np.ones(12), 3, 0.0)
    assert np.allclose(a, b) and np.allclose((a.reshape(2, 3, 4) ** 2).mean(-1), 1.0)


def test_oracle_streams_are_causal():
    cfg = du.config([du.layer(mlp=du.moe()), du.layer(mlp=du.dense())])
    w = du.random_weights(cfg, seed=4)
    toks = [int(t) for t in np.random.default_rng(5).integers(0, cfg["vocab"], size=30)]
    full = ref.forward(cfg, w, toks)
    assert np.allclose(ref.forward(cfg, w, toks[:17]), full[:17], atol=1e-10)
