"""Dibesun through the native engine against the float64 oracle (oracle/dibesun_ref.py), on small random models the tests
make themselves: the mixer's branches and each feed-forward block alone, prompt against token-by-token decoding, portions
down to two tokens, unequal batches against each request alone, slots and pages used again, keys just inside and just
outside a chunk and at page borders, far tokens through the linear-attention state, the first tokens, long decoding,
degenerate and odd sizes, random configurations, the trace replay program, and greedy generation through `Llama` and the
scheduler."""
import copy
import threading

import numpy as np
import pytest

import dibesun_util as du
from oracle import dibesun_ref as ref

pytestmark = pytest.mark.gpu

TOL = {"float32": 3e-4, "bfloat16": 6e-2}


def open_engine(path, dtype="float32", n_ctx=512, max_seqs=4, kv_tokens=None, max_step_tokens=None, flags=0):
    from llama_cpp import models
    return models.open_engine(models.open_model(path), n_ctx=n_ctx, max_seqs=max_seqs, dtype=dtype, kv_tokens=kv_tokens,
                              max_step_tokens=max_step_tokens, flags=flags)


def run_cut(eng, seqs, key, tokens, cuts):
    """All logits of `tokens`, fed in portions of the given sizes (cycled)."""
    rows, pos, k = [], 0, 0
    seqs.open(key)
    while pos < len(tokens):
        n = min(cuts[k % len(cuts)], len(tokens) - pos)
        k += 1
        slot = seqs.extend(key, n)
        lg, _ = eng.step([(slot, tokens[pos:pos + n])], want=[list(range(n))])
        rows.append(lg)
        pos += n
    seqs.close(key)
    return np.concatenate(rows)


def close(got, want, dtype):
    """float32: every row within the tolerance. bfloat16: the rounded activations can tip a near-tie of the router the other
    way than the oracle's, which moves that row (and, slightly, later ones) by a whole expert; so the typical row must be
    well inside the tolerance and at most one row in twenty may leave it."""
    if dtype == "float32":
        return du.rel_err(got, want) < TOL[dtype]
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    ref_rms = np.sqrt(((want - want.mean(-1, keepdims=True)) ** 2).mean())
    rows = np.sqrt((d ** 2).mean(-1)) / ref_rms
    return np.median(rows) < TOL[dtype] / 4 and (rows > TOL[dtype]).mean() <= 0.05


def tokens_for(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], size=n)]


@pytest.fixture(scope="module")
def hybrid(native_lib, tmp_path_factory):
    cfg = du.config([du.layer(mlp=du.dense(40)), du.layer(mlp=du.moe(), l=du.left(heads=3, kv_heads=3, dim=16, vdim=24, chunk=70), r=du.right(heads=2, dim=16, vdim=24)),
                     du.layer(mlp=None, l=du.left(heads=6, kv_heads=2, dim=20, vdim=12, chunk=7)),
                     du.layer(mlp=du.moe(experts=9, top=4, ff=16, shared=0), l=du.left(heads=2, kv_heads=1, dim=32, vdim=32, chunk=64, softcap=2.0))])
    w = du.random_weights(cfg, seed=3)
    path = du.write_model(str(tmp_path_factory.mktemp("dibesun_hybrid")), cfg, w)
    return cfg, w, path


LAYERS = {
    "attention_only": lambda: du.layer(right_scale=0.0),
    "linear_only": lambda: du.layer(left_scale=0.0),
    "both": lambda: du.layer(l=du.left(heads=2, kv_heads=1, dim=40, vdim=36, chunk=33), r=du.right(heads=4, dim=12, vdim=20)),
    "dense_ff": lambda: du.layer(mlp=du.dense(52)),
    "moe_shared": lambda: du.layer(mlp=du.moe(experts=10, top=4, ff=20, shared=28)),
    "moe_plain": lambda: du.layer(mlp=du.moe(experts=5, top=2, ff=12, shared=0)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", sorted(LAYERS))
def test_each_mechanism_alone(native_lib, tmp_path, layer, dtype):
    from llama_cpp.kv_pages import SequenceSlots
    cfg = du.config([LAYERS[layer]()])
    w = du.random_weights(cfg, seed=11)
    eng = open_engine(du.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 90, 1)
    want_logits, want_layers = ref.forward(cfg, w, toks, return_layers=True)
    seqs = SequenceSlots(eng)
    eng.trace_layers(True)
    seqs.open("a")
    slot = seqs.extend("a", len(toks))
    got, _ = eng.step([(slot, toks)], want=[list(range(len(toks)))])
    layers = eng.layer_outputs(len(toks))
    eng.close()
    assert close(layers[0], want_layers[0], dtype)
    assert close(got, want_logits, dtype)


def test_mechanisms_are_not_trivial(hybrid):
    """The test weights make the mechanisms matter: the router bias changes choices, the chosen weights are far from uniform,
    scores reach the bend of the cap, and sigmoid weights spread over (0, 1)."""
    cfg, w, _ = hybrid
    wd = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    h = np.random.default_rng(0).standard_normal((200, cfg["width"]))
    r = cfg["layers"][1]["mlp"]["router"]
    chosen, weight = ref.route(h, wd, "l1.mlp.", r)
    flat = dict(wd)
    flat["l1.mlp.router.b"] = np.zeros_like(wd["l1.mlp.router.b"])
    assert (np.sort(ref.route(h, flat, "l1.mlp.", r)[0]) != np.sort(chosen)).any()
    assert weight.max() > 0.8 and np.allclose(weight.sum(-1), 1.0)
    m = cfg["layers"][3]["mixer"]["left"]
    q = ref.unit_rms(h @ wd["l3.mix.left.q"].T, 1e-6) * wd["l3.mix.left.q.norm"]
    k = ref.unit_rms(h @ wd["l3.mix.left.k"].T, 1e-6) * wd["l3.mix.left.k.norm"]
    s = (q[:, :32] @ k[:, :32].T) * m["scale"]
    assert (np.abs(s) > m["softcap"]).mean() > 0.01
    p = ref.sigmoid(m["softcap"] * np.tanh(s / m["softcap"]) + wd["l3.mix.left.pb"][0])
    assert p.min() < 0.3 and p.max() > 0.7


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_against_token_by_token(hybrid, dtype):
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, dtype)
    seqs = SequenceSlots(eng)
    toks = tokens_for(cfg, 150, 2)
    want = ref.forward(cfg, w, toks)
    whole = run_cut(eng, seqs, "w", toks, [len(toks)])
    single = run_cut(eng, seqs, "s", toks, [1])
    eng.close()
    assert close(whole, want, dtype)
    assert close(single, want, dtype)
    assert close(single, whole, dtype)


@pytest.mark.parametrize("cuts", [[2], [3, 2, 5, 1], [17, 64, 2, 9], [63, 1, 1, 70]])
def test_portions(hybrid, cuts):
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32")
    toks = tokens_for(cfg, 140, 4)
    got = run_cut(eng, SequenceSlots(eng), "p", toks, cuts)
    eng.close()
    assert du.rel_err(got, ref.forward(cfg, w, toks)) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone(hybrid, dtype):
    """Three requests of different lengths advance together, portions of some beside single tokens of others."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, dtype)
    seqs = SequenceSlots(eng)
    reqs = {"a": tokens_for(cfg, 131, 5), "b": tokens_for(cfg, 40, 6), "c": tokens_for(cfg, 77, 7)}
    alone = {k: run_cut(eng, seqs, k + "_alone", t, [len(t)]) for k, t in reqs.items()}
    plan = {"a": [50, 1, 1, 30, 2, 1], "b": [1, 1, 9, 1], "c": [2, 40, 1, 1, 20]}
    at = {k: 0 for k in reqs}
    turn = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    for k in reqs:
        seqs.open(k)
    while any(at[k] < len(reqs[k]) for k in reqs):
        entries, want, who = [], [], []
        for k, t in reqs.items():
            if at[k] >= len(t):
                continue
            n = min(plan[k][turn[k] % len(plan[k])], len(t) - at[k])
            turn[k] += 1
            entries.append((seqs.extend(k, n), t[at[k]:at[k] + n]))
            want.append(list(range(n)))
            who.append((k, n))
            at[k] += n
        lg, _ = eng.step(entries, want=want)
        r = 0
        for k, n in who:
            got[k].append(lg[r:r + n])
            r += n
    eng.close()
    for k, t in reqs.items():
        mixed = np.concatenate(got[k])
        assert du.rel_err(mixed, alone[k]) < 2e-5 if dtype == "float32" else close(mixed, alone[k], dtype)
        assert close(mixed, ref.forward(cfg, w, t), dtype)


def test_slots_and_pages_used_again(hybrid):
    """One slot, a pool of three pages: every sequence runs in the pages and the state slot the previous one left."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32", n_ctx=192, max_seqs=1, kv_tokens=192)
    seqs = SequenceSlots(eng)
    for i, n in enumerate([150, 70, 192, 3]):
        toks = tokens_for(cfg, n, 20 + i)
        got = run_cut(eng, seqs, f"s{i}", toks, [40, 1, 23])
        assert seqs.free_slots == 1 and eng.pages.free_pages == 3
        assert du.rel_err(got, ref.forward(cfg, w, toks)) < TOL["float32"], i
    eng.close()


def _peaky_attention_model(tmp_path, chunk):
    """One layer in which a token attends to earlier copies of itself whenever the mask lets it: keys are made by the query's
    own map and norm weight, so a copy's key is parallel to the query and its capped score is far above the per-head bias,
    which keeps the weights of all other keys near zero. The linear branch is turned down so that only the mask decides
    whether the copy is seen."""
    H, d = 2, 32
    cfg = du.config([du.layer(l=du.left(heads=H, kv_heads=H, dim=d, vdim=24, chunk=chunk, scale=0.4, softcap=12.0), right_scale=0.05)],
                    width=64, groups=2)
    w = du.random_weights(cfg, seed=5)
    w["l0.mix.left.k"] = w["l0.mix.left.q"].copy()
    w["l0.mix.left.k.norm"] = w["l0.mix.left.q.norm"].copy()
    w["l0.mix.left.pb"] = du.bf16_round(np.array([-6.0, -5.0]))
    return cfg, w, du.write_model(str(tmp_path / "peaky"), cfg, w)


def _with_chunk(cfg, size):
    c = copy.deepcopy(cfg)
    c["layers"][0]["mixer"]["left"]["mask"]["size"] = size
    return c


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode", [False, True])
def test_chunk_edges(native_lib, tmp_path, decode, dtype):
    """The marked token is the first of the probing position's chunk, or the last of the chunk before, or sits at a page border;
    a mask that is one position off changes the logits by far more than the tolerance. The chunk size is no multiple of the
    page size, and the prompt is cut inside the chunk."""
    from llama_cpp.kv_pages import SequenceSlots
    chunk, n = 70, 200
    cfg, w, path = _peaky_attention_model(tmp_path, chunk)
    eng = open_engine(path, dtype)
    tol = TOL["float32"] if dtype == "float32" else 0.02
    seqs = SequenceSlots(eng)
    mark = 7
    base = [int(t) for t in np.random.default_rng(9).integers(8, cfg["vocab"], size=n)]
    probe = n - 1
    first = probe // chunk * chunk
    cases = {"first_of_chunk": (first, chunk + 1), "last_of_chunk_before": (first - 1, chunk - 1), "at_page_border": (191, None), "after_page_border": (192, None)}
    for name, (at, other_chunk) in cases.items():
        toks = list(base)
        toks[at] = mark
        toks[probe] = mark
        true = ref.forward(cfg, w, toks)[probe]
        seqs.open(name)
        if decode:
            slot = seqs.extend(name, probe - 20)
            eng.step([(slot, toks[:probe - 20])])
            for t in range(probe - 20, probe):
                eng.step([(seqs.extend(name, 1), [toks[t]])])
            got, _ = eng.step([(seqs.extend(name, 1), [toks[probe]])], want=[[0]])
        else:
            slot = seqs.extend(name, first + 9)
            eng.step([(slot, toks[:first + 9])])
            slot = seqs.extend(name, n - first - 9)
            got, _ = eng.step([(slot, toks[first + 9:])], want=[[n - first - 10]])
        seqs.close(name)
        err = du.rel_err(got[0], true)
        assert err < tol, (name, err)
        if other_chunk is not None:
            assert du.rel_err(ref.forward(_with_chunk(cfg, other_chunk), w, toks)[probe], true) > 0.05, f"{name}: the test model does not show the edge"
    eng.close()


def test_far_token_through_the_state(native_lib, tmp_path):
    """A token 600 positions back reaches the last logits only through the linear-attention state (decays close to one, an
    embedding row large enough that its write stands out); attention chunks are 32 positions. The prompt is cut at odd places."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg = du.config([du.layer(l=du.left(chunk=32), r=du.right(heads=2, dim=24, vdim=16, decay=[0.999, 0.9995]), left_scale=0.3, right_scale=1.5)],
                    width=48, groups=1)
    w = du.random_weights(cfg, seed=6)
    e = w["embed"].copy()
    e[5] *= 12
    e[6] *= 12
    w["embed"] = du.bf16_round(e)
    n = 600
    toks = [int(t) for t in np.random.default_rng(12).integers(8, cfg["vocab"], size=n)]
    toks[1] = 5
    changed = list(toks)
    changed[1] = 6
    true = ref.forward(cfg, w, toks)[n - 1]
    assert du.rel_err(ref.forward(cfg, w, changed)[n - 1], true) > 0.02, "the test model forgets the far token"
    eng = open_engine(du.write_model(str(tmp_path / "far"), cfg, w), "float32", n_ctx=640)
    got = run_cut(eng, SequenceSlots(eng), "far", toks, [257, 64, 1, 2])
    eng.close()
    assert du.rel_err(got[n - 1], true) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [16, 64, 100, 1000])
def test_prompt_tiles(native_lib, tmp_path, chunk, dtype):
    """Sizes the tensor-core prompt kernels take: chunks narrower and wider than the 64-query tile and than the prompt, enough
    (token, expert) pairs for 128-row expert tiles; a 300-token prompt at once and in portions that straddle the tiles."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg = du.config([du.layer(mlp=du.moe(experts=6, top=4, ff=16, shared=32), l=du.left(heads=4, kv_heads=2, dim=32, vdim=16, chunk=chunk)),
                     du.layer(mlp=du.dense(64), l=du.left(heads=2, kv_heads=2, dim=48, vdim=64, chunk=chunk), r=du.right(heads=2, dim=32, vdim=32))], width=64, groups=2)
    w = du.random_weights(cfg, seed=13)
    eng = open_engine(du.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 300, 14)
    want = ref.forward(cfg, w, toks)
    seqs = SequenceSlots(eng)
    whole = run_cut(eng, seqs, "w", toks, [300])
    parts = run_cut(eng, seqs, "p", toks, [100, 7, 64, 129])
    eng.close()
    assert close(whole, want, dtype)
    assert close(parts, want, dtype)


def test_steps_larger_than_the_engine_takes_at_once(hybrid):
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32", max_step_tokens=16)
    seqs = SequenceSlots(eng)
    reqs = {"a": tokens_for(cfg, 50, 70), "b": tokens_for(cfg, 3, 71), "c": tokens_for(cfg, 37, 72)}
    for k in reqs:
        seqs.open(k)
    entries = [(seqs.extend(k, len(t)), t) for k, t in reqs.items()]
    want = [[0, 17, 49], [2], list(range(37))]
    got, _ = eng.step(entries, want=want)
    eng.close()
    expect = np.concatenate([ref.forward(cfg, w, t)[wi] for t, wi in zip(reqs.values(), want)])
    assert got.shape == expect.shape and du.rel_err(got, expect) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replayed_steps_equal_direct_launches(hybrid, dtype):
    """Repeating small steps are replayed as CUDA graphs; the logits are bit-identical to launching the kernels directly."""
    from llama_cpp import _cabi
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    toks = {"a": tokens_for(cfg, 40, 80), "b": tokens_for(cfg, 30, 81)}
    outs = []
    for flags in (0, _cabi.B2_FLAG_NO_GRAPH):
        eng = open_engine(path, dtype, n_ctx=256, max_seqs=2, flags=flags)
        seqs = SequenceSlots(eng)
        rows = []
        for k, t in toks.items():
            seqs.open(k)
            eng.step([(seqs.extend(k, 5), t[:5])])
        for i in range(5, 30):
            lg, _ = eng.step([(seqs.extend(k, 1), [t[i]]) for k, t in toks.items()], want=[[0], [0]])
            rows.append(lg)
        eng.close()
        outs.append(np.concatenate(rows))
    assert np.array_equal(outs[0], outs[1])
    want = np.concatenate([np.stack([ref.forward(cfg, w, t)[i] for t in toks.values()]) for i in range(5, 30)])
    assert close(outs[0], want, dtype)


def test_first_tokens(hybrid):
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32")
    seqs = SequenceSlots(eng)
    for n in (1, 2, 3, 5):
        toks = tokens_for(cfg, n, 30 + n)
        want = ref.forward(cfg, w, toks)
        assert du.rel_err(run_cut(eng, seqs, f"w{n}", toks, [n]), want) < TOL["float32"]
        assert du.rel_err(run_cut(eng, seqs, f"s{n}", toks, [1]), want) < TOL["float32"]
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(hybrid, dtype):
    """A short prompt and 300 single-token steps: chunks begin and end among decoded tokens, and pages fill up."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, dtype)
    toks = tokens_for(cfg, 310, 40)
    got = run_cut(eng, SequenceSlots(eng), "d", toks, [10] + [1] * 300)
    eng.close()
    assert close(got, ref.forward(cfg, w, toks), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_one_odd_or_large(native_lib, tmp_path, dtype):
    """One head, one key head, one expert, one choice, one norm part, a chunk of one token, branch weights and embedding scale 1,
    no cap, no mask entry (attention over the whole sequence), no shared expert, no feed-forward; key and value sizes that
    differ both ways; odd sizes that no vector path takes; keys and values wider than 128; memories with more than 128 rows."""
    from llama_cpp.kv_pages import SequenceSlots
    whole = du.left(heads=2, kv_heads=1, dim=12, vdim=20, softcap=0.0)
    del whole["mask"]
    cfg = du.config([
        du.layer(mlp=du.moe(experts=1, top=1, ff=8, shared=0), l=du.left(heads=1, kv_heads=1, dim=1, vdim=1, chunk=1), r=du.right(heads=1, dim=1, vdim=1, decay=[1.0]),
                 left_scale=1.0, right_scale=1.0),
        du.layer(mlp=None, l=whole, r=du.right(heads=5, dim=7, vdim=9)),
        du.layer(mlp=du.moe(experts=33, top=5, ff=11, shared=3), l=du.left(heads=6, kv_heads=3, dim=13, vdim=7, chunk=500)),
        du.layer(mlp=du.dense(1), l=du.left(heads=2, kv_heads=2, dim=160, vdim=24, chunk=37), r=du.right(heads=2, dim=150, vdim=20)),
        du.layer(mlp=du.dense(9), l=du.left(heads=1, kv_heads=1, dim=24, vdim=200, chunk=65), r=du.right(heads=1, dim=33, vdim=131, decay=[0.5])),
    ], width=40, vocab=50, groups=1, eps=1e-5, embed_scale=1.0)
    w = du.random_weights(cfg, seed=8)
    eng = open_engine(du.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 100, 3)
    got = run_cut(eng, SequenceSlots(eng), "x", toks, [5, 1, 2, 30])
    eng.close()
    assert close(got, ref.forward(cfg, w, toks), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [45, 50])
def test_widths_no_vector_path_takes(native_lib, tmp_path, width, dtype):
    """A model width that is odd, or even but no multiple of four: every product over the width takes its scalar path, in
    prompts (tiles) and in few-token steps (rows); as many norm parts as the width has divisors to offer."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg = du.config([du.layer(mlp=du.moe(experts=4, top=2, ff=10, shared=7), l=du.left(heads=2, kv_heads=2, dim=12, vdim=10, chunk=40)),
                     du.layer(mlp=du.dense(13), r=du.right(heads=3, dim=9, vdim=11))], width=width, vocab=77, groups=5)
    w = du.random_weights(cfg, seed=21)
    eng = open_engine(du.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 150, 22)
    got = run_cut(eng, SequenceSlots(eng), "x", toks, [70, 1, 3, 20, 1])
    eng.close()
    assert close(got, ref.forward(cfg, w, toks), dtype)


def random_config(seed):
    """A random model: layer count, every size and constant drawn anew (sizes of the scale small real models have)."""
    rng = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(rng.integers(0, len(xs)))]

    def block():
        kind = pick("none", "dense", "moe", "moe")
        if kind == "none":
            return None
        if kind == "dense":
            return du.dense(pick(24, 64, 100, 256))
        experts = pick(2, 4, 8, 12, 16)
        return du.moe(experts=experts, top=int(rng.integers(1, min(experts, 6) + 1)), ff=pick(8, 24, 40, 64), shared=pick(0, 16, 48, 96))

    layers = []
    for _ in range(int(rng.integers(2, 6))):
        g = pick(1, 2, 4)
        hr = pick(1, 2, 4, 6)
        layers.append(du.layer(mlp=block(),
                               l=du.left(heads=g * pick(1, 2, 4), kv_heads=g, dim=pick(16, 32, 48, 64, 128), vdim=pick(16, 32, 64, 80, 128),
                                         chunk=pick(1, 7, 24, 64, 65, 100, 128, 300), scale=float(rng.uniform(0.05, 0.4)), softcap=pick(5.0, 30.0, 50.0)),
                               r=du.right(heads=hr, dim=pick(16, 32, 64, 96), vdim=pick(16, 32, 48, 64), decay=rng.uniform(0.5, 0.999, size=hr)),
                               left_scale=float(rng.uniform(0.3, 1.5)), right_scale=float(rng.uniform(0.3, 1.5))))
    width = pick(64, 96, 128, 192, 200, 320)
    return du.config(layers, width=width, vocab=pick(97, 256, 500), groups=pick(1, 2, 4, 8), eps=pick(1e-5, 1e-6), embed_scale=float(rng.uniform(1.0, 20.0)))


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(native_lib, tmp_path, seed):
    """Eight models nobody chose: each runs a 330-token prompt at once and in uneven portions with decoded tokens at the end,
    in both modes, from a pool that forces page reuse."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg = random_config(200 + seed)
    w = du.random_weights(cfg, seed=seed)
    path = du.write_model(str(tmp_path / "m"), cfg, w)
    toks = tokens_for(cfg, 330, seed)
    want = ref.forward(cfg, w, toks)
    for dtype in ("float32", "bfloat16"):
        eng = open_engine(path, dtype, n_ctx=384, max_seqs=2, kv_tokens=384 + 128)
        seqs = SequenceSlots(eng)
        whole = run_cut(eng, seqs, "w", toks, [330])
        parts = run_cut(eng, seqs, "p", toks, [61, 3, 128, 2, 70, 37] + [1] * 29)
        eng.close()
        assert close(whole, want, dtype), (seed, dtype, "whole")
        assert close(parts, want, dtype), (seed, dtype, "parts")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(hybrid, tmp_path, dtype):
    """`bin/trace_run` as a user starts it: six requests, at most four live, portions of some beside single tokens of others, a
    request that sits out steps, a pool of --max-tokens sized for the live ones only, so pages and slots are used again; every
    written row against the oracle."""
    import json
    import os
    import subprocess
    import sys
    cfg, w, path = hybrid
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    reqs = {f"r{i}": tokens_for(cfg, n, 90 + i) for i, n in enumerate([130, 7, 64, 201, 33, 90])}
    plans = {"r0": [64, 2, 1, 1, 40, 1], "r1": [1, 1], "r2": [3, 61], "r3": [100, 1, 1, 64, 2], "r4": [33], "r5": [2, 1, 50, 1]}
    order, live, at, turn, steps, wanted = list(reqs), [], {k: 0 for k in reqs}, {k: 0 for k in reqs}, [], []
    most = 0
    while order or live:
        while order and len(live) < 4:
            live.append(order.pop(0))
        entries, end = [], []
        for k in list(live):
            if k == "r3" and len(steps) % 3 == 1:          # sits this step out
                continue
            n = min(plans[k][turn[k] % len(plans[k])], len(reqs[k]) - at[k])
            turn[k] += 1
            want = sorted({0, n - 1})
            entries.append({"id": k, "tokens": reqs[k][at[k]:at[k] + n], "want": want})
            wanted.append((len(steps), k, [at[k] + x for x in want]))
            at[k] += n
        most = max(most, sum((at[k] + 63) // 64 * 64 for k in live))
        for k in list(live):
            if at[k] == len(reqs[k]):
                end.append(k)
                live.remove(k)
        steps.append({"step": len(steps), "entries": entries, "end": end})
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(most)], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.split("\n") if ln.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    refs = {k: ref.forward(cfg, w, t) for k, t in reqs.items()}
    for i in range(len(steps)):
        rows = [(k, pos) for st, k, ps in wanted if st == i for pos in ps]
        got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(len(rows), cfg["vocab"])
        expect = np.stack([refs[k][pos] for k, pos in rows])
        assert close(got, expect, dtype) if len(rows) >= 20 else du.rel_err(got, expect) < (TOL[dtype] if dtype == "float32" else 0.2), i


def test_greedy_generation_through_llama_and_the_scheduler(hybrid):
    """`Llama(model_path=<folder>)`: three callers at once, prompts of different lengths, greedy. Every generated token is
    the oracle's argmax for the sequence so far wherever the oracle's top-two margin is clear."""
    from llama_cpp import Llama
    cfg, w, path = hybrid
    llm = Llama(model_path=path, n_gpu_layers=-1, n_ctx=256, n_seq_max=3, verbose=False, dtype="float32")
    prompts = [tokens_for(cfg, n, 50 + n) for n in (9, 70, 33)]
    outs = [None] * len(prompts)

    def call(i):
        outs[i] = llm.create_completion(prompts[i], max_tokens=12, temperature=0.0, repeat_penalty=1.0)

    threads = [threading.Thread(target=call, args=(i,)) for i in range(len(prompts))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    stats = llm._scheduler.stats
    llm.close()
    assert stats["max_batch"] >= 2
    for p, o in zip(prompts, outs):
        assert o["usage"]["completion_tokens"] == 12
        gen = [int(x[1:-1]) for x in o["choices"][0]["text"].replace("><", "> <").split()]
        logits = ref.forward(cfg, w, p + gen)
        for i, g in enumerate(gen):
            row = logits[len(p) + i - 1]
            top = np.sort(row)[-2:]
            if top[1] - top[0] > 1e-3:
                assert int(np.argmax(row)) == g


def test_direct_eval_and_scores(hybrid):
    from llama_cpp import Llama
    cfg, w, path = hybrid
    llm = Llama(model_path=path, n_gpu_layers=-1, n_ctx=128, verbose=False, dtype="float32")
    toks = tokens_for(cfg, 40, 60)
    llm.eval(toks[:30])
    for t in toks[30:]:
        llm.eval([t])
    got = llm.scores[0]
    llm.close()
    assert du.rel_err(got, ref.forward(cfg, w, toks)[-1]) < TOL["float32"]
