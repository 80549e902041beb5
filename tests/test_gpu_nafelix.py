"""Nafelix through the native engine against the float64 oracle (oracle/nafelix_ref.py), on small random models the tests
make themselves: each mixer and feed-forward block alone, stream copies and the input convolution on and off, repeated runs of
layers, prompt against token-by-token decoding, portions down to two tokens, unequal batches against each request alone, slots
and pages used again, keys just inside and just outside the window and at page borders, far tokens through the delta-rule
state, the first tokens, long decoding, degenerate and odd sizes, random configurations, the trace replay program, and greedy
generation through `Llama` and the scheduler."""
import copy
import threading

import numpy as np
import pytest

import nafelix_util as nu
from oracle import nafelix_ref as ref

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


def close(got, want, dtype, touchy=False):
    """float32: every row within the tolerance. bfloat16: the rounded activations can tip a near-tie of the router the other
    way than the oracle's, which moves that row (and, through the repeated layers and the stream copies, later ones) by a whole
    expert: the oracle itself moves as much when its matrices are disturbed by one part in 2^9 (median row 1.2 %, one row in
    eight above 6 % on the touchiest of the random models). So the typical row must be well inside the tolerance and at most
    one row in five may leave it. `touchy`: a model of degenerate sizes, which answers to the same disturbance with a median row
    of 2.6 % and rows of up to 90 %: the median must stay inside the tolerance and nine rows in ten within five times it."""
    if dtype == "float32":
        return nu.rel_err(got, want) < TOL[dtype]
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    ref_rms = np.sqrt(((want - want.mean(-1, keepdims=True)) ** 2).mean())
    rows = np.sqrt((d ** 2).mean(-1)) / ref_rms
    ok = np.median(rows) < TOL[dtype] / 3 and (rows > TOL[dtype]).mean() <= 0.2
    if touchy:
        ok = np.median(rows) < TOL[dtype] and (rows > 5 * TOL[dtype]).mean() <= 0.1
    if not ok:
        print(f"bfloat16 rows: median {np.median(rows):.4f}, share above {TOL[dtype]}: {(rows > TOL[dtype]).mean():.3f}, worst {rows.max():.3f}")
    return ok


def tokens_for(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], size=n)]


@pytest.fixture(scope="module")
def hybrid(native_lib, tmp_path_factory):
    """Five layers, the middle two run twice: both mixers, every feed-forward kind, a layer without one."""
    cfg = nu.config([nu.parallel(mlp=nu.dense(40)),
                     nu.parallel(mlp=nu.moe(), left=nu.attn(heads=3, kv_heads=3, dim=16, vdim=24, window=70, rot=6), right=nu.delta(heads=2, kv_heads=2, dim=16, vdim=24, conv=4)),
                     nu.attention(mlp=nu.moe(experts=9, top=4, ff=16, limit=0.8)),
                     nu.attention(mlp=None, m=nu.attn(heads=2, kv_heads=1, dim=32, vdim=20, window=7, rot=32)),
                     nu.parallel(mlp=nu.dense(24), left=nu.attn(heads=6, kv_heads=2, dim=20, vdim=12, window=64, rot=10))],
                    streams=3, taps=3, loop=(1, 3, 2))
    w = nu.random_weights(cfg, seed=3)
    path = nu.write_model(str(tmp_path_factory.mktemp("nafelix_hybrid")), cfg, w)
    return cfg, w, path


MODELS = {
    "attention_alone": lambda: nu.config([nu.attention()]),
    "parallel_alone": lambda: nu.config([nu.parallel()]),
    "dense_ff": lambda: nu.config([nu.attention(mlp=nu.dense(52))]),
    "moe_ff": lambda: nu.config([nu.parallel(mlp=nu.moe(experts=10, top=4, ff=20, limit=0.7))]),
    "one_copy_no_convolution": lambda: nu.config([nu.parallel(mlp=nu.moe())], streams=0, taps=0),
    "five_copies_five_taps": lambda: nu.config([nu.attention(mlp=nu.dense(30)), nu.parallel()], streams=5, taps=5),
    "repeated_run": lambda: nu.config([nu.parallel(mlp=nu.dense(20)), nu.attention(mlp=nu.moe())], loop=(0, 2, 3)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("model", sorted(MODELS))
def test_each_mechanism_alone(native_lib, tmp_path, model, dtype):
    from llama_cpp.kv_pages import SequenceSlots
    cfg = MODELS[model]()
    w = nu.random_weights(cfg, seed=11)
    eng = open_engine(nu.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 90, 1)
    want_logits, want_layers = ref.forward(cfg, w, toks, return_layers=True)
    seqs = SequenceSlots(eng)
    eng.trace_layers(True)
    seqs.open("a")
    slot = seqs.extend("a", len(toks))
    got, _ = eng.step([(slot, toks)], want=[list(range(len(toks)))])
    layers = eng.layer_outputs(len(toks))
    eng.close()
    assert layers.shape == want_layers.shape
    for i in range(len(layers)):
        assert close(layers[i], want_layers[i], dtype), i
    assert close(got, want_logits, dtype)


def test_mechanisms_are_not_trivial(hybrid):
    """The test weights make the mechanisms matter: the sink holds a visible share of the denominators, mixing the heads'
    weights moves the logits, expert inputs reach the clamp, the chosen scores are far from uniform, both branches of the
    activation are used, and the stream copies differ from one another."""
    cfg, w, _ = hybrid
    toks = tokens_for(cfg, 60, 0)
    true = ref.forward(cfg, w, toks)

    def moved(changes):
        w2 = dict(w)
        w2.update(changes)
        return nu.rel_err(ref.forward(cfg, w2, toks), true)

    assert moved({"l0.mix.left.sink": np.full(4, -30.0, dtype=np.float32)}) > 0.01
    assert moved({"l2.mix.sink": np.full(6, -30.0, dtype=np.float32)}) > 0.01
    assert moved({"l0.mix.left.talk": np.eye(4, dtype=np.float32)}) > 0.01
    assert moved({"l1.hc2.mix": np.eye(3, dtype=np.float32)}) > 0.01
    assert moved({"l1.canon1": np.zeros_like(w["l1.canon1"])}) > 0.01
    wd = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    h = np.random.default_rng(0).standard_normal((200, cfg["width"]))
    lim = cfg["layers"][2]["mlp"]["expert"]["limit"]
    g = h @ wd["l2.mlp.e0.gate"].T
    assert (g > lim).mean() > 0.02 and (g < lim).mean() > 0.5
    _, weight = ref.route(h, wd, "l2.mlp.", cfg["layers"][2]["mlp"]["router"])
    assert weight.max() > 0.7 and np.allclose(weight.sum(-1), 1.0)
    z = h @ wd["l0.mlp.up"].T
    assert (z > 0).mean() > 0.3 and (z < 0).mean() > 0.3


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
    assert nu.rel_err(got, ref.forward(cfg, w, toks)) < TOL["float32"]


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
        assert nu.rel_err(mixed, alone[k]) < 2e-5 if dtype == "float32" else close(mixed, alone[k], dtype)
        assert close(mixed, ref.forward(cfg, w, t), dtype)


def test_slots_and_pages_used_again(hybrid):
    """One slot, a pool of three pages: every sequence runs in the pages and the state slot the previous one left (delta-rule
    memories, both kinds of convolution state, every run of the repeated layers)."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, "float32", n_ctx=192, max_seqs=1, kv_tokens=192)
    seqs = SequenceSlots(eng)
    for i, n in enumerate([150, 70, 192, 3]):
        toks = tokens_for(cfg, n, 20 + i)
        got = run_cut(eng, seqs, f"s{i}", toks, [40, 1, 23])
        assert seqs.free_slots == 1 and eng.pages.free_pages == 3
        assert nu.rel_err(got, ref.forward(cfg, w, toks)) < TOL["float32"], i
    eng.close()


PROBE, MARK = 7, 6


def _peaky_attention_model(tmp_path, kind, window):
    """One layer in which token PROBE attends to token MARK whenever the mask lets it: the two embedding rows are the same
    vector in the two halves of the width, and the key map is the query map with the halves of its input swapped, so MARK's key
    is parallel to PROBE's query (PROBE's own key is not). The input convolution is turned down so that the neighbours do not
    blur this, and in the two-branch layer the delta rule is turned down so that only the mask decides what is seen."""
    H, d = 2, 32
    a = nu.attn(heads=H, kv_heads=H, dim=d, vdim=24, window=window, rot=8, scale=0.4)
    layer = nu.attention(m=a) if kind == "attention" else nu.parallel(left=a, right=nu.delta(heads=1, kv_heads=1, dim=8, vdim=8))
    cfg = nu.config([layer], width=64, streams=2, taps=3)
    w = nu.random_weights(cfg, seed=5)
    p = "l0.mix." if kind == "attention" else "l0.mix.left."
    W = cfg["width"]
    w[p + "k"] = np.concatenate([w[p + "q"][:, W // 2:], w[p + "q"][:, :W // 2]], 1)
    if kind == "attention":
        w[p + "k.b"] = w[p + "q.b"].copy()
    else:
        w["l0.mix.right.out"] = nu.bf16_round(w["l0.mix.right.out"] * 0.05)
    w["l0.norm1"] = np.ones(W, dtype=np.float32)
    w["l0.hc1.in"] = np.array([0.625, 0.375], dtype=np.float32)
    half = w["embed"][MARK, :W // 2].copy()
    w["embed"][MARK] = np.concatenate([half, 0 * half])
    w["embed"][PROBE] = np.concatenate([0 * half, half])
    w["l0.canon1"] = nu.bf16_round(w["l0.canon1"] * 0.1)
    w[p + "sink"] = nu.bf16_round(np.array([6.0, 7.0]))
    return cfg, w, nu.write_model(str(tmp_path / "peaky"), cfg, w), p


def _with_window(cfg, kind, size):
    c = copy.deepcopy(cfg)
    m = c["layers"][0]["mixer"]
    (m if kind == "attention" else m["left"])["mask"]["size"] = size
    return c


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("kind", ["attention", "parallel"])
def test_window_edges_and_sink(native_lib, tmp_path, kind, decode, dtype):
    """The marked token is the oldest one the probing position's window keeps, or the one just before it, or sits at a page
    border; a window that is one position off changes the logits by far more than the tolerance, and so does leaving the sink
    out where no key stands out. The window is no multiple of the page size and the prompt is cut inside it."""
    from llama_cpp.kv_pages import SequenceSlots
    window, n = 70, 200
    cfg, w, path, p = _peaky_attention_model(tmp_path, kind, window)
    eng = open_engine(path, dtype)
    tol = TOL["float32"] if dtype == "float32" else 0.03
    seqs = SequenceSlots(eng)
    base = [int(t) for t in np.random.default_rng(9).integers(8, cfg["vocab"], size=n)]
    probe = n - 1
    cases = {"oldest_in_window": (probe - window + 1, window - 1), "just_outside": (probe - window, window + 1), "at_page_border": (191, None),
             "after_page_border": (192, None)}
    for name, (at, other_window) in cases.items():
        toks = list(base)
        toks[at] = MARK
        toks[probe] = PROBE
        true = ref.forward(cfg, w, toks)[probe]
        seqs.open(name)
        if decode:
            slot = seqs.extend(name, probe - 90)
            eng.step([(slot, toks[:probe - 90])])
            for t in range(probe - 90, probe):               # the window's tail passes over decoded tokens
                eng.step([(seqs.extend(name, 1), [toks[t]])])
            got, _ = eng.step([(seqs.extend(name, 1), [toks[probe]])], want=[[0]])
        else:
            cut = probe - window + 9
            slot = seqs.extend(name, cut)
            eng.step([(slot, toks[:cut])])
            slot = seqs.extend(name, n - cut)
            got, _ = eng.step([(slot, toks[cut:])], want=[[n - cut - 1]])
        seqs.close(name)
        err = nu.rel_err(got[0], true)
        assert err < tol, (name, err)
        if other_window is not None:
            assert nu.rel_err(ref.forward(_with_window(cfg, kind, other_window), w, toks)[probe], true) > 0.3, f"{name}: the test model does not show the edge"
        if name == "just_outside":
            no_sink = dict(w)
            no_sink[p + "sink"] = np.full(2, -30.0, dtype=np.float32)
            assert nu.rel_err(ref.forward(cfg, no_sink, toks)[probe], true) > 0.08, "the test model does not show the sink"
    eng.close()


def test_far_token_through_the_state(native_lib, tmp_path):
    """A token 600 positions back reaches the last logits only through the delta-rule memory (decays close to one; the filler
    uses three tokens, so its keys leave most directions of the memory alone); the attention window is 32 positions. The
    prompt is cut at odd places."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg = nu.config([nu.parallel(left=nu.attn(window=32), right=nu.delta(heads=2, kv_heads=1, dim=24, vdim=16, conv=3))], width=48, streams=2, taps=2)
    w = nu.random_weights(cfg, seed=6)
    w["l0.mix.right.A_log"] = nu.bf16_round(np.array([-9.0, -8.0]))
    w["l0.mix.left.out"] = nu.bf16_round(w["l0.mix.left.out"] * 0.3)
    n = 600
    toks = [int(t) for t in np.random.default_rng(12).integers(9, 12, size=n)]
    toks[1] = 5
    changed = list(toks)
    changed[1] = 6
    true = ref.forward(cfg, w, toks)[n - 1]
    assert nu.rel_err(ref.forward(cfg, w, changed)[n - 1], true) > 0.02, "the test model forgets the far token"
    eng = open_engine(nu.write_model(str(tmp_path / "far"), cfg, w), "float32", n_ctx=640)
    got = run_cut(eng, SequenceSlots(eng), "far", toks, [257, 64, 1, 2])
    eng.close()
    assert nu.rel_err(got[n - 1], true) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [16, 64, 100, 0])
def test_prompt_tiles(native_lib, tmp_path, window, dtype):
    """Sizes the tensor-core prompt kernels take: windows narrower and wider than the 64-query tile and none at all, key and
    value sizes that are multiples of 16, mixed heads over two key/value heads (one weighted sum per pair of query head and
    value head) and over four (weights mixed before the values, through the scratch), enough (token, expert) pairs for 128-row
    expert tiles; a 300-token prompt at once and in portions that straddle the tiles."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg = nu.config([nu.parallel(mlp=nu.moe(experts=6, top=4, ff=16), left=nu.attn(heads=4, kv_heads=2, dim=32, vdim=16, window=window, rot=16)),
                     nu.attention(mlp=nu.dense(64), m=nu.attn(heads=2, kv_heads=2, dim=48, vdim=64, window=window, rot=8)),
                     nu.parallel(left=nu.attn(heads=8, kv_heads=4, dim=64, vdim=80, window=window, rot=64), right=nu.delta(heads=2, kv_heads=2, dim=32, vdim=32)),
                     nu.parallel(left=nu.attn(heads=3, kv_heads=3, dim=16, vdim=128, window=window, rot=2))], width=64)
    w = nu.random_weights(cfg, seed=13)
    eng = open_engine(nu.write_model(str(tmp_path / "m"), cfg, w), dtype)
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
    assert got.shape == expect.shape and nu.rel_err(got, expect) < TOL["float32"]


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
        assert nu.rel_err(run_cut(eng, seqs, f"w{n}", toks, [n]), want) < TOL["float32"]
        assert nu.rel_err(run_cut(eng, seqs, f"s{n}", toks, [1]), want) < TOL["float32"]
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(hybrid, dtype):
    """A short prompt and 300 single-token steps: windows slide over decoded tokens, and pages fill up."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg, w, path = hybrid
    eng = open_engine(path, dtype)
    toks = tokens_for(cfg, 310, 40)
    got = run_cut(eng, SequenceSlots(eng), "d", toks, [10] + [1] * 300)
    eng.close()
    assert close(got, ref.forward(cfg, w, toks), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_one_odd_or_large(native_lib, tmp_path, dtype):
    """One head, one key head, one expert, one choice, one copy of the stream, one tap, a window of one token, a run repeated
    once, no mask entry (attention over the whole sequence), no rotation and a rotation of the whole head, no feed-forward; key
    and value sizes that differ both ways; odd sizes that no vector path takes; keys and values wider than 128; memories with
    more than 128 rows."""
    from llama_cpp.kv_pages import SequenceSlots
    # a unit vector of one entry is a sign: under 16-bit rounding it flips where the oracle's does not, so that size is
    # compared in float32 only
    one = 1 if dtype == "float32" else 8
    cfg = nu.config([
        nu.parallel(mlp=nu.moe(experts=1, top=1, ff=8), left=nu.attn(heads=1, kv_heads=1, dim=2, vdim=1, window=1, rot=2), right=nu.delta(heads=1, kv_heads=1, dim=one, vdim=1, conv=1)),
        nu.attention(mlp=None, m=nu.attn(heads=2, kv_heads=1, dim=12, vdim=20, window=0, rot=0)),
        nu.parallel(mlp=nu.moe(experts=33, top=5, ff=11), left=nu.attn(heads=6, kv_heads=3, dim=13, vdim=7, window=500, rot=12), right=nu.delta(heads=5, kv_heads=5, dim=7, vdim=9, conv=2)),
        nu.parallel(mlp=nu.dense(1), left=nu.attn(heads=2, kv_heads=2, dim=160, vdim=24, window=37, rot=160), right=nu.delta(heads=2, kv_heads=1, dim=150, vdim=20, conv=6)),
        nu.attention(mlp=nu.dense(9), m=nu.attn(heads=1, kv_heads=1, dim=24, vdim=200, window=65, rot=2)),
        nu.parallel(left=nu.attn(heads=3, kv_heads=1, dim=8, vdim=8, window=3, rot=4), right=nu.delta(heads=1, kv_heads=1, dim=33, vdim=131, conv=4)),
    ], width=40, vocab=50, streams=1, taps=1, loop=(2, 4, 1), eps=1e-5)
    w = nu.random_weights(cfg, seed=8)
    eng = open_engine(nu.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 100, 3)
    got = run_cut(eng, SequenceSlots(eng), "x", toks, [5, 1, 2, 30])
    eng.close()
    assert close(got, ref.forward(cfg, w, toks), dtype, touchy=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [45, 50])
def test_widths_no_vector_path_takes(native_lib, tmp_path, width, dtype):
    """A model width that is odd, or even but no multiple of four: every product over the width takes its scalar path, in
    prompts (tiles) and in few-token steps (rows); eight and eleven copies of the stream."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg = nu.config([nu.parallel(mlp=nu.moe(experts=4, top=2, ff=10), left=nu.attn(heads=2, kv_heads=2, dim=12, vdim=10, window=40, rot=6)),
                     nu.attention(mlp=nu.dense(13))], width=width, vocab=77, streams=8 if width == 45 else 11, taps=4)
    w = nu.random_weights(cfg, seed=21)
    eng = open_engine(nu.write_model(str(tmp_path / "m"), cfg, w), dtype)
    toks = tokens_for(cfg, 150, 22)
    got = run_cut(eng, SequenceSlots(eng), "x", toks, [70, 1, 3, 20, 1])
    eng.close()
    assert close(got, ref.forward(cfg, w, toks), dtype)


def random_config(seed):
    """A random model: layer count and order, the repeated run, every size and constant drawn anew (sizes of the scale small
    real models have)."""
    rng = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(rng.integers(0, len(xs)))]

    def block():
        kind = pick("none", "dense", "moe", "moe")
        if kind == "none":
            return None
        if kind == "dense":
            return nu.dense(pick(24, 64, 100, 256))
        experts = pick(2, 4, 8, 12, 16)
        return nu.moe(experts=experts, top=int(rng.integers(1, min(experts, 6) + 1)), ff=pick(8, 24, 40, 64), limit=pick(0.5, 1.0, 7.0))

    def att():
        g = pick(1, 2, 4)
        d = pick(16, 32, 48, 64, 128)
        return nu.attn(heads=g * pick(1, 2, 4), kv_heads=g, dim=d, vdim=pick(16, 32, 64, 80, 128), window=pick(1, 7, 24, 64, 65, 72, 100, 128, 300),
                       rot=pick(0, 2, 8, 16, d), base=pick(1e4, 2.5e5, 5e5), scale=float(rng.uniform(0.05, 0.4)))

    layers = []
    for _ in range(int(rng.integers(2, 6))):
        if rng.random() < 0.4:
            layers.append(nu.attention(mlp=block(), m=att()))
        else:
            g = pick(1, 2, 3)
            layers.append(nu.parallel(mlp=block(), left=att(), right=nu.delta(heads=g * pick(1, 2), kv_heads=g, dim=pick(16, 32, 64, 96), vdim=pick(16, 32, 48, 64), conv=pick(2, 3, 4))))
    a = int(rng.integers(0, len(layers)))
    b = int(rng.integers(a, len(layers) + 1))
    width = pick(64, 96, 128, 192, 200, 320)
    return nu.config(layers, width=width, vocab=pick(97, 256, 500), streams=pick(0, 1, 2, 4, 6), taps=pick(0, 2, 3, 4), loop=pick(None, (a, b, int(rng.integers(1, 4)))),
                     eps=pick(1e-5, 1e-6))


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(native_lib, tmp_path, seed):
    """Eight models nobody chose: each runs a 330-token prompt at once and in uneven portions with decoded tokens at the end,
    in both modes, from a pool that forces page reuse."""
    from llama_cpp.kv_pages import SequenceSlots
    cfg = random_config(200 + seed)
    w = nu.random_weights(cfg, seed=seed)
    path = nu.write_model(str(tmp_path / "m"), cfg, w)
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
        assert close(got, expect, dtype) if len(rows) >= 20 else nu.rel_err(got, expect) < (TOL[dtype] if dtype == "float32" else 0.2), i


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
    assert nu.rel_err(got, ref.forward(cfg, w, toks)[-1]) < TOL["float32"]
