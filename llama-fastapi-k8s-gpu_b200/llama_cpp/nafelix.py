"""Nafelix: a decoder with several copies of the residual stream, served by the layer-list graph of the native engine.

A model folder holds `config.json` and `model.safetensors`. The stream exists in `streams` copies, all equal to the
embedding at first. A sublayer reads the normed weighted sum of the copies (RMS norm with a plain weight), passed through
a short causal convolution with a skip (`canon.taps` taps per channel, tensors `l<i>.canon1` / `canon2`); what it returns
is written back to every copy through the layer's `hc1` / `hc2` tensors (`in` [S], `mix` [S, S] indexed [from, to],
`out` [S]). The output norm reads the sum of the copies. Token mixers:
  "parallel":  softmax attention (`left`: grouped query heads, value size of its own, rotate-half rotation of the first
               `rot.dims` entries, sliding window `mask.size`, a learned sink term in every head's denominator, the heads'
               weights mixed by `talk` [H, H] after the softmax, one sigmoid gate per head) beside a gated delta rule
               (`right`: convolution + SiLU on q, k, v, unit-length q and k, ONE decay per head and token, per-head RMS norm
               times SiLU gate); both outputs are RMS-normed over the width and averaged
  "attention": the same attention alone, with biases on q, k, v, unit-RMS q and k after the rotation, no mixing of the
               heads and a gate per output entry
Feed-forward: "dense" (`down(act(up h))` with a piecewise quadratic / exponential activation whose two numbers are the
tensor `mlp.act`) or "moe" (softmax over all experts, the `top` largest renormalised, clamped gated experts). `loop`
repeats layers start .. stop-1 `times` times with the same weights; every pass keeps a cache and state of its own, which
is why the engine gets one layer entry per RUN with `weights_of` naming the layer whose tensors it uses.

This module turns the config into the C ABI's `b2_layer_desc` list (every size and constant comes from the file) and
checks the tensor set; the arithmetic is in csrc/layered.cu, sink_attn.cu, hyper.cu, state_mixers.cu, moe.cu, dense.cu.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

from . import _cabi
from .goponex import LayeredDims, _need
from .models import Family, register

EXPERT_ALPHA = 1.702          # slope inside the sigmoid of a clamped expert (fixed by the design)


def layer_runs(cfg: dict) -> List[int]:
    """Layer indices in the order they run."""
    n = len(_need(cfg, "layers", "the config"))
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop")), int(_need(loop, "times", "loop"))
    if not (0 <= a <= b <= n) or times < 1:
        raise ValueError(f"config.json: loop {loop!r} does not fit {n} layers")
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def _attention(d: _cabi.B2LayerDesc, m: dict, where: str, flags: int):
    d.n_head, d.head_dim = int(_need(m, "heads", where)), int(_need(m, "dim", where))
    d.n_head_kv = int(m.get("kv_heads", d.n_head))
    d.attn_vdim = int(m.get("vdim", d.head_dim))
    rot = m.get("rot") or {}
    d.rot_dims = int(rot.get("dims", 0))
    d.rope_base = float(rot.get("base", 10000.0))
    d.rope_factor = 0.0
    mask = m.get("mask")
    d.window = int(mask["size"]) if mask else 0
    d.attn_scale = float(_need(m, "scale", where))
    d.attn_flags = flags


def layer_desc(i: int, layer: dict, weights_of: int = 0) -> _cabi.B2LayerDesc:
    where = f"layers[{i}]"
    kind = _need(layer, "type", where)
    mix = _need(layer, "mixer", where)
    d = _cabi.B2LayerDesc()
    d.weights_of = weights_of
    if kind == "parallel":
        d.mixer = _cabi.B2_MIX_SINK_DELTA
        _attention(d, _need(mix, "left", where + ".mixer"), where + ".mixer.left", _cabi.B2_ATTN_TALK | _cabi.B2_ATTN_HEAD_GATE)
        r = _need(mix, "right", where + ".mixer")
        d.mm_heads, d.mm_dim, d.mm_vdim = int(r["heads"]), int(r["dim"]), int(r["vdim"])
        d.key_heads = int(r.get("kv_heads", d.mm_heads))
        d.conv_taps = int(_need(r, "conv", where + ".mixer.right"))
    elif kind == "attention":
        d.mixer = _cabi.B2_MIX_SINK_ATTN
        _attention(d, mix, where + ".mixer", _cabi.B2_ATTN_BIAS | _cabi.B2_ATTN_UNIT_QK)
    else:
        raise ValueError(f"config.json: {where}: unknown layer type {kind!r}")
    mlp = layer.get("mlp")
    if mlp:
        fk = mlp.get("kind", "dense")
        if fk == "dense":
            d.ff_kind, d.n_ff = _cabi.B2_FF_PIECEWISE, int(_need(mlp, "ff", where + ".mlp"))
        elif fk == "moe":
            r, ex = _need(mlp, "router", where + ".mlp"), _need(mlp, "expert", where + ".mlp")
            d.ff_kind, d.n_ff = _cabi.B2_FF_MOE, int(_need(ex, "ff", where + ".mlp.expert"))
            d.moe_experts, d.moe_identity, d.moe_top = int(r["experts"]), 0, int(r["top"])
            d.moe_groups = d.moe_keep = 1
            d.moe_scale = 1.0
            d.moe_route, d.moe_renorm = _cabi.B2_ROUTE_SOFTMAX_ALL, 1
            d.moe_expert, d.moe_limit, d.moe_alpha = _cabi.B2_EXPERT_CLAMPED, float(_need(ex, "limit", where + ".mlp.expert")), EXPERT_ALPHA
        else:
            raise ValueError(f"config.json: {where}: unknown feed-forward kind {fk!r}")
    return d


def read_dims(cfg: dict) -> LayeredDims:
    layers = _need(cfg, "layers", "the config")
    runs = layer_runs(cfg)
    first: Dict[int, int] = {}
    descs = []
    for r, li in enumerate(runs):
        descs.append(layer_desc(li, layers[li], weights_of=li + 1))
        first.setdefault(li, r)
    canon = cfg.get("canon") or {}
    return LayeredDims(n_layer=len(descs), n_embd=int(_need(cfg, "width", "the config")), n_vocab=int(_need(cfg, "vocab", "the config")),
                       norm_eps=float(_need(_need(cfg, "norm", "the config"), "eps", "norm")), residual_scale=1.0, layers=descs,
                       block_style=_cabi.B2_BLOCK_HYPER_RMS, n_streams=int(cfg.get("streams", 1)), canon_taps=int(canon.get("taps", 0)))


def _attention_shapes(out: dict, p: str, m: dict, W: int, biases: bool, talk: bool, head_gate: bool):
    H, d = int(m["heads"]), int(m["dim"])
    G, dv = int(m.get("kv_heads", H)), int(m.get("vdim", d))
    out.update({p + "q": (H * d, W), p + "k": (G * d, W), p + "v": (G * dv, W), p + "sink": (H,),
                p + "g": (H if head_gate else H * dv, W), p + "o": (W, H * dv)})
    if biases:
        out.update({p + "q.b": (H * d,), p + "k.b": (G * d,), p + "v.b": (G * dv,)})
    if talk:
        out[p + "talk"] = (H, H)


def tensor_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
    """Every tensor the design needs, with its shape ([out, in] for linear maps)."""
    W, V, S = int(cfg["width"]), int(cfg["vocab"]), int(cfg.get("streams", 1))
    taps = int((cfg.get("canon") or {}).get("taps", 0))
    out: Dict[str, Tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        subs = ("1", "2") if L.get("mlp") else ("1",)
        for q in subs:
            out[p + "norm" + q] = (W,)
            if "streams" in cfg:
                out.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
            if taps > 0:
                out[p + "canon" + q] = (W, taps)
        if L["type"] == "parallel":
            _attention_shapes(out, p + "mix.left.", m["left"], W, biases=False, talk=True, head_gate=True)
            r = m["right"]
            H, G, d, dv, ct = int(r["heads"]), int(r.get("kv_heads", r["heads"])), int(r["dim"]), int(r["vdim"]), int(r["conv"])
            b = p + "mix.right."
            out.update({b + "q": (G * d, W), b + "q.conv": (G * d, ct), b + "k": (G * d, W), b + "k.conv": (G * d, ct),
                        b + "v": (H * dv, W), b + "v.conv": (H * dv, ct), b + "b": (H, W), b + "A_log": (H,), b + "norm": (dv,),
                        b + "a": (H, W), b + "dt_bias": (H,), b + "g": (H * dv, W), b + "o": (W, H * dv),
                        p + "mix.left.out": (W,), p + "mix.right.out": (W,)})
        elif L["type"] == "attention":
            _attention_shapes(out, p + "mix.", m, W, biases=True, talk=False, head_gate=False)
        else:
            raise ValueError(f"config.json: layers[{i}]: unknown layer type {L['type']!r}")
        mlp = L.get("mlp")
        if mlp and mlp.get("kind", "dense") == "dense":
            F = int(mlp["ff"])
            out.update({p + "mlp.up": (F, W), p + "mlp.down": (W, F), p + "mlp.act": (2,)})
        elif mlp:
            E, F = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            out[p + "mlp.router"] = (E, W)
            for e in range(E):
                out.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
    return out


def synthetic(width: int, heads: int, ff: int, vocab: int, pattern: str = "papa", experts: int = 16, top: int = 4,
              window: int = 1024, streams: int = 4, seed: int = 0):
    """A random-weight model of realistic layer sizes, in memory (timing only). `pattern` lists the layers: "p" parallel,
    "a" attention; the first layer has a dense block of width 4 * `ff`, the others a mixture of `experts` experts of width
    `ff`. Returns (config dict, {name: tensor})."""
    import numpy as np
    from .safetensors_file import STensor
    kv = max(1, heads // 4)
    att = {"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "mask": {"size": window}, "rot": {"base": 5e5, "dims": 64}, "scale": 128 ** -0.5}
    dl = {"heads": max(1, width // 256), "kv_heads": max(1, width // 512), "dim": 128, "vdim": 128, "conv": 4}
    moe = {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": experts, "top": top}}
    layers = []
    for n, ch in enumerate(pattern):
        mlp = {"kind": "dense", "ff": 4 * ff} if n == 0 else moe
        layers.append({"type": "parallel", "mixer": {"left": att, "right": dl}, "mlp": mlp} if ch == "p" else
                      {"type": "attention", "mixer": att, "mlp": mlp})
    cfg = {"architecture": "Nafelix", "canon": {"taps": 4}, "layers": layers, "norm": {"eps": 1e-6}, "streams": streams,
           "vocab": vocab, "width": width}
    rng = np.random.default_rng(seed)
    tensors = {}
    for name, shape in tensor_shapes(cfg).items():
        n = int(np.prod(shape))
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "A_log":
            a = np.log(rng.uniform(0.5, 4.0, size=n)).astype(np.float32)
        elif leaf == "dt_bias":
            a = np.log(np.expm1(rng.uniform(0.01, 0.2, size=n))).astype(np.float32)
        elif leaf == "conv" or "canon" in leaf:
            a = rng.standard_normal(n, dtype=np.float32) * 0.3
        elif leaf == "mix" and ".hc" in name:
            a = (np.eye(shape[0], dtype=np.float32) + rng.standard_normal(shape, dtype=np.float32) * 0.05).reshape(-1)
        elif leaf == "talk":
            a = (np.eye(shape[0], dtype=np.float32) + rng.standard_normal(shape, dtype=np.float32) * 0.1).reshape(-1)
        elif leaf == "in" and ".hc" in name:
            a = np.full(n, 1.0 / n, dtype=np.float32) + rng.standard_normal(n, dtype=np.float32) * 0.02
        elif len(shape) == 2:
            a = rng.standard_normal(n, dtype=np.float32) / np.sqrt(shape[1])
        elif leaf in ("norm", "norm1", "norm2", "out") and ".hc" not in name:
            a = np.ones(n, dtype=np.float32)
        elif leaf == "out":
            a = np.full(n, 0.5, dtype=np.float32)
        else:                       # sinks, biases, activation numbers
            a = rng.standard_normal(n, dtype=np.float32) * 0.05
        bits = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)       # truncation is fine for random weights
        tensors[name] = STensor(name, "BF16", tuple(shape), bits.reshape(shape))
    return cfg, tensors


def open_synthetic(cfg, tensors, **kw):
    from .engine import LayeredEngine
    return LayeredEngine(read_dims(cfg), tensors, **kw)


def _open(src, **kw):
    from .engine import LayeredEngine
    have = src.weights.tensors
    dims = read_dims(src.config)
    want = tensor_shapes(src.config)
    for name, shape in want.items():
        if name not in have:
            raise ValueError(f"{src.path}: tensor {name} is missing")
        if tuple(have[name].shape) != tuple(shape):
            raise ValueError(f"{src.path}: tensor {name} has shape {tuple(have[name].shape)}, the config asks for {tuple(shape)}")
    return LayeredEngine(dims, {n: have[n] for n in want}, **kw)


NAFELIX = register(Family(name="Nafelix", source="folder", open_engine=_open))
