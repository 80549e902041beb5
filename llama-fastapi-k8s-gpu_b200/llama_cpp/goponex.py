"""Goponex: a hybrid decoder served by the layer-list graph of the native engine.

A model folder holds `config.json` and `model.safetensors`. The config lists the layers; each is either
  "parallel": sliding-window attention with a kept prefix (grouped query heads, per-head query/key RMS norm, partial
              interleaved rotary with blended frequencies, values = the keys as projected) beside a Mamba selective
              scan, the two outputs RMS-normed over the width and averaged, or
  "mlstm":    an mLSTM matrix memory with capped exponential gating,
optionally followed by a squared-ReLU feed-forward block; every sublayer is x <- LayerNorm(alpha * x + f(x)).
This module turns the config into the C ABI's `b2_layer_desc` list and checks the tensor set; the arithmetic is in
csrc/layered.cu, csrc/mixers.cu and csrc/dense.cu.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

from . import _cabi
from .models import Family, register


@dataclass
class LayeredDims:
    """What the host side needs to know of a layer-list model (the engine-facing counterpart of `ModelDims`)."""
    n_layer: int
    n_embd: int
    n_vocab: int
    norm_eps: float
    residual_scale: float
    layers: List[_cabi.B2LayerDesc]
    n_ctx_train: int = 0
    block_style: int = _cabi.B2_BLOCK_POSTSUM_LN
    logit_scale: float = 1.0
    embed_scale: float = 1.0
    norm_groups: int = 1
    tie_head: bool = False
    n_streams: int = 1
    canon_taps: int = 0


def _need(d: dict, key: str, where: str):
    if key not in d:
        raise ValueError(f"config.json: {where} lacks {key!r}")
    return d[key]


def layer_desc(i: int, layer: dict) -> _cabi.B2LayerDesc:
    where = f"layers[{i}]"
    kind = _need(layer, "type", where)
    mix = _need(layer, "mixer", where)
    d = _cabi.B2LayerDesc()
    mlp = layer.get("mlp")
    if mlp:
        if mlp.get("kind", "dense") != "dense":
            raise ValueError(f"config.json: {where}: feed-forward kind {mlp.get('kind')!r} is not supported")
        d.n_ff = int(_need(mlp, "ff", where + ".mlp"))
    if kind == "parallel":
        a, s = _need(mix, "left", where), _need(mix, "right", where)
        d.mixer = _cabi.B2_MIX_WINDOW_SCAN
        d.n_head, d.n_head_kv, d.head_dim = int(a["heads"]), int(a["kv_heads"]), int(a["dim"])
        if int(a.get("vdim", a["dim"])) != d.head_dim:
            raise ValueError(f"config.json: {where}: the values are the projected keys, so vdim must equal dim")
        rot = a.get("rot") or {}
        d.rot_dims = int(rot.get("dims", 0))
        d.rope_base = float(rot.get("base", 10000.0))
        sc = rot.get("scaling")
        if sc:
            d.rope_factor, d.rope_orig_ctx = float(sc["factor"]), int(sc["original"])
            d.rope_fast, d.rope_slow = float(sc["fast"]), float(sc["slow"])
        else:
            d.rope_factor = 0.0
        mask = _need(a, "mask", where + ".left")
        d.window, d.keep_first = int(mask["size"]), int(mask.get("keep_first", 0))
        d.attn_scale = float(_need(a, "scale", where + ".left"))
        d.conv_taps, d.dt_rank, d.d_inner, d.d_state = int(s["conv"]), int(s["dt_rank"]), int(s["inner"]), int(s["state"])
    elif kind == "mlstm":
        d.mixer = _cabi.B2_MIX_MATRIX_MEMORY
        d.mm_heads, d.mm_dim, d.mm_vdim = int(mix["heads"]), int(mix["dim"]), int(mix["vdim"])
        d.gate_cap = float(mix["gate_cap"])
    else:
        raise ValueError(f"config.json: {where}: unknown layer type {kind!r}")
    return d


def read_dims(cfg: dict) -> LayeredDims:
    layers = _need(cfg, "layers", "the config")
    descs = [layer_desc(i, L) for i, L in enumerate(layers)]
    return LayeredDims(n_layer=len(descs), n_embd=int(_need(cfg, "width", "the config")), n_vocab=int(_need(cfg, "vocab", "the config")),
                       norm_eps=float(_need(_need(cfg, "norm", "the config"), "eps", "norm")),
                       residual_scale=float(_need(cfg, "postln_alpha", "the config")), layers=descs)


def tensor_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
    """Every tensor the design needs, with its shape ([out, in] for linear maps)."""
    W, V = int(cfg["width"]), int(cfg["vocab"])
    out: Dict[str, Tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = (W,)
        if L["type"] == "parallel":
            a, s = m["left"], m["right"]
            H, G, d = int(a["heads"]), int(a["kv_heads"]), int(a["dim"])
            inner, N, R, taps = int(s["inner"]), int(s["state"]), int(s["dt_rank"]), int(s["conv"])
            out.update({p + "mix.left.q": (H * d, W), p + "mix.left.k": (G * d, W), p + "mix.left.q.norm": (d,),
                        p + "mix.left.k.norm": (d,), p + "mix.left.o": (W, H * d), p + "mix.left.out": (W,),
                        p + "mix.right.in": (2 * inner, W), p + "mix.right.conv": (inner, taps), p + "mix.right.conv.b": (inner,),
                        p + "mix.right.x": (R + 2 * N, inner), p + "mix.right.dt": (inner, R), p + "mix.right.dt.b": (inner,),
                        p + "mix.right.A_log": (inner, N), p + "mix.right.D": (inner,), p + "mix.right.o": (W, inner),
                        p + "mix.right.out": (W,)})
        else:
            H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * dv, W), p + "mix.g": (H * dv, W),
                        p + "mix.o": (W, H * dv), p + "mix.norm": (H * dv,), p + "mix.i": (H, W), p + "mix.i.b": (H,),
                        p + "mix.f": (H, W), p + "mix.f.b": (H,)})
        if L.get("mlp"):
            F = int(L["mlp"]["ff"])
            out.update({p + "norm2": (W,), p + "mlp.up": (F, W), p + "mlp.up.b": (F,), p + "mlp.down": (W, F), p + "mlp.down.b": (W,)})
    return out


def synthetic(width: int, n_heads: int, n_kv: int, ff: int, vocab: int, pattern: str = "mppm", seed: int = 0):
    """A random-weight model of realistic layer sizes, in memory (timing only): `pattern` lists the layers, "m" = mLSTM
    without feed-forward, "p" = attention + scan with feed-forward. Returns (config dict, {name: tensor})."""
    import numpy as np
    from .safetensors_file import STensor
    head = 128
    left = {"heads": n_heads, "kv_heads": n_kv, "dim": head, "vdim": head,
            "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 4.0, "fast": 16.0, "original": 8192, "slow": 2.0}},
            "mask": {"size": 1024, "keep_first": 4}, "scale": head ** -0.5}
    right = {"inner": 2 * width, "state": 16, "dt_rank": max(16, width // 16), "conv": 4}
    mm = {"heads": max(1, width // 256), "dim": 128, "vdim": 256, "gate_cap": 12.0}
    layers = [{"type": "mlstm", "mixer": mm, "mlp": None} if ch == "m" else
              {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": {"kind": "dense", "ff": ff}} for ch in pattern]
    cfg = {"architecture": "Goponex", "layers": layers, "norm": {"eps": 1e-5}, "postln_alpha": 1.0, "vocab": vocab, "width": width}
    rng = np.random.default_rng(seed)
    tensors = {}
    for name, shape in tensor_shapes(cfg).items():
        n = int(np.prod(shape))
        if len(shape) == 2 and not name.endswith(("conv", "A_log")):
            a = rng.standard_normal(n, dtype=np.float32) / np.sqrt(shape[1])
        elif name.endswith("A_log"):
            a = np.log(rng.uniform(1.0, 16.0, size=n)).astype(np.float32)
        elif name.endswith("dt.b"):
            a = np.log(np.expm1(rng.uniform(0.001, 0.1, size=n))).astype(np.float32)
        elif name.endswith("f.b"):
            a = rng.uniform(3.0, 6.0, size=n).astype(np.float32)
        elif name.endswith((".b", "conv")):
            a = (rng.standard_normal(n, dtype=np.float32) * 0.1)
        else:
            a = np.ones(n, dtype=np.float32)
        bits = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)       # truncation is fine for random weights
        tensors[name] = STensor(name, "BF16", tuple(shape), bits.reshape(shape))
    return cfg, tensors


def open_synthetic(cfg, tensors, **kw):
    from .engine import LayeredEngine
    return LayeredEngine(read_dims(cfg), tensors, **kw)


def _open(src, **kw):
    from .engine import LayeredEngine
    dims = read_dims(src.config)
    want = tensor_shapes(src.config)
    have = src.weights.tensors
    for name, shape in want.items():
        if name not in have:
            raise ValueError(f"{src.path}: tensor {name} is missing")
        if tuple(have[name].shape) != tuple(shape):
            raise ValueError(f"{src.path}: tensor {name} has shape {tuple(have[name].shape)}, the config asks for {tuple(shape)}")
    return LayeredEngine(dims, {n: have[n] for n in want}, **kw)


GOPONEX = register(Family(name="Goponex", source="folder", open_engine=_open))
