"""Dibesun: a decoder that norms what its sublayers RETURN, served by the layer-list graph of the native engine.

A model folder holds `config.json` and `model.safetensors`. Every layer is
    x <- x + norm1(mixer(x)),   x <- x + norm2(ff(x))        (`mlp` may be null)
where both sublayers read the stream itself and the norm is an RMS norm over `norm.groups` equal consecutive parts of the
vector, each part scaled by its own root mean square, the whole times a plain weight. The embedding row is multiplied by
`embedding.scale`; the embedding table, unscaled, is also the output map (after the same norm with `final.norm`).

The one token mixer, "parallel", adds two branches with fixed weights (`left_scale`, `right_scale`):
  left:  attention inside chunks of `mask.size` positions counted from the start of the sequence; grouped query heads, value
         size independent of the key size; queries and keys RMS-normed over the whole projection (all heads at once); no
         rotation; score = q.k * scale, capped as softcap * tanh(score / softcap); a key's weight is sigmoid(score + pb[head])
         and nothing is normalised over the keys
  right: linear attention with SiLU feature maps on q, k and v and one fixed decay per head (S <- decay S + k v^T, read-out
         S^T q after the write), the heads RMS-normed together, times sigmoid(W_g h)
The feed-forward block is a gated SiLU unit ("dense"), or a routed mixture of such units ("moe": the `top` largest biased
router logits choose, their softmax weighs, a shared expert is added for every token).

This module turns the config into the C ABI's `b2_layer_desc` list (every size and constant comes from the file) and checks
the tensor set; the arithmetic is in csrc/layered.cu, sigmoid_attn.cu, state_mixers.cu, moe.cu and dense.cu.
"""
from __future__ import annotations

from typing import Dict, Tuple

from . import _cabi
from .goponex import LayeredDims, _need
from .models import Family, register


def layer_desc(i: int, layer: dict) -> _cabi.B2LayerDesc:
    where = f"layers[{i}]"
    kind = _need(layer, "type", where)
    mix = _need(layer, "mixer", where)
    d = _cabi.B2LayerDesc()
    mlp = layer.get("mlp")
    if mlp:
        ff_kind = mlp.get("kind", "dense")
        if ff_kind == "dense":
            d.ff_kind = _cabi.B2_FF_GLU
            d.n_ff = int(_need(mlp, "ff", where + ".mlp"))
        elif ff_kind == "moe":
            r = _need(mlp, "router", where + ".mlp")
            d.ff_kind = _cabi.B2_FF_MOE
            d.n_ff = int(_need(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert"))
            d.moe_experts, d.moe_identity, d.moe_top = int(_need(r, "experts", where + ".mlp.router")), 0, int(_need(r, "top", where + ".mlp.router"))
            d.moe_groups, d.moe_keep, d.moe_scale = 1, 1, 1.0
            d.moe_route = _cabi.B2_ROUTE_TOPK_SOFTMAX
            shared = mlp.get("shared")
            d.moe_shared_ff = int(_need(shared, "ff", where + ".mlp.shared")) if shared else 0
        else:
            raise ValueError(f"config.json: {where}: feed-forward kind {ff_kind!r} is not supported")
    if kind != "parallel":
        raise ValueError(f"config.json: {where}: unknown layer type {kind!r}")
    a, b = _need(mix, "left", where + ".mixer"), _need(mix, "right", where + ".mixer")
    d.mixer = _cabi.B2_MIX_CHUNK_LINEAR
    d.n_head, d.n_head_kv = int(_need(a, "heads", where + ".left")), int(a.get("kv_heads", a["heads"]))
    d.head_dim = int(_need(a, "dim", where + ".left"))
    d.attn_vdim = int(a.get("vdim", d.head_dim))
    mask = a.get("mask")
    d.window = int(mask["size"]) if mask else 0
    d.attn_scale = float(_need(a, "scale", where + ".left"))
    d.softcap = float(a.get("softcap", 0.0))
    d.mm_heads, d.mm_dim, d.mm_vdim = int(_need(b, "heads", where + ".right")), int(_need(b, "dim", where + ".right")), int(_need(b, "vdim", where + ".right"))
    if len(_need(b, "decay", where + ".right")) != d.mm_heads:
        raise ValueError(f"config.json: {where}.right: one decay per head")
    d.branch_scale[0], d.branch_scale[1] = float(mix.get("left_scale", 1.0)), float(mix.get("right_scale", 1.0))
    return d


def read_dims(cfg: dict) -> LayeredDims:
    layers = _need(cfg, "layers", "the config")
    descs = [layer_desc(i, L) for i, L in enumerate(layers)]
    norm = _need(cfg, "norm", "the config")
    return LayeredDims(n_layer=len(descs), n_embd=int(_need(cfg, "width", "the config")), n_vocab=int(_need(cfg, "vocab", "the config")),
                       norm_eps=float(_need(norm, "eps", "norm")), residual_scale=1.0, layers=descs,
                       block_style=_cabi.B2_BLOCK_OUTNORM_RMS, logit_scale=1.0,
                       embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)), norm_groups=int(norm.get("groups", 1)), tie_head=True)


def tensor_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
    """Every tensor of the file that the design needs, with its shape ([out, in] for linear maps)."""
    W, V = int(cfg["width"]), int(cfg["vocab"])
    out: Dict[str, Tuple[int, ...]] = {"embed": (V, W), "final.norm": (W,)}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        if L["type"] != "parallel":
            raise ValueError(f"config.json: layers[{i}]: unknown layer type {L['type']!r}")
        a, b = L["mixer"]["left"], L["mixer"]["right"]
        H, G, d = int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"])
        dv = int(a.get("vdim", d))
        Hr, dr, dvr = int(b["heads"]), int(b["dim"]), int(b["vdim"])
        out.update({p + "norm1": (W,),
                    p + "mix.left.q": (H * d, W), p + "mix.left.k": (G * d, W), p + "mix.left.v": (G * dv, W),
                    p + "mix.left.q.norm": (H * d,), p + "mix.left.k.norm": (G * d,), p + "mix.left.pb": (H,), p + "mix.left.o": (W, H * dv),
                    p + "mix.right.q": (Hr * dr, W), p + "mix.right.k": (Hr * dr, W), p + "mix.right.v": (Hr * dvr, W),
                    p + "mix.right.g": (Hr * dvr, W), p + "mix.right.o": (W, Hr * dvr), p + "mix.right.norm": (Hr * dvr,)})
        mlp = L.get("mlp")
        if not mlp:
            continue
        out[p + "norm2"] = (W,)
        if mlp.get("kind", "dense") == "dense":
            F = int(mlp["ff"])
            out.update({p + "mlp.gate": (F, W), p + "mlp.up": (F, W), p + "mlp.down": (W, F)})
        else:
            E, F = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            out.update({p + "mlp.router": (E, W), p + "mlp.router.b": (E,)})
            for e in range(E):
                out.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
            if mlp.get("shared"):
                Fs = int(mlp["shared"]["ff"])
                out.update({p + "mlp.shared.gate": (Fs, W), p + "mlp.shared.up": (Fs, W), p + "mlp.shared.down": (W, Fs)})
    return out


def config_tensors(cfg: dict) -> dict:
    """Constants of the config that the engine takes as tensors: the per-head decays of every layer's linear attention."""
    import numpy as np
    from .safetensors_file import STensor
    out = {}
    for i, L in enumerate(cfg["layers"]):
        dec = np.asarray(L["mixer"]["right"]["decay"], dtype=np.float32)
        out[f"l{i}.mix.right.decay"] = STensor(f"l{i}.mix.right.decay", "F32", tuple(dec.shape), dec)
    return out


def synthetic(width: int, heads: int, kv_heads: int, ff: int, vocab: int, pattern: str = "dmmm", experts: int = 16, top: int = 4,
              chunk: int = 1024, seed: int = 0):
    """A random-weight model of realistic layer sizes, in memory (timing only). `pattern` lists the layers' feed-forward
    blocks: "d" a dense gated unit of width `ff`, "m" a mixture of `experts` experts of width ff // 4 with a shared expert of
    width ff // 2, "n" none. Returns (config dict, {name: tensor})."""
    import numpy as np
    from .safetensors_file import STensor
    hr = max(1, width // 256)
    mixer = {"left": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "mask": {"size": chunk}, "scale": 128 ** -0.5, "softcap": 30.0},
             "right": {"heads": hr, "dim": 128, "vdim": 128, "decay": [float(1.0 - 2.0 ** -(3 + 5 * h / max(1, hr - 1))) for h in range(hr)]},
             "left_scale": 0.5, "right_scale": 0.5}
    ffs = {"d": {"kind": "dense", "ff": ff}, "n": None,
           "m": {"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": experts, "top": top}, "shared": {"ff": ff // 2}}}
    cfg = {"architecture": "Dibesun", "embedding": {"scale": float(width) ** 0.5},
           "layers": [{"type": "parallel", "mixer": mixer, "mlp": ffs[ch]} for ch in pattern],
           "norm": {"eps": 1e-5, "groups": 2}, "vocab": vocab, "width": width}
    rng = np.random.default_rng(seed)
    tensors = {}
    for name, shape in tensor_shapes(cfg).items():
        n = int(np.prod(shape))
        if len(shape) == 2:
            a = rng.standard_normal(n, dtype=np.float32) / np.sqrt(shape[1])
        elif name.endswith((".pb", "router.b")):
            a = rng.standard_normal(n, dtype=np.float32) * 0.5 - (3.0 if name.endswith(".pb") else 0.0)
        else:
            a = np.ones(n, dtype=np.float32)
        bits = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)       # truncation is fine for random weights
        tensors[name] = STensor(name, "BF16", tuple(shape), bits.reshape(shape))
    return cfg, tensors


def open_synthetic(cfg, tensors, **kw):
    from .engine import LayeredEngine
    return LayeredEngine(read_dims(cfg), {**tensors, **config_tensors(cfg)}, **kw)


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
    return LayeredEngine(dims, {**{n: have[n] for n in want}, **config_tensors(src.config)}, **kw)


DIBESUN = register(Family(name="Dibesun", source="folder", open_engine=_open))
