"""Small random Dibesun models for the tests: a config, bf16-rounded random weights, the folder the product loads."""
import numpy as np

from goponex_util import bf16_round, rel_err, write_model  # noqa: F401  (shared helpers)


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, shared=20):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def left(heads=4, kv_heads=2, dim=24, vdim=16, chunk=16, scale=None, softcap=8.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
            "scale": float(scale if scale is not None else dim ** -0.5), "softcap": softcap}


def right(heads=3, dim=20, vdim=12, decay=None):
    return {"heads": heads, "dim": dim, "vdim": vdim,
            "decay": [float(x) for x in (decay if decay is not None else np.linspace(0.7, 0.995, heads))]}


def layer(mlp=None, l=None, r=None, left_scale=0.7, right_scale=1.2):
    return {"type": "parallel", "mixer": {"left": l or left(), "right": r or right(), "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def config(layers, width=72, vocab=131, groups=3, eps=1e-6, embed_scale=5.0):
    return {"architecture": "Dibesun", "embedding": {"scale": embed_scale}, "layers": layers, "norm": {"eps": eps, "groups": groups},
            "vocab": vocab, "width": width}


def random_weights(cfg, seed=0):
    """Weights at a scale that keeps every mechanism alive (sigmoid weights neither 0 nor 1, capped scores on both sides of the
    cap's bend, router biases large enough to change choices), rounded to bf16 so the file and the oracle hold the same
    numbers."""
    from llama_cpp.dibesun import tensor_shapes
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "pb":
            a = rng.uniform(-3.0, 0.5, size=shape)
        elif name.endswith("router.b"):
            a = rng.standard_normal(shape) * 0.8
        elif leaf == "router":
            a = rng.standard_normal(shape) * 2.0 / np.sqrt(shape[1])
        elif len(shape) == 2:
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        else:                                   # norm weights
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        w[name] = bf16_round(a)
    w["embed"] = bf16_round(rng.standard_normal(w["embed"].shape) * 0.3)
    return w
