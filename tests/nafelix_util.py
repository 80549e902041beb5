"""Small random Nafelix models for the tests: a config, bf16-rounded random weights, the folder the product loads."""
import numpy as np

from goponex_util import bf16_round, rel_err, write_model  # noqa: F401  (shared helpers)


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24, limit=1.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def attn(heads=4, kv_heads=2, dim=24, vdim=16, window=16, rot=8, base=5000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5)}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    return m


def delta(heads=4, kv_heads=2, dim=20, vdim=12, conv=3):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(mlp=None, left=None, right=None):
    return {"type": "parallel", "mixer": {"left": left or attn(), "right": right or delta()}, "mlp": mlp}


def attention(mlp=None, m=None):
    return {"type": "attention", "mixer": m or attn(heads=6, kv_heads=3, dim=16, vdim=16, window=23, rot=16), "mlp": mlp}


def config(layers, width=72, vocab=131, streams=3, taps=3, loop=None, eps=1e-6):
    cfg = {"architecture": "Nafelix", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if streams:
        cfg["streams"] = streams
    if taps:
        cfg["canon"] = {"taps": taps}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(cfg, seed=0):
    """Weights at a scale that keeps every mechanism alive (sinks that hold a visible share of the denominator, a head-mixing
    matrix far from the identity, mixing matrices of the stream copies that really mix, gates unsaturated, expert inputs on
    both sides of the clamp, decays neither 0 nor 1), rounded to bf16 so the file and the oracle hold the same numbers."""
    from llama_cpp.nafelix import tensor_shapes
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if ".hc" in name:
            S = shape[0]
            if leaf == "mix":
                a = np.eye(S) * 0.8 + rng.standard_normal(shape) * 0.25
            elif leaf == "in":
                a = 1.0 / S + rng.standard_normal(shape) * 0.3
            else:
                a = 0.7 + rng.standard_normal(shape) * 0.4
        elif leaf == "talk":
            a = np.eye(shape[0]) * 0.7 + rng.standard_normal(shape) * 0.3
        elif leaf == "sink":
            a = rng.uniform(-1.0, 2.0, size=shape)
        elif leaf == "A_log":
            a = np.log(rng.uniform(0.3, 4.0, size=shape))
        elif leaf == "dt_bias":
            a = np.log(np.expm1(rng.uniform(0.02, 0.5, size=shape)))
        elif leaf == "conv" or leaf.startswith("canon"):
            a = rng.standard_normal(shape) * 0.5
        elif leaf == "act":
            a = rng.standard_normal(shape)
        elif leaf == "router":
            a = rng.standard_normal(shape) * 2.0 / np.sqrt(shape[1])
        elif leaf in ("gate", "up") and ".mlp.e" in name:
            a = rng.standard_normal(shape) * 1.5 / np.sqrt(shape[1])
        elif leaf == "b" and len(shape) == 1:
            a = rng.standard_normal(shape) * 0.3
        elif len(shape) == 2:
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        else:                                   # norm weights
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        w[name] = bf16_round(a)
    w["embed"] = bf16_round(rng.standard_normal(w["embed"].shape))
    return w
