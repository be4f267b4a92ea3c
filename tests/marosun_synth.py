"""Small Marosun configurations with random weights for the tests, and the glue between the library and the oracle.

Weights are drawn in float32 and rounded to bfloat16-representable values, so that the library (either compute mode) and the float64
oracle hold exactly the same numbers."""
import numpy as np

import llama_gguf_b200 as B
from llama_gguf_b200 import marosun
from llama_gguf_b200.safetensors_io import bf16_bits, bf16_to_f32


def dense(ff=72, limit=1.25):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=5, top=2, ff=24):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def rot(dims=12, base=900.0, scaling=True):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = scaling if isinstance(scaling, dict) else {"factor": 3.0, "original": 48, "fast": 8.0, "slow": 2.0}
    return r


def layer_a(heads=4, kv_heads=2, dim=24, vdim=40, r=None, scale=None, mlp=None):
    """softmax attention alone: biases, q / k norm, stretched rotation, turned values, learned extra denominator term"""
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": r if r is not None else rot(),
                      "scale": scale if scale is not None else dim ** -0.5},
            "mlp": mlp}


def layer_p(heads=4, kv_heads=2, dim=24, vdim=40, chunk=7, scale=None, r_heads=3, r_dim=20, r_vdim=12, left_scale=0.7, right_scale=1.3, mlp=None):
    """chunked gated attention beside a gated linear memory, weighted sum"""
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
                               "scale": scale if scale is not None else dim ** -0.5},
                      "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim}, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def layer_q(heads=4, kv_heads=2, dim=24, vdim=40, r=None, scale=None, r_width=56, mlp=None):
    """attention with one added to the denominator beside a gated unit per channel, both normed, half their sum"""
    return {"type": "parallel_2",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": r if r is not None else rot(dims=dim, scaling=False),
                               "scale": scale if scale is not None else 1.5 * dim ** -0.5},
                      "right": {"width": r_width}},
            "mlp": mlp}


def config(layers, width=64, vocab=96, eps=1e-5):
    return {"architecture": "Marosun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


def random_weights(cfg, seed=0):
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in marosun.tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last == "norm1" or name == "final.norm":
            a = 0.25 * rng.standard_normal(shape)                 # stored around zero
        elif name.endswith((".q.norm", ".k.norm", ".left.out", ".right.out", ".right.norm")):
            a = 1.0 + 0.3 * rng.standard_normal(shape)
        elif last == "b":
            a = 0.3 * rng.standard_normal(shape)
        elif last == "sink":
            a = 1.5 * rng.standard_normal(shape)
        elif last == "lower":
            a = rng.uniform(0.05, 0.9, shape)
        elif name == "embed":
            a = rng.standard_normal(shape)
        elif last == "router":
            a = rng.standard_normal(shape) * (6.0 / np.sqrt(shape[-1]))
        else:
            a = rng.standard_normal(shape) * (2.0 / np.sqrt(shape[-1]))
        w[name] = bf16_to_f32(bf16_bits(np.asarray(a, dtype=np.float32))).reshape(shape)
    return w


def round_bf16(a):
    return bf16_to_f32(bf16_bits(np.asarray(a, dtype=np.float32))).reshape(np.shape(a))


def gpu_model(cfg, weights, compute="float32", max_seq_len=256, max_batch=4, taps=False):
    program, layers = marosun.parse_config(cfg, max_seq_len, max_batch, compute)
    tensors = {n: (B.F32, list(reversed(a.shape)) if a.shape else [1], np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
                   if not a.shape else np.ascontiguousarray(a, dtype=np.float32)) for n, a in weights.items()}
    return B.LayerProgramInference(program, layers, tensors, taps=taps)


def rel_err(got, want):
    """Row-wise: rms of the difference (mean removed) over the rms of the wanted row (mean removed); the largest row."""
    got, want = np.atleast_2d(got).astype(np.float64), np.atleast_2d(want).astype(np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    s = want - want.mean(-1, keepdims=True)
    return float(np.max(np.sqrt((d * d).mean(-1)) / np.sqrt((s * s).mean(-1) + 1e-30)))
