"""Small Madudra configurations with random weights for the tests, and the glue between the library and the oracle.

Weights are drawn in float32 and rounded to bfloat16-representable values, so that the library (either compute mode) and the float64
oracle hold exactly the same numbers."""
import math

import numpy as np

import llama_gguf_b200 as B
from llama_gguf_b200 import madudra
from llama_gguf_b200.safetensors_io import bf16_bits, bf16_to_f32


def moe(experts=5, top=2, ff=24, scale=1.3):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff}}


def latent(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=32, window=9, scale=None, base=1000.0, scaling="default", kv_from=None,
           rot_dims=None, mlp=None):
    rot = {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}
    if scaling == "default":
        scaling = {"factor": 3.0, "original": 64, "fast": 16.0, "slow": 1.0}
    if scaling:
        rot["scaling"] = scaling
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "mask": {"size": window},
          "rot": rot, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def scan(heads=4, vdim=12, state=16, groups=2, conv=4, norm_groups=2, mlp=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups},
            "mlp": mlp}


def config(layers, width=64, vocab=96, eps=1e-5, streams=2, mult=0.6, embed_scale=3.0):
    cfg = {"architecture": "Madudra", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
           "residual_mult": mult, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    return cfg


def random_weights(cfg, seed=0):
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in madudra.tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        part = name.split(".")[1] if "." in name else ""
        if part in ("hc1", "hc2"):
            if last == "mix":
                a = np.eye(shape[0]) + 0.3 * rng.standard_normal(shape)
            elif last == "in":
                a = 1.0 / shape[0] + 0.3 * rng.standard_normal(shape)
            else:
                a = 1.0 + 0.3 * rng.standard_normal(shape)
        elif last in ("norm1", "norm2", "norm") or name == "final.norm":
            a = 1.0 + 0.3 * rng.standard_normal(shape)
        elif last == "conv":
            a = 0.6 * rng.standard_normal(shape)
        elif last == "b":
            a = 0.3 * rng.standard_normal(shape)
        elif last == "dt_bias":
            a = rng.uniform(-3.0, 0.5, shape)
        elif last == "A_log":
            a = rng.uniform(-1.5, 1.0, shape)
        elif last == "D":
            a = rng.standard_normal(shape)
        elif name == "embed":
            a = rng.standard_normal(shape)
        elif last == "router":
            a = rng.standard_normal(shape) * (4.0 / math.sqrt(shape[-1]))
        else:
            a = rng.standard_normal(shape) * (1.5 / math.sqrt(shape[-1]))
        w[name] = bf16_to_f32(bf16_bits(np.asarray(a, dtype=np.float32))).reshape(shape)
    return w


def gpu_model(cfg, weights, compute="float32", max_seq_len=256, max_batch=4, taps=False):
    program, layers = madudra.parse_config(cfg, max_seq_len, max_batch, compute)
    tensors = {n: (B.F32, list(reversed(a.shape)) if a.shape else [1], np.ascontiguousarray(a, dtype=np.float32)) for n, a in weights.items()}
    return B.LayerProgramInference(program, layers, tensors, taps=taps)


def f64(weights):
    return {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}


def rel_err(got, want):
    """Row-wise: rms of the difference (mean removed) over the rms of the wanted row (mean removed); the largest row."""
    got, want = np.atleast_2d(got).astype(np.float64), np.atleast_2d(want).astype(np.float64)
    d = got - want
    d = d - d.mean(axis=1, keepdims=True)
    w = want - want.mean(axis=1, keepdims=True)
    return float((np.sqrt((d * d).mean(axis=1)) / np.maximum(np.sqrt((w * w).mean(axis=1)), 1e-30)).max())
