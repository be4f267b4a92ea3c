"""Madudra: a small hybrid decoder whose layers mix tokens either by latent attention or by a state-space recurrence, with several
residual streams, layer norms and a mixture-of-experts feed-forward.  config.json -> the library's layer program; model.safetensors
-> its tensors.

The design in the library's terms (include/llama_b200.h, "layer-program models"):
  * x = embedding row * `embedding.scale`; the residual is `streams` copies of it (program.streams, residual_mult = `residual_mult`):
    sublayer q of layer i reads layernorm(sum_s hc<q>.in[s] x_s) and its output y makes x_t <- sum_s hc<q>.mix[s][t] x_s +
    residual_mult * hc<q>.out[t] * y; without `streams` there is one copy and x += residual_mult * y; norms are layer norms with a
    weight and no bias (norm_kind = NORM_LAYER), eps = `norm.eps`;
  * `layers[i].type`:
      "latent_attention"  B200_MIX_LATENT_ATTN: queries through a normed latent of `q_rank`, keys and values out of a normed latent of
                          `kv_rank` plus one rotated key part of `rot_dim` shared by the heads (only these are cached), `dim` plain
                          query / key channels and `vdim` value channels per head, rotary positions in the half-split layout with
                          `rot` {dims, base, scaling {factor, original, fast, slow}}, `scale` as given, sliding window `mask.size`,
                          sigmoid gate per value channel from the mixer's input; `kv_from`: j reads layer j's cached rows;
      "mamba2"            B200_MIX_STATE_SPACE: `heads` x `vdim` channels, `state` rows per head, `groups` of B / C, `conv` taps,
                          gated rms norm in `norm_groups` parts;
  * `mlp`: null or {"kind": "moe", "router": {experts, top, scale}, "expert": {ff}}: softmax over all experts, the `top` largest
    weighted by probability * scale, experts W_down gelu(W_up h) with the exact GELU;
  * final layer norm, head.
Tensor names are the file's own (`l<i>.norm1`, `l<i>.hc1.in`, `l<i>.mix.dq`, `l<i>.mix.in`, `l<i>.mlp.e<j>.up`, ..., `embed`, `head`,
`final.norm`)."""
import json
import os

from . import (ACT_GELU, COMPUTE_BF16, COMPUTE_F32, FF_MOE, FF_RELU2, GATE_CHANNEL, MIX_LATENT_ATTN, MIX_STATE_SPACE, NORM_LAYER,
               ROUTE_SOFTMAX_TOP, InvalidArgument, LayerProgramInference, Unsupported)
from .safetensors_io import SafetensorsFile

ARCHITECTURE = "Madudra"


def parse_config(cfg, max_seq_len, max_batch, compute="bfloat16"):
    """config.json (dict) -> (program dict, layer dicts) for LayerProgramInference.  Every size and constant is read from cfg."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise InvalidArgument(f"not a {ARCHITECTURE} config: architecture = {cfg.get('architecture')!r}")
    if compute not in ("bfloat16", "float32"):
        raise Unsupported(f"compute {compute!r}: bfloat16 or float32")
    program = {
        "width": int(cfg["width"]), "vocab": int(cfg["vocab"]), "max_seq_len": int(max_seq_len), "max_batch": int(max_batch),
        "norm_eps": float(cfg["norm"]["eps"]), "embed_scale": float((cfg.get("embedding") or {}).get("scale", 1.0)), "logit_scale": 1.0,
        "pos_sinusoid": 0, "loop_start": 0, "loop_stop": 0, "loop_times": 1,
        "compute": COMPUTE_F32 if compute == "float32" else COMPUTE_BF16, "post_norm": 0, "residual_alpha": 1.0, "norm_weight_offset": 0.0,
        "norm_kind": NORM_LAYER, "streams": int(cfg.get("streams", 1)), "residual_mult": float(cfg.get("residual_mult", 1.0)),
    }
    layers = []
    for i, L in enumerate(cfg["layers"]):
        m = L["mixer"]
        if L["type"] == "latent_attention":
            rot = m.get("rot") or {}
            sc = rot.get("scaling") or {}
            r = {"dims": int(rot.get("dims", 0)), "base": float(rot.get("base", 0.0)), "yarn_factor": float(sc.get("factor", 0.0)),
                 "yarn_original": float(sc.get("original", 0.0)), "yarn_fast": float(sc.get("fast", 0.0)), "yarn_slow": float(sc.get("slow", 0.0))}
            src = m.get("kv_from")
            d = {"mixer": MIX_LATENT_ATTN,
                 "latent": {"heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]), "vdim": int(m["vdim"]),
                            "q_rank": int(m["q_rank"]), "kv_rank": int(m["kv_rank"]), "mask_size": int((m.get("mask") or {}).get("size", 0)),
                            "scale": float(m["scale"]), "rot": r, "kv_from": -1 if src is None else int(src), "out_gate": GATE_CHANNEL}}
        elif L["type"] == "mamba2":
            d = {"mixer": MIX_STATE_SPACE,
                 "ssd": {"heads": int(m["heads"]), "vdim": int(m["vdim"]), "state": int(m["state"]), "groups": int(m["groups"]),
                         "conv": int(m["conv"]), "norm_groups": int(m.get("norm_groups", 1))}}
        else:
            raise Unsupported(f"layer {i}: mixer type {L['type']!r}")
        d.update(ff=0, ff_kind=FF_RELU2)
        mlp = L.get("mlp")
        if mlp is not None:
            if mlp.get("kind") != "moe":
                raise Unsupported(f"layer {i}: feed-forward kind {mlp.get('kind')!r}")
            rt = mlp["router"]
            d.update(ff_kind=FF_MOE, moe={"experts": int(rt["experts"]), "top": int(rt["top"]), "expert_ff": int(mlp["expert"]["ff"]), "shared_ff": 0,
                                          "act": ACT_GELU, "route": ROUTE_SOFTMAX_TOP, "route_scale": float(rt.get("scale", 1.0))})
        layers.append(d)
    return program, layers


def tensor_shapes(cfg):
    """name -> shape of every tensor a model of this config must hold."""
    W, V = cfg["width"], cfg["vocab"]
    S = cfg.get("streams")
    out = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        x = p + "mix."
        out[p + "norm1"] = (W,)
        subs = ["hc1."]
        if L["type"] == "latent_attention":
            H, per = m["heads"], m["dim"] + m["rot_dim"]
            out.update({x + "dq": (m["q_rank"], W), x + "dq.norm": (m["q_rank"],), x + "uq": (H * per, m["q_rank"]),
                        x + "uk": (H * m["dim"], m["kv_rank"]), x + "uv": (H * m["vdim"], m["kv_rank"]), x + "g": (H * m["vdim"], W),
                        x + "o": (W, H * m["vdim"])})
            if m.get("kv_from") is None:
                out.update({x + "dkv": (m["kv_rank"] + m["rot_dim"], W), x + "dkv.norm": (m["kv_rank"],)})
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            out.update({x + "in": (2 * inner + 2 * gn + m["heads"], W), x + "conv": (inner + 2 * gn, m["conv"]), x + "conv.b": (inner + 2 * gn,),
                        x + "dt_bias": (m["heads"],), x + "A_log": (m["heads"],), x + "D": (m["heads"],), x + "norm": (inner,),
                        x + "o": (W, inner)})
        mlp = L.get("mlp")
        if mlp is not None:
            subs.append("hc2.")
            out[p + "norm2"] = (W,)
            ff = mlp["expert"]["ff"]
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for e in range(mlp["router"]["experts"]):
                out.update({p + "mlp.e%d.up" % e: (ff, W), p + "mlp.e%d.down" % e: (W, ff)})
        if S is not None:
            for hc in subs:
                out.update({p + hc + "in": (S,), p + hc + "out": (S,), p + hc + "mix": (S, S)})
    return out


def load(model_dir, max_seq_len=4096, max_batch=8, compute="bfloat16", device=0, taps=False):
    """A folder with config.json and model.safetensors -> a finalized context."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    program, layers = parse_config(cfg, max_seq_len, max_batch, compute)
    st = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))

    want = tensor_shapes(cfg)
    missing = sorted(set(want) - set(st.names()))
    if missing:
        raise InvalidArgument(f"{model_dir}: model.safetensors lacks {missing[:4]}{' ...' if len(missing) > 4 else ''}")
    for name, shape in want.items():
        if tuple(st.shape(name)) != tuple(shape):
            raise InvalidArgument(f"{model_dir}: tensor {name} has shape {st.shape(name)}, the config wants {tuple(shape)}")

    def feeder(upload):
        for name in st.names():
            if name not in want:
                continue
            gg, shape, arr = st.tensor(name)
            if gg is None:
                continue
            upload(name, gg, list(reversed(shape)) if shape else [1], arr)

    try:
        gpu = LayerProgramInference(program, layers, device=device, taps=taps, feeder=feeder)
    finally:
        try:
            st.close()
        except BufferError:
            pass
    gpu.arch = ARCHITECTURE
    gpu.config = cfg
    return gpu
