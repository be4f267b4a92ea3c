"""Marosun: a small hybrid decoder whose layers have ONE norm that both sublayers read, x <- x + mixer(N(x)) + ff(N(x)).
config.json -> the library's layer program; model.safetensors -> its tensors.

The design in the library's terms (include/llama_b200.h, "layer-program models"):
  * x = embedding row; norm weights are stored around zero (norm_weight_offset = 1); program.parallel_ff = 1: the feed-forward's first
    projection joins the layer's input projection, and both outputs add into the residual stream;
  * `layers[i].type` picks the mixer:
      "attention"    B200_MIX_SOFTMAX_ATTN: biases on q / k / v and on the output, per-head RMS norm of q and k with a weight, THEN
                     rotary positions on the first rot.dims channels (interleaved pairs, frequencies stretched by rot.scaling), every
                     earlier position visible, a learned extra term per head in the softmax's denominator ('.sink'), and values that
                     carry positions: turned by their own position when cached (all pairs, base rot.base, never stretched), the summed
                     output turned back by the query's position;
      "parallel"     B200_MIX_ATTN_RECURRENT, weighted sum of the branches (left_scale, right_scale): left = softmax attention without
                     biases, norm or rotation over chunks of mask.size positions with a learned extra term and a sigmoid gate per
                     value channel; right = B200_REC_GATED_LINEAR, a matrix memory per head whose forget gate (with a stored lower
                     bound) also says what is written;
      "parallel_2"   B200_MIX_ATTN_RECURRENT, each branch RMS-normed over the width with its own weight, half their sum: left = softmax
                     attention with biases, q / k norm, rotation of q and k only, every earlier position visible, the constant 1 added to
                     the softmax's denominator; right = B200_REC_GATED_UNIT, one gated state per channel;
    all: grouped K/V heads, separate key and value sizes, `scale` from the config;
  * `mlp`: null, {"kind": "dense", "ff", "limit"} = B200_FF_CLAMPED_GLU, or {"kind": "moe", "router": {experts, top}, "expert": {ff}} =
    gated SiLU experts chosen by the largest sigmoid scores, the score multiplying the expert's input;
  * final norm, head.
Tensor names are the file's own (`l<i>.norm1`, `l<i>.mix.q`, `l<i>.mix.left.q.b`, `l<i>.mix.right.lower`, `l<i>.mlp.e<j>.gate`, ...,
`embed`, `head`, `final.norm`)."""
import json
import os

from . import (ACT_SILU_GLU, COMBINE_NORMED_MEAN, COMBINE_WEIGHTED, COMPUTE_BF16, COMPUTE_F32, FF_CLAMPED_GLU, FF_MOE, FF_RELU2, GATE_CHANNEL,
               GATE_NONE, MASK_CAUSAL, MASK_CHUNK, MIX_ATTN_RECURRENT, MIX_SOFTMAX_ATTN, QKNORM_HEAD_WEIGHT, QKNORM_NONE, REC_GATED_LINEAR,
               REC_GATED_UNIT, ROUTE_SIGMOID_TOP, SINK_LEARNED, SINK_ZERO, VMIX_NONE, InvalidArgument, LayerProgramInference, Unsupported)
from .safetensors_io import SafetensorsFile

ARCHITECTURE = "Marosun"
GATE_SLOPE = 1.702      # the dense layer's gate: g * sigmoid(1.702 g)


def _rotation(a, rot):
    """rotary fields of a softmax mixer from a config's "rot" entry (dims, base, optional scaling)"""
    sc = rot.get("scaling") or {}
    a.update(rot_dims=int(rot["dims"]), rot_base=float(rot["base"]), rot_after_norm=1, yarn_factor=float(sc.get("factor", 0.0)),
             yarn_original=float(sc.get("original", 0.0)), yarn_fast=float(sc.get("fast", 0.0)), yarn_slow=float(sc.get("slow", 0.0)))


def _softmax_branch(m, kind):
    """b200_softmax_attn_desc fields of the softmax mixer of layer type `kind` with the sizes and constants of the config entry m"""
    a = {"heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]), "vdim": int(m["vdim"]), "scale": float(m["scale"]),
         "conv": 0, "softcap": 0.0, "dist_bias_exp": 0.0, "v_mix": VMIX_NONE, "rot_dims": 0, "rot_base": 0.0, "v_rot_base": 0.0}
    if kind == "parallel":
        a.update(mask=MASK_CHUNK, mask_size=int(m["mask"]["size"]), qkv_bias=0, o_bias=0, qk_norm=QKNORM_NONE, sink=SINK_LEARNED,
                 out_gate=GATE_CHANNEL)
        return a
    a.update(mask=MASK_CAUSAL, mask_size=0, qkv_bias=1, o_bias=1, qk_norm=QKNORM_HEAD_WEIGHT, out_gate=GATE_NONE)
    _rotation(a, m["rot"])
    if kind == "attention":
        a.update(sink=SINK_LEARNED, v_rot_base=float(m["rot"]["base"]))
    else:
        a.update(sink=SINK_ZERO)
    return a


def parse_config(cfg, max_seq_len, max_batch, compute="bfloat16"):
    """config.json (dict) -> (program dict, layer dicts) for LayerProgramInference.  Every size and constant is read from cfg."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise InvalidArgument(f"not a {ARCHITECTURE} config: architecture = {cfg.get('architecture')!r}")
    if compute not in ("bfloat16", "float32"):
        raise Unsupported(f"compute {compute!r}: bfloat16 or float32")
    program = {
        "width": int(cfg["width"]), "vocab": int(cfg["vocab"]), "max_seq_len": int(max_seq_len), "max_batch": int(max_batch),
        "norm_eps": float(cfg["norm"]["eps"]), "embed_scale": 1.0, "logit_scale": 1.0, "pos_sinusoid": 0,
        "loop_start": 0, "loop_stop": 0, "loop_times": 1, "compute": COMPUTE_F32 if compute == "float32" else COMPUTE_BF16,
        "post_norm": 0, "norm_weight_offset": 1.0, "parallel_ff": 1,
    }
    layers = []
    for i, L in enumerate(cfg["layers"]):
        m, kind = L["mixer"], L["type"]
        if kind == "attention":
            d = {"mixer": MIX_SOFTMAX_ATTN, "sattn": _softmax_branch(m, kind)}
        elif kind == "parallel":
            r = m["right"]
            d = {"mixer": MIX_ATTN_RECURRENT, "sattn": _softmax_branch(m["left"], kind), "rec_kind": REC_GATED_LINEAR,
                 "glin": {"heads": int(r["heads"]), "dim": int(r["dim"]), "vdim": int(r["vdim"])}, "combine": COMBINE_WEIGHTED,
                 "attn_scale": float(m["left_scale"]), "mem_scale": float(m["right_scale"])}
        elif kind == "parallel_2":
            d = {"mixer": MIX_ATTN_RECURRENT, "sattn": _softmax_branch(m["left"], kind), "rec_kind": REC_GATED_UNIT,
                 "gunit": {"width": int(m["right"]["width"])}, "combine": COMBINE_NORMED_MEAN}
        else:
            raise Unsupported(f"layer {i}: mixer type {kind!r}")
        d.update(ff=0, ff_kind=FF_RELU2)
        mlp = L.get("mlp")
        if mlp is not None:
            if mlp.get("kind") == "dense":
                d.update(ff=int(mlp["ff"]), ff_kind=FF_CLAMPED_GLU, ff_limit=float(mlp["limit"]), ff_slope=GATE_SLOPE)
            elif mlp.get("kind") == "moe":
                d.update(ff_kind=FF_MOE, moe={"experts": int(mlp["router"]["experts"]), "top": int(mlp["router"]["top"]),
                                              "expert_ff": int(mlp["expert"]["ff"]), "shared_ff": 0, "act": ACT_SILU_GLU,
                                              "route": ROUTE_SIGMOID_TOP, "route_scale": 0.0, "weight_input": 1})
            else:
                raise Unsupported(f"layer {i}: feed-forward kind {mlp.get('kind')!r}")
        layers.append(d)
    return program, layers


def _softmax_shapes(out, x, m, kind, W):
    nq, nk, nv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
    out.update({x + "q": (nq, W), x + "k": (nk, W), x + "v": (nv, W), x + "o": (W, m["heads"] * m["vdim"])})
    if kind == "parallel":
        out.update({x + "g": (m["heads"] * m["vdim"], W), x + "sink": (m["heads"],)})
        return
    out.update({x + "q.b": (nq,), x + "k.b": (nk,), x + "v.b": (nv,), x + "o.b": (W,), x + "q.norm": (m["dim"],), x + "k.norm": (m["dim"],)})
    if kind == "attention":
        out[x + "sink"] = (m["heads"],)


def tensor_shapes(cfg):
    """name -> shape of every tensor a model of this config must hold"""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    for i, L in enumerate(cfg["layers"]):
        p, m, kind = "l%d." % i, L["mixer"], L["type"]
        out[p + "norm1"] = (W,)
        if kind == "attention":
            _softmax_shapes(out, p + "mix.", m, kind, W)
        else:
            _softmax_shapes(out, p + "mix.left.", m["left"], kind, W)
            r, x = m["right"], p + "mix.right."
            if kind == "parallel":
                n = r["heads"] * r["dim"]
                out.update({x + "q": (n, W), x + "v": (r["heads"] * r["vdim"], W), x + "f": (n, W), x + "f.b": (n,), x + "lower": (n,),
                            x + "norm": (r["vdim"],), x + "o": (W, r["heads"] * r["vdim"])})
            else:
                n = r["width"]
                out.update({x + "z": (n, W), x + "z.b": (n,), x + "x": (n, W), x + "x.b": (n,), x + "g": (n, W), x + "o": (W, n),
                            p + "mix.left.out": (W,), p + "mix.right.out": (W,)})
        mlp = L.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            ff = mlp["expert"]["ff"]
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for e in range(mlp["router"]["experts"]):
                out.update({p + "mlp.e%d.gate" % e: (ff, W), p + "mlp.e%d.up" % e: (ff, W), p + "mlp.e%d.down" % e: (W, ff)})
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
