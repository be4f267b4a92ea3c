"""bench.py --design lazilorn | mefurax | madudra | marosun: prefill and decode throughput of a layer-program design at sizes that resemble a real model's
layers (random weights), beside the library's closest existing model -- a llama-architecture transformer of the same width, depth
and parameter count in Q8_0 blocks (the densest weight type its tensor-core prompt path takes); Mefurax also beside Lazilorn at
the same width and depth (the other bf16 layer program, whose attention and GEMM kernels it shares); Madudra beside Lazilorn (the
other hybrid of attention and recurrent scans) and Mefurax (the other mixture of experts) at the same width and depth; Marosun beside
the same two (Lazilorn: attention beside a matrix memory; Mefurax: softmax mixers with rotation and experts).

Per size and model: prompt tokens/s for one prompt of --prefill-len tokens, decode tokens/s at batch 1 and at --batch sequences
after prompts of --prompt-len tokens.  Every number is host wall clock around the library call (each call ends with a stream
synchronisation), after warm-up calls, so launch overhead and the copies of tokens and results are inside.  One JSON line."""
import json
import sys
import time

import numpy as np

SIZES = {
    # name: width, layers (p = attention beside a matrix memory, d = gated delta rule), attention heads / kv heads, ff
    "w1024": dict(width=1024, pattern="pdppdp", heads=8, kv_heads=2, ff=4096, vocab=32000),
    "w2048": dict(width=2048, pattern="pdppdppd", heads=16, kv_heads=4, ff=8192, vocab=32000),
}


def lazilorn_config(s, window=1024, keep_first=4):
    layers = []
    for ch in s["pattern"]:
        if ch == "p":
            layers.append({"type": "parallel", "mlp": {"kind": "dense", "ff": s["ff"]},
                           "mixer": {"left": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": 128, "vdim": 128,
                                              "mask": {"size": window, "keep_first": keep_first}, "scale": 128 ** -0.5},
                                     "right": {"heads": s["heads"] // 2, "dim": 64, "vdim": 128, "gate_cap": 15.0},
                                     "left_scale": 0.7, "right_scale": 0.7}})
        else:
            layers.append({"type": "delta", "mlp": {"kind": "dense", "ff": s["ff"]},
                           "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": 128, "vdim": 128, "conv": 4}})
    return {"architecture": "Lazilorn", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "logit_scale": 1.0, "loop": {"start": 0, "stop": 0, "times": 1}, "layers": layers}


MEFURAX_SIZES = {
    # name: width, layers (a = windowed mixer with convolution and distance bias, b = chunked rotary mixer; the first layer's feed-forward
    # is dense, the others are mixtures), heads / kv heads, dense ff, experts / chosen / expert ff / always-on ff
    "w1024": dict(width=1024, pattern="bbabba", heads=8, kv_heads=2, ff=4096, experts=8, top=2, eff=1024, sff=1024, vocab=32000),
    "w2048": dict(width=2048, pattern="bbabbbab", heads=16, kv_heads=4, ff=8192, experts=8, top=2, eff=2048, sff=2048, vocab=32000),
}


def mefurax_config(s, span=1024):
    layers = []
    for i, ch in enumerate(s["pattern"]):
        mlp = {"kind": "dense", "ff": s["ff"]} if i == 0 else {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]},
                                                               "expert": {"ff": s["eff"]}, "shared": {"ff": s["sff"]}}
        m = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": 128, "vdim": 128, "mask": {"size": span}, "scale": 128 ** -0.5, "v_mix": True}
        if ch == "a":
            m["conv"] = 4
        else:
            m.update(rot={"dims": 64, "base": 10000.0}, softcap=50.0)
        layers.append({"type": "attention" if ch == "a" else "attention_2", "mixer": m, "mlp": mlp})
    return {"architecture": "Mefurax", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-6}, "postln_alpha": 2.0, "layers": layers}


MADUDRA_SIZES = {
    # name: width, layers (l = latent attention with its own cache rows, k = latent attention on layer 0's rows, m = state-space mixer; every
    # layer with a mixture of experts), attention heads, query latent, state-space heads, experts / chosen / expert ff, residual streams
    "w1024": dict(width=1024, pattern="lmmkmm", heads=8, q_rank=512, ssd_heads=16, experts=8, top=2, eff=1024, streams=4, vocab=32000),
    "w2048": dict(width=2048, pattern="lmmkmmkm", heads=16, q_rank=768, ssd_heads=32, experts=8, top=2, eff=2048, streams=4, vocab=32000),
}


def madudra_config(s, span=1024):
    # cached row = 96 latent + 32 rotated = 128 floats (the width the tile attention kernel takes); heads of 64 + 32 query / key and 128
    # value channels; state-space heads of 128 channels with 128 state rows (inner = 2 x width)
    layers = []
    mlp = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"], "scale": 1.0}, "expert": {"ff": s["eff"]}}
    for ch in s["pattern"]:
        if ch == "m":
            layers.append({"type": "mamba2", "mlp": mlp,
                           "mixer": {"heads": s["ssd_heads"], "vdim": 128, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1}})
            continue
        m = {"heads": s["heads"], "dim": 64, "rot_dim": 32, "vdim": 128, "q_rank": s["q_rank"], "kv_rank": 96, "mask": {"size": span},
             "scale": 96 ** -0.5, "rot": {"dims": 32, "base": 10000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
        if ch == "k":
            m["kv_from"] = 0
        layers.append({"type": "latent_attention", "mixer": m, "mlp": mlp})
    return {"architecture": "Madudra", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "residual_mult": 0.5, "streams": s["streams"], "layers": layers}


MAROSUN_SIZES = {
    # name: width, layers (a = attention with turned values, q = attention beside a gated unit, p = chunked attention beside a gated linear
    # memory; D = dense clamped feed-forward, M = mixture of gated experts), heads / kv heads, dense ff, experts / chosen / expert ff
    "w1024": dict(width=1024, pattern=["aD", "aM", "qD", "pM", "aD", "pM"], heads=8, kv_heads=2, ff=4096, experts=8, top=2, eff=1024, vocab=32000),
    "w2048": dict(width=2048, pattern=["aD", "aM", "qD", "pM", "aD", "aM", "qD", "pM"], heads=16, kv_heads=4, ff=8192, experts=8, top=2, eff=2048,
                  vocab=32000),
}


def marosun_config(s, span=1024):
    # heads of 128 key and 128 value channels; the memory branch has as many heads of 128 x 128 state; the gated unit is twice the width
    layers = []
    rot = {"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    for ch, ff in s["pattern"]:
        mlp = {"kind": "dense", "ff": s["ff"], "limit": 7.0} if ff == "D" else {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]},
                                                                                "expert": {"ff": s["eff"]}}
        soft = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": 128, "vdim": 128, "scale": 128 ** -0.5}
        if ch == "a":
            layers.append({"type": "attention", "mixer": dict(soft, rot=rot), "mlp": mlp})
        elif ch == "q":
            layers.append({"type": "parallel_2", "mlp": mlp,
                           "mixer": {"left": dict(soft, rot={"dims": 128, "base": 10000.0}), "right": {"width": 2 * s["width"]}}})
        else:
            layers.append({"type": "parallel", "mlp": mlp,
                           "mixer": {"left": dict(soft, mask={"size": span}), "right": {"heads": s["heads"], "dim": 128, "vdim": 128},
                                     "left_scale": 0.7, "right_scale": 0.7}})
    return {"architecture": "Marosun", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-6}, "layers": layers}


def lazilorn_feeder(cfg, seed, tensor_shapes=None):
    """upload(name, type, ne, data) for every tensor of cfg: bf16 bit patterns of N(0, 1/fan_in) matrices, f32 vectors."""
    import llama_gguf_b200 as B
    from llama_gguf_b200.safetensors_io import bf16_bits
    if tensor_shapes is None:
        from llama_gguf_b200.lazilorn import tensor_shapes

    def feed(upload):
        rng = np.random.default_rng(seed)
        for name, shape in tensor_shapes(cfg).items():
            last = name.split(".")[-1]
            if ".hc" in name:      # stream weights near the plain residual
                a = {"mix": lambda: np.eye(shape[0]) + 0.05 * rng.standard_normal(shape), "in": lambda: np.full(shape, 1.0 / shape[0]),
                     "out": lambda: np.ones(shape)}[last]()
                upload(name, B.F32, list(reversed(shape)), np.ascontiguousarray(a, dtype=np.float32))
                continue
            if len(shape) == 2 and last != "conv" and name != "loop.step":
                a = rng.standard_normal(shape, dtype=np.float32) * np.float32(1.0 / np.sqrt(shape[-1]))
                upload(name, B.BF16, list(reversed(shape)), bf16_bits(a).reshape(shape))
                continue
            if last == "conv":
                a = 0.5 * rng.standard_normal(shape)
            elif name.endswith("f.b"):
                a = rng.uniform(1.0, 4.0, shape)
            elif last == "lower":
                a = rng.uniform(0.0, 0.9, shape)
            elif last in ("A_log", "dt_bias", "b") and len(shape) == 1:
                a = rng.uniform(-2.0, 0.5, shape)
            elif (last in ("norm1", "norm2", "vmix") or name == "final.norm") and cfg["architecture"] in ("Mefurax", "Marosun"):
                a = 0.1 * rng.standard_normal(shape) + (0.4 if last == "vmix" else 0.0)
            else:
                a = 1.0 + 0.1 * rng.standard_normal(shape)
            upload(name, B.F32, list(reversed(shape)) if shape else [1], np.ascontiguousarray(a, dtype=np.float32).reshape(shape if shape else (1,)))
    return feed


def design_module(cfg):
    from llama_gguf_b200 import lazilorn, madudra, marosun, mefurax
    return {"Lazilorn": lazilorn, "Mefurax": mefurax, "Madudra": madudra, "Marosun": marosun}[cfg["architecture"]]


def n_params(cfg):
    return int(sum(np.prod(s) for n, s in design_module(cfg).tensor_shapes(cfg).items() if n != "embed"))


def timed(fn, warm, reps):
    for _ in range(warm):
        fn()
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    return (time.perf_counter() - t0) / reps


def bench_lazilorn(cfg, args, max_seq):
    import llama_gguf_b200 as B
    mod = design_module(cfg)
    program, layers = mod.parse_config(cfg, max_seq, max(args.batch, 1) + 1, "bfloat16")
    gpu = B.LayerProgramInference(program, layers, feeder=lazilorn_feeder(cfg, args.seed, mod.tensor_shapes))
    V = cfg["vocab"]
    rng = np.random.default_rng(args.seed + 1)
    out = {}
    if args.prefill_len:
        toks = [int(t) for t in rng.integers(0, V, args.prefill_len)]

        def one():
            gpu.reset(0)
            gpu.step([(0, toks)], [len(toks) - 1])
        out["prefill_tok_s"] = args.prefill_len / timed(one, 2, 4)
    st0 = gpu.stats()["kernel_launches"]
    for nb, key in ((1, "decode_b1_tok_s"), (args.batch, "decode_b%d_tok_s" % args.batch)):
        if nb < 1:
            continue
        for s in range(nb):
            gpu.reset(s)
        gpu.step([(s, [int(t) for t in rng.integers(0, V, args.prompt_len)]) for s in range(nb)])
        state = {"t": [1] * nb}

        def one():
            state["t"] = gpu.decode_batch_greedy(list(range(nb)), state["t"])
        out[key] = nb / timed(one, args.warmup, args.steps)
    out["kernel_launches"] = gpu.stats()["kernel_launches"] - st0
    out["weight_bytes_per_token"] = gpu.stats()["weight_bytes_per_token"]
    gpu.close()
    return out


def bench_llama(s, n_layers, ffn, args, max_seq):
    import llama_gguf_b200 as B
    from llama_gguf_b200.presets import make_desc
    from llama_gguf_b200.randmodel import random_model
    preset = dict(arch="llama", hidden=s["width"], n_layers=n_layers, n_heads=s["width"] // 128, n_kv_heads=s["kv_heads"], head_dim=128,
                  ffn=ffn, vocab=s["vocab"], norm_eps=1e-5, rope_base=1e4, rope_neox=0, bias=False, tied=False)
    desc = make_desc(preset, max_seq, max(args.batch, 1))
    gpu = B.GpuOnlyInference(desc, None, feeder=lambda up: random_model(preset, "Q8_0", max_seq, seed=args.seed, upload=up))
    V = s["vocab"]
    rng = np.random.default_rng(args.seed + 1)
    out = {"path": gpu.path()}
    if args.prefill_len:
        toks = [int(t) for t in rng.integers(0, V, args.prefill_len)]

        def one():
            gpu.reset(0)
            gpu.forward_batch(toks, 0)
        out["prefill_tok_s"] = args.prefill_len / timed(one, 2, 4)
    for nb, key in ((1, "decode_b1_tok_s"), (args.batch, "decode_b%d_tok_s" % args.batch)):
        if nb < 1:
            continue
        for q in range(nb):
            gpu.reset(q)
            gpu.forward_batch([int(t) for t in rng.integers(0, V, args.prompt_len)], q)
        state = {"t": [1] * nb}

        def one():
            state["t"] = gpu.decode_batch_greedy(list(range(nb)), state["t"])
        out[key] = nb / timed(one, args.warmup, args.steps)
    out["weight_bytes_per_token"] = gpu.stats()["weight_bytes_per_token"]
    gpu.close()
    return out


def main(args):
    import llama_gguf_b200 as B
    if B.device_count() == 0:
        print("bench.py --design: no CUDA device", file=sys.stderr)
        return 2
    if args.design == "mefurax":
        return main_mefurax(args)
    if args.design == "madudra":
        return main_madudra(args)
    if args.design == "marosun":
        return main_marosun(args)
    sizes = [x for x in (args.sizes.split(",") if args.sizes else SIZES) if x]
    max_seq = max(args.prefill_len, args.prompt_len + args.warmup + args.steps + 8) + 8
    res = {}
    for name in sizes:
        s = SIZES[name]
        cfg = lazilorn_config(s)
        params = n_params(cfg)
        # llama layer: 4 w^2 (1 + kv/heads)/2-ish attention + 3 w ffn; pick ffn so that the parameter counts match
        w, L = s["width"], len(s["pattern"])
        attn = w * w * 2 + 2 * w * s["kv_heads"] * 128
        ffn = max(256, int(round(((params - s["vocab"] * w) / L - attn) / (3 * w) / 256)) * 256)
        r = {"params_without_embedding": params, "layers": s["pattern"], "lazilorn_bf16": bench_lazilorn(cfg, args, max_seq),
             "llama_q8_0": dict(bench_llama(s, L, ffn, args, max_seq), ffn=ffn)}
        res[name] = r
        print(name, json.dumps(r), file=sys.stderr, flush=True)
    print(json.dumps({"bench": "design", "design": "lazilorn", "unit": "tok/s", "prefill_len": args.prefill_len, "prompt_len": args.prompt_len,
                      "batch": args.batch, "steps": args.steps, "warmup": args.warmup, "timing": "host wall clock around the library calls",
                      "dtype": "bf16 (lazilorn) / Q8_0 (llama)", "data": "synthetic", "sizes": res}))
    return 0


def main_mefurax(args):
    sizes = [x for x in (args.sizes.split(",") if args.sizes else MEFURAX_SIZES) if x]
    max_seq = max(args.prefill_len, args.prompt_len + args.warmup + args.steps + 8) + 8
    res = {}
    for name in sizes:
        s = MEFURAX_SIZES[name]
        cfg = mefurax_config(s)
        params = n_params(cfg)
        # parameters a token multiplies with: every mixer, the dense layer, router + `top` experts + the always-on expert of the others
        w, L = s["width"], len(s["pattern"])
        active = params - (L - 1) * (s["experts"] - s["top"]) * 2 * w * s["eff"]
        attn = w * w * 2 + 2 * w * s["kv_heads"] * 128
        ffn = max(256, int(round(((active - s["vocab"] * w) / L - attn) / (3 * w) / 256)) * 256)
        r = {"params_without_embedding": params, "active_params_without_embedding": active, "layers": s["pattern"],
             "mefurax_bf16": bench_lazilorn(cfg, args, max_seq)}
        print(name, json.dumps(r), file=sys.stderr, flush=True)
        r["lazilorn_bf16"] = bench_lazilorn(lazilorn_config(SIZES[name]), args, max_seq)
        r["llama_q8_0"] = dict(bench_llama(s, L, ffn, args, max_seq), ffn=ffn)
        res[name] = r
        print(name, json.dumps(r), file=sys.stderr, flush=True)
    print(json.dumps({"bench": "design", "design": "mefurax", "unit": "tok/s", "prefill_len": args.prefill_len, "prompt_len": args.prompt_len,
                      "batch": args.batch, "steps": args.steps, "warmup": args.warmup, "timing": "host wall clock around the library calls",
                      "dtype": "bf16 (mefurax, lazilorn) / Q8_0 (llama, sized to mefurax's active parameters)", "data": "synthetic", "sizes": res}))
    return 0


def main_madudra(args):
    sizes = [x for x in (args.sizes.split(",") if args.sizes else MADUDRA_SIZES) if x]
    max_seq = max(args.prefill_len, args.prompt_len + args.warmup + args.steps + 8) + 8
    res = {}
    for name in sizes:
        s = MADUDRA_SIZES[name]
        cfg = madudra_config(s)
        params = n_params(cfg)
        active = params - len(s["pattern"]) * (s["experts"] - s["top"]) * 2 * s["width"] * s["eff"]
        r = {"params_without_embedding": params, "active_params_without_embedding": active, "layers": s["pattern"],
             "madudra_bf16": bench_lazilorn(cfg, args, max_seq)}
        print(name, json.dumps(r), file=sys.stderr, flush=True)
        r["lazilorn_bf16"] = bench_lazilorn(lazilorn_config(SIZES[name]), args, max_seq)
        r["mefurax_bf16"] = bench_lazilorn(mefurax_config(MEFURAX_SIZES[name]), args, max_seq)
        res[name] = r
        print(name, json.dumps(r), file=sys.stderr, flush=True)
    print(json.dumps({"bench": "design", "design": "madudra", "unit": "tok/s", "prefill_len": args.prefill_len, "prompt_len": args.prompt_len,
                      "batch": args.batch, "steps": args.steps, "warmup": args.warmup, "timing": "host wall clock around the library calls",
                      "dtype": "bf16 (madudra, lazilorn, mefurax at the same width and depth)", "data": "synthetic", "sizes": res}))
    return 0


def main_marosun(args):
    sizes = [x for x in (args.sizes.split(",") if args.sizes else MAROSUN_SIZES) if x]
    max_seq = max(args.prefill_len, args.prompt_len + args.warmup + args.steps + 8) + 8
    res = {}
    for name in sizes:
        s = MAROSUN_SIZES[name]
        cfg = marosun_config(s)
        params = n_params(cfg)
        n_moe = sum(1 for p in s["pattern"] if p[1] == "M")
        active = params - n_moe * (s["experts"] - s["top"]) * 3 * s["width"] * s["eff"]
        r = {"params_without_embedding": params, "active_params_without_embedding": active, "layers": ",".join(s["pattern"]),
             "marosun_bf16": bench_lazilorn(cfg, args, max_seq)}
        print(name, json.dumps(r), file=sys.stderr, flush=True)
        r["lazilorn_bf16"] = bench_lazilorn(lazilorn_config(SIZES[name]), args, max_seq)
        r["mefurax_bf16"] = bench_lazilorn(mefurax_config(MEFURAX_SIZES[name]), args, max_seq)
        res[name] = r
        print(name, json.dumps(r), file=sys.stderr, flush=True)
    print(json.dumps({"bench": "design", "design": "marosun", "unit": "tok/s", "prefill_len": args.prefill_len, "prompt_len": args.prompt_len,
                      "batch": args.batch, "steps": args.steps, "warmup": args.warmup, "timing": "host wall clock around the library calls",
                      "dtype": "bf16 (marosun, lazilorn, mefurax at the same width and depth)", "data": "synthetic", "sizes": res}))
    return 0
